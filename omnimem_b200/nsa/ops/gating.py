"""Gate + sum of the three attention branches, differentiable.

The reference does this with eager tensor ops inside the attention module
(models/transformers/causal_wan_nsa_model.py:378-386 and 541-546):

    g = clamp(g_proj(x).view(..., H, 3), -10, 10)
    g_cmp, g_slc, g_swa = g.sigmoid().unbind(-1)        # or softmax(-1) for gate_mode == 'softmax'
    x = g_cmp[..., None] * o_cmp + g_slc[..., None] * o_slc + g_swa[..., None] * o_swa
    # skip_module == 'cmp' / 'slc' drops that term

`gated_branch_sum` takes the raw gate logits and the branch outputs and does clamp, gate and
sum in one pass (and their gradients in one pass in backward).
"""
from __future__ import annotations

from typing import Optional

import torch

from ... import ops


class _GatedSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g_logits, o_cmp, o_slc, o_swa, gate_mode):
        ctx.gate_mode = gate_mode
        ctx.save_for_backward(g_logits, o_cmp, o_slc, o_swa)
        return ops.gate_combine(g_logits, o_cmp, o_slc, o_swa, gate_mode)

    @staticmethod
    def backward(ctx, dx):
        g_logits, o_cmp, o_slc, o_swa = ctx.saved_tensors
        dg, da, db, dc = ops.gate_combine_bwd(g_logits, o_cmp, o_slc, o_swa, dx, ctx.gate_mode)
        return dg, da, db, dc, None


def gated_branch_sum(g_logits: torch.Tensor, o_cmp: Optional[torch.Tensor], o_slc: Optional[torch.Tensor],
                     o_swa: Optional[torch.Tensor], gate_mode: str = "sigmoid",
                     skip_module: Optional[str] = None) -> torch.Tensor:
    """g_logits [B, M, H, 3] (the output of g_proj, not yet clamped), branches [B, M, H, D]."""
    if skip_module == "cmp":
        o_cmp = None
    elif skip_module == "slc":
        o_slc = None
    return _GatedSum.apply(g_logits, o_cmp, o_slc, o_swa, gate_mode)
