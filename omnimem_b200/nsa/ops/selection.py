"""Dense selection attention facade; same signature, validation and error behaviour as the
reference's ``omnimem/nsa/ops/selection/__init__.py`` (selection_attention :56-100,
_validate_common :16-44) with the autograd function of ``cuda_backend/autograd.py:9-43``.

One extension: ``allow_ragged=True`` accepts M that is not a multiple of group_size (a short
last query group)."""
import math
import os

import torch

from ... import ops as _ops

__all__ = ["selection_attention", "SelectionAttentionB200"]


def _debug_checks_enabled() -> bool:
    return os.environ.get("OMNIMEM_NSA_DEBUG", "0") not in ("", "0", "false", "False")


def _validate_common(q, k, v, block_indices, block_size, chunk_size, group_size, causal, allow_ragged=False):
    B, M, H, D = q.shape
    N = k.shape[1]
    G = group_size
    assert k.shape == (B, N, H, D), f"expected k {(B, N, H, D)}, got {tuple(k.shape)}"
    assert v.shape == (B, N, H, D), f"expected v {(B, N, H, D)}, got {tuple(v.shape)}"
    assert D >= 16, f"expected D >= 16, but got {D}"
    if not allow_ragged:
        assert M % G == 0, f"M ({M}) must be divisible by group_size ({G})"
    MG = -(-M // G)
    assert block_indices.dim() == 4 and block_indices.shape[:3] == (B, MG, H), (
        f"Expected block_indices {(B, MG, H, '*')}, got {tuple(block_indices.shape)}")
    if chunk_size <= 0:
        raise ValueError(f"chunk_size must be > 0, got {chunk_size}")
    if causal and G > 1 and not allow_ragged:
        assert chunk_size % G == 0, (
            f"causal + group requires chunk_size ({chunk_size}) divisible by group_size ({G})")
    if block_indices.shape[-1] == 0:
        raise ValueError("top_idx last dim T must be > 0")
    num_blocks = math.ceil(N / block_size)
    valid_mask = block_indices >= 0                     # one host sync per call, as the reference
    if valid_mask.any() and torch.any(block_indices[valid_mask] >= num_blocks):
        raise ValueError(
            f"top_idx out of range: expected in [-1, {num_blocks - 1}] "
            f"but got [{block_indices.min()}, {block_indices.max()}]")
    return num_blocks


def _debug_check_unique(block_indices):
    ids = block_indices.to(torch.int64)
    sorted_ids, _ = ids.sort(dim=-1)
    dup = (sorted_ids[..., 1:] == sorted_ids[..., :-1]) & (sorted_ids[..., 1:] >= 0)
    if dup.any():
        raise ValueError("duplicate valid block ids within a row are not allowed (OMNIMEM_NSA_DEBUG)")


class SelectionAttentionB200(torch.autograd.Function):
    """Autograd wrapper over nsa_sel_fwd / nsa_sel_bwd."""

    @staticmethod
    def forward(ctx, q, k, v, block_indices, block_size, chunk_size, scale, causal, return_lse, group_size):
        if scale is None:
            scale = q.shape[-1] ** -0.5
        # fp32 tensors are computed on bf16 operands with fp32 accumulation (the kernels are 16-bit;
        # the reference's default for fp32 is TF32, also a reduced-precision product) and the results
        # are returned in fp32.
        io_dtype = q.dtype
        if io_dtype == torch.float32:
            q, k, v = q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)
        kv = _ops.DenseKV(k, v)
        out, lse = _ops.sel_fwd(q, kv, block_indices, block_size, chunk_size, scale, causal, group_size)
        ctx.save_for_backward(q, k, v, block_indices, out, lse)
        ctx.cfg = (block_size, chunk_size, scale, causal, group_size, io_dtype)
        ctx.mark_non_differentiable(lse)
        out = out.to(io_dtype)
        return (out, lse) if return_lse else out

    @staticmethod
    def backward(ctx, d_out, *unused):
        q, k, v, block_indices, out, lse = ctx.saved_tensors
        block_size, chunk_size, scale, causal, group_size, io_dtype = ctx.cfg
        dq, dk, dv = _ops.sel_bwd(q, _ops.DenseKV(k, v), block_indices, out, lse, d_out.to(q.dtype),
                                  block_size, chunk_size, scale, causal, group_size)
        return dq.to(io_dtype), dk.to(io_dtype), dv.to(io_dtype), None, None, None, None, None, None, None


def selection_attention(q, k, v, block_indices, block_count, block_size, chunk_size=1, scale=None,
                        variant='two-pass', causal=False, return_lse=False, allow_tf32=True,
                        bwd_method='auto', group_size=1, allow_ragged=False):
    """out [B,M,H,D] (and lse fp32 [B,H,M] when return_lse), differentiable in q, k, v.

    ``variant``, ``allow_tf32`` and ``bwd_method`` are validated like the reference and
    otherwise ignored: there is one forward and one (atomics-free) backward."""
    if variant not in ('one-pass', 'two-pass'):
        raise ValueError(f"Invalid variant: {variant!r}, expected 'one-pass' or 'two-pass'")
    if group_size < 1:
        raise ValueError(f"Invalid group_size: {group_size}, expected >= 1")
    if variant == 'one-pass':
        raise NotImplementedError(f"{variant=} is not supported")
    if bwd_method not in ('auto', 'mask', 'inverted'):
        raise ValueError(f"Unknown bwd_method '{bwd_method}', expected 'auto', 'inverted' or 'mask'")
    _validate_common(q, k, v, block_indices, block_size, chunk_size, group_size, causal, allow_ragged)
    if _debug_checks_enabled():
        _debug_check_unique(block_indices)
    if block_indices.dtype != torch.int32:
        block_indices = block_indices.to(torch.int32)
    return SelectionAttentionB200.apply(q, k, v, block_indices, block_size, chunk_size, scale, causal,
                                        return_lse, group_size)
