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


def _fail(kind, text):
    raise kind(text)


def _check_arguments(q, k, v, block_indices, block_size, chunk_size, group_size, causal, allow_ragged):
    """The reference facade's argument contract (selection/__init__.py:16-44), with its exception
    types and messages, checked shape first, values last; the id range check costs one host
    synchronisation, as it does there.  Returns the number of key blocks."""
    B, M, H, D = q.shape
    N, G = k.shape[1], group_size
    kv_shape = (B, N, H, D)
    for name, t in (("k", k), ("v", v)):
        if tuple(t.shape) != kv_shape:
            _fail(AssertionError, f"expected {name} {kv_shape}, got {tuple(t.shape)}")
    if D < 16:
        _fail(AssertionError, f"expected D >= 16, but got {D}")
    if M % G and not allow_ragged:
        _fail(AssertionError, f"M ({M}) must be divisible by group_size ({G})")
    rows = (M + G - 1) // G
    if block_indices.dim() != 4 or tuple(block_indices.shape[:3]) != (B, rows, H):
        _fail(AssertionError, f"Expected block_indices {(B, rows, H, '*')}, got {tuple(block_indices.shape)}")
    if chunk_size <= 0:
        _fail(ValueError, f"chunk_size must be > 0, got {chunk_size}")
    if causal and G > 1 and chunk_size % G and not allow_ragged:
        _fail(AssertionError, f"causal + group requires chunk_size ({chunk_size}) divisible by group_size ({G})")
    if block_indices.shape[-1] == 0:
        _fail(ValueError, "top_idx last dim T must be > 0")
    n_blocks = math.ceil(N / block_size)
    if block_indices.numel():
        lo, hi = (int(x) for x in torch.aminmax(block_indices))
        if hi >= n_blocks:
            _fail(ValueError, f"top_idx out of range: expected in [-1, {n_blocks - 1}] but got [{lo}, {hi}]")
    return n_blocks


def _check_no_duplicates(block_indices):
    """OMNIMEM_NSA_DEBUG: a row must not list a valid block twice (selection/__init__.py:47-53)."""
    ordered = block_indices.to(torch.int64).sort(dim=-1).values
    same = ordered.diff(dim=-1) == 0
    if bool((same & (ordered[..., 1:] >= 0)).any()):
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
    # option checks in the reference's order, with its exception types and messages (:70-77)
    problems = (
        (variant not in ('one-pass', 'two-pass'), ValueError,
         f"Invalid variant: {variant!r}, expected 'one-pass' or 'two-pass'"),
        (group_size < 1, ValueError, f"Invalid group_size: {group_size}, expected >= 1"),
        (variant == 'one-pass', NotImplementedError, f"{variant=} is not supported"),
        (bwd_method not in ('auto', 'mask', 'inverted'), ValueError,
         f"Unknown bwd_method '{bwd_method}', expected 'auto', 'inverted' or 'mask'"),
    )
    for bad, kind, text in problems:
        if bad:
            _fail(kind, text)
    _check_arguments(q, k, v, block_indices, block_size, chunk_size, group_size, causal, allow_ragged)
    if _debug_checks_enabled():
        _check_no_duplicates(block_indices)
    if block_indices.dtype != torch.int32:
        block_indices = block_indices.to(torch.int32)
    return SelectionAttentionB200.apply(q, k, v, block_indices, block_size, chunk_size, scale, causal,
                                        return_lse, group_size)
