"""Tensor-level wrappers over the C ABI (one Python function per entry point).

Every function runs on the current CUDA stream of its first tensor's device, allocates
its outputs and scratch with torch's caching allocator, and never synchronises.  Inputs
whose innermost stride is not 1 or whose rows are not 16-byte aligned are copied once
(`_rows16`); everything else is passed by stride.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import NSABackendError, KVSource, TopkMask, call, strides3, strides4

_DTYPES = {torch.bfloat16: _lib.NSA_BF16, torch.float16: _lib.NSA_F16, torch.float32: _lib.NSA_F32}


def _dtype(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise NSABackendError(f"unsupported dtype {t.dtype}") from None


def _require_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise NSABackendError("omnimem_b200 ops need CUDA tensors (there is no CPU path)")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _rows16(t: torch.Tensor) -> torch.Tensor:
    """Return t or a contiguous copy such that stride(-1) == 1 and every leading stride
    and the base address are multiples of 16 bytes."""
    esz = t.element_size()
    ok = t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and all((s * esz) % 16 == 0 for s in t.stride()[:-1])
    return t if ok else t.contiguous()


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _i32(x, what: str) -> int:
    x = int(x)
    if not -2 ** 31 <= x < 2 ** 31:
        raise NSABackendError(f"{what}={x} does not fit in int32")
    return x


# ------------------------------------------------------------------------------------ pooling
def pool_rows(x: torch.Tensor, size: int) -> torch.Tensor:
    """Mean over runs of `size` rows of dim 1 of x [B,N,H,D] -> [B,ceil(N/size),H,D]."""
    _require_cuda(x)
    B, N, H, D = x.shape
    x = _rows16(x)
    nb = (N + size - 1) // size
    out = torch.empty(B, nb, H, D, dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        call("nsa_pool_rows", x.data_ptr(), strides3(x), out.data_ptr(), strides3(out), B, N, H, D,
             _i32(size, "size"), _dtype(x), _stream(x))
    return out


# -------------------------------------------------------------------------------------- top-k
def _mask(block_size, chunk_size, chunk_size_k, q_group_size, q_chunk_offset, ex_win, ex_sink,
          causal, tf_mask, prog_excl, id_base=0, id_stride=1) -> TopkMask:
    return TopkMask(_i32(block_size, "block_size"), _i32(chunk_size, "chunk_size"),
                    _i32(chunk_size_k, "chunk_size_k"), _i32(q_group_size, "q_group_size"),
                    _i32(q_chunk_offset, "q_chunk_offset"), _i32(ex_win, "ex_win"),
                    _i32(ex_sink, "ex_sink"), int(bool(causal)), int(bool(tf_mask)),
                    int(bool(prog_excl)), _i32(id_base, "id_base"), _i32(id_stride, "id_stride"))


def topk(q_pooled: torch.Tensor, k_pooled: torch.Tensor, topk: int, scale: float, block_size: int,
         chunk_size: int, chunk_size_k: int, causal: bool, ex_win: int = 0, ex_sink: int = 0,
         prog_excl: bool = False, tf_mask: bool = False, q_chunk_offset: int = 0,
         q_group_size: int = 1, id_base: int = 0, id_stride: int = 1, return_scores: bool = False):
    """int32 [B,MG,H,topk] block ids by (score desc, id asc), -1 padded; optionally the scores.
    `chunk_size` counts query tokens; a pooled row stands for `q_group_size` tokens."""
    _require_cuda(q_pooled, k_pooled)
    if q_pooled.dtype != k_pooled.dtype:
        raise NSABackendError(f"topk: q and k must share a dtype, got {q_pooled.dtype} vs {k_pooled.dtype}")
    B, MG, H, D = q_pooled.shape
    NC = k_pooled.shape[1]
    if k_pooled.shape[0] != B or k_pooled.shape[2] != H or k_pooled.shape[3] != D:
        raise NSABackendError(f"topk: incompatible shapes q={tuple(q_pooled.shape)} k={tuple(k_pooled.shape)}")
    q_pooled = q_pooled if q_pooled.stride(-1) == 1 else q_pooled.contiguous()
    k_pooled = k_pooled if k_pooled.stride(-1) == 1 else k_pooled.contiguous()
    dev = q_pooled.device
    out = torch.empty(B, MG, H, topk, dtype=torch.int32, device=dev)
    scores = torch.empty(B, MG, H, topk, dtype=torch.float32, device=dev) if return_scores else None
    m = _mask(block_size, chunk_size, chunk_size_k, q_group_size, q_chunk_offset, ex_win, ex_sink,
              causal, tf_mask, prog_excl, id_base, id_stride)
    with torch.cuda.device(dev):
        wsb = _lib.load().nsa_topk_workspace_bytes(B, MG, H, NC)
        ws = torch.empty(max(wsb, 1), dtype=torch.uint8, device=dev)
        call("nsa_topk", q_pooled.data_ptr(), strides3(q_pooled), k_pooled.data_ptr(), strides3(k_pooled),
             B, MG, H, D, NC, _i32(topk, "topk"), float(scale), C.byref(m), out.data_ptr(), _ptr(scores),
             ws.data_ptr(), wsb, _dtype(q_pooled), _stream(q_pooled))
    return (out, scores) if return_scores else out


def pool_score_topk(q_pooled: torch.Tensor, k: torch.Tensor, topk: int, scale: float, block_size: int,
                    chunk_size: int, chunk_size_k: int, causal: bool, ex_win: int = 0, ex_sink: int = 0,
                    prog_excl: bool = False, tf_mask: bool = False, q_chunk_offset: int = 0,
                    q_group_size: int = 1, return_scores: bool = False):
    """Pool raw keys k [B,N,H,D] per block, score against q_pooled and select.
    Returns (idx, k_pooled[, scores])."""
    _require_cuda(q_pooled, k)
    B, MG, H, D = q_pooled.shape
    N = k.shape[1]
    k = _rows16(k)
    q_pooled = q_pooled if q_pooled.stride(-1) == 1 else q_pooled.contiguous()
    NC = (N + block_size - 1) // block_size
    dev = k.device
    kp = torch.empty(B, NC, H, D, dtype=k.dtype, device=dev)
    out = torch.empty(B, MG, H, topk, dtype=torch.int32, device=dev)
    scores = torch.empty(B, MG, H, topk, dtype=torch.float32, device=dev) if return_scores else None
    m = _mask(block_size, chunk_size, chunk_size_k, q_group_size, q_chunk_offset, ex_win, ex_sink,
              causal, tf_mask, prog_excl)
    with torch.cuda.device(dev):
        wsb = _lib.load().nsa_topk_workspace_bytes(B, MG, H, NC)
        ws = torch.empty(max(wsb, 1), dtype=torch.uint8, device=dev)
        call("nsa_pool_score_topk", q_pooled.data_ptr(), strides3(q_pooled), k.data_ptr(), strides3(k),
             B, MG, H, D, N, _i32(topk, "topk"), float(scale), C.byref(m), kp.data_ptr(), out.data_ptr(),
             _ptr(scores), ws.data_ptr(), wsb, _dtype(k), _stream(k))
    return (out, kp, scores) if return_scores else (out, kp)


def select_blocks(q: torch.Tensor, k: torch.Tensor, topk: int, scale: float, block_size: int, group_size: int,
                  chunk_size: int, chunk_size_k: int, causal: bool, ex_win: int = 0, ex_sink: int = 0,
                  prog_excl: bool = False, tf_mask: bool = False, q_chunk_offset: int = 0,
                  return_scores: bool = False, id_base: int = 0, id_stride: int = 1):
    """Block selection from the raw tensors in one call: q [B,M,H,D] pooled per query group, k
    [B,N,H,D] pooled per key block and scored in the same pass, top-k per (group, head).
    Returns (idx int32 [B,MG,H,topk], q_pooled, k_pooled[, scores])."""
    _require_cuda(q, k)
    if q.dtype != k.dtype:
        raise NSABackendError(f"select_blocks: q and k must share a dtype, got {q.dtype} vs {k.dtype}")
    B, M, H, D = q.shape
    N = k.shape[1]
    q, k = _rows16(q), _rows16(k)
    MG = (M + group_size - 1) // group_size
    NC = (N + block_size - 1) // block_size
    dev = k.device
    qp = torch.empty(B, MG, H, D, dtype=q.dtype, device=dev)
    kp = torch.empty(B, NC, H, D, dtype=k.dtype, device=dev)
    out = torch.empty(B, MG, H, topk, dtype=torch.int32, device=dev)
    scores = torch.empty(B, MG, H, topk, dtype=torch.float32, device=dev) if return_scores else None
    m = _mask(block_size, chunk_size, chunk_size_k, group_size, q_chunk_offset, ex_win, ex_sink,
              causal, tf_mask, prog_excl, id_base, id_stride)
    with torch.cuda.device(dev):
        wsb = _lib.load().nsa_topk_workspace_bytes(B, MG, H, NC)
        ws = torch.empty(max(wsb, 1), dtype=torch.uint8, device=dev)
        call("nsa_select_blocks", q.data_ptr(), strides3(q), k.data_ptr(), strides3(k), B, M, H, D, N,
             _i32(topk, "topk"), float(scale), C.byref(m), qp.data_ptr(), kp.data_ptr(), out.data_ptr(),
             _ptr(scores), ws.data_ptr(), wsb, _dtype(k), _stream(k))
    return (out, qp, kp, scores) if return_scores else (out, qp, kp)


def local_block_ids(idx: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """Ids of a block-sharded memory as rank `rank` of `world` sees them: idx // world where the block
    is this rank's (idx % world == rank), else -1; int32, same shape."""
    _require_cuda(idx)
    if idx.dtype != torch.int32:
        raise NSABackendError("local_block_ids: ids must be int32")
    idx = idx.contiguous()
    out = torch.empty_like(idx)
    with torch.cuda.device(idx.device):
        call("nsa_local_block_ids", idx.data_ptr(), idx.numel(), _i32(world, "world"), _i32(rank, "rank"),
             out.data_ptr(), _stream(idx))
    return out


def merge_candidates(idx: torch.Tensor, scores: torch.Tensor, topk: int):
    """idx / scores [R, ..., T] (global ids, -1 = none) -> merged ([..., topk], [..., topk])."""
    _require_cuda(idx, scores)
    idx = idx.contiguous()
    scores = scores.contiguous()
    R, T = idx.shape[0], idx.shape[-1]
    rows = idx[0].numel() // T
    out_i = torch.empty(*idx.shape[1:-1], topk, dtype=torch.int32, device=idx.device)
    out_s = torch.empty(*idx.shape[1:-1], topk, dtype=torch.float32, device=idx.device)
    with torch.cuda.device(idx.device):
        call("nsa_merge_candidates", idx.data_ptr(), scores.data_ptr(), R, rows, T, _i32(topk, "topk"),
             out_i.data_ptr(), out_s.data_ptr(), _stream(idx))
    return out_i, out_s


# --------------------------------------------------------------------------------- K/V sources
class DenseKV:
    """k, v [B,N,H,D] addressed by stride."""

    def __init__(self, k: torch.Tensor, v: torch.Tensor):
        _require_cuda(k, v)
        if k.shape != v.shape:
            raise NSABackendError("k and v must have the same shape")
        self.k, self.v = _rows16(k), _rows16(v)
        self.n_tokens = k.shape[1]

    def struct(self) -> KVSource:
        s = KVSource()
        s.mode = _lib.NSA_KV_DENSE
        s.k, s.v = self.k.data_ptr(), self.v.data_ptr()
        s.k_stride = strides3(self.k)
        s.v_stride = strides3(self.v)
        s.n_tokens = self.n_tokens
        return s


class PagedKV:
    """Fixed-page pool + block table (see omnimem_b200.cache.BlockKVCache)."""

    def __init__(self, k_pool, v_pool, block_table, n_tokens: int, page_tokens: int):
        _require_cuda(k_pool, v_pool, block_table)
        self.k_pool, self.v_pool, self.block_table = k_pool, v_pool, block_table
        self.n_tokens, self.page_tokens = int(n_tokens), int(page_tokens)

    def struct(self) -> KVSource:
        s = KVSource()
        s.mode = _lib.NSA_KV_PAGED
        s.k, s.v = self.k_pool.data_ptr(), self.v_pool.data_ptr()
        s.n_tokens = self.n_tokens
        s.block_table = self.block_table.data_ptr()
        s.max_blocks = self.block_table.shape[-1]
        s.page_tokens = self.page_tokens
        s.num_pages = self.k_pool.shape[0]
        return s


class PtrKV:
    """int64 byte-address tables [B,MG,H,T] (0 = skip), whole blocks, `stride_bn` elements
    between tokens - the reference's pointer-table contract."""

    def __init__(self, ptr_k: torch.Tensor, ptr_v: torch.Tensor, stride_bn: int):
        _require_cuda(ptr_k, ptr_v)
        if ptr_k.dtype != torch.int64 or ptr_v.dtype != torch.int64:
            raise NSABackendError("pointer tables must be int64 byte addresses")
        if ptr_k.shape != ptr_v.shape or ptr_k.stride() != ptr_v.stride():
            raise NSABackendError("ptr_k / ptr_v must be [B,MG,H,T] with identical layout")
        self.ptr_k, self.ptr_v, self.stride_bn = ptr_k, ptr_v, int(stride_bn)

    def struct(self) -> KVSource:
        s = KVSource()
        s.mode = _lib.NSA_KV_PTR
        s.ptr_k, s.ptr_v = self.ptr_k.data_ptr(), self.ptr_v.data_ptr()
        s.ptr_stride_n = self.stride_bn
        s.n_tokens = 0
        return s


# ------------------------------------------------------------------------- selection attention
def sel_fwd(q: torch.Tensor, kv, block_indices: Optional[torch.Tensor], block_size: int,
            chunk_size: int, scale: float, causal: bool, group_size: int,
            out: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """(out [B,M,H,D] in q.dtype, lse fp32 [B,H,M]).  `out` may be given: a [B,M,H,D] tensor or
    view (innermost stride 1, 16-byte aligned rows) that the kernel writes in place."""
    _require_cuda(q, block_indices)
    B, M, H, D = q.shape
    q = _rows16(q)
    if out is None:
        out = torch.empty(B, M, H, D, dtype=q.dtype, device=q.device)
    elif out.shape != q.shape or out.dtype != q.dtype or _rows16(out) is not out:
        raise NSABackendError("sel_fwd: `out` must have q's shape and dtype, unit innermost stride and 16-byte aligned rows")
    lse = torch.empty(B, H, M, dtype=torch.float32, device=q.device)
    table = kv.ptr_k if isinstance(kv, PtrKV) else block_indices
    if table.dim() != 4:
        raise NSABackendError("block_indices must be [B,MG,H,T]")
    if block_indices is not None and block_indices.dtype != torch.int32:
        raise NSABackendError("block_indices must be int32")
    T = table.shape[-1]
    src = kv.struct()
    with torch.cuda.device(q.device):
        call("nsa_sel_fwd", q.data_ptr(), strides3(q), C.byref(src), _ptr(block_indices), strides4(table),
             out.data_ptr(), strides3(out), lse.data_ptr(), B, M, H, D, T, _i32(block_size, "block_size"),
             _i32(chunk_size, "chunk_size"), int(bool(causal)), _i32(group_size, "group_size"), float(scale),
             _dtype(q), _stream(q))
    return out, lse


def range_fwd(q: torch.Tensor, kv, first_block: int, n_blocks: int, block_size: int, scale: float,
              out: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Attention of every query over the blocks [first_block, first_block + n_blocks) of `kv`, not
    causal: (out [B,M,H,D], lse fp32 [B,H,M]), what sel_fwd returns when every query group lists
    exactly those blocks.  Shapes the range kernel is not built for (anything but bf16, D = 128,
    64-token blocks, H > 1, dense or paged K/V, <= 1024 blocks) go to sel_fwd with the list spelt out."""
    _require_cuda(q)
    B, M, H, D = q.shape
    first_block, n_blocks = _i32(first_block, "first_block"), _i32(n_blocks, "n_blocks")
    if first_block < 0 or n_blocks < 0:
        raise NSABackendError(f"range_fwd: first_block {first_block}, n_blocks {n_blocks}")
    covered = (q.dtype == torch.bfloat16 and D == 128 and block_size == 64 and H > 1 and scale > 0
               and isinstance(kv, (DenseKV, PagedKV)) and n_blocks <= 1024 and kv.n_tokens > 0
               and os.environ.get("OMNIMEM_B200_RANGE_KERNEL", "") != "listed")   # test hook: always list the blocks
    if not covered:
        G = 64
        ids = torch.arange(first_block, first_block + max(n_blocks, 1), dtype=torch.int32, device=q.device)
        if n_blocks == 0:
            ids = torch.full_like(ids, -1)
        ids = ids.expand(B, -(-M // G), H, ids.numel())
        return sel_fwd(q, kv, ids, block_size, 1, scale, False, G, out=out)
    q = _rows16(q)
    if out is None:
        out = torch.empty(B, M, H, D, dtype=q.dtype, device=q.device)
    elif out.shape != q.shape or out.dtype != q.dtype or _rows16(out) is not out:
        raise NSABackendError("range_fwd: `out` must have q's shape and dtype, unit innermost stride and 16-byte aligned rows")
    lse = torch.empty(B, H, M, dtype=torch.float32, device=q.device)
    src = kv.struct()
    with torch.cuda.device(q.device):
        nbytes = _lib.load().nsa_range_fwd_workspace_bytes(B, M, H, D, n_blocks) if out.is_contiguous() else 0
        ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device) if nbytes else None
        call("nsa_range_fwd", q.data_ptr(), strides3(q), C.byref(src), first_block, n_blocks, out.data_ptr(),
             strides3(out), lse.data_ptr(), B, M, H, D, _i32(block_size, "block_size"), float(scale), _ptr(ws), nbytes,
             _dtype(q), _stream(q))
    return out, lse


def sel_bwd(q, kv, block_indices, out, lse, d_out, block_size: int, chunk_size: int, scale: float,
            causal: bool, group_size: int):
    """(dq [B,M,H,D] q.dtype, dk, dv [B,N,H,D] k dtype, contiguous)."""
    _require_cuda(q, block_indices, out, lse, d_out)
    B, M, H, D = q.shape
    q, out, d_out = _rows16(q), _rows16(out), _rows16(d_out)
    lse = lse.contiguous()
    if block_indices.dtype != torch.int32:
        raise NSABackendError("block_indices must be int32")
    N = kv.n_tokens
    T = block_indices.shape[-1]
    dev = q.device
    dq = torch.empty(B, M, H, D, dtype=q.dtype, device=dev)
    dk = torch.empty(B, N, H, D, dtype=q.dtype, device=dev)
    dv = torch.empty(B, N, H, D, dtype=q.dtype, device=dev)
    nbytes = stored_probabilities_bytes(q, kv, block_indices, block_size, group_size)
    if nbytes:
        # P and dS computed once: the dQ kernel stores them, the dK/dV kernel streams them
        pds = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        NS = -(-N // block_size)
        groups, offsets, slots = inverted_index(block_indices, NS, block_size, chunk_size, causal, group_size,
                                                with_slots=True)
        dq, delta, written = sel_bwd_dq(q, kv, block_indices, out, lse, d_out, block_size, chunk_size, scale, causal,
                                        group_size, pds=pds)
        dk, dv = sel_bwd_dkv(q, kv, groups, offsets, lse, delta, d_out, T, block_size, chunk_size, scale, causal,
                             group_size, slots=slots if written else None, pds=pds if written else None)
        return dq, dk, dv
    src = kv.struct()
    with torch.cuda.device(dev):
        wsb = _lib.load().nsa_sel_bwd_workspace_bytes(B, M, H, N, T, block_size, group_size)
        ws = torch.empty(max(wsb, 1), dtype=torch.uint8, device=dev)
        call("nsa_sel_bwd", q.data_ptr(), strides3(q), C.byref(src), block_indices.data_ptr(),
             strides4(block_indices), out.data_ptr(), strides3(out), lse.data_ptr(), d_out.data_ptr(),
             strides3(d_out), dq.data_ptr(), strides3(dq), dk.data_ptr(), dv.data_ptr(), B, M, H, D, T,
             _i32(block_size, "block_size"), _i32(chunk_size, "chunk_size"), int(bool(causal)),
             _i32(group_size, "group_size"), float(scale), ws.data_ptr(), wsb, _dtype(q), _stream(q))
    return dq, dk, dv


def stored_probabilities_bytes(q, kv, block_indices, block_size: int, group_size: int) -> int:
    """Size of the P / dS buffer when the backward of this call can compute them once (dQ kernel
    stores, dK/dV kernel streams), else 0.  The buffer holds 16 KiB per (query group, head, slot);
    OMNIMEM_B200_BWD_STORED_MB caps it (default 4096, 0 turns the path off)."""
    cap_mb = int(os.environ.get("OMNIMEM_B200_BWD_STORED_MB", "4096"))
    B, M, H, D = q.shape
    T = block_indices.shape[-1]
    if (cap_mb <= 0 or q.dtype != torch.bfloat16 or D != 128 or block_size != 64 or not 16 <= group_size <= 64
            or H == 1 or T > 64 or not isinstance(kv, (DenseKV, PagedKV))):
        return 0
    with torch.cuda.device(q.device):
        n = _lib.load().nsa_sel_bwd_pds_bytes(B, M, H, T, group_size)
    return n if 0 < n <= cap_mb << 20 else 0


def inverted_index(block_indices: torch.Tensor, NS: int, block_size: int, chunk_size: int, causal: bool,
                   group_size: int, with_slots: bool = False):
    """CSR block -> query groups: (groups int32 [B,H,MG*T], offsets int32 [B,H,NS+1]), every bucket in
    ascending group order; with_slots adds slots int32 [B,H,MG*T], the position of each entry in its
    group's id list (buckets then ordered by (group, slot))."""
    _require_cuda(block_indices)
    B, MG, H, T = block_indices.shape
    dev = block_indices.device
    groups = torch.full((B, H, MG * T), -1, dtype=torch.int32, device=dev)
    offsets = torch.zeros(B, H, NS + 1, dtype=torch.int32, device=dev)
    slots = torch.full((B, H, MG * T), -1, dtype=torch.int32, device=dev) if with_slots else None
    with torch.cuda.device(dev):
        wsb = _lib.load().nsa_inverted_index_workspace_bytes(B, H, NS)
        ws = torch.empty(max(wsb, 1), dtype=torch.uint8, device=dev)
        args = (block_indices.data_ptr(), strides4(block_indices), B, MG, H, T, NS,
                _i32(block_size, "block_size"), _i32(chunk_size, "chunk_size"), int(bool(causal)),
                _i32(group_size, "group_size"), groups.data_ptr(), offsets.data_ptr())
        if with_slots:
            call("nsa_inverted_index_slots", *args, slots.data_ptr(), ws.data_ptr(), wsb, _stream(block_indices))
        else:
            call("nsa_inverted_index", *args, ws.data_ptr(), wsb, _stream(block_indices))
    return (groups, offsets, slots) if with_slots else (groups, offsets)


def merge_partials(outs: torch.Tensor, lses: torch.Tensor):
    """outs [R,B,M,H,D], lses [R,B,H,M] -> (out [B,M,H,D], lse [B,H,M])."""
    _require_cuda(outs, lses)
    outs, lses = outs.contiguous(), lses.contiguous().float()
    R, B, M, H, D = outs.shape
    out = torch.empty(B, M, H, D, dtype=outs.dtype, device=outs.device)
    lse = torch.empty(B, H, M, dtype=torch.float32, device=outs.device)
    with torch.cuda.device(outs.device):
        call("nsa_merge_partials", outs.data_ptr(), lses.data_ptr(), R, B, M, H, D, out.data_ptr(),
             lse.data_ptr(), _dtype(outs), _stream(outs))
    return out, lse


def packed_row_elems(H: int, D: int) -> int:
    """Elements (of a 16-bit dtype) of one packed row: H*D outputs, H fp32 log-sum-exps, and padding
    to a multiple of 16 bytes."""
    return (H * D + 2 * H + 7) // 8 * 8


def merge_packed_rows(parts: torch.Tensor, H: int, D: int) -> torch.Tensor:
    """parts [R, rows, packed_row_elems(H, D)] (16-bit dtype; elements [H*D, H*D + 2*H) of a row are
    H fp32 log-sum-exps) -> merged [rows, ...] in the same format: attention partials over disjoint
    key sets merged exactly, row by row."""
    _require_cuda(parts)
    if parts.dim() != 3 or parts.shape[-1] != packed_row_elems(H, D) or not parts.is_contiguous():
        raise NSABackendError("merge_packed_rows: parts must be contiguous [R, rows, packed_row_elems(H, D)]")
    R, rows, _ = parts.shape
    merged = torch.empty(rows, parts.shape[-1], dtype=parts.dtype, device=parts.device)
    with torch.cuda.device(parts.device):
        call("nsa_merge_packed_rows", parts.data_ptr(), R, rows, H, D, merged.data_ptr(), _dtype(parts), _stream(parts))
    return merged


def build_ptr_table(block_indices, base_k, base_v, n_blocks_per_head, batch_stride: int,
                    blocks_per_chunk: int, in_chunk_block_bytes: int):
    """Block id -> int64 byte address tables (0 = invalid / not resident)."""
    _require_cuda(block_indices, base_k, base_v, n_blocks_per_head)
    if block_indices.dtype != torch.int32:
        block_indices = block_indices.to(torch.int32)
    base_k, base_v = base_k.contiguous(), base_v.contiguous()
    nb = n_blocks_per_head.to(torch.int32).contiguous()
    B, MG, H, T = block_indices.shape
    pk = torch.empty(B, MG, H, T, dtype=torch.int64, device=block_indices.device)
    pv = torch.empty_like(pk)
    with torch.cuda.device(block_indices.device):
        call("nsa_build_ptr_table", block_indices.data_ptr(), strides4(block_indices), base_k.data_ptr(),
             base_v.data_ptr(), nb.data_ptr(), B, MG, H, T, base_k.shape[1], int(batch_stride),
             _i32(blocks_per_chunk, "blocks_per_chunk"), int(in_chunk_block_bytes), pk.data_ptr(),
             pv.data_ptr(), _stream(block_indices))
    return pk, pv


# ------------------------------------------------------------ reference block-KV entry points
def gather_publish_clear(desc: torch.Tensor, n_fetch: int, n_clear: int, block_bytes: int, wide: bool,
                         num_warps: int = 1) -> int:
    """K1 with the reference contract; returns the number of thread blocks launched."""
    n_fetch, n_clear = int(n_fetch), int(n_clear)
    if n_fetch == 0 and n_clear == 0:
        return 0
    _require_cuda(desc)
    if desc.dtype != torch.int64 or not desc.is_contiguous() or desc.numel() < 6 * n_fetch + n_clear:
        raise NSABackendError("gather_publish_clear: desc must be contiguous int64 with 6*n_fetch + n_clear entries")
    ctas = C.c_int64(0)
    with torch.cuda.device(desc.device):
        call("nsa_gather_publish_clear", desc.data_ptr(), n_fetch, n_clear, int(block_bytes), int(bool(wide)),
             int(num_warps), C.byref(ctas), _stream(desc))
    return int(ctas.value)


def block_range(table: torch.Tensor, n_valid: torch.Tensor, first_bid: int, n_blocks: int, k_base: int,
                v_base: int, head_stride_bytes: int, block_bytes: int, n_valid_value: int, write_k: bool,
                write_v: bool, clear: bool) -> None:
    """K2 with the reference contract on table int64 [2,H,MB], n_valid int32 [H]."""
    _require_cuda(table, n_valid)
    if table.dtype != torch.int64 or table.dim() != 3 or table.shape[0] != 2 or not table.is_contiguous():
        raise NSABackendError("block_range: table must be contiguous int64 [2,H,MB]")
    with torch.cuda.device(table.device):
        call("nsa_block_range", table.data_ptr(), n_valid.data_ptr(), table.shape[1], table.shape[2],
             int(first_bid), int(n_blocks), int(k_base), int(v_base), int(head_stride_bytes), int(block_bytes),
             int(n_valid_value), int(bool(write_k)), int(bool(write_v)), int(bool(clear)), _stream(table))


def dedup_run(block_indices_flat: torch.Tensor, stamp: torch.Tensor, out: torch.Tensor, epoch: int, mb: int,
              heads: int, t: int, bpc: int, cap: int) -> None:
    """K3 with the reference contract: out[0] = unique count, out[1..cap] ascending keys."""
    _require_cuda(block_indices_flat, stamp, out)
    if block_indices_flat.dim() != 1:
        raise NSABackendError("block_indices must be flattened to 1-D")
    dev = stamp.device
    with torch.cuda.device(dev):
        wsb = _lib.load().nsa_cache_dedup_workspace_bytes(heads * mb)
        ws = torch.empty(max(wsb, 1), dtype=torch.uint8, device=dev)
        call("nsa_cache_dedup_touch", block_indices_flat.data_ptr(), block_indices_flat.numel(), heads, t, mb,
             bpc, stamp.data_ptr(), _i32(epoch, "epoch"), None, None, 0, out.data_ptr(), None, _i32(cap, "cap"),
             None, ws.data_ptr(), wsb, _stream(stamp))


def sel_bwd_dq(q, kv, block_indices, out, lse, d_out, block_size: int, chunk_size: int, scale: float,
               causal: bool, group_size: int, pds: Optional[torch.Tensor] = None):
    """First half of the backward: (dq, delta fp32 [B,H,M]).  With a PtrKV source block_indices may
    be None: the address tables define the slots (the reference's pointer path).  With `pds` (a
    uint8 buffer of stored_probabilities_bytes) the result is (dq, delta, written): written says
    whether the kernel stored P and dS of every pair there for sel_bwd_dkv."""
    layout = block_indices if block_indices is not None else kv.ptr_k
    _require_cuda(q, layout, out, lse, d_out)
    B, M, H, D = q.shape
    q, out, d_out = _rows16(q), _rows16(out), _rows16(d_out)
    lse = lse.contiguous()
    dq = torch.empty(B, M, H, D, dtype=q.dtype, device=q.device)
    delta = torch.empty(B, H, M, dtype=torch.float32, device=q.device)
    src = kv.struct()
    with torch.cuda.device(q.device):
        args = (q.data_ptr(), strides3(q), C.byref(src), _ptr(block_indices),
                strides4(layout), out.data_ptr(), strides3(out), lse.data_ptr(), d_out.data_ptr(),
                strides3(d_out), dq.data_ptr(), strides3(dq), delta.data_ptr(), B, M, H, D, layout.shape[-1],
                _i32(block_size, "block_size"), _i32(chunk_size, "chunk_size"), int(bool(causal)),
                _i32(group_size, "group_size"), float(scale))
        if pds is None:
            call("nsa_sel_bwd_dq", *args, _dtype(q), _stream(q))
            return dq, delta
        written = C.c_int32(0)
        call("nsa_sel_bwd_dq_pds", *args, pds.data_ptr(), pds.numel() * pds.element_size(), C.byref(written),
             _dtype(q), _stream(q))
    return dq, delta, bool(written.value)


def sel_bwd_dkv(q, kv, groups, offsets, lse, delta, d_out, T: int, block_size: int, chunk_size: int,
                scale: float, causal: bool, group_size: int, slots: Optional[torch.Tensor] = None,
                pds: Optional[torch.Tensor] = None):
    """Second half of the backward: (dk, dv) [B,N,H,D] from the CSR index and delta; with `slots` and
    `pds` (after a sel_bwd_dq call that reported written) from the stored P / dS tiles."""
    _require_cuda(q, groups, offsets, lse, delta, d_out)
    B, M, H, D = q.shape
    q, d_out = _rows16(q), _rows16(d_out)
    N = kv.n_tokens
    dk = torch.empty(B, N, H, D, dtype=q.dtype, device=q.device)
    dv = torch.empty(B, N, H, D, dtype=q.dtype, device=q.device)
    src = kv.struct()
    with torch.cuda.device(q.device):
        ws = torch.empty(256, dtype=torch.uint8, device=q.device)
        stored = slots is not None and pds is not None
        call("nsa_sel_bwd_dkv_pds", q.data_ptr(), strides3(q), C.byref(src), groups.data_ptr(), offsets.data_ptr(),
             slots.data_ptr() if stored else None, pds.data_ptr() if stored else None,
             pds.numel() * pds.element_size() if stored else 0,
             lse.contiguous().data_ptr(), delta.data_ptr(), d_out.data_ptr(), strides3(d_out), dk.data_ptr(),
             dv.data_ptr(), B, M, H, D, _i32(T, "T"), _i32(block_size, "block_size"),
             _i32(chunk_size, "chunk_size"), int(bool(causal)), _i32(group_size, "group_size"), float(scale),
             ws.data_ptr(), 256, _dtype(q), _stream(q))
    return dk, dv


def _gate_args(g_logits, o_cmp, o_slc, o_swa):
    present = [t for t in (o_cmp, o_slc, o_swa) if t is not None]
    if not present:
        raise ValueError("gate_combine: at least one branch is needed")
    ref = present[0]
    _require_cuda(g_logits, *present)
    if g_logits.shape[-1] != 3 or tuple(g_logits.shape[:-1]) != tuple(ref.shape[:-1]):
        raise ValueError(f"gate_combine: gate logits {tuple(g_logits.shape)} do not match branches {tuple(ref.shape)}")
    for t in present:
        if t.shape != ref.shape or t.dtype != ref.dtype:
            raise ValueError("gate_combine: branches must share shape and dtype")
    if g_logits.dtype != ref.dtype:
        raise ValueError("gate_combine: gate logits must have the branches' dtype")
    cont = lambda t: None if t is None else t.contiguous()
    return g_logits.contiguous(), cont(o_cmp), cont(o_slc), cont(o_swa), ref


def gate_combine(g_logits: torch.Tensor, o_cmp: Optional[torch.Tensor], o_slc: Optional[torch.Tensor],
                 o_swa: Optional[torch.Tensor], gate_mode: str = "sigmoid") -> torch.Tensor:
    """x = g_cmp*o_cmp + g_slc*o_slc + g_swa*o_swa with (g_cmp, g_slc, g_swa) = sigmoid / softmax of
    clamp(g_logits, -10, 10); g_logits [..., H, 3], branches [..., H, D]; None skips a branch
    (causal_wan_nsa_model.py:378-386, 541-546)."""
    if gate_mode not in ("sigmoid", "softmax"):
        raise NotImplementedError(f"gate_mode={gate_mode!r} not implemented")
    g, a, b, c, ref = _gate_args(g_logits, o_cmp, o_slc, o_swa)
    x = torch.empty_like(ref, memory_format=torch.contiguous_format)
    D = ref.shape[-1]
    with torch.cuda.device(ref.device):
        call("nsa_gate_combine", g.data_ptr(), _ptr(a), _ptr(b), _ptr(c), x.data_ptr(), ref.numel() // D, D,
             1 if gate_mode == "softmax" else 0, _dtype(ref), _stream(ref))
    return x


def gate_combine_bwd(g_logits, o_cmp, o_slc, o_swa, dx: torch.Tensor, gate_mode: str = "sigmoid"):
    """Gradients of gate_combine: (d_g_logits, d_o_cmp, d_o_slc, d_o_swa); None for skipped branches."""
    if gate_mode not in ("sigmoid", "softmax"):
        raise NotImplementedError(f"gate_mode={gate_mode!r} not implemented")
    g, a, b, c, ref = _gate_args(g_logits, o_cmp, o_slc, o_swa)
    _require_cuda(dx)
    dx = dx.contiguous()
    dg = torch.empty_like(g)
    outs = [None if t is None else torch.empty_like(t) for t in (a, b, c)]
    D = ref.shape[-1]
    with torch.cuda.device(ref.device):
        call("nsa_gate_combine_bwd", g.data_ptr(), _ptr(a), _ptr(b), _ptr(c), dx.data_ptr(), dg.data_ptr(),
             _ptr(outs[0]), _ptr(outs[1]), _ptr(outs[2]), ref.numel() // D, D,
             1 if gate_mode == "softmax" else 0, _dtype(ref), _stream(ref))
    return dg, outs[0], outs[1], outs[2]


def sel_bwd_dkv_ptr(q, base_k, base_v, base_dk, base_dv, n_blocks_per_head, groups, offsets, lse, delta, d_out,
                    T: int, block_size: int, group_size: int, scale: float, batch_stride_kv_bytes: int,
                    batch_stride_dkv_bytes: int, stride_bn: int, stride_dbn: int, blocks_per_chunk: int = 0,
                    in_chunk_block_bytes_kv: int = 0, in_chunk_block_bytes_dkv: int = 0) -> None:
    """dK/dV of the pointer path, written as fp32 tiles into the scratch the base_dk / base_dv tables
    point at (sel_bwd_ptr_cuda, selection_bwd.cu:1409-1527).  base_* int64 [H, MAXB]; groups / offsets
    from inverted_index(block_indices, NS, block_size, 1, False, group_size)."""
    _require_cuda(q, base_k, base_v, base_dk, base_dv, groups, offsets, lse, delta, d_out)
    for t in (base_k, base_v, base_dk, base_dv):
        if t.dtype != torch.int64 or t.dim() != 2 or t.shape != base_k.shape or t.stride() != base_k.stride():
            raise NSABackendError("sel_bwd_dkv_ptr: base tables must be int64 [H, MAXB] with identical layout")
    B, M, H, D = q.shape
    if base_k.shape[0] != H:
        raise NSABackendError("sel_bwd_dkv_ptr: base_k must be [H, MAXB]")
    q, d_out = _rows16(q), _rows16(d_out)
    NS = offsets.shape[-1] - 1
    nbph = None
    if n_blocks_per_head is not None and n_blocks_per_head.numel() != 0:
        if n_blocks_per_head.dtype != torch.int32 or n_blocks_per_head.shape != (H,):
            raise NSABackendError("sel_bwd_dkv_ptr: n_blocks_per_head must be int32 [H]")
        nbph = n_blocks_per_head.contiguous()
    bs = (C.c_int64 * 3)(base_k.stride(0), base_k.stride(1), 0)
    with torch.cuda.device(q.device):
        call("nsa_sel_bwd_dkv_ptr", q.data_ptr(), _lib.strides3(q), base_k.data_ptr(), base_v.data_ptr(),
             base_dk.data_ptr(), base_dv.data_ptr(), bs, base_k.shape[1], _ptr(nbph), batch_stride_kv_bytes,
             batch_stride_dkv_bytes, stride_bn, stride_dbn, blocks_per_chunk, in_chunk_block_bytes_kv,
             in_chunk_block_bytes_dkv, groups.data_ptr(), offsets.data_ptr(), NS, lse.data_ptr(), delta.data_ptr(),
             d_out.data_ptr(), _lib.strides3(d_out), B, M, H, D, T, block_size, group_size, float(scale),
             _dtype(q), _stream(q))
