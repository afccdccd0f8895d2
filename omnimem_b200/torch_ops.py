"""Registers the reference's operator schemas under ``torch.ops.omnimem_nsa`` on top of the
C ABI, so code that calls ``torch.ops.omnimem_nsa.{topk,build_ptr_table,sel_fwd,sel_fwd_ptr,
sel_bwd,sel_bwd_ptr}`` (nsa/cuda_backend/csrc/bindings.cpp:7-36) runs on this library unchanged.  Shapes
and dtypes of the fake (meta) kernels follow nsa/cuda_backend/ops.py:199-235.

Importing this module in a process that has also loaded the reference's own extension would
define the namespace twice; use one or the other.
"""
from __future__ import annotations

import torch

from . import ops as _ops

_lib = torch.library.Library("omnimem_nsa", "DEF")

_lib.define("topk(Tensor q, Tensor k, int topk, float scale, int block_size, int chunk_size, "
            "int chunk_size_k, bool causal, int ex_win, int ex_sink, bool prog_excl, bool tf_mask, "
            "int q_chunk_offset, bool allow_tf32) -> Tensor")
_lib.define("build_ptr_table(Tensor block_indices, Tensor base_k, Tensor base_v, Tensor n_blocks_per_head, "
            "int batch_stride, int blocks_per_chunk, int in_chunk_block_bytes) -> (Tensor, Tensor)")
_lib.define("sel_fwd(Tensor q, Tensor k, Tensor v, Tensor block_indices, int block_size, int chunk_size, "
            "float scale, bool causal, int group_size, bool allow_tf32) -> (Tensor, Tensor)")
_lib.define("sel_fwd_ptr(Tensor q, Tensor ptr_k, Tensor ptr_v, int block_size, int group_size, int stride_bn, "
            "int stride_bd, float scale, str input_precision, Tensor[] owners) -> (Tensor, Tensor)")
_lib.define("sel_bwd(Tensor q, Tensor k, Tensor v, Tensor block_indices, Tensor out, Tensor lse, Tensor d_out, "
            "int block_size, int chunk_size, float scale, bool causal, int group_size, bool allow_tf32) "
            "-> (Tensor, Tensor, Tensor)")
_lib.define("sel_bwd_ptr(Tensor q, Tensor out, Tensor lse, Tensor d_out, Tensor block_indices, Tensor ptr_k, "
            "Tensor ptr_v, Tensor base_k, Tensor base_v, Tensor base_dk, Tensor base_dv, Tensor n_blocks_per_head, "
            "int block_size, int group_size, int batch_stride_kv_bytes, int batch_stride_dkv_bytes, int stride_bn, "
            "int stride_bd, int stride_dbn, int stride_dbd, int blocks_per_chunk, int in_chunk_block_bytes_kv, "
            "int in_chunk_block_bytes_dkv, float scale, str input_precision, bool compute_dkv, Tensor[] owners, "
            "Tensor(a!)[] grad_buffers) -> (Tensor, Tensor)")


def _topk(q, k, topk, scale, block_size, chunk_size, chunk_size_k, causal, ex_win, ex_sink, prog_excl,
          tf_mask, q_chunk_offset, allow_tf32):
    # operator convention: rows of q are already pooled and chunk_size counts rows
    return _ops.topk(q, k, topk, scale, block_size, chunk_size, chunk_size_k, causal, ex_win, ex_sink,
                     prog_excl, tf_mask, q_chunk_offset, q_group_size=1)


def _build_ptr_table(block_indices, base_k, base_v, n_blocks_per_head, batch_stride, blocks_per_chunk,
                     in_chunk_block_bytes):
    return _ops.build_ptr_table(block_indices, base_k, base_v, n_blocks_per_head, batch_stride,
                                blocks_per_chunk, in_chunk_block_bytes)


def _sel_fwd(q, k, v, block_indices, block_size, chunk_size, scale, causal, group_size, allow_tf32):
    return _ops.sel_fwd(q, _ops.DenseKV(k, v), block_indices, block_size, chunk_size, scale, causal, group_size)


def _sel_fwd_ptr(q, ptr_k, ptr_v, block_size, group_size, stride_bn, stride_bd, scale, input_precision, owners):
    if input_precision not in ("tf32", "ieee", "tf32x3"):
        raise RuntimeError(f"unsupported input_precision '{input_precision}' (expected 'tf32', 'ieee' or 'tf32x3')")
    if q.dtype != torch.bfloat16:
        raise RuntimeError(f"sel_fwd_ptr: q must be bfloat16, got {q.dtype}")
    if stride_bd != 1:
        raise RuntimeError("sel_fwd_ptr: blocks must have unit stride along the head dimension")
    return _ops.sel_fwd(q, _ops.PtrKV(ptr_k, ptr_v, stride_bn), None, block_size, 1, scale, False, group_size)


def _sel_bwd(q, k, v, block_indices, out, lse, d_out, block_size, chunk_size, scale, causal, group_size,
             allow_tf32):
    dq, dk, dv = _ops.sel_bwd(q, _ops.DenseKV(k, v), block_indices, out, lse, d_out, block_size, chunk_size,
                              scale, causal, group_size)
    return dq, dk.to(k.dtype), dv.to(v.dtype)


def _sel_bwd_ptr(q, out, lse, d_out, block_indices, ptr_k, ptr_v, base_k, base_v, base_dk, base_dv,
                 n_blocks_per_head, block_size, group_size, batch_stride_kv_bytes, batch_stride_dkv_bytes, stride_bn,
                 stride_bd, stride_dbn, stride_dbd, blocks_per_chunk, in_chunk_block_bytes_kv,
                 in_chunk_block_bytes_dkv, scale, input_precision, compute_dkv, owners, grad_buffers):
    """dq and delta are returned; dK / dV tiles are written as fp32 into the scratch the base_dk / base_dv
    tables address (selection_bwd.cu:1409-1527).  `owners` / `grad_buffers` only pin lifetimes."""
    if input_precision not in ("tf32", "ieee", "tf32x3"):
        raise RuntimeError(f"unsupported input_precision '{input_precision}' (expected 'tf32', 'ieee' or 'tf32x3')")
    if q.dtype != torch.bfloat16:
        raise RuntimeError(f"sel_bwd_ptr: q must be bfloat16, got {q.dtype}")
    if ptr_k.dtype != torch.int64 or ptr_v.dtype != torch.int64:
        raise RuntimeError("sel_bwd_ptr: ptr tables must be int64 byte addresses")
    if stride_bd != 1 or (compute_dkv and stride_dbd != 1):
        raise RuntimeError("sel_bwd_ptr: blocks must have unit stride along the head dimension")
    dq, delta = _ops.sel_bwd_dq(q, _ops.PtrKV(ptr_k, ptr_v, stride_bn), None, out, lse, d_out, block_size, 1, scale,
                                False, group_size)
    if not compute_dkv:
        return dq, delta
    max_n = base_k.shape[1] * (blocks_per_chunk if blocks_per_chunk > 0 else 1)
    groups, offsets = _ops.inverted_index(block_indices, max_n, block_size, 1, False, group_size)
    _ops.sel_bwd_dkv_ptr(q, base_k, base_v, base_dk, base_dv, n_blocks_per_head, groups, offsets, lse, delta, d_out,
                         block_indices.shape[-1], block_size, group_size, scale, batch_stride_kv_bytes,
                         batch_stride_dkv_bytes, stride_bn, stride_dbn, blocks_per_chunk, in_chunk_block_bytes_kv,
                         in_chunk_block_bytes_dkv)
    return dq, delta


for _name, _fn in (("topk", _topk), ("build_ptr_table", _build_ptr_table), ("sel_fwd", _sel_fwd),
                   ("sel_fwd_ptr", _sel_fwd_ptr), ("sel_bwd", _sel_bwd), ("sel_bwd_ptr", _sel_bwd_ptr)):
    _lib.impl(_name, _fn, "CUDA")


@torch.library.register_fake("omnimem_nsa::topk")
def _topk_fake(q, k, topk, scale, block_size, chunk_size, chunk_size_k, causal, ex_win, ex_sink, prog_excl,
               tf_mask, q_chunk_offset, allow_tf32):
    B, MG, H, _ = q.shape
    return q.new_empty((B, MG, H, topk), dtype=torch.int32)


@torch.library.register_fake("omnimem_nsa::build_ptr_table")
def _ptr_fake(block_indices, base_k, base_v, n_blocks_per_head, batch_stride, blocks_per_chunk,
              in_chunk_block_bytes):
    e = block_indices.new_empty(block_indices.shape, dtype=torch.int64)
    return e, block_indices.new_empty(block_indices.shape, dtype=torch.int64)


@torch.library.register_fake("omnimem_nsa::sel_fwd")
def _fwd_fake(q, k, v, block_indices, block_size, chunk_size, scale, causal, group_size, allow_tf32):
    B, M, H, _ = q.shape
    return torch.empty_like(q), q.new_empty((B, H, M), dtype=torch.float32)


@torch.library.register_fake("omnimem_nsa::sel_fwd_ptr")
def _fwd_ptr_fake(q, ptr_k, ptr_v, block_size, group_size, stride_bn, stride_bd, scale, input_precision, owners):
    B, M, H, _ = q.shape
    return torch.empty_like(q), q.new_empty((B, H, M), dtype=torch.float32)


@torch.library.register_fake("omnimem_nsa::sel_bwd")
def _bwd_fake(q, k, v, block_indices, out, lse, d_out, block_size, chunk_size, scale, causal, group_size,
              allow_tf32):
    return torch.empty_like(q), k.new_empty(k.shape), v.new_empty(v.shape)


@torch.library.register_fake("omnimem_nsa::sel_bwd_ptr")
def _bwd_ptr_fake(q, out, lse, d_out, block_indices, ptr_k, ptr_v, base_k, base_v, base_dk, base_dv,
                  n_blocks_per_head, block_size, group_size, batch_stride_kv_bytes, batch_stride_dkv_bytes, stride_bn,
                  stride_bd, stride_dbn, stride_dbd, blocks_per_chunk, in_chunk_block_bytes_kv,
                  in_chunk_block_bytes_dkv, scale, input_precision, compute_dkv, owners, grad_buffers):
    return torch.empty_like(q), lse.new_empty(lse.shape)
