"""Selection attention over cache-resident K/V: the two inference facades of the reference's
``omnimem/nsa/ops/selection/padded_ptr`` package with their signatures, argument checks and
return values, on this library's kernels.

* ``selection_attention_block_store`` (padded_ptr/block_wrapper.py:15-89): K/V live in a block-level
  store.  Here the store is a ``BlockKVStore`` (one fixed-page ``BlockKVCache`` per layer); the call
  LRU-touches the selected blocks, fetches the ones that were evicted and runs the forward through
  the block table - the reference's prepare_selection / table_views / build_ptr_table /
  launch_ptr_fwd / release_selection sequence as two device-side steps without a pointer table.
* ``selection_attention_padded_ptr_fast`` (padded_ptr/wrapper.py:458-553): K/V live in per-head chunk
  tensors described by int64 base-address tables.  The pointer table is built on the device
  (nsa_build_ptr_table) and the forward reads the blocks through it (NSA_KV_PTR), as the reference
  does; the optional MMCache LRU touch / reload of that wrapper belongs to the reference's cache and
  is not repeated here (pass a BlockKVStore to the other facade for a managed cache).
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from ... import ops as _ops

__all__ = ["selection_attention_block_store", "selection_attention_padded_ptr_fast", "build_ptr_table"]

build_ptr_table = _ops.build_ptr_table


def _check_common(q, block_indices, group_size, what):
    B, M, H, D = q.shape
    if not (q.is_cuda and q.dtype == torch.bfloat16):
        raise AssertionError(f"{what} needs bf16 CUDA queries, got {q.dtype}")
    if M % group_size:
        raise AssertionError(f"M ({M}) must be divisible by group_size ({group_size})")
    want = (B, M // group_size, H, block_indices.shape[-1])
    if tuple(block_indices.shape) != want:
        raise AssertionError(f"block_indices {tuple(block_indices.shape)} != {want}")
    if block_indices.dtype != torch.int32:
        raise AssertionError(f"block_indices must be int32, got {block_indices.dtype}")


def selection_attention_block_store(q: torch.Tensor, block_indices: torch.Tensor, block_size: int, group_size: int,
                                    kv_cache, layer_idx: int, softmax_scale: Optional[float] = None,
                                    return_lse: bool = False, input_precision: str = "tf32"):
    """One selection-attention call with the block store as the only address source.  `kv_cache` is a
    BlockKVStore or an object whose ``block_store`` attribute is one."""
    B, M, H, D = q.shape
    if B != 1:
        raise AssertionError(f"the block KV store requires batch size 1, got B={B}: a page holds one batch "
                             f"element's block and the block table adds no batch stride")
    _check_common(q, block_indices, group_size, "block-store selection attention")
    if torch.is_grad_enabled() and q.requires_grad:
        raise RuntimeError("the block KV cache is inference-only: selection_attention_block_store was called with "
                           "grad enabled.  Wrap the forward in torch.no_grad(), or use selection_attention for training")
    store = getattr(kv_cache, "block_store", kv_cache)
    if store is None:
        raise AssertionError("selection_attention_block_store needs a configured store")
    if not (store.block_tokens == block_size and store.head_dim == D and store.num_heads == H):
        raise AssertionError(f"store geometry (bt={store.block_tokens}, D={store.head_dim}, H={store.num_heads}) != "
                             f"({block_size}, {D}, {H})")
    return store.layer(layer_idx).selection_attention(q, block_indices, scale=softmax_scale, group_size=group_size,
                                                      return_lse=return_lse)


def selection_attention_padded_ptr_fast(q: torch.Tensor, block_indices: torch.Tensor, block_size: int, group_size: int,
                                        chunk_len: int, chunk_base_ptrs_k: torch.Tensor, chunk_base_ptrs_v: torch.Tensor,
                                        n_chunks_per_head: torch.Tensor, chunk_strides: Dict[str, Any],
                                        softmax_scale: Optional[float] = None, return_lse: bool = False,
                                        input_precision: str = "tf32", verify_complete: bool = False, kv_cache=None,
                                        layer_idx: Optional[int] = None):
    """Forward over K/V chunks addressed by int64 base tables [H, max_chunks] (0 = chunk not on the
    device).  chunk_strides carries 'batch_stride_bytes', 'token_stride_bytes', 'stride_bn', 'stride_bd'."""
    B, M, H, D = q.shape
    _check_common(q, block_indices, group_size, "pointer-table selection attention")
    for name, t in (("chunk_base_ptrs_k", chunk_base_ptrs_k), ("chunk_base_ptrs_v", chunk_base_ptrs_v)):
        if t.dtype != torch.int64 or t.shape[0] != H:
            raise AssertionError(f"{name} must be int64 [H, max_chunks], got {t.dtype} {tuple(t.shape)}")
    if n_chunks_per_head.dtype != torch.int32 or tuple(n_chunks_per_head.shape) != (H,):
        raise AssertionError("n_chunks_per_head must be int32 [H]")
    if chunk_len % block_size:
        raise AssertionError(f"chunk_len ({chunk_len}) must be a multiple of block_size ({block_size})")
    if chunk_strides["stride_bd"] != 1:
        raise AssertionError("blocks must have unit stride along the head dimension")
    scale = D ** -0.5 if softmax_scale is None else softmax_scale
    blocks_per_chunk = chunk_len // block_size
    ptr_k, ptr_v = _ops.build_ptr_table(block_indices, chunk_base_ptrs_k, chunk_base_ptrs_v,
                                        n_chunks_per_head * blocks_per_chunk, chunk_strides["batch_stride_bytes"],
                                        blocks_per_chunk, block_size * chunk_strides["token_stride_bytes"])
    out, lse = _ops.sel_fwd(q, _ops.PtrKV(ptr_k, ptr_v, chunk_strides["stride_bn"]), None, block_size, 1, scale, False,
                            group_size)
    return (out, lse) if return_lse else out
