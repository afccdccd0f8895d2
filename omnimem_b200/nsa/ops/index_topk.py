"""Top-K block selection facade; same names, arguments and checks as the reference's
``omnimem/nsa/ops/index_topk.py`` (parallel_nsa_topk :43-105, parallel_nsa_topk_grouped_heads
:108-162, should_use_selection_attention :165-176), running on the sm_100a kernels.

One extension: ``allow_ragged=True`` lifts the reference's divisibility asserts so a last
query group shorter than ``group_size`` (and a chunk length that is not a multiple of it) is
accepted; the short group is pooled over the queries that exist and its chunk is that of its
first token.
"""
import math
from typing import Optional

import torch

from ... import ops as _ops

__all__ = ["parallel_nsa_topk", "parallel_nsa_topk_grouped_heads", "should_use_selection_attention"]


def parallel_nsa_topk(
        q: torch.Tensor,       # [B, T, H, K]
        k: torch.Tensor,       # [B, TC, H, K]  block-pooled keys
        block_counts: int,
        block_size: int = 64,
        scale: Optional[float] = None,
        chunk_size: int = 64,
        causal: bool = True,
        bt_chunk: int = 512,
        allow_tf32: bool = True,
        group_size: int = 1,
        exclude_window_chunks: int = 0,
        exclude_sink_chunks: int = 0,
        progressive_exclude: bool = False,
        tf_mask: bool = False,
        q_chunk_offset: int = 0,
        allow_ragged: bool = False,
) -> torch.Tensor:
    """Select the top ``block_counts`` pooled-key blocks per (pooled) query row.

    Returns int32 [B, ceil(T/G), H, block_counts]; visible blocks ordered by descending score
    (ties: lowest id first), -1 in unused slots.  ``bt_chunk`` and ``allow_tf32`` are accepted
    for compatibility: scores are always exact fp32 sums of the stored operands."""
    assert not (tf_mask and q_chunk_offset), "tf_mask assumes a full [clean|noisy] layout; q_chunk_offset must be 0"
    B, T, H, K = q.shape
    G = group_size
    if G > 1:
        if not allow_ragged:
            assert T % G == 0
            assert chunk_size % G == 0
        q = _ops.pool_rows(q, G)
    if causal and not allow_ragged:
        assert chunk_size % block_size == 0
    if tf_mask:
        # teacher forcing: pooled rows and key blocks both come as [clean | noisy] halves of whole
        # chunks (messages of reference index_topk.py:86-97)
        for what, have, per_chunk, unit, side in (
                ("T", q.shape[1], chunk_size // G, "2*chunk_size", "Q must be laid out as"),
                ("TC", k.shape[1], chunk_size // block_size, "2 * (chunk_size_k/block_size)", "K layout must be")):
            if have % (2 * per_chunk):
                raise AssertionError(f"tf_mask=True requires {what} ({have}) divisible by {unit} ({2 * per_chunk}); "
                                     f"{side} [clean | noisy] with equal halves.")
    sc = scale if scale is not None else K ** -0.5
    return _ops.topk(q, k, block_counts, sc, block_size, chunk_size, chunk_size, causal,
                     ex_win=exclude_window_chunks, ex_sink=exclude_sink_chunks,
                     prog_excl=progressive_exclude, tf_mask=tf_mask, q_chunk_offset=q_chunk_offset,
                     q_group_size=G)


def parallel_nsa_topk_grouped_heads(
        q: torch.Tensor,           # [B, T, H, K]
        k: torch.Tensor,           # [B, TC, H, K]
        num_kv_head_groups: int,
        block_counts: int,
        block_size: int,
        chunk_size: int,
        causal: bool = False,
        group_size: int = 1,
        tf_mask=False,
        **topk_kwargs,
) -> torch.Tensor:
    """GQA-style head pooling: pool heads per KV group, select, broadcast the indices."""
    B, T, H, K = q.shape
    TC = k.shape[1]
    assert H % num_kv_head_groups == 0
    if num_kv_head_groups == H:
        return parallel_nsa_topk(q=q, k=k, block_counts=block_counts, block_size=block_size,
                                 chunk_size=chunk_size, causal=causal, group_size=group_size,
                                 tf_mask=tf_mask, **topk_kwargs)
    hpg = H // num_kv_head_groups
    # head pooling first, then query pooling, each rounded to the input dtype (reference order).
    # The heads of a group are neighbouring rows of the [B*T*H, K] matrix, so the row-pooling
    # kernel does it (fp32 sum, one rounding), like the mean over dim 3 of the 5-D view.
    q_grouped = _ops.pool_rows(q.reshape(1, B * T * H, 1, K), hpg).view(B, T, num_kv_head_groups, K)
    k_grouped = _ops.pool_rows(k.reshape(1, B * TC * H, 1, K), hpg).view(B, TC, num_kv_head_groups, K)
    idx = parallel_nsa_topk(q=q_grouped, k=k_grouped, block_counts=block_counts, block_size=block_size,
                            chunk_size=chunk_size, causal=causal, group_size=group_size, tf_mask=tf_mask,
                            **topk_kwargs)
    return (idx.unsqueeze(-2).expand(-1, -1, -1, hpg, -1)
            .reshape(idx.shape[0], idx.shape[1], H, idx.shape[-1]))


def should_use_selection_attention(seq_len, chunk_size, exclude_window_chunks, exclude_sink_chunks,
                                   causal=True):
    """False when the sink and window exclusions hide every chunk, so the caller can return zeros
    for the selection branch without a launch (reference index_topk.py:165-176).  Under the causal
    rule an exclusion cannot hide more chunks than exist; without it the two counts simply add."""
    n_chunks = math.ceil(seq_len / chunk_size)
    sink, window = exclude_sink_chunks, exclude_window_chunks
    hidden = min(sink, n_chunks) + min(window, n_chunks) if causal else sink + window
    return n_chunks > hidden
