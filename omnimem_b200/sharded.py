"""Block-sharded selection attention over several GPUs of one node.

For memories too long for one device the KV blocks are dealt round-robin to the ranks
(global block ``b`` lives on rank ``b % R`` as local block ``b // R``); Q is replicated.
One call does, on every rank:

1. pool the local keys (or take the cached pooled keys), score them against the pooled queries
   and take the local top-k (``id_base = rank, id_stride = R`` turns local columns into global
   block ids, so the visibility rules see true positions);
2. ONE all-gather of the candidate lists (ids and scores packed into one buffer, ``R x 2 x B x MG
   x H x T`` words) and a merge with the same (score desc, id asc) rule - every rank ends with the
   identical global top-k, which is exact because the global top-k is a subset of the union of the
   local ones;
3. run the selection forward over the selected blocks this rank owns, writing the partial output
   straight into packed rows (a token's H x D outputs followed by its H log-sum-exps);
4. ONE all-to-all that hands every rank its ``M / R`` share of the rows from all ranks, an exact
   merge of those rows (``O = sum_r exp(LSE_r - LSE) O_r``), and ONE all-gather of the merged
   rows.  A rank receives ``2 (R-1)/R`` x 14.6 MB at the Wan layer shape whatever R is, where an
   all-gather of the partials would deliver ``R`` x 14.6 MB and make every rank merge all rows.

The three exchanges are NCCL collectives into local buffers; no kernel reads peer memory.
The reference has no multi-GPU mode for this path (its long-memory answer is host offload,
models/cache.py:1032-1142); the semantics are those of its single-device operators
(nsa/ops/index_topk.py:43-105, nsa/ops/selection/__init__.py:56-100) applied to the whole KV.

Token-level causal clipping inside a block needs global token positions, which a shard does
not have; as in the reference's rollout path the forward therefore runs with ``causal=False``
and visibility is decided per block by the top-k mask.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def local_block_ids(n_blocks_global: int, rank: int, world: int) -> torch.Tensor:
    """Global ids of the blocks rank `rank` owns, in local order."""
    return torch.arange(rank, n_blocks_global, world)


def shard_kv(x: torch.Tensor, block_size: int, rank: int, world: int) -> torch.Tensor:
    """The rows of x [B,N,H,D] that belong to `rank` (blocks rank, rank+R, ...), concatenated."""
    B, N, H, D = x.shape
    nb = -(-N // block_size)
    parts = [x[:, b * block_size:min(N, (b + 1) * block_size)] for b in range(rank, nb, world)]
    if not parts:
        return x[:, :0]
    return torch.cat(parts, dim=1).contiguous()


class ShardedSelection:
    """Selection top-k + forward over a KV cache sharded by block across a process group.

    `ops` is the operator module to run on (``omnimem_b200.ops`` by default; the CPU tests
    pass an oracle-backed stand-in to exercise the exchange logic over gloo).  Without an
    initialised process group the object serves a single rank (no exchange at all)."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None, ops=None):
        if ops is None:
            from . import ops as _ops
            ops = _ops
        self.ops = ops
        self.group = group
        live = dist.is_available() and dist.is_initialized()
        self.rank = dist.get_rank(group) if live else 0
        self.world = dist.get_world_size(group) if live else 1

    def _all_gather(self, t: torch.Tensor) -> torch.Tensor:
        t = t.contiguous()
        out = torch.empty((self.world * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t, group=self.group)
        return out.view((self.world,) + tuple(t.shape))

    def select(self, q: torch.Tensor, k_local: torch.Tensor, topk: int, block_size: int, group_size: int,
               chunk_size: int, causal: bool, q_chunk_offset: int = 0, scale: Optional[float] = None,
               k_pooled_local: Optional[torch.Tensor] = None, exclude_window_chunks: int = 0,
               exclude_sink_chunks: int = 0, progressive_exclude: bool = False):
        """Global top-k block ids int32 [B,MG,H,topk] (identical on every rank) and their scores.
        `k_pooled_local` (the pooled keys of this rank's blocks, e.g. a cache's) skips the pass
        over the local keys."""
        ops = self.ops
        sc = q.shape[-1] ** -0.5 if scale is None else scale
        if k_pooled_local is None and group_size > 1:
            # both poolings in one launch, then scoring + selection
            idx, _, _, val = ops.select_blocks(q, k_local, topk, sc, block_size, group_size, chunk_size, chunk_size, causal,
                                               ex_win=exclude_window_chunks, ex_sink=exclude_sink_chunks,
                                               prog_excl=progressive_exclude, q_chunk_offset=q_chunk_offset,
                                               return_scores=True, id_base=self.rank, id_stride=self.world)
        else:
            qp = ops.pool_rows(q, group_size) if group_size > 1 else q
            kp = k_pooled_local if k_pooled_local is not None else ops.pool_rows(k_local, block_size)
            idx, val = ops.topk(qp, kp, topk, sc, block_size, chunk_size, chunk_size, causal,
                                ex_win=exclude_window_chunks, ex_sink=exclude_sink_chunks, prog_excl=progressive_exclude,
                                q_chunk_offset=q_chunk_offset, q_group_size=group_size, id_base=self.rank,
                                id_stride=self.world, return_scores=True)
        if self.world == 1:
            return idx, val
        # ids and scores travel as one buffer of 32-bit words
        both = self._all_gather(torch.stack([idx, val.view(torch.int32)]))          # [R, 2, B, MG, H, T]
        return ops.merge_candidates(both[:, 0].contiguous(), both[:, 1].contiguous().view(torch.float32), topk)

    def attend(self, q: torch.Tensor, k_local: torch.Tensor, v_local: torch.Tensor, idx_global: torch.Tensor,
               block_size: int, group_size: int, scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        """(out [B,M,H,D], lse [B,H,M]) of attention over the globally selected blocks.  With more
        than one rank both are views into the gathered packed rows (unit innermost stride)."""
        ops = self.ops
        sc = q.shape[-1] ** -0.5 if scale is None else scale
        R, r = self.world, self.rank
        local_ids = ops.local_block_ids(idx_global, R, r)
        kv = ops.DenseKV(k_local, v_local)
        if R == 1:
            return ops.sel_fwd(q, kv, local_ids, block_size, 1, sc, False, group_size)
        B, M, H, D = q.shape
        if B != 1 or q.element_size() != 2:
            raise ValueError("the row-split exchange serves batch size 1 and 16-bit tensors")
        HD, row = H * D, ops.packed_row_elems(H, D)
        rows_per = -(-M // R)
        # rows beyond M (padding up to R equal shares) start as "no key seen": out 0, lse -inf
        packed = torch.empty(R * rows_per, row, dtype=q.dtype, device=q.device)
        if R * rows_per > M:
            packed[M:, :HD] = 0
            packed[M:, HD:HD + 2 * H].view(torch.float32).fill_(float("-inf"))
        _, lse = ops.sel_fwd(q, kv, local_ids, block_size, 1, sc, False, group_size,
                             out=packed[:M, :HD].view(1, M, H, D))
        packed[:M, HD:HD + 2 * H].view(torch.float32).copy_(lse[0].t())
        parts = torch.empty_like(packed)                                  # [R][rows_per] rows of my share
        dist.all_to_all_single(parts, packed, group=self.group)
        merged = ops.merge_packed_rows(parts.view(R, rows_per, row), H, D)
        rows = torch.empty_like(packed)
        dist.all_gather_into_tensor(rows, merged, group=self.group)
        out = rows[:M, :HD].view(1, M, H, D)
        return out, rows[:M, HD:HD + 2 * H].view(torch.float32).t().unsqueeze(0)

    def forward(self, q, k_local, v_local, topk: int, block_size: int, group_size: int, chunk_size: int,
                causal: bool, q_chunk_offset: int = 0, scale: Optional[float] = None, **mask_kw):
        idx, _ = self.select(q, k_local, topk, block_size, group_size, chunk_size, causal, q_chunk_offset, scale,
                             **mask_kw)
        out, lse = self.attend(q, k_local, v_local, idx, block_size, group_size, scale)
        return out, lse, idx
