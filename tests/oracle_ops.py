"""A stand-in for ``omnimem_b200.ops`` backed by the CPU oracle, for tests of host-side logic
that must run without a GPU (the multi-rank exchange of ``omnimem_b200.sharded`` over gloo).
Test infrastructure only - it mirrors just the functions that module calls."""
import torch

from oracle import nsa_oracle as O


class DenseKV:
    def __init__(self, k, v):
        self.k, self.v, self.n_tokens = k, v, k.shape[1]


def pool_rows(x, size):
    return O.pool_rows(x, size)


def topk(q_pooled, k_pooled, topk, scale, block_size, chunk_size, chunk_size_k, causal, ex_win=0, ex_sink=0,
         prog_excl=False, tf_mask=False, q_chunk_offset=0, q_group_size=1, id_base=0, id_stride=1,
         return_scores=False):
    cols = id_base + id_stride * torch.arange(k_pooled.shape[1])
    return O.topk_select(q_pooled, k_pooled, topk, scale, block_size=block_size, chunk_size=chunk_size,
                         chunk_size_k=chunk_size_k, causal=causal, ex_win=ex_win, ex_sink=ex_sink,
                         prog_excl=prog_excl, tf_mask=tf_mask, q_chunk_offset=q_chunk_offset,
                         q_group_size=q_group_size, return_scores=return_scores, col_ids=cols)


def select_blocks(q, k, topk_, scale, block_size, group_size, chunk_size, chunk_size_k, causal, ex_win=0, ex_sink=0,
                  prog_excl=False, tf_mask=False, q_chunk_offset=0, return_scores=False, id_base=0, id_stride=1):
    qp = O.pool_rows(q, group_size) if group_size > 1 else q
    kp = O.pool_rows(k, block_size)
    r = topk(qp, kp, topk_, scale, block_size, chunk_size, chunk_size_k, causal, ex_win, ex_sink, prog_excl, tf_mask,
             q_chunk_offset, group_size, id_base, id_stride, return_scores)
    return (r[0], qp, kp, r[1]) if return_scores else (r, qp, kp)


def local_block_ids(idx, world, rank):
    mine = (idx >= 0) & (idx % world == rank)
    return torch.where(mine, torch.div(idx, world, rounding_mode="floor"), torch.full_like(idx, -1)).to(torch.int32)


def merge_candidates(idx, scores, topk):
    return O.merge_candidates(list(idx), list(scores), topk)


def sel_fwd(q, kv, block_indices, block_size, chunk_size, scale, causal, group_size, out=None):
    o, lse = O.selection_fwd(q.float(), kv.k.float(), kv.v.float(), block_indices, block_size, chunk_size, scale,
                             causal, group_size)
    if out is not None:
        out.copy_(o)
        return out, lse
    return o.to(q.dtype), lse


def packed_row_elems(H, D):
    return (H * D + 2 * H + 7) // 8 * 8


def merge_packed_rows(parts, H, D):
    """[R, rows, H*D + 2*H] packed rows (16-bit outputs, fp32 log-sum-exps in the tail) -> [rows, ...]."""
    R, rows, _ = parts.shape
    outs = [parts[r, :, :H * D].reshape(1, rows, H, D).float() for r in range(R)]
    lses = [parts[r, :, H * D:H * D + 2 * H].contiguous().view(torch.float32).t().unsqueeze(0) for r in range(R)]
    out, lse = O.merge_partials(outs, lses)
    merged = torch.empty(rows, parts.shape[-1], dtype=parts.dtype)
    merged[:, :H * D] = out.reshape(rows, H * D).to(parts.dtype)
    merged[:, H * D:H * D + 2 * H].view(torch.float32).copy_(lse[0].t())
    return merged


def merge_partials(outs, lses):
    out, lse = O.merge_partials(list(outs), list(lses))
    return out.to(outs.dtype), lse
