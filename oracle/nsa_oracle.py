"""CPU oracle for the NSA selection path.  TEST INFRASTRUCTURE ONLY.

This module restates, on the CPU with plain torch ops, what the reference computes on
the selection path: block/group mean pooling, pooled-key scoring with the visibility
rules, top-k block selection, selection attention forward (out + log-sum-exp) and
backward (dQ, dK, dV), the inverted (block -> query group) index, and the LRU block
cache policy.  Nothing under ``omnimem_b200`` imports it; only the tests, the smoke
check and the CPU-baseline legs of the benchmark do, and only as the checker or as the
thing timed as "CPU baseline" - never as the shipped compute path.

Semantics follow the reference's CUDA backend (the documented one), extended to ragged
tails (a last block / last query group that is shorter than the others), which the
reference rejects but the 64-token geometry needs.

Pinning: ``tests/golden/make_golden.py`` imports the reference's own pure-torch path
(``omnimem.nsa.naive``) and stores its outputs; ``tests/test_oracle.py`` checks this
module against those stored vectors (ids as sets per row, outputs to 1e-5).

Reference anchors (paths inside the reference project):
  pooling        src/omnimem/models/transformers/causal_wan_nsa_model.py:408-409,481,487
                 src/omnimem/nsa/ops/index_topk.py:72-79,136-141
  visibility     src/omnimem/nsa/cuda_backend/csrc/topk.cu:36-97
  order / -1     src/omnimem/nsa/cuda_backend/csrc/topk.cu:100-102, csrc/ops.h:11-12
  forward        src/omnimem/nsa/cuda_backend/csrc/common.cuh:158-190,326-332
                 src/omnimem/nsa/cuda_backend/csrc/selection_fwd.cu:1-3,595,794-805
                 src/omnimem/nsa/naive/select_attention.py:53-149
  backward       src/omnimem/nsa/cuda_backend/csrc/selection_bwd.cu:122-135,243-292
  inverted index src/omnimem/nsa/cuda_backend/csrc/inverted_index.cu:14-34
  pointer table  src/omnimem/nsa/cuda_backend/csrc/ptr_table.cu:29-53
  LRU policy     src/omnimem/models/cache.py:673-699,1018-1142
  block-KV K1-K3 src/omnimem/nsa/cuda_backend/csrc/block_kv_ops.h:12-31
"""
from __future__ import annotations

import math
from collections import OrderedDict
from typing import List, Optional, Tuple

import torch

NEG_INF = float("-inf")


# --------------------------------------------------------------------------------------
# pooling (a1, a2, a3)
# --------------------------------------------------------------------------------------
def pool_rows(x: torch.Tensor, size: int) -> torch.Tensor:
    """Mean over consecutive runs of ``size`` rows of dim 1; a ragged last run averages
    only the rows that exist.  fp32 accumulation, result rounded to ``x.dtype``
    (what ``x.view(b, n // size, size, h, d).mean(2)`` gives on whole runs;
    causal_wan_nsa_model.py:408-409, index_topk.py:72-79)."""
    B, N, H, D = x.shape
    nb = (N + size - 1) // size
    out = torch.empty(B, nb, H, D, dtype=x.dtype)
    full = N // size
    if full:
        out[:, :full] = x[:, : full * size].reshape(B, full, size, H, D).float().mean(2).to(x.dtype)
    if nb > full:
        out[:, full] = x[:, full * size:].float().mean(1).to(x.dtype)
    return out


def pool_heads(x: torch.Tensor, num_groups: int) -> torch.Tensor:
    """Head-group mean (index_topk.py:136-141); result in ``x.dtype``."""
    B, N, H, D = x.shape
    return x.view(B, N, num_groups, H // num_groups, D).float().mean(3).to(x.dtype)


# --------------------------------------------------------------------------------------
# visibility (a5) - a direct restatement of topk.cu:36-81
# --------------------------------------------------------------------------------------
def visibility_mask(MG: int, NC: int, *, block_size: int, chunk_size: int, chunk_size_k: int,
                    causal: bool, ex_win: int = 0, ex_sink: int = 0, prog_excl: bool = False,
                    tf_mask: bool = False, q_chunk_offset: int = 0,
                    q_group_size: int = 1, col_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bool [MG, NC]; True where key block c is a candidate for query row g.
    `col_ids` gives the global block id of every column (a shard of a block-sharded cache);
    default 0..NC-1.

    ``chunk_size`` is measured in query tokens and row g stands for tokens
    [g*q_group_size, ...): q_cid = (g*q_group_size)//chunk_size + q_chunk_offset.  With
    q_group_size == 1 this is the reference operator's convention (rows already pooled,
    chunk_size in rows).  k_cid = (c*block_size)//chunk_size_k."""
    g = torch.arange(MG, dtype=torch.int64)
    c = torch.arange(NC, dtype=torch.int64) if col_ids is None else col_ids.to(torch.int64)
    q_cid = (g * q_group_size) // chunk_size + q_chunk_offset
    k_cid = (c * block_size) // chunk_size_k
    if tf_mask:
        rows_per_chunk = max(chunk_size // q_group_size, 1)
        q_half = MG // (2 * rows_per_chunk)
        k_half = (NC * block_size) // (2 * chunk_size_k)
        q_clean = q_cid < q_half
        q_rel = torch.where(q_clean, q_cid, q_cid - q_half)
        k_clean = k_cid < k_half
        k_rel = torch.where(k_clean, k_cid, k_cid - k_half)
    else:
        q_clean = torch.ones(MG, dtype=torch.bool)
        q_rel = q_cid
        k_clean = torch.ones(NC, dtype=torch.bool)
        k_rel = k_cid
    do_excl = (q_rel >= (ex_sink + ex_win)) if prog_excl else torch.ones(MG, dtype=torch.bool)
    qc, qr, de = q_clean[:, None], q_rel[:, None], do_excl[:, None]
    kc, kr = k_clean[None, :], k_rel[None, :]
    if tf_mask:
        valid = (qc & kc & (kr <= qr)) | (~qc & kc & (kr < qr)) | (~qc & ~kc & (kr == qr))
    elif causal:
        valid = k_cid[None, :] <= q_cid[:, None]
    else:
        valid = torch.ones(MG, NC, dtype=torch.bool)
    if ex_sink > 0:
        sink_ok = (~kc) | (kr >= ex_sink)
        valid = valid & (sink_ok | ~de)
    if ex_win > 0:
        if tf_mask:
            in_win = kc & (kr >= qr - ex_win + 1)
        else:
            in_win = k_cid[None, :] >= (q_cid[:, None] - ex_win + 1)
            if not causal:
                in_win = in_win & (k_cid[None, :] <= (q_cid[:, None] + ex_win - 1))
        valid = valid & (~in_win | ~de)
    return valid


# --------------------------------------------------------------------------------------
# scoring + top-k (a4)
# --------------------------------------------------------------------------------------
def scores(q_pooled: torch.Tensor, k_pooled: torch.Tensor, scale: float) -> torch.Tensor:
    """fp32 [B, H, MG, NC] = (q̄ · k̄) * scale; operands are used at their stored
    precision, products and sums in fp32 (topk.cu:179-291)."""
    s = torch.einsum("bghd,bchd->bhgc", q_pooled.float(), k_pooled.float())
    return s * scale


def topk_select(q_pooled: torch.Tensor, k_pooled: torch.Tensor, topk: int, scale: Optional[float] = None,
                *, block_size: int, chunk_size: int, chunk_size_k: Optional[int] = None,
                causal: bool = True, ex_win: int = 0, ex_sink: int = 0, prog_excl: bool = False,
                tf_mask: bool = False, q_chunk_offset: int = 0, q_group_size: int = 1,
                return_scores: bool = False, col_ids: Optional[torch.Tensor] = None):
    """int32 [B, MG, H, topk]: visible blocks ordered by (score descending, id ascending),
    -1 in the unused slots (topk.cu:100-102,388-392; ops.h:11-12)."""
    B, MG, H, D = q_pooled.shape
    NC = k_pooled.shape[1]
    if scale is None:
        scale = D ** -0.5
    if chunk_size_k is None:
        chunk_size_k = chunk_size
    idx = torch.full((B, MG, H, topk), -1, dtype=torch.int32)
    val = torch.full((B, MG, H, topk), NEG_INF, dtype=torch.float32)
    if NC == 0 or MG == 0:
        return (idx, val) if return_scores else idx
    s = scores(q_pooled, k_pooled, scale) + 0.0  # canonical +0.0
    vis = visibility_mask(MG, NC, block_size=block_size, chunk_size=chunk_size,
                          chunk_size_k=chunk_size_k, causal=causal, ex_win=ex_win,
                          ex_sink=ex_sink, prog_excl=prog_excl, tf_mask=tf_mask,
                          q_chunk_offset=q_chunk_offset, q_group_size=q_group_size)
    s = s.masked_fill(~vis[None, None], NEG_INF)
    # stable sort on descending score keeps ascending ids among equal scores
    order = torch.sort(s, dim=-1, descending=True, stable=True)
    kk = min(topk, NC)
    top_i = order.indices[..., :kk]
    top_v = order.values[..., :kk]
    top_i = torch.where(torch.gather(vis[None, None].expand(B, H, MG, NC), -1, top_i), top_i,
                        torch.full_like(top_i, -1))
    top_v = torch.where(top_i >= 0, top_v, torch.full_like(top_v, NEG_INF))
    if col_ids is not None:                                  # local column -> global block id
        top_i = torch.where(top_i >= 0, col_ids.to(torch.int64)[top_i.clamp_min(0)], top_i)
    idx[..., :kk] = top_i.permute(0, 2, 1, 3).to(torch.int32)
    val[..., :kk] = top_v.permute(0, 2, 1, 3)
    return (idx, val) if return_scores else idx


def parallel_nsa_topk(q: torch.Tensor, k_pooled: torch.Tensor, block_counts: int, block_size: int = 64,
                      scale: Optional[float] = None, chunk_size: int = 64, causal: bool = True,
                      group_size: int = 1, exclude_window_chunks: int = 0,
                      exclude_sink_chunks: int = 0, progressive_exclude: bool = False,
                      tf_mask: bool = False, q_chunk_offset: int = 0) -> torch.Tensor:
    """Facade-level restatement of index_topk.py:43-105 (query pooling, then top-k),
    tail-aware: a ragged last query group is pooled over the queries that exist."""
    qp = pool_rows(q, group_size) if group_size > 1 else q
    return topk_select(qp, k_pooled, block_counts, scale, block_size=block_size,
                       chunk_size=chunk_size, chunk_size_k=chunk_size, causal=causal,
                       ex_win=exclude_window_chunks, ex_sink=exclude_sink_chunks,
                       prog_excl=progressive_exclude, tf_mask=tf_mask,
                       q_chunk_offset=q_chunk_offset, q_group_size=group_size)


def merge_candidates(idx_parts: List[torch.Tensor], val_parts: List[torch.Tensor], topk: int):
    """Merge per-shard candidate lists [B,MG,H,T] (global ids) into the global top-k with
    the same (score desc, id asc) rule; the exact result because the global top-k is a
    subset of the union of the local top-k lists."""
    idx = torch.cat(idx_parts, dim=-1).to(torch.int64)
    val = torch.cat(val_parts, dim=-1).clone()
    val[idx < 0] = NEG_INF
    big = torch.where(idx < 0, torch.full_like(idx, 2 ** 40), idx)
    o1 = torch.sort(big, dim=-1, stable=True)
    val1 = torch.gather(val, -1, o1.indices)
    o2 = torch.sort(val1, dim=-1, descending=True, stable=True)
    ids = torch.gather(o1.values, -1, o2.indices)[..., :topk]
    vals = o2.values[..., :topk]
    ids = torch.where(vals == NEG_INF, torch.full_like(ids, -1), ids)
    return ids.to(torch.int32), vals


# --------------------------------------------------------------------------------------
# selection attention forward / backward (a7, a10)
# --------------------------------------------------------------------------------------
def _row_tokens(ids_row, N: int, block_size: int, causal: bool, chunk_size: int, q_chunk: int):
    """Token indices a (b, g, h) row attends to, in slot order, duplicates kept
    (common.cuh:168-187: skip id<0, token0>=N, block-level causal; common.cuh:326-332:
    visible prefix)."""
    toks = []
    for bid in ids_row:
        bid = int(bid)
        if bid < 0:
            continue
        t0 = bid * block_size
        if t0 >= N:
            continue
        n_valid = min(block_size, N - t0)
        if causal:
            if t0 // chunk_size > q_chunk:
                continue
            n_valid = min(n_valid, (q_chunk + 1) * chunk_size - t0)
            if n_valid <= 0:
                continue
        toks.append(torch.arange(t0, t0 + n_valid, dtype=torch.int64))
    if toks:
        return torch.cat(toks)
    return torch.empty(0, dtype=torch.int64)


def selection_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, block_indices: torch.Tensor,
                  block_size: int, chunk_size: int = 1, scale: Optional[float] = None,
                  causal: bool = False, group_size: int = 1,
                  compute_dtype: torch.dtype = torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    """(out [B,M,H,D] in q.dtype, lse fp32 [B,H,M], natural log).  Rows with no visible key
    give out = 0 and lse = -inf (selection_fwd.cu:1-3,794-805).  The query chunk of a
    group is that of its first token (selection_fwd.cu:595)."""
    B, M, H, D = q.shape
    N = k.shape[1]
    G = group_size
    MG = (M + G - 1) // G
    if scale is None:
        scale = D ** -0.5
    out = torch.zeros(B, M, H, D, dtype=compute_dtype)
    lse = torch.full((B, H, M), NEG_INF, dtype=torch.float32)
    qf, kf, vf = q.to(compute_dtype), k.to(compute_dtype), v.to(compute_dtype)
    ids = block_indices.cpu()
    for b in range(B):
        for h in range(H):
            kh, vh = kf[b, :, h], vf[b, :, h]
            for g in range(MG):
                m0, m1 = g * G, min(M, g * G + G)
                toks = _row_tokens(ids[b, g, h].tolist(), N, block_size, causal, chunk_size,
                                   (g * G) // chunk_size)
                if toks.numel() == 0:
                    continue
                s = (qf[b, m0:m1, h] @ kh[toks].T) * scale
                mx = s.max(dim=-1, keepdim=True).values
                p = torch.exp(s - mx)
                l = p.sum(-1, keepdim=True)
                out[b, m0:m1, h] = (p @ vh[toks]) / l
                lse[b, h, m0:m1] = (mx + torch.log(l)).squeeze(-1).float()
    return out.to(q.dtype), lse


def selection_bwd(q, k, v, block_indices, out, lse, d_out, block_size: int, chunk_size: int = 1,
                  scale: Optional[float] = None, causal: bool = False, group_size: int = 1,
                  compute_dtype: torch.dtype = torch.float32):
    """(dq, dk, dv) in the input dtypes, accumulated in ``compute_dtype``
    (selection_bwd.cu:122-135: delta = sum(O*dO), P = exp(S*scale - LSE), dP = dO V^T,
    dS = P (dP - delta) scale, dQ = dS K; :243-292: dK = dS^T Q, dV = P^T dO, summed over
    every group that selected the block)."""
    B, M, H, D = q.shape
    N = k.shape[1]
    G = group_size
    MG = (M + G - 1) // G
    if scale is None:
        scale = D ** -0.5
    cd = compute_dtype
    qf, kf, vf, of, dof = (t.to(cd) for t in (q, k, v, out, d_out))
    dq = torch.zeros(B, M, H, D, dtype=cd)
    dk = torch.zeros(B, N, H, D, dtype=cd)
    dv = torch.zeros(B, N, H, D, dtype=cd)
    delta = (of * dof).sum(-1)  # [B,M,H]
    ids = block_indices.cpu()
    for b in range(B):
        for h in range(H):
            kh, vh = kf[b, :, h], vf[b, :, h]
            for g in range(MG):
                m0, m1 = g * G, min(M, g * G + G)
                toks = _row_tokens(ids[b, g, h].tolist(), N, block_size, causal, chunk_size,
                                   (g * G) // chunk_size)
                if toks.numel() == 0:
                    continue
                s = (qf[b, m0:m1, h] @ kh[toks].T) * scale
                p = torch.exp(s - lse[b, h, m0:m1].to(cd)[:, None])
                dp = dof[b, m0:m1, h] @ vh[toks].T
                ds = p * (dp - delta[b, m0:m1, h][:, None]) * scale
                dq[b, m0:m1, h] = ds @ kh[toks]
                dk[b, :, h].index_add_(0, toks, ds.T @ qf[b, m0:m1, h])
                dv[b, :, h].index_add_(0, toks, p.T @ dof[b, m0:m1, h])
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


def selection_flops(block_indices: torch.Tensor, M: int, N: int, D: int, block_size: int,
                    chunk_size: int, causal: bool, group_size: int) -> int:
    """Executed forward FLOPs 4*D*sum(n_q * n_visible_keys) over all (b, g, h) rows."""
    ids = block_indices.cpu().to(torch.int64)
    B, MG, H, T = ids.shape
    G = group_size
    g = torch.arange(MG, dtype=torch.int64)
    n_q = torch.clamp(torch.full((MG,), M, dtype=torch.int64) - g * G, max=G)
    t0 = ids * block_size
    n_valid = torch.clamp(N - t0, min=0, max=block_size)
    ok = (ids >= 0) & (t0 < N)
    if causal:
        q_chunk = ((g * G) // chunk_size).view(1, MG, 1, 1)
        ok = ok & ((t0 // chunk_size) <= q_chunk)
        n_valid = torch.minimum(n_valid, torch.clamp((q_chunk + 1) * chunk_size - t0, min=0))
    n_keys = torch.where(ok, n_valid, torch.zeros_like(n_valid)).sum(-1)  # [B,MG,H]
    return int(4 * D * (n_keys * n_q.view(1, MG, 1)).sum())


def merge_partials(outs: List[torch.Tensor], lses: List[torch.Tensor]):
    """Exact merge of attention partials over disjoint key sets:
    LSE = logsumexp_r LSE_r, O = sum_r exp(LSE_r - LSE) O_r; all -inf -> O = 0."""
    L = torch.stack([x.float() for x in lses])              # [R,B,H,M]
    O = torch.stack([x.float() for x in outs])              # [R,B,M,H,D]
    mx = L.max(0).values
    safe = torch.where(mx == NEG_INF, torch.zeros_like(mx), mx)
    w = torch.exp(L - safe[None])
    w = torch.where(L == NEG_INF, torch.zeros_like(w), w)
    den = w.sum(0)
    lse = torch.where(den > 0, safe + torch.log(den), torch.full_like(den, NEG_INF))
    wn = torch.where(den > 0, w / den.clamp_min(1e-38), torch.zeros_like(w))
    out = (O * wn.permute(0, 1, 3, 2)[..., None]).sum(0)
    return out, lse


# --------------------------------------------------------------------------------------
# rotary embedding of a key chunk in the reordered token order
# --------------------------------------------------------------------------------------
def rope_params(max_seq_len: int, dim: int, theta: float = 10000.0) -> torch.Tensor:
    """complex128 [max_seq_len, dim/2] table (models/transformers/wan_model.py:37-43)."""
    freqs = torch.outer(torch.arange(max_seq_len),
                        1.0 / torch.pow(theta, torch.arange(0, dim, 2).to(torch.float64).div(dim)))
    return torch.polar(torch.ones_like(freqs), freqs)


def reorder_rope_apply(x: torch.Tensor, grid, freqs: torch.Tensor, start_frame: int = 0, pool=(1, 1, 1)):
    """One sample of causal_reorder_rope_apply (models/transformers/causal_wan_nsa_model.py:72-105):
    x [S, H, D] with S = f*h*w tokens in the order (f h w fs hs ws) of the pooling windows; the
    frame / row / column parts of the table multiply the complex pairs in float64."""
    f, h, w = grid
    pf, ph, pw = pool
    S, H, D = x.shape
    assert S == f * h * w and f % pf == 0 and h % ph == 0 and w % pw == 0
    c = D // 2
    parts = freqs.split([c - 2 * (c // 3), c // 3, c // 3], dim=1)
    t = torch.arange(S)
    ws = t % pw; t = t // pw
    hs = t % ph; t = t // ph
    fs = t % pf; t = t // pf
    wo = t % (w // pw); t = t // (w // pw)
    ho = t % (h // ph); t = t // (h // ph)
    fr, hr, wr = t * pf + fs, ho * ph + hs, wo * pw + ws
    fac = torch.cat([parts[0][start_frame + fr], parts[1][hr], parts[2][wr]], dim=1)      # [S, c]
    xc = torch.view_as_complex(x.to(torch.float64).reshape(S, H, c, 2))
    return torch.view_as_real(xc * fac[:, None, :]).flatten(2).type_as(x)


# --------------------------------------------------------------------------------------
# gate + sum of the three branches (a16)
# --------------------------------------------------------------------------------------
def gate_combine(g_logits: torch.Tensor, o_cmp, o_slc, o_swa, gate_mode: str = "sigmoid"):
    """The reference's expression, on CPU tensors of the activations' dtype
    (causal_wan_nsa_model.py:378-386 for the gates, 541-546 for the sum; a None branch is the
    skipped module).  g_logits [..., H, 3], branches [..., H, D]."""
    g = torch.clamp(g_logits, min=-10.0, max=10.0)
    if gate_mode == "sigmoid":
        g_cmp, g_slc, g_swa = g.sigmoid().unbind(-1)
    elif gate_mode == "softmax":
        g_cmp, g_slc, g_swa = g.softmax(dim=-1).unbind(-1)
    else:
        raise NotImplementedError(f"{gate_mode=} not implemented")
    x = None
    for gt, o in ((g_cmp, o_cmp), (g_slc, o_slc), (g_swa, o_swa)):
        if o is None:
            continue
        term = gt.unsqueeze(-1) * o
        x = term if x is None else x + term
    return x


# --------------------------------------------------------------------------------------
# inverted index (a11) and pointer table (a9)
# --------------------------------------------------------------------------------------
def inverted_index(block_indices: torch.Tensor, NS: int, block_size: int, chunk_size: int,
                   causal: bool, group_size: int):
    """CSR block -> query groups, buckets sorted by (group, slot) (the reference's bucket
    order is arrival order; inverted_index.cu:14-34 gives the filter).
    Returns (groups int32 [B,H,MG*T] padded with -1, offsets int32 [B,H,NS+1])."""
    ids = block_indices.cpu()
    B, MG, H, T = ids.shape
    groups = torch.full((B, H, MG * T), -1, dtype=torch.int32)
    offsets = torch.zeros((B, H, NS + 1), dtype=torch.int32)
    for b in range(B):
        for h in range(H):
            buckets = [[] for _ in range(NS)]
            for g in range(MG):
                for t in range(T):
                    bid = int(ids[b, g, h, t])
                    if bid < 0 or bid >= NS:
                        continue
                    if causal and (bid * block_size) // chunk_size > (g * group_size) // chunk_size:
                        continue
                    buckets[bid].append(g)
            pos = 0
            for s in range(NS):
                offsets[b, h, s] = pos
                for g in buckets[s]:
                    groups[b, h, pos] = g
                    pos += 1
            offsets[b, h, NS] = pos
    return groups, offsets


def build_ptr_table(block_indices, base_k, base_v, n_blocks_per_head, batch_stride: int,
                    blocks_per_chunk: int, in_chunk_block_bytes: int):
    """int64 byte addresses [B,MG,H,T] (ptr_table.cu:29-53): 0 when the id is negative,
    not below n_blocks_per_head[h], its chunk is past the table, or the chunk base is 0."""
    ids = block_indices.cpu().to(torch.int64)
    B, MG, H, T = ids.shape
    max_chunks = base_k.shape[1]
    pk = torch.zeros(B, MG, H, T, dtype=torch.int64)
    pv = torch.zeros(B, MG, H, T, dtype=torch.int64)
    for b in range(B):
        for h in range(H):
            nb = int(n_blocks_per_head[h])
            for g in range(MG):
                for t in range(T):
                    bid = int(ids[b, g, h, t])
                    if bid < 0 or bid >= nb:
                        continue
                    cid, loc = divmod(bid, blocks_per_chunk)
                    if cid >= max_chunks:
                        continue
                    off = b * batch_stride + loc * in_chunk_block_bytes
                    bk, bv = int(base_k[h, cid]), int(base_v[h, cid])
                    if bk != 0:
                        pk[b, g, h, t] = bk + off
                    if bv != 0:
                        pv[b, g, h, t] = bv + off
    return pk, pv


# --------------------------------------------------------------------------------------
# LRU block-cache policy model (a13, a14)
# --------------------------------------------------------------------------------------
class LRUBlockCacheModel:
    """Host model of the fixed-page pool with an LRU block table.

    Unit of residency = one (head, block) page.  Touch order follows
    cache.py:673-699 (an OrderedDict per head: a hit moves the key to the end, a miss
    inserts it and, when the set is full, pops the oldest).  Evicted pages keep their
    pooled key (history is never dropped from the candidate set; cache.py:1032-1142 moves
    the full-resolution K/V to a fixed host slot) and are fetched back when selected
    (padded_ptr/wrapper.py:253-362).  Pages inside the protected tail window are never
    chosen as victims."""

    def __init__(self, num_heads: int, capacity_pages_per_head: int, protect_last_blocks: int = 0):
        self.H = num_heads
        self.cap = capacity_pages_per_head
        self.protect = protect_last_blocks
        self.lru = [OrderedDict() for _ in range(num_heads)]
        self.n_blocks = 0
        self.hits = 0
        self.misses = 0
        self.evictions: List[Tuple[int, int]] = []
        self.fetches: List[Tuple[int, int]] = []

    def _protected(self, bid: int) -> bool:
        return bid >= self.n_blocks - self.protect

    def _insert(self, h: int, bid: int):
        lru = self.lru[h]
        while len(lru) >= self.cap:
            victim = next((x for x in lru if not self._protected(x) and x != bid), None)
            if victim is None:
                raise RuntimeError("page pool exhausted: every resident page is protected")
            del lru[victim]
            self.evictions.append((h, victim))
        lru[bid] = None

    def append(self, first_block: int, n_blocks: int):
        """Blocks [first_block, first_block+n_blocks) were (re)written for every head."""
        self.n_blocks = max(self.n_blocks, first_block + n_blocks)
        for h in range(self.H):
            for bid in range(first_block, first_block + n_blocks):
                if bid in self.lru[h]:
                    self.lru[h].move_to_end(bid)
                else:
                    self._insert(h, bid)

    def touch(self, h: int, bids):
        """Selection touched blocks ``bids`` of head h (ascending unique ids)."""
        for bid in bids:
            lru = self.lru[h]
            if bid in lru:
                lru.move_to_end(bid)
                self.hits += 1
            else:
                self.misses += 1
                self._insert(h, bid)
                self.fetches.append((h, bid))

    def resident(self, h: int):
        return sorted(self.lru[h].keys())


def dedup_keys(block_indices: torch.Tensor, heads: int, mb: int) -> torch.Tensor:
    """Ascending unique keys h*mb + bid of the valid ids of a [B,MG,H,T] table
    (block_kv_ops.h:26-31 with one block per chunk slot)."""
    ids = block_indices.cpu().to(torch.int64)
    h = torch.arange(heads, dtype=torch.int64).view(1, 1, heads, 1).expand_as(ids)
    ok = (ids >= 0) & (ids < mb)
    return torch.unique(h[ok] * mb + ids[ok])


class EpochLRUPagePool:
    """Host model of the device page pool's policy, page ids included, for parity tests of
    the cache kernels.  The LRU clock is an epoch counter bumped once per append / touch call;
    a page for a new or returning block is a free page (lowest id first) or, when none is free,
    the owned, unprotected page not stamped in the current epoch with the lowest (stamp, page id).
    With one key touched per epoch and one pool per head this is exactly the OrderedDict LRU of
    cache.py:673-699 (`LRUBlockCacheModel`); tests replay the reference's own trace through it."""

    def __init__(self, num_heads: int, num_pages: int, max_blocks: int, page_tokens: int,
                 protect_blocks: int = 0):
        self.H, self.P, self.MB, self.PT = num_heads, num_pages, max_blocks, page_tokens
        self.protect = protect_blocks
        self.table = {}                 # key -> page
        self.owner = [-1] * num_pages
        self.stamp = [0] * num_pages
        self.n_tokens = 0
        self.epoch = 0
        self.host = set()               # keys whose K/V were saved to the host tier
        self.evicted_any = False
        self.hits = self.misses = self.pages_evicted = self.pages_fetched = 0
        self.last_evicted = []          # keys evicted by the latest call

    @property
    def n_blocks(self):
        return -(-self.n_tokens // self.PT)

    def _victims(self, n, protect_from=None):
        if protect_from is None:
            protect_from = max(self.n_blocks - self.protect, 0)
        cand = [(0, p) for p in range(self.P) if self.owner[p] < 0]
        cand += [(self.stamp[p] + 1, p) for p in range(self.P)
                 if self.owner[p] >= 0 and self.owner[p] % self.MB < protect_from and self.stamp[p] < self.epoch]
        cand.sort()
        out = [p for _, p in cand[:n]]
        return out + [-1] * (n - len(out))

    def _evict(self, pages):
        for p in pages:
            if p < 0 or self.owner[p] < 0:
                continue
            key = self.owner[p]
            self.host.add(key)
            self.last_evicted.append(key)
            self.pages_evicted += 1
            del self.table[key]
            self.owner[p] = -1

    def _make_resident(self, uniq, count, protect_from=None):
        miss = [k for k in uniq if k not in self.table]
        if count:
            self.hits += len(uniq) - len(miss)
            self.misses += len(miss)
        for k in uniq:
            if k in self.table:
                self.stamp[self.table[k]] = self.epoch
        if self.evicted_any and miss:
            v = self._victims(len(miss), protect_from)
            self._evict(v)
            for k, p in zip(miss, v):
                if p < 0:
                    continue
                self.table[k] = p
                self.owner[p] = k
                self.stamp[p] = self.epoch
                self.pages_fetched += 1
        return miss

    def append(self, S, pos0=None):
        pos0 = self.n_tokens if pos0 is None else pos0
        first, last = pos0 // self.PT, (pos0 + S - 1) // self.PT
        n_touched = last - first + 1
        n_new = max(0, last + 1 - self.n_blocks)
        n_exist = n_touched - n_new
        self.epoch += 1
        self.last_evicted = []
        protect_from = max(min(first, self.n_blocks - self.protect), 0)
        if n_exist and self.evicted_any:
            keys = sorted(h * self.MB + bid for h in range(self.H) for bid in range(first, first + n_exist))
            self._make_resident(keys, False, protect_from)
        ids = []
        need = n_new * self.H
        if need:
            ids = self._victims(need, protect_from)
            self._evict(ids)
            if self.n_blocks * self.H + need > self.P:
                self.evicted_any = True
        for h in range(self.H):
            for j in range(n_touched):
                bid = first + j
                key = h * self.MB + bid
                page = self.table.get(key, -1)
                if page < 0:
                    jn = j - n_exist
                    page = ids[h * n_new + jn] if jn >= 0 else -1
                    if page >= 0:
                        self.table[key] = page
                        self.owner[page] = key
                if page >= 0:
                    self.stamp[page] = self.epoch
        self.n_tokens = max(self.n_tokens, pos0 + S)

    def evict_all(self):
        self.last_evicted = []
        self._evict(list(range(self.P)))
        self.evicted_any = True

    def touch(self, block_indices):
        """block_indices [1,MG,H,T]; returns (unique keys, missing keys), both ascending."""
        self.epoch += 1
        self.last_evicted = []
        uniq = [int(x) for x in dedup_keys(block_indices, self.H, self.MB).tolist()]
        miss = self._make_resident(uniq, True)
        return uniq, miss
