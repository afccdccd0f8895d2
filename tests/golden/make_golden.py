"""Generate the golden vectors under tests/golden/ from the REFERENCE's own code.

Run once, in a container that has the reference checked out (it is not available where
the GPU tests run, so the outputs are committed):

    python tests/golden/make_golden.py --reference /path/to/reference

It imports the reference's pure-torch path (``omnimem.nsa.naive``: index_selection_topk,
inflate_indices, select_attention_torch_chunk), the facade's pooling expression and the
``MMCache`` LRU, runs them on small seeded inputs at geometries the reference accepts
(whole blocks, whole groups) and stores inputs and outputs.  Inputs are rounded to bf16
so the same vectors can be fed to the bf16 kernels; bf16 tensors are stored as their
16-bit patterns (key suffix ``_bf16``).
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bf16_bits(x: torch.Tensor) -> np.ndarray:
    return x.to(torch.bfloat16).view(torch.int16).numpy().copy()


def rb(x: torch.Tensor) -> torch.Tensor:
    """Round to bf16, keep fp32 storage."""
    return x.to(torch.bfloat16).float()


def case_topk(naive_topk, seed, B, M, NC, H, D, T, block_size, chunk_size, causal):
    g = torch.Generator().manual_seed(seed)
    q = rb(torch.randn(B, M, H, D, generator=g))
    kc = rb(torch.randn(B, NC, H, D, generator=g))
    idx = naive_topk(q, kc, None, T, causal=causal, chunk_size=chunk_size, block_size=block_size)
    return dict(q_bf16=bf16_bits(q), k_cmp_bf16=bf16_bits(kc), top_idx_sorted=idx.numpy(),
                meta=np.array([B, M, NC, H, D, T, block_size, chunk_size, int(causal)]))


def case_pool(seed, B, N, H, D, bs, G, M):
    """The reference's pooling expressions, in bf16 (causal_wan_nsa_model.py:408-409 and
    index_topk.py:76)."""
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(B, N, H, D, generator=g).to(torch.bfloat16)
    q = torch.randn(B, M, H, D, generator=g).to(torch.bfloat16)
    k_cmp = k.view(B, N // bs, bs, H, D).mean(2)
    q_grp = q.reshape(B, M // G, G, H, D).mean(dim=2)
    return dict(k_bf16=bf16_bits(k), q_bf16=bf16_bits(q), k_cmp_bf16=bf16_bits(k_cmp),
                q_grp_bf16=bf16_bits(q_grp), meta=np.array([B, N, H, D, bs, G, M]))


def case_attention(naive_topk, inflate, naive_attn, seed, B, M, N, H, D, T, bs, G, chunk, causal):
    g = torch.Generator().manual_seed(seed)
    q = rb(torch.randn(B, M, H, D, generator=g))
    k = rb(torch.randn(B, N, H, D, generator=g))
    v = rb(torch.randn(B, N, H, D, generator=g))
    do = rb(torch.randn(B, M, H, D, generator=g))
    k_cmp = k.view(B, N // bs, bs, H, D).mean(2)
    q_grp = q.reshape(B, M // G, G, H, D).mean(dim=2)
    # group rows: chunk measured in rows for q and in tokens for k, so use the facade's
    # convention by scaling block ids into row units: k_chunk = (c*bs)//chunk tokens and
    # q_chunk = (g*G)//chunk.  The naive function uses one chunk_size for both sides, so it
    # is fed rows expanded back to tokens (one pooled row repeated G times).
    q_rows = q_grp.repeat_interleave(G, dim=1)
    idx_tok = naive_topk(q_rows, k_cmp, None, T, causal=causal, chunk_size=chunk, block_size=bs)
    idx_grp = idx_tok[:, ::G].contiguous()           # [B,MG,H,T], ascending ids
    tok = inflate(idx_tok.to(torch.int64), bs)
    q_ = q.clone().requires_grad_(True)
    k_ = k.clone().requires_grad_(True)
    v_ = v.clone().requires_grad_(True)
    o = naive_attn(q_, k_, v_, tok, causal=causal, q_chunk_size=G, chunk_size=chunk)
    (o * do).sum().backward()
    return dict(q_bf16=bf16_bits(q), k_bf16=bf16_bits(k), v_bf16=bf16_bits(v), do_bf16=bf16_bits(do),
                idx_grp=idx_grp.numpy(), out=o.detach().numpy(), dq=q_.grad.numpy(),
                dk=k_.grad.numpy(), dv=v_.grad.numpy(),
                meta=np.array([B, M, N, H, D, T, bs, G, chunk, int(causal)]))


def case_lru(MMCache, seed, heads, cap, n_ids, n_touch):
    """Trace of MMCache.lru_touch_per_head (cache.py:673-699): the touched ids and, after
    each touch, nothing; at the end the per-head LRU order and the offload queue."""
    cache = MMCache(config={"cache_type": ["k_cache"]}, seq_dim=1,
                    available_shape={"k_cache": (1, 8, 4)}, device="cpu", num_layers=1,
                    lru_max_size=cap, chunk_per_head_types=["k_cache"], num_heads=heads,
                    block_seqlen_config={"k_cache": 4})
    rng = np.random.RandomState(seed)
    trace = np.stack([rng.randint(0, heads, n_touch), rng.randint(0, n_ids, n_touch)], 1)
    evicted = []
    for h, cid in trace:
        cache._to_offload.clear()          # so a repeated victim shows up again
        cache.lru_touch_per_head(0, "k_cache", int(h), int(cid))
        new = sorted(cache._to_offload.get((0, "k_cache"), set()))
        evicted.append(new[0][1] if new else -1)
    final = np.full((heads, cap), -1, dtype=np.int64)
    for h in range(heads):
        lru = cache._lru.get((0, "k_cache", h), {})
        order = list(lru.keys())
        final[h, :len(order)] = order
    return dict(trace=trace.astype(np.int64), evicted=np.array(evicted, dtype=np.int64),
                final_order=final, hits=np.array([cache._lru_total_hits]),
                meta=np.array([heads, cap, n_ids, n_touch]))


def _reference_function(path, name):
    """Executes one top-level function of a reference module from its source text (the module
    itself imports packages that are not installed here)."""
    import re
    from einops import rearrange
    src = open(path).read()
    m = re.search(r"^def %s\(.*?(?=^(?:def |class |@))" % name, src, re.S | re.M)
    ns = {"torch": torch, "rearrange": rearrange}
    exec(m.group(0), ns)
    return ns[name]


def case_rope(ref_root):
    """causal_reorder_rope_apply on small bf16 chunks: plain and pooled token order."""
    base = os.path.join(ref_root, "src", "omnimem", "models", "transformers")
    rope_apply = _reference_function(os.path.join(base, "causal_wan_nsa_model.py"), "causal_reorder_rope_apply")
    rope_params = _reference_function(os.path.join(base, "wan_model.py"), "rope_params")
    D, H = 32, 2
    c = D // 2
    freqs = torch.cat([rope_params(64, D - 4 * (D // 6)), rope_params(64, 2 * (D // 6)), rope_params(64, 2 * (D // 6))],
                      dim=1)                                  # the layout WanModel builds (wan_model.py)
    assert freqs.shape[1] == c
    out = {"freqs": torch.view_as_real(freqs).numpy()}
    g = torch.Generator().manual_seed(21)
    for tag, (f, h, w), pool, start in (("plain", (2, 4, 6), (1, 1, 1), 3), ("pooled", (2, 4, 6), (2, 2, 2), 5)):
        x = torch.randn(1, f * h * w, H, D, generator=g).to(torch.bfloat16)
        y = rope_apply(x, torch.tensor([[f, h, w]]), freqs, start_frame=start, pool_f=pool[0], pool_h=pool[1],
                       pool_w=pool[2])
        out[f"{tag}_x"] = x[0].float().numpy()
        out[f"{tag}_y"] = y[0].float().numpy()
        out[f"{tag}_meta"] = np.array([f, h, w, *pool, start])
    return out


def case_early_out(ref_root):
    """Truth table of should_use_selection_attention (nsa/ops/index_topk.py:165-176) over a grid of
    sequence lengths (in tokens, chunk 10: whole and ragged chunk counts) and exclusion counts."""
    import math
    path = os.path.join(ref_root, "src", "omnimem", "nsa", "ops", "index_topk.py")
    src = open(path).read()
    body = src[src.index("def should_use_selection_attention("):]
    ns = {"math": math}
    exec(body, ns)
    fn = ns["should_use_selection_attention"]
    rows = []
    for seq_len in (1, 9, 10, 11, 20, 35, 40, 70):
        for ex_win in range(0, 5):
            for ex_sink in range(0, 4):
                for causal in (False, True):
                    rows.append([seq_len, 10, ex_win, ex_sink, int(causal), int(bool(fn(seq_len, 10, ex_win, ex_sink, causal)))])
    return {"table": np.array(rows, dtype=np.int64)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (its src/ is imported)")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, "src"))
    from omnimem.nsa.naive.index_selection import index_selection_topk, inflate_indices
    from omnimem.nsa.naive.select_attention import select_attention_torch_chunk
    from omnimem.models.cache import MMCache

    torch.set_num_threads(max(1, os.cpu_count() or 1))
    out = {}
    out["topk_causal"] = case_topk(index_selection_topk, 11, 1, 96, 24, 3, 64, 4, 16, 32, True)
    out["topk_full"] = case_topk(index_selection_topk, 12, 2, 40, 50, 2, 128, 16, 64, 64, False)
    out["pool"] = case_pool(13, 1, 60 * 5, 3, 128, 60, 15, 90)
    out["attn_6464"] = case_attention(index_selection_topk, inflate_indices,
                                      select_attention_torch_chunk, 14, 1, 256, 1024, 2, 128,
                                      4, 64, 64, 256, True)
    out["attn_native"] = case_attention(index_selection_topk, inflate_indices,
                                        select_attention_torch_chunk, 15, 1, 120, 480, 2, 128,
                                        5, 30, 15, 120, True)
    out["attn_full_d64"] = case_attention(index_selection_topk, inflate_indices,
                                          select_attention_torch_chunk, 16, 2, 64, 256, 2, 64,
                                          3, 32, 16, 64, False)
    out["lru"] = case_lru(MMCache, 17, 3, 4, 9, 200)
    out["rope"] = case_rope(args.reference)
    out["early_out"] = case_early_out(args.reference)
    for name, d in out.items():
        path = os.path.join(HERE, f"{name}.npz")
        np.savez_compressed(path, **d)
        print(name, os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main()
