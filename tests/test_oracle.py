"""The CPU oracle against vectors produced by the reference's own pure-torch path
(tests/golden/make_golden.py) and against brute-force restatements."""
import itertools

import pytest
import torch

from oracle import nsa_oracle as O


def _sets(idx):
    return [set(int(x) for x in row if x >= 0) for row in idx.reshape(-1, idx.shape[-1]).tolist()]


@pytest.mark.parametrize("name", ["topk_causal", "topk_full"])
def test_topk_matches_reference_naive(golden, name):
    d = golden(name)
    B, M, NC, H, D, T, bs, chunk, causal = d["meta"].tolist()
    idx = O.topk_select(d["q"].float(), d["k_cmp"].float(), T, block_size=bs, chunk_size=chunk,
                        chunk_size_k=chunk, causal=bool(causal))
    ref = d["top_idx_sorted"]
    # the naive path sorts ids ascending and fills rows that see fewer than T blocks with
    # arbitrary masked ids; compare the visible ids as sets
    vis = O.visibility_mask(M, NC, block_size=bs, chunk_size=chunk, chunk_size_k=chunk,
                            causal=bool(causal))
    n_vis = vis.sum(-1)
    for b, g, h in itertools.product(range(B), range(M), range(H)):
        mine = set(int(x) for x in idx[b, g, h].tolist() if x >= 0)
        theirs = set(int(x) for x in ref[b, g, h].tolist() if vis[g, int(x)])
        assert mine == theirs, (b, g, h)
        assert len(mine) == min(T, int(n_vis[g]))
        assert (idx[b, g, h, len(mine):] == -1).all()


def test_pooling_matches_reference_expression(golden):
    d = golden("pool")
    B, N, H, D, bs, G, M = d["meta"].tolist()
    assert torch.equal(O.pool_rows(d["k"], bs), d["k_cmp"])
    assert torch.equal(O.pool_rows(d["q"], G), d["q_grp"])


@pytest.mark.parametrize("name", ["attn_6464", "attn_native", "attn_full_d64"])
def test_attention_fwd_bwd_matches_reference_naive(golden, name):
    d = golden(name)
    B, M, N, H, D, T, bs, G, chunk, causal = d["meta"].tolist()
    q, k, v, do = (d[x].float() for x in ("q", "k", "v", "do"))
    ids = d["idx_grp"].to(torch.int32)
    out, lse = O.selection_fwd(q, k, v, ids, bs, chunk, None, bool(causal), G)
    assert torch.allclose(out, d["out"], atol=1e-5, rtol=1e-5)
    dq, dk, dv = O.selection_bwd(q, k, v, ids, out, lse, do, bs, chunk, None, bool(causal), G)
    assert torch.allclose(dq, d["dq"], atol=2e-5, rtol=1e-4)
    assert torch.allclose(dk, d["dk"], atol=2e-5, rtol=1e-4)
    assert torch.allclose(dv, d["dv"], atol=2e-5, rtol=1e-4)
    # the top-k of the oracle (pooled operands in fp32 here) picks the same sets
    idx = O.parallel_nsa_topk(q, O.pool_rows(k, bs), T, bs, None, chunk, bool(causal), G)
    vis = O.visibility_mask(M // G, N // bs, block_size=bs, chunk_size=chunk, chunk_size_k=chunk,
                            causal=bool(causal), q_group_size=G)
    for b, g, h in itertools.product(range(B), range(M // G), range(H)):
        mine = set(int(x) for x in idx[b, g, h].tolist() if x >= 0)
        theirs = set(int(x) for x in ids[b, g, h].tolist() if vis[g, int(x)])
        assert mine == theirs


def test_lru_model_matches_reference_mmcache(golden):
    d = golden("lru")
    heads, cap, n_ids, n_touch = d["meta"].tolist()
    m = O.LRUBlockCacheModel(heads, cap, protect_last_blocks=0)
    m.n_blocks = n_ids
    for (h, cid), ev in zip(d["trace"].tolist(), d["evicted"].tolist()):
        n0 = len(m.evictions)
        m.touch(h, [cid])
        got = m.evictions[n0][1] if len(m.evictions) > n0 else -1
        assert got == ev
    for h in range(heads):
        order = [x for x in d["final_order"][h].tolist() if x >= 0]
        assert list(m.lru[h].keys()) == order
    assert m.hits == int(d["hits"][0])


def test_page_pool_model_replays_the_reference_lru_trace(golden):
    """The policy model the device cache is compared with, pinned to the reference: the trace of
    MMCache.lru_touch_per_head (models/cache.py:673-699) replayed through one page pool per head
    (capacity = the LRU size, every block starting in the host tier) evicts the same ids in the
    same order, ends with the same LRU order and counts the same hits."""
    d = golden("lru")
    heads, cap, n_ids, n_touch = d["meta"].tolist()
    pools = []
    for _ in range(heads):
        m = O.EpochLRUPagePool(1, cap, n_ids, 64)
        m.n_tokens = n_ids * 64
        m.evict_all()
        pools.append(m)
    for (h, cid), ev in zip(d["trace"].tolist(), d["evicted"].tolist()):
        m = pools[h]
        m.touch(torch.tensor([[[[cid]]]], dtype=torch.int32))
        got = m.last_evicted[0] if m.last_evicted else -1
        assert got == ev and len(m.last_evicted) <= 1
    for h, m in enumerate(pools):
        order = [x for x in d["final_order"][h].tolist() if x >= 0]
        resident = sorted(m.table, key=lambda k: m.stamp[m.table[k]])
        assert resident == order
    assert sum(m.hits for m in pools) == int(d["hits"][0])


def test_early_out_matches_the_reference_truth_table(golden):
    """should_use_selection_attention against the table the reference's own function produced
    (nsa/ops/index_topk.py:165-176): host integer logic, no device involved."""
    from omnimem_b200.nsa.ops.index_topk import should_use_selection_attention
    table = golden("early_out")["table"].tolist()
    assert len(table) == 8 * 5 * 4 * 2
    for seq_len, chunk, ex_win, ex_sink, causal, want in table:
        assert bool(should_use_selection_attention(seq_len, chunk, ex_win, ex_sink, bool(causal))) == bool(want)


def _visible_bruteforce(g, c, bs, cs, csk, causal, ex_win, ex_sink, prog, off, G):
    q_cid = (g * G) // cs + off
    k_cid = (c * bs) // csk
    do_excl = (q_cid >= ex_sink + ex_win) if prog else True
    valid = (k_cid <= q_cid) if causal else True
    if ex_sink > 0:
        valid = valid and ((k_cid >= ex_sink) or not do_excl)
    if ex_win > 0:
        in_win = k_cid >= q_cid - ex_win + 1
        if not causal:
            in_win = in_win and (k_cid <= q_cid + ex_win - 1)
        valid = valid and ((not in_win) or not do_excl)
    return valid


@pytest.mark.parametrize("causal,ex_win,ex_sink,prog,off,G",
                         [(True, 0, 0, False, 0, 1), (False, 3, 0, True, 4, 4),
                          (True, 2, 1, False, 0, 2), (False, 1, 2, True, 2, 1),
                          (True, 3, 1, True, 1, 4)])
def test_visibility_truth_table(causal, ex_win, ex_sink, prog, off, G):
    MG, NC, bs, cs = 24, 40, 8, 16
    vis = O.visibility_mask(MG, NC, block_size=bs, chunk_size=cs, chunk_size_k=cs, causal=causal,
                            ex_win=ex_win, ex_sink=ex_sink, prog_excl=prog, q_chunk_offset=off,
                            q_group_size=G)
    for g in range(MG):
        for c in range(NC):
            assert bool(vis[g, c]) == _visible_bruteforce(g, c, bs, cs, cs, causal, ex_win,
                                                         ex_sink, prog, off, G)


def test_tie_rule_and_padding():
    # duplicate pooled keys -> equal scores -> lowest id first; fewer visible than T -> -1
    q = torch.randn(1, 2, 1, 16)
    k = torch.randn(1, 3, 1, 16).repeat(1, 2, 1, 1)          # ids j and j+3 tie
    idx = O.topk_select(q, k, 8, block_size=4, chunk_size=1, chunk_size_k=4, causal=False)
    for g in range(2):
        row = idx[0, g, 0].tolist()
        assert row[6:] == [-1, -1]
        for a in range(0, 6, 2):
            assert row[a + 1] == row[a] + 3


def test_ragged_forward_against_dense_masked_softmax():
    torch.manual_seed(0)
    B, M, N, H, D, bs, G, T, chunk = 1, 100, 200, 2, 32, 64, 64, 2, 50
    q, k, v = torch.randn(B, M, H, D), torch.randn(B, N, H, D), torch.randn(B, N, H, D)
    ids = O.parallel_nsa_topk(q, O.pool_rows(k, bs), T, bs, None, chunk, True, G)
    out, lse = O.selection_fwd(q, k, v, ids, bs, chunk, None, True, G)
    # dense restatement with an explicit token mask and autograd for the gradients
    qa, ka, va = (t.clone().double().requires_grad_(True) for t in (q, k, v))
    mask = torch.zeros(B, H, M, N, dtype=torch.bool)
    for g in range((M + G - 1) // G):
        qc = (g * G) // chunk
        for h in range(H):
            for bid in ids[0, g, h].tolist():
                if bid < 0:
                    continue
                t0 = bid * bs
                hi = min(N, t0 + bs, (qc + 1) * chunk)
                mask[0, h, g * G:(g + 1) * G, t0:hi] = True
    s = torch.einsum("bmhd,bnhd->bhmn", qa, ka) * D ** -0.5
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, -1)
    o = torch.einsum("bhmn,bnhd->bmhd", p, va)
    assert torch.allclose(out.double(), o, atol=1e-5)
    assert torch.allclose(lse.double(), torch.logsumexp(s, -1), atol=1e-5)
    do = torch.randn(B, M, H, D)
    (o * do.double()).sum().backward()
    dq, dk, dv = O.selection_bwd(q, k, v, ids, out, lse, do, bs, chunk, None, True, G)
    assert torch.allclose(dq.double(), qa.grad, atol=1e-4)
    assert torch.allclose(dk.double(), ka.grad, atol=1e-4)
    assert torch.allclose(dv.double(), va.grad, atol=1e-4)


def test_empty_rows_and_invalid_ids():
    torch.manual_seed(1)
    q, k, v = torch.randn(1, 8, 1, 16), torch.randn(1, 32, 1, 16), torch.randn(1, 32, 1, 16)
    ids = torch.tensor([[[[-1, -1]], [[9, 1]]]], dtype=torch.int32)   # group 0 empty; id 9 out of range
    out, lse = O.selection_fwd(q, k, v, ids, 8, 1, None, False, 4)
    assert torch.all(out[0, :4] == 0) and torch.all(lse[0, 0, :4] == float("-inf"))
    assert torch.isfinite(lse[0, 0, 4:]).all()


def test_merges_are_exact():
    torch.manual_seed(2)
    B, M, N, H, D, bs, G, T = 1, 32, 256, 2, 32, 16, 16, 4
    q, k, v = torch.randn(B, M, H, D), torch.randn(B, N, H, D), torch.randn(B, N, H, D)
    kp = O.pool_rows(k, bs)
    qp = O.pool_rows(q, G)
    full_i, full_s = O.topk_select(qp, kp, T, block_size=bs, chunk_size=M, chunk_size_k=N,
                                   causal=False, q_group_size=G, return_scores=True)
    R = 4
    parts_i, parts_s = [], []
    for r in range(R):
        own = torch.arange(r, N // bs, R)
        li, ls = O.topk_select(qp, kp[:, own], T, block_size=bs, chunk_size=M, chunk_size_k=N,
                               causal=False, q_group_size=G, return_scores=True)
        gi = torch.where(li >= 0, own[li.clamp_min(0).long()].to(torch.int32), li)
        parts_i.append(gi)
        parts_s.append(ls)
    mi, ms = O.merge_candidates(parts_i, parts_s, T)
    assert torch.equal(mi, full_i)
    out, lse = O.selection_fwd(q, k, v, full_i, bs, 1, None, False, G)
    outs, lses = [], []
    for r in range(R):
        mine = torch.where((full_i >= 0) & (full_i % R == r), full_i, torch.full_like(full_i, -1))
        o_r, l_r = O.selection_fwd(q, k, v, mine, bs, 1, None, False, G)
        outs.append(o_r)
        lses.append(l_r)
    mo, ml = O.merge_partials(outs, lses)
    assert torch.allclose(mo, out, atol=1e-5) and torch.allclose(ml, lse, atol=1e-5)


def test_inverted_index_and_ptr_table():
    ids = torch.tensor([[[[0, 3]], [[3, -1]], [[1, 3]]]], dtype=torch.int32)  # [1,3,1,2]
    groups, offsets = O.inverted_index(ids, 4, 8, 1, False, 1)
    assert offsets[0, 0].tolist() == [0, 1, 2, 2, 5]
    assert groups[0, 0, :5].tolist() == [0, 2, 0, 1, 2]
    base_k = torch.tensor([[4096, 0]], dtype=torch.int64)
    base_v = torch.tensor([[8192, 0]], dtype=torch.int64)
    pk, pv = O.build_ptr_table(ids, base_k, base_v, torch.tensor([4]), 0, 2, 16)
    assert pk[0, :, 0].tolist() == [[4096, 0], [0, 0], [4096 + 16, 0]]
    assert pv[0, 2, 0, 0] == 8192 + 16


def test_gate_combine_matches_the_written_out_formula():
    """oracle.gate_combine against the reference expression evaluated term by term in float64
    (causal_wan_nsa_model.py:378-386, 541-546), all gate modes and skipped modules."""
    g = torch.Generator().manual_seed(0)
    gl = torch.randn(2, 5, 3, 3, generator=g, dtype=torch.float64) * 8        # some logits beyond +-10
    o = [torch.randn(2, 5, 3, 16, generator=g, dtype=torch.float64) for _ in range(3)]
    gc = gl.clamp(-10, 10)
    for mode in ("sigmoid", "softmax"):
        gates = 1 / (1 + torch.exp(-gc)) if mode == "sigmoid" else torch.exp(gc) / torch.exp(gc).sum(-1, keepdim=True)
        for skip in (None, 0, 1):
            want = sum(gates[..., i:i + 1] * o[i] for i in range(3) if i != skip)
            got = O.gate_combine(gl, *[None if i == skip else o[i] for i in range(3)], mode)
            assert torch.allclose(got, want, atol=1e-12)
    with pytest.raises(NotImplementedError):
        O.gate_combine(gl, *o, "tanh")


def test_rope_matches_the_reference_function(golden):
    """oracle.reorder_rope_apply against vectors produced by the reference's own
    causal_reorder_rope_apply (tests/golden/make_golden.py, case_rope): bit-exact in bf16."""
    g = golden("rope")
    freqs = torch.view_as_complex(torch.as_tensor(g["freqs"]).double().contiguous())
    for tag in ("plain", "pooled"):
        f, h, w, pf, ph, pw, start = (int(v) for v in g[f"{tag}_meta"])
        x = torch.as_tensor(g[f"{tag}_x"]).to(torch.bfloat16)
        want = torch.as_tensor(g[f"{tag}_y"]).to(torch.bfloat16)
        got = O.reorder_rope_apply(x, (f, h, w), freqs, start, (pf, ph, pw))
        assert torch.equal(got, want), tag
    # the table builder restates rope_params
    d = 32
    table = torch.cat([O.rope_params(64, d - 4 * (d // 6)), O.rope_params(64, 2 * (d // 6)), O.rope_params(64, 2 * (d // 6))], 1)
    assert torch.equal(torch.view_as_real(table), torch.view_as_real(freqs))
