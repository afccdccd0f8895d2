"""Selection attention forward / backward kernels against the CPU oracle and the vectors
produced by the reference's naive torch path (through the C ABI and the facade)."""
import pytest
import torch

from oracle import nsa_oracle as O
from tests.helpers import assert_close_bf16

pytestmark = pytest.mark.gpu


def _ops():
    from omnimem_b200 import ops
    return ops


def _rand_case(seed, B, M, N, H, D, T, bs, G, chunk, causal, dtype=torch.bfloat16, q_off=0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, M, H, D, generator=g).to(dtype)
    k = torch.randn(B, N, H, D, generator=g).to(dtype)
    v = torch.randn(B, N, H, D, generator=g).to(dtype)
    do = torch.randn(B, M, H, D, generator=g).to(dtype)
    ids = O.parallel_nsa_topk(q, O.pool_rows(k, bs), T, bs, None, chunk, causal, G, q_chunk_offset=q_off)
    return q, k, v, do, ids


def _check(dev, q, k, v, do, ids, bs, chunk, causal, G, what):
    ops = _ops()
    scale = q.shape[-1] ** -0.5
    out, lse = ops.sel_fwd(q.to(dev), ops.DenseKV(k.to(dev), v.to(dev)), ids.to(dev), bs, chunk, scale, causal, G)
    o_ref, l_ref = O.selection_fwd(q.float(), k.float(), v.float(), ids, bs, chunk, scale, causal, G)
    assert_close_bf16(out, o_ref, f"{what} out")
    fin = torch.isfinite(l_ref)
    assert torch.equal(torch.isfinite(lse.cpu()), fin), f"{what}: -inf pattern of lse"
    assert torch.allclose(lse.cpu()[fin], l_ref[fin], atol=2e-3, rtol=1e-4), f"{what} lse"
    dq, dk, dv = ops.sel_bwd(q.to(dev), ops.DenseKV(k.to(dev), v.to(dev)), ids.to(dev), out, lse, do.to(dev), bs,
                             chunk, scale, causal, G)
    # oracle gradients use the kernel's own out / lse rounding of the forward as the reference does
    dq_r, dk_r, dv_r = O.selection_bwd(q.float(), k.float(), v.float(), ids, o_ref, l_ref, do.float(), bs, chunk,
                                       scale, causal, G)
    # gradients at the contract's tolerance for outputs AND gradients: max abs 2e-2, mean abs 2e-3
    assert_close_bf16(dq, dq_r, f"{what} dq")
    assert_close_bf16(dk, dk_r, f"{what} dk")
    assert_close_bf16(dv, dv_r, f"{what} dv")
    return out, lse, dq, dk, dv


@pytest.mark.parametrize("name", ["attn_6464", "attn_native", "attn_full_d64"])
def test_golden_from_reference_naive(dev, golden, name):
    d = golden(name)
    B, M, N, H, D, T, bs, G, chunk, causal = d["meta"].tolist()
    ops = _ops()
    ids = d["idx_grp"].to(torch.int32)
    q, k, v, do = d["q"], d["k"], d["v"], d["do"]
    scale = D ** -0.5
    out, lse = ops.sel_fwd(q.to(dev), ops.DenseKV(k.to(dev), v.to(dev)), ids.to(dev), bs, chunk, scale, bool(causal), G)
    assert_close_bf16(out, d["out"], f"{name} out vs reference naive")
    dq, dk, dv = ops.sel_bwd(q.to(dev), ops.DenseKV(k.to(dev), v.to(dev)), ids.to(dev), out, lse, do.to(dev), bs,
                             chunk, scale, bool(causal), G)
    assert_close_bf16(dq, d["dq"], f"{name} dq vs reference naive")
    assert_close_bf16(dk, d["dk"], f"{name} dk vs reference naive")
    assert_close_bf16(dv, d["dv"], f"{name} dv vs reference naive")


GEOMS = [
    # seed, B, M, N, H, D, T, bs, G, chunk, causal
    (1, 1, 256, 1024, 2, 128, 4, 64, 64, 256, True),       # the 64/64 page geometry
    (2, 1, 200, 1000, 2, 128, 5, 64, 64, 100, True),       # ragged last group (8) and last block (40)
    (3, 2, 120, 480, 2, 128, 5, 30, 15, 120, True),        # reference-native 30/15
    (4, 1, 64, 256, 3, 64, 3, 16, 1, 64, False),           # one query per group
    (5, 1, 256, 512, 1, 128, 3, 64, 128, 256, True),       # 128-query groups (8 warps)
    (6, 1, 180, 600, 2, 128, 4, 60, 60, 180, True),        # 60/60
    (7, 1, 99, 700, 2, 64, 6, 100, 33, 99, False),         # block longer than a tile, odd group
    (8, 1, 130, 390, 2, 128, 20, 13, 10, 130, True),       # many small blocks packed into tiles
    (9, 2, 192, 640, 2, 128, 4, 64, 64, 192, True),        # the page geometry with a batch dimension
    (10, 3, 100, 300, 2, 128, 3, 64, 50, 100, False),      # batch of 3, 50-query groups, ragged last block
]


@pytest.mark.parametrize("case", GEOMS, ids=[f"g{c[8]}_bs{c[7]}_d{c[5]}_t{c[6]}" for c in GEOMS])
def test_forward_backward_geometries(dev, case):
    seed, B, M, N, H, D, T, bs, G, chunk, causal = case
    q, k, v, do, ids = _rand_case(seed, B, M, N, H, D, T, bs, G, chunk, causal)
    _check(dev, q, k, v, do, ids, bs, chunk, causal, G, f"case{seed}")


def test_tensor_core_kernel_agrees_with_general_kernel(dev, monkeypatch):
    """The tcgen05 forward (64-token blocks, 64-query groups, D=128, bf16) against the general
    kernel on the same inputs: dense and paged sources, ragged tails, odd block counts, -1 slots."""
    ops = _ops()
    for seed, M, N, T, chunk, causal in ((41, 256, 4096, 16, 256, False), (42, 200, 1000, 5, 100, True),
                                          (43, 150, 3000, 1, 150, False), (44, 4680, 6000, 7, 1560, True),
                                          (45, 128, 64 * 1500, 8, 128, False),    # long runs of unselected blocks
                                          (46, 3072, 384, 4, 3072, False)):       # 32 query groups per block bucket
        q, k, v, do, ids = _rand_case(seed, 1, M, N, 3, 128, T, 64, 64, chunk, causal)
        ids[0, 0, 0, T // 2:] = -1
        args = (q.to(dev), ops.DenseKV(k.to(dev), v.to(dev)), ids.to(dev), 64, chunk, 128 ** -0.5, causal, 64)
        monkeypatch.setenv("OMNIMEM_B200_FWD_KERNEL", "general")
        o_g, l_g = ops.sel_fwd(*args)
        monkeypatch.delenv("OMNIMEM_B200_FWD_KERNEL")
        o_t, l_t = ops.sel_fwd(*args)
        assert_close_bf16(o_t, o_g, f"tc vs general out (seed {seed})", max_abs=1.6e-2, mean_abs=1e-3)
        fin = torch.isfinite(l_g)
        assert torch.equal(torch.isfinite(l_t), fin)
        assert torch.allclose(l_t[fin], l_g[fin], atol=1e-3, rtol=1e-4)
        o_ref, l_ref = O.selection_fwd(q.float(), k.float(), v.float(), ids, 64, chunk, None, causal, 64)
        assert_close_bf16(o_t, o_ref, f"tc out vs oracle (seed {seed})")
        # dQ half of the backward: tensor-core kernel against the general kernel and the oracle
        bargs = (q.to(dev), ops.DenseKV(k.to(dev), v.to(dev)), ids.to(dev), o_t, l_t, do.to(dev), 64, chunk,
                 128 ** -0.5, causal, 64)
        monkeypatch.setenv("OMNIMEM_B200_BWD_KERNEL", "general")
        dq_g, dl_g = ops.sel_bwd_dq(*bargs)
        monkeypatch.delenv("OMNIMEM_B200_BWD_KERNEL")
        dq_t, dl_t = ops.sel_bwd_dq(*bargs)
        assert torch.allclose(dl_t, dl_g, atol=2e-3, rtol=1e-3), f"delta (seed {seed})"
        assert_close_bf16(dq_t, dq_g, f"tc vs general dq (seed {seed})", mean_abs=1.5e-3)
        dq_r, _, _ = O.selection_bwd(q.float(), k.float(), v.float(), ids, o_ref, l_ref, do.float(), 64, chunk, None,
                                     causal, 64)
        assert_close_bf16(dq_t, dq_r, f"tc dq vs oracle (seed {seed})")
        # dK / dV half: tensor-core kernel against the general kernel and the oracle
        NS = -(-N // 64)
        groups, offsets = ops.inverted_index(ids.to(dev), NS, 64, chunk, causal, 64)
        kargs = (q.to(dev), ops.DenseKV(k.to(dev), v.to(dev)), groups, offsets, l_t, dl_t, do.to(dev), T, 64, chunk,
                 128 ** -0.5, causal, 64)
        monkeypatch.setenv("OMNIMEM_B200_BWD_KERNEL", "general")
        dk_g, dv_g = ops.sel_bwd_dkv(*kargs)
        monkeypatch.delenv("OMNIMEM_B200_BWD_KERNEL")
        dk_t, dv_t = ops.sel_bwd_dkv(*kargs)
        dk_t2, dv_t2 = ops.sel_bwd_dkv(*kargs)
        assert torch.equal(dk_t, dk_t2) and torch.equal(dv_t, dv_t2), "dk/dv not bit-reproducible"
        _, dk_r, dv_r = O.selection_bwd(q.float(), k.float(), v.float(), ids, o_ref, l_ref, do.float(), 64, chunk,
                                        None, causal, 64)
        assert_close_bf16(dk_t, dk_g, f"tc vs general dk (seed {seed})")
        assert_close_bf16(dv_t, dv_g, f"tc vs general dv (seed {seed})")
        assert_close_bf16(dk_t, dk_r, f"tc dk vs oracle (seed {seed})")
        assert_close_bf16(dv_t, dv_r, f"tc dv vs oracle (seed {seed})")


def test_fp16(dev):
    q, k, v, do, ids = _rand_case(21, 1, 128, 512, 2, 128, 4, 64, 64, 128, True, dtype=torch.float16)
    _check(dev, q, k, v, do, ids, 64, 128, True, 64, "fp16")


def test_invalid_duplicate_and_empty_rows(dev):
    g = torch.Generator().manual_seed(22)
    B, M, N, H, D, bs, G = 1, 96, 250, 2, 128, 32, 32
    q = torch.randn(B, M, H, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, N, H, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, N, H, D, generator=g).to(torch.bfloat16)
    do = torch.randn(B, M, H, D, generator=g).to(torch.bfloat16)
    ids = torch.tensor([[[[-1, -1, -1, -1], [3, 3, -1, 7]],          # group 0: empty row / duplicate + last partial block
                         [[99, 2, -1, 0], [-1, -1, 5, -1]],          # out-of-range id is skipped
                         [[7, 6, 5, 4], [-1, -1, -1, -1]]]], dtype=torch.int32)
    out, lse, dq, dk, dv = _check(dev, q, k, v, do, ids, bs, 1, False, G, "edge")
    assert (out[0, :32, 0] == 0).all() and torch.isinf(lse[0, 0, :32]).all()
    assert (dq[0, :32, 0] == 0).all()
    assert (dk[0, :, 0][32:64] == 0).all()           # block 1 of head 0 was never selected


def test_causal_prefix_inside_a_block(dev):
    # chunk boundaries cut through blocks: 100-token chunks, 64-token blocks
    q, k, v, do, ids = _rand_case(23, 1, 300, 300, 2, 128, 3, 64, 50, 100, True)
    _check(dev, q, k, v, do, ids, 64, 100, True, 50, "prefix")


def test_strided_inputs(dev):
    g = torch.Generator().manual_seed(24)
    B, M, N, H, D, bs, G, T = 1, 128, 512, 2, 128, 64, 64, 3
    big_q = torch.randn(B, M, H, 3 * D, generator=g).to(torch.bfloat16)
    big_kv = torch.randn(B, N, H, 2 * D, generator=g).to(torch.bfloat16)
    q, k, v = big_q[..., D:2 * D], big_kv[..., :D], big_kv[..., D:]
    ids = O.parallel_nsa_topk(q, O.pool_rows(k.contiguous(), bs), T, bs, None, 128, True, G)
    ops = _ops()
    qd, kvd = big_q.to(dev), big_kv.to(dev)
    out, lse = ops.sel_fwd(qd[..., D:2 * D], ops.DenseKV(kvd[..., :D], kvd[..., D:]), ids.to(dev), bs, 128, D ** -0.5, True, G)
    o_ref, _ = O.selection_fwd(q.float(), k.float(), v.float(), ids, bs, 128, None, True, G)
    assert_close_bf16(out, o_ref, "strided out")
    # backward with strided q / k / v / dO (views into wider tensors)
    big_do = torch.randn(B, M, H, 2 * D, generator=g).to(torch.bfloat16)
    dod = big_do.to(dev)
    dq, dk, dv = ops.sel_bwd(qd[..., D:2 * D], ops.DenseKV(kvd[..., :D], kvd[..., D:]), ids.to(dev), out, lse,
                             dod[..., D:], bs, 128, D ** -0.5, True, G)
    dq_c, dk_c, dv_c = ops.sel_bwd(qd[..., D:2 * D].contiguous(), ops.DenseKV(kvd[..., :D].contiguous(), kvd[..., D:].contiguous()),
                                   ids.to(dev), out, lse, dod[..., D:].contiguous(), bs, 128, D ** -0.5, True, G)
    assert torch.equal(dq, dq_c) and torch.equal(dk, dk_c) and torch.equal(dv, dv_c), "strided backward differs from contiguous"


def test_dkdv_bit_reproducible(dev):
    q, k, v, do, ids = _rand_case(25, 1, 512, 1024, 2, 128, 8, 64, 64, 512, False)
    ops = _ops()
    kv = ops.DenseKV(k.to(dev), v.to(dev))
    out, lse = ops.sel_fwd(q.to(dev), kv, ids.to(dev), 64, 512, 0.0884, False, 64)
    runs = [ops.sel_bwd(q.to(dev), kv, ids.to(dev), out, lse, do.to(dev), 64, 512, 0.0884, False, 64) for _ in range(3)]
    for r in runs[1:]:
        for a, b in zip(runs[0], r):
            assert torch.equal(a, b)


def test_inverted_index(dev):
    g = torch.Generator().manual_seed(26)
    ids = torch.randint(-1, 20, (2, 7, 3, 5), generator=g, dtype=torch.int32)
    groups, offsets = _ops().inverted_index(ids.to(dev), 16, 8, 16, True, 4)
    g_ref, o_ref = O.inverted_index(ids, 16, 8, 16, True, 4)
    assert torch.equal(offsets.cpu(), o_ref)
    groups = groups.cpu()
    for b in range(2):
        for h in range(3):
            for s in range(16):
                lo, hi = int(o_ref[b, h, s]), int(o_ref[b, h, s + 1])
                assert groups[b, h, lo:hi].tolist() == g_ref[b, h, lo:hi].tolist()   # ascending inside a bucket


def test_inverted_index_many_blocks(dev):
    """More blocks than one thread block can count in shared memory: the multi-kernel path."""
    g = torch.Generator().manual_seed(31)
    NS = 45000
    ids = torch.randint(-1, NS, (1, 40, 2, 6), generator=g, dtype=torch.int32)
    ids[0, :, :, 0] = 7                                     # one long bucket
    groups, offsets = _ops().inverted_index(ids.to(dev), NS, 64, 1, False, 64)
    g_ref, o_ref = O.inverted_index(ids, NS, 64, 1, False, 64)
    assert torch.equal(offsets.cpu(), o_ref)
    n = int(o_ref[0, 0, -1])
    assert torch.equal(groups.cpu()[:, :, :n], g_ref[:, :, :n])


def test_inverted_index_slots(dev):
    """The slot output: entry e of a bucket names (group, slot) with ids[b, group, h, slot] == the
    bucket's block; groups as without slots, buckets ordered by (group, slot), duplicates kept apart."""
    g = torch.Generator().manual_seed(27)
    for NS, T, MG in ((16, 5, 7), (45000, 6, 40)):                     # one-kernel and multi-kernel index
        ids = torch.randint(-1, NS if NS < 100 else 60, (2, MG, 3, T), generator=g, dtype=torch.int32)
        ids[0, 1, 0, :2] = 3                                            # a duplicate inside a row
        plain_g, plain_o = _ops().inverted_index(ids.to(dev), NS, 8, 16, False, 4)
        groups, offsets, slots = _ops().inverted_index(ids.to(dev), NS, 8, 16, False, 4, with_slots=True)
        assert torch.equal(offsets, plain_o)
        n = int(offsets[0, 0, -1])
        assert torch.equal(groups[:, :, :n], plain_g[:, :, :n])
        groups, offsets, slots = groups.cpu(), offsets.cpu(), slots.cpu()
        for b in range(2):
            for h in range(3):
                seen = set()
                for blk in ids[b, :, h].unique().tolist():
                    if blk < 0:
                        continue
                    lo, hi = int(offsets[b, h, blk]), int(offsets[b, h, blk + 1])
                    pairs = list(zip(groups[b, h, lo:hi].tolist(), slots[b, h, lo:hi].tolist()))
                    assert pairs == sorted(pairs) and len(set(pairs)) == len(pairs)
                    for gg, tt in pairs:
                        assert int(ids[b, gg, h, tt]) == blk
                    seen.update(pairs)
                want = {(gg, tt) for gg in range(MG) for tt in range(T) if 0 <= int(ids[b, gg, h, tt]) < NS}
                assert seen == want


@pytest.mark.parametrize("case", [
    # seed, M, N, H, T, chunk, causal, paged
    (61, 4680, 6000, 3, 7, 1560, True, False),
    (62, 200, 1000, 2, 5, 100, True, True),
    (63, 3072, 384, 2, 4, 3072, False, False),           # 48 query groups per block bucket: long buckets
    (64, 150, 64 * 40 + 9, 4, 16, 150, False, True),     # ragged last block and group
])
def test_backward_from_stored_probabilities(dev, monkeypatch, case):
    """The backward that computes P and dS once (dQ kernel stores the tiles, dK/dV kernel streams
    them) against the backward that recomputes them and against the oracle; twice, bit for bit."""
    seed, M, N, H, T, chunk, causal, paged = case
    ops = _ops()
    q, k, v, do, ids = _rand_case(seed, 1, M, N, H, 128, T, 64, 64, chunk, causal)
    ids[0, 0, 0, T // 2:] = -1
    ids[0, 1, 1, 1] = ids[0, 1, 1, 0]                                   # a block listed twice in one row
    scale = 128 ** -0.5
    qd, kd, vd, dod, idd = (t.to(dev) for t in (q, k, v, do, ids))
    if paged:
        from omnimem_b200.cache import BlockKVCache
        nb = -(-N // 64)
        cache = BlockKVCache(H, 128, num_pages=H * nb + 3, max_blocks=nb + 2, page_tokens=64, device=dev, host_tier=False)
        cache.append(kd[0], vd[0])
        kv = cache.kv_source()
    else:
        kv = ops.DenseKV(kd, vd)
    out, lse = ops.sel_fwd(qd, kv, idd, 64, chunk, scale, causal, 64)
    assert ops.stored_probabilities_bytes(qd, kv, idd, 64, 64) == (-(-M // 64)) * H * T * 16384
    got = ops.sel_bwd(qd, kv, idd, out, lse, dod, 64, chunk, scale, causal, 64)
    again = ops.sel_bwd(qd, kv, idd, out, lse, dod, 64, chunk, scale, causal, 64)
    for a, b in zip(got, again):
        assert torch.equal(a, b), "not bit-reproducible"
    monkeypatch.setenv("OMNIMEM_B200_BWD_STORED_MB", "0")
    assert ops.stored_probabilities_bytes(qd, kv, idd, 64, 64) == 0
    ref = ops.sel_bwd(qd, kv, idd, out, lse, dod, 64, chunk, scale, causal, 64)
    monkeypatch.delenv("OMNIMEM_B200_BWD_STORED_MB")
    o_ref, l_ref = O.selection_fwd(q.float(), k.float(), v.float(), ids, 64, chunk, scale, causal, 64)
    orc = O.selection_bwd(q.float(), k.float(), v.float(), ids, o_ref, l_ref, do.float(), 64, chunk, scale, causal, 64)
    for name, a, b, c in zip(("dq", "dk", "dv"), got, ref, orc):
        assert_close_bf16(a, b, f"stored vs recomputed {name} (seed {seed})")
        assert_close_bf16(a, c, f"stored {name} vs oracle (seed {seed})")


def test_pointer_table_source(dev):
    g = torch.Generator().manual_seed(27)
    B, M, N, H, D, bs, G, T = 1, 128, 512, 2, 128, 64, 64, 3
    q = torch.randn(B, M, H, D, generator=g).to(torch.bfloat16)
    # chunk-per-head storage: one [N, D] tensor per head, as the reference's pointer path expects
    ks = [torch.randn(N, D, generator=g).to(torch.bfloat16) for _ in range(H)]
    vs = [torch.randn(N, D, generator=g).to(torch.bfloat16) for _ in range(H)]
    k = torch.stack(ks, 1).unsqueeze(0)
    v = torch.stack(vs, 1).unsqueeze(0)
    ids = O.parallel_nsa_topk(q, O.pool_rows(k, bs), T, bs, None, N, False, G)
    ids[0, 1, 0, 2] = -1
    ops = _ops()
    kd, vd = [t.to(dev) for t in ks], [t.to(dev) for t in vs]
    base_k = torch.tensor([[t.data_ptr()] for t in kd], dtype=torch.int64, device=dev)
    base_v = torch.tensor([[t.data_ptr()] for t in vd], dtype=torch.int64, device=dev)
    nb = torch.full((H,), N // bs, dtype=torch.int32, device=dev)
    pk, pv = ops.build_ptr_table(ids.to(dev), base_k, base_v, nb, 0, N // bs, bs * D * 2)
    pk_ref, pv_ref = O.build_ptr_table(ids, base_k.cpu(), base_v.cpu(), nb.cpu(), 0, N // bs, bs * D * 2)
    assert torch.equal(pk.cpu(), pk_ref) and torch.equal(pv.cpu(), pv_ref)
    out, lse = ops.sel_fwd(q.to(dev), ops.PtrKV(pk, pv, D), None, bs, 1, D ** -0.5, False, G)
    o_ref, l_ref = O.selection_fwd(q.float(), k.float(), v.float(), ids, bs, 1, None, False, G)
    assert_close_bf16(out, o_ref, "ptr out")


def test_partials_merge_exactly(dev):
    q, k, v, do, ids = _rand_case(28, 1, 192, 2048, 2, 128, 8, 64, 64, 192, False)
    ops = _ops()
    kv = ops.DenseKV(k.to(dev), v.to(dev))
    full, full_l = ops.sel_fwd(q.to(dev), kv, ids.to(dev), 64, 1, 0.0884, False, 64)
    R = 4
    outs, lses = [], []
    for r in range(R):
        mine = torch.where((ids >= 0) & (ids % R == r), ids, torch.full_like(ids, -1))
        o_r, l_r = ops.sel_fwd(q.to(dev), kv, mine.to(dev), 64, 1, 0.0884, False, 64)
        outs.append(o_r)
        lses.append(l_r)
    mo, ml = ops.merge_partials(torch.stack(outs), torch.stack(lses))
    assert_close_bf16(mo, full, "merged out", max_abs=1.6e-2)
    assert torch.allclose(ml, full_l, atol=1e-4)
    ro, rl = O.merge_partials([o.cpu() for o in outs], [l.cpu() for l in lses])
    assert_close_bf16(mo, ro, "merged out vs oracle merge", max_abs=8e-3)


def test_facade_autograd_and_errors(dev):
    from omnimem_b200.nsa.ops import selection_attention
    q, k, v, do, ids = _rand_case(29, 1, 128, 512, 2, 128, 4, 64, 64, 128, True)
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    out, lse = selection_attention(qd, kd, vd, ids.to(dev), 4, 64, chunk_size=128, causal=True, return_lse=True,
                                   group_size=64)
    (out.float() * do.to(dev).float()).sum().backward()
    o_ref, l_ref = O.selection_fwd(q.float(), k.float(), v.float(), ids, 64, 128, None, True, 64)
    dq_r, dk_r, dv_r = O.selection_bwd(q.float(), k.float(), v.float(), ids, o_ref, l_ref, do.float(), 64, 128,
                                       None, True, 64)
    assert_close_bf16(out, o_ref, "facade out")
    assert_close_bf16(qd.grad, dq_r, "facade dq")
    assert_close_bf16(kd.grad, dk_r, "facade dk")
    assert_close_bf16(vd.grad, dv_r, "facade dv")
    with pytest.raises(ValueError, match="out of range"):
        selection_attention(qd, kd, vd, torch.full_like(ids, 99).to(dev), 4, 64, group_size=64)
    with pytest.raises(AssertionError, match="divisible"):
        selection_attention(qd[:, :100], kd, vd, ids.to(dev), 4, 64, group_size=64)
    with pytest.raises(NotImplementedError):
        selection_attention(qd, kd, vd, ids.to(dev), 4, 64, variant="one-pass", group_size=64)


def test_config1_shape_fp32_tensors(dev):
    """B=1, H=12, D=128, fp32, one 1560-token frame of queries (frame 3) against 4 frames of keys
    in 64-token blocks, top-16 per 64-query group, block-causal by frame, seed 0 - the reference's
    CPU-runnable case.  fp32 tensors are computed on bf16 operands; compared with the fp32 oracle."""
    from omnimem_b200.nsa.ops import parallel_nsa_topk, selection_attention
    ops = _ops()
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 1560, 12, 128, generator=g)
    k = torch.randn(1, 6240, 12, 128, generator=g)
    v = torch.randn(1, 6240, 12, 128, generator=g)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    idx = parallel_nsa_topk(qd, ops.pool_rows(kd, 64), 16, 64, None, 1560, True, group_size=64, q_chunk_offset=3,
                            allow_ragged=True)
    out, lse = selection_attention(qd, kd, vd, idx, 16, 64, chunk_size=1, causal=False, return_lse=True, group_size=64,
                                   allow_ragged=True)
    assert out.dtype == torch.float32 and out.shape == q.shape
    o_ref, l_ref = O.selection_fwd(q, k, v, idx.cpu(), 64, 1, None, False, 64)
    assert_close_bf16(out, o_ref, "config 1 out (fp32 tensors, bf16 operands)")
    assert torch.allclose(lse.cpu(), l_ref, atol=1e-2)


def test_torch_ops_namespace(dev):
    import omnimem_b200.torch_ops  # noqa: F401
    q, k, v, do, ids = _rand_case(30, 1, 128, 512, 2, 128, 4, 64, 64, 128, True)
    out, lse = torch.ops.omnimem_nsa.sel_fwd(q.to(dev), k.to(dev), v.to(dev), ids.to(dev), 64, 128, 128 ** -0.5,
                                             True, 64, True)
    dq, dk, dv = torch.ops.omnimem_nsa.sel_bwd(q.to(dev), k.to(dev), v.to(dev), ids.to(dev), out, lse, do.to(dev),
                                               64, 128, 128 ** -0.5, True, 64, True)
    assert out.shape == q.shape and lse.shape == (1, 2, 128) and lse.dtype == torch.float32
    assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == v.shape
    qp = _ops().pool_rows(q.to(dev), 64)
    kp = _ops().pool_rows(k.to(dev), 64)
    idx = torch.ops.omnimem_nsa.topk(qp, kp, 4, 128 ** -0.5, 64, 2, 128, True, 0, 0, False, False, 0, True)
    assert idx.shape == (1, 2, 2, 4) and idx.dtype == torch.int32
    want = O.topk_select(qp.cpu(), kp.cpu(), 4, 128 ** -0.5, block_size=64, chunk_size=2, chunk_size_k=128, causal=True)
    assert (idx.cpu() == want).float().mean() > 0.95


def test_config2_full_size_properties(dev):
    """B=1, H=12, D=128, M=4680 (3 latent frames), N=32760 (21 frames), 64-token blocks,
    top-16 per 64-query group, block-causal by frame.  Checked through size-independent
    properties plus the oracle on a sample of rows."""
    ops = _ops()
    g = torch.Generator().manual_seed(0)
    B, M, N, H, D, bs, G, T, frame = 1, 4680, 32760, 12, 128, 64, 64, 16, 1560
    q = torch.randn(B, M, H, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, N, H, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, N, H, D, generator=g).to(torch.bfloat16)
    do = torch.randn(B, M, H, D, generator=g).to(torch.bfloat16)
    qd, kd, vd, dod = (t.to(dev) for t in (q, k, v, do))
    qp = ops.pool_rows(qd, G)
    idx, kp = ops.pool_score_topk(qp, kd, T, D ** -0.5, bs, frame, frame, True, q_chunk_offset=18, q_group_size=G)
    assert idx.shape == (1, 74, 12, 16) and (idx >= 0).all() and (idx < 512).all()
    srt = idx.sort(-1).values
    assert (srt[..., 1:] != srt[..., :-1]).all()                        # no duplicates in a row
    # the selection kernels see queries at frames 18..20: pass the global chunk through causal=False
    kv = ops.DenseKV(kd, vd)
    out, lse = ops.sel_fwd(qd, kv, idx, bs, 1, D ** -0.5, False, G)
    # property 1: splitting every row's blocks in two and merging the partials gives the same result
    half = torch.where(torch.arange(T, device=dev) < 8, idx, torch.full_like(idx, -1))
    rest = torch.where(torch.arange(T, device=dev) >= 8, idx, torch.full_like(idx, -1))
    o1, l1 = ops.sel_fwd(qd, kv, half, bs, 1, D ** -0.5, False, G)
    o2, l2 = ops.sel_fwd(qd, kv, rest, bs, 1, D ** -0.5, False, G)
    mo, ml = ops.merge_partials(torch.stack([o1, o2]), torch.stack([l1, l2]))
    assert_close_bf16(mo, out, "split/merge", max_abs=1.6e-2)
    assert torch.allclose(ml, lse, atol=1e-4)
    # property 2: linear in V
    out2, _ = ops.sel_fwd(qd, ops.DenseKV(kd, vd * 2), idx, bs, 1, D ** -0.5, False, G)
    assert_close_bf16(out2, out.float() * 2, "linearity in V")
    # property 3: sum over tokens of dV rows equals P^T dO column sums -> sum(dv) = sum over rows of dO weighted by 1
    dq, dk, dv = ops.sel_bwd(qd, kv, idx, out, lse, dod, bs, 1, D ** -0.5, False, G)
    assert torch.allclose(dv.float().sum((0, 1)), dod.float().sum((0, 1)), rtol=2e-2, atol=1.0)
    # oracle on a sample: 3 groups (incl. the ragged last one) x all heads
    for grp in (0, 37, 73):
        m0, m1 = grp * G, min(M, grp * G + G)
        ids_g = idx[:, grp:grp + 1].cpu()
        o_ref, l_ref = O.selection_fwd(q[:, m0:m1].float(), k.float(), v.float(), ids_g, bs, 1, None, False, G)
        assert_close_bf16(out[:, m0:m1], o_ref, f"group {grp} out")
        assert torch.allclose(lse[:, :, m0:m1].cpu(), l_ref, atol=2e-3)
        dq_r, _, _ = O.selection_bwd(q[:, m0:m1].float(), k.float(), v.float(), ids_g, o_ref, l_ref,
                                     do[:, m0:m1].float(), bs, 1, None, False, G)
        assert_close_bf16(dq[:, m0:m1], dq_r, f"group {grp} dq")
    # the whole backward of three heads (first, middle, last) against the oracle: every dK / dV row of
    # the 32760 tokens, summed over all the groups that selected its block, and all of dQ
    hs = [0, 5, 11]
    qh, kh, vh, doh = (t[:, :, hs].float() for t in (q, k, v, do))
    ids_h = idx[:, :, hs].cpu()
    o_ref, l_ref = O.selection_fwd(qh, kh, vh, ids_h, bs, 1, None, False, G)
    dq_r, dk_r, dv_r = O.selection_bwd(qh, kh, vh, ids_h, o_ref, l_ref, doh, bs, 1, None, False, G)
    assert_close_bf16(out[:, :, hs], o_ref, "config 2 out, heads 0/5/11")
    assert_close_bf16(dq[:, :, hs], dq_r, "config 2 dq, heads 0/5/11")
    assert_close_bf16(dk[:, :, hs], dk_r, "config 2 dk, heads 0/5/11")
    assert_close_bf16(dv[:, :, hs], dv_r, "config 2 dv, heads 0/5/11")
    # top-k parity on the same pooled operands
    from tests.helpers import assert_topk_parity, masked_scores
    s = masked_scores(qp.cpu(), kp.cpu(), D ** -0.5, block_size=bs, chunk_size=frame, chunk_size_k=frame,
                      causal=True, q_chunk_offset=18, q_group_size=G)
    assert_topk_parity(idx, s, T)


@pytest.mark.gpu
def test_captured_step_replays_the_eager_result():
    """A CUDA-graph replay of pooling + top-k + forward + backward gives the eager tensors."""
    from omnimem_b200 import ops
    from omnimem_b200.graph import CapturedStep
    torch.manual_seed(7)
    dev = torch.device("cuda")
    B, M, N, H, D, T = 1, 256, 1024, 4, 128, 4
    q = torch.randn(B, M, H, D, device=dev, dtype=torch.bfloat16)
    k = torch.randn(B, N, H, D, device=dev, dtype=torch.bfloat16)
    v = torch.randn(B, N, H, D, device=dev, dtype=torch.bfloat16)
    do = torch.randn(B, M, H, D, device=dev, dtype=torch.bfloat16)
    scale = D ** -0.5

    def step():
        qp, kp = ops.pool_rows(q, 64), ops.pool_rows(k, 64)
        idx = ops.topk(qp, kp, T, scale, 64, 1 << 30, 1 << 30, False, q_group_size=64)
        kv = ops.DenseKV(k, v)
        out, lse = ops.sel_fwd(q, kv, idx, 64, 1, scale, False, 64)
        groups, offsets = ops.inverted_index(idx, N // 64, 64, 1, False, 64)
        dq, delta = ops.sel_bwd_dq(q, kv, idx, out, lse, do, 64, 1, scale, False, 64)
        dk, dv = ops.sel_bwd_dkv(q, kv, groups, offsets, lse, delta, do, T, 64, 1, scale, False, 64)
        return idx, out, dq, dk, dv

    eager = [x.clone() for x in step()]
    cap = CapturedStep(step)
    q.copy_(torch.randn_like(q))          # new inputs at the same addresses
    eager2 = [x.clone() for x in step()]
    replayed = [x.clone() for x in cap.replay()]
    torch.cuda.synchronize()
    assert any(not torch.equal(a, b) for a, b in zip(eager, eager2))
    for a, b in zip(eager2, replayed):
        assert torch.equal(a, b)
