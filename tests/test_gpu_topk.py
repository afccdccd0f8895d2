"""Pooling, scoring and top-k selection kernels against the CPU oracle (through the C ABI)."""
import pytest
import torch

from oracle import nsa_oracle as O
from tests.helpers import assert_topk_parity, masked_scores, separated_keys

pytestmark = pytest.mark.gpu


def _ops():
    from omnimem_b200 import ops
    return ops


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("N,size,H,D", [(300, 60, 3, 128), (1560, 64, 2, 128), (70, 64, 1, 64), (33, 1, 2, 96), (40, 15, 2, 32)])
def test_pool_rows(dev, dtype, N, size, H, D):
    g = torch.Generator().manual_seed(N + size)
    x = torch.randn(2, N, H, D, generator=g).to(dtype)
    want = O.pool_rows(x, size)
    got = _ops().pool_rows(x.to(dev), size).cpu()
    assert got.shape == want.shape and got.dtype == dtype
    # fp32 sums in a different order may round a value to the neighbouring representable number
    ulp = {torch.bfloat16: 2 ** -7, torch.float16: 2 ** -10, torch.float32: 2 ** -20}[dtype]
    err = (got.float() - want.float()).abs()
    assert (err <= ulp * want.float().abs() + (2e-6 if dtype == torch.float32 else 1e-6)).all()
    if dtype != torch.float32:          # fp32 sums in another order rarely match to the last bit
        assert (err == 0).float().mean() > 0.97


def test_pool_rows_matches_reference_expression(dev, golden):
    d = golden("pool")
    B, N, H, D, bs, G, M = d["meta"].tolist()
    kc = _ops().pool_rows(d["k"].to(dev), bs).cpu()
    qg = _ops().pool_rows(d["q"].to(dev), G).cpu()
    assert ((kc.float() - d["k_cmp"].float()).abs() <= 2 ** -7 * d["k_cmp"].float().abs() + 1e-6).all()
    assert ((qg.float() - d["q_grp"].float()).abs() <= 2 ** -7 * d["q_grp"].float().abs() + 1e-6).all()
    assert (kc == d["k_cmp"]).float().mean() > 0.97


def test_pool_rows_strided_input(dev):
    x = torch.randn(1, 128, 4, 256).to(torch.bfloat16)
    xs = x.to(dev)[..., :128]                       # rows 256 B apart in a 512 B pitch
    assert not xs.is_contiguous()
    got = _ops().pool_rows(xs, 32).cpu()
    assert torch.equal(got, O.pool_rows(x[..., :128].contiguous(), 32)) or \
        (got.float() - O.pool_rows(x[..., :128].contiguous(), 32).float()).abs().max() < 2 ** -7


@pytest.mark.parametrize("name", ["topk_causal", "topk_full"])
def test_topk_golden_from_reference_naive(dev, golden, name):
    d = golden(name)
    B, M, NC, H, D, T, bs, chunk, causal = d["meta"].tolist()
    idx = _ops().topk(d["q"].to(dev), d["k_cmp"].to(dev), T, D ** -0.5, bs, chunk, chunk, bool(causal)).cpu()
    vis = O.visibility_mask(M, NC, block_size=bs, chunk_size=chunk, chunk_size_k=chunk, causal=bool(causal))
    ref = d["top_idx_sorted"]
    s = masked_scores(d["q"].float(), d["k_cmp"].float(), D ** -0.5, block_size=bs, chunk_size=chunk,
                      chunk_size_k=chunk, causal=bool(causal))
    assert_topk_parity(idx, s, T)
    same = 0
    for b in range(B):
        for g in range(M):
            for h in range(H):
                mine = set(idx[b, g, h].tolist()) - {-1}
                theirs = set(int(x) for x in ref[b, g, h].tolist() if vis[g, int(x)])
                same += mine == theirs
    assert same >= 0.98 * B * M * H           # the rest are ties inside the band (checked above)


MASKS = [
    dict(causal=True, ex_win=0, ex_sink=0, prog_excl=False, q_chunk_offset=0, q_group_size=1),
    dict(causal=False, ex_win=3, ex_sink=0, prog_excl=True, q_chunk_offset=4, q_group_size=4),
    dict(causal=True, ex_win=2, ex_sink=1, prog_excl=False, q_chunk_offset=0, q_group_size=2),
    dict(causal=False, ex_win=1, ex_sink=2, prog_excl=True, q_chunk_offset=2, q_group_size=1),
    dict(causal=True, ex_win=3, ex_sink=1, prog_excl=True, q_chunk_offset=1, q_group_size=4),
    dict(causal=False, ex_win=0, ex_sink=0, prog_excl=False, q_chunk_offset=0, q_group_size=8),
]


@pytest.mark.parametrize("mk", MASKS)
def test_topk_mask_modes_exact_on_separated_scores(dev, mk):
    g = torch.Generator().manual_seed(5)
    B, MG, NC, H, D, T, bs, cs = 2, 24, 40, 3, 64, 6, 8, 16
    q = torch.randn(B, MG, H, D, generator=g).to(torch.bfloat16)
    k = separated_keys(B, NC, H, D, g)
    kw = dict(block_size=bs, chunk_size=cs, chunk_size_k=cs, causal=mk["causal"], ex_win=mk["ex_win"],
              ex_sink=mk["ex_sink"], prog_excl=mk["prog_excl"], q_chunk_offset=mk["q_chunk_offset"],
              q_group_size=mk["q_group_size"])
    want, want_s = O.topk_select(q, k, T, 0.125, return_scores=True, **kw)
    got, got_s = _ops().topk(q.to(dev), k.to(dev), T, 0.125, bs, cs, cs, mk["causal"], mk["ex_win"], mk["ex_sink"],
                             mk["prog_excl"], False, mk["q_chunk_offset"], mk["q_group_size"], return_scores=True)
    s = masked_scores(q, k, 0.125, **kw)
    assert_topk_parity(got, s, T)
    assert (got.cpu() == want).float().mean() > 0.995
    fin = torch.isfinite(want_s)
    assert torch.equal(torch.isfinite(got_s.cpu()), fin)
    assert torch.allclose(got_s.cpu()[fin], want_s[fin], atol=1e-4, rtol=1e-5)


def test_topk_tf_mask(dev):
    g = torch.Generator().manual_seed(6)
    B, MG, NC, H, D, T, bs, cs = 1, 32, 32, 2, 32, 5, 4, 8       # 2 clean + 2 noisy chunks
    q = torch.randn(B, MG, H, D, generator=g).to(torch.bfloat16)
    k = separated_keys(B, NC, H, D, g)
    kw = dict(block_size=bs, chunk_size=cs, chunk_size_k=cs, causal=False, tf_mask=True, ex_win=1, ex_sink=0)
    want = O.topk_select(q, k, T, 0.2, **kw)
    got = _ops().topk(q.to(dev), k.to(dev), T, 0.2, bs, cs, cs, False, 1, 0, False, True, 0, 1).cpu()
    assert (got == want).float().mean() > 0.99
    assert_topk_parity(got, masked_scores(q, k, 0.2, **kw), T)


def test_topk_ties_pick_lowest_id_and_pad_with_minus_one(dev):
    g = torch.Generator().manual_seed(7)
    q = torch.randn(1, 2, 1, 16, generator=g).to(torch.bfloat16)
    k = torch.randn(1, 3, 1, 16, generator=g).to(torch.bfloat16).repeat(1, 2, 1, 1)   # ids j and j+3 tie exactly
    got = _ops().topk(q.to(dev), k.to(dev), 8, 0.25, 4, 1, 4, False).cpu()
    want = O.topk_select(q, k, 8, 0.25, block_size=4, chunk_size=1, chunk_size_k=4, causal=False)
    assert torch.equal(got, want)
    for r in range(2):
        row = got[0, r, 0].tolist()
        assert row[6:] == [-1, -1]
        assert all(row[a + 1] == row[a] + 3 for a in range(0, 6, 2))


def test_topk_edge_sizes(dev):
    q = torch.randn(1, 3, 2, 32).to(torch.bfloat16).to(dev)
    empty = torch.empty(1, 0, 2, 32, dtype=torch.bfloat16, device=dev)
    got, sc = _ops().topk(q, empty, 4, 1.0, 8, 8, 8, False, return_scores=True)
    assert (got == -1).all() and got.shape == (1, 3, 2, 4)
    assert torch.isinf(sc).all() and (sc < 0).all()
    # a row that sees nothing (causal, query chunk before every key chunk)
    k = torch.randn(1, 4, 2, 32).to(torch.bfloat16).to(dev)
    got = _ops().topk(q[:, :0], k, 4, 1.0, 8, 8, 8, True)
    assert got.shape == (1, 0, 2, 4)


def test_topk_fp32_inputs(dev):
    g = torch.Generator().manual_seed(8)
    q = torch.randn(1, 25, 12, 128, generator=g)
    k = torch.randn(1, 98, 12, 128, generator=g)
    kw = dict(block_size=64, chunk_size=1560, chunk_size_k=1560, causal=True, q_chunk_offset=3, q_group_size=64)
    got = _ops().topk(q.to(dev), k.to(dev), 16, 128 ** -0.5, 64, 1560, 1560, True, q_chunk_offset=3, q_group_size=64)
    assert_topk_parity(got, masked_scores(q, k, 128 ** -0.5, **kw), 16)


def test_facade_config1_shape_ragged(dev):
    """B=1, H=12, D=128, one 1560-token frame of queries against 4 frames of keys in 64-token
    blocks: last block has 32 tokens, last query group 24 queries."""
    from omnimem_b200.nsa.ops import parallel_nsa_topk
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 1560, 12, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(1, 6240, 12, 128, generator=g).to(torch.bfloat16)
    kp_gpu = _ops().pool_rows(k.to(dev), 64)
    idx = parallel_nsa_topk(q.to(dev), kp_gpu, 16, 64, None, 1560, True, group_size=64, q_chunk_offset=3,
                            allow_ragged=True)
    assert idx.shape == (1, 25, 12, 16) and idx.dtype == torch.int32
    # oracle on the SAME pooled operands (pooling parity is tested separately)
    qp = _ops().pool_rows(q.to(dev), 64).cpu()
    s = masked_scores(qp, kp_gpu.cpu(), 128 ** -0.5, block_size=64, chunk_size=1560, chunk_size_k=1560,
                      causal=True, q_chunk_offset=3, q_group_size=64)
    assert_topk_parity(idx, s, 16)
    with pytest.raises(AssertionError):
        parallel_nsa_topk(q.to(dev), kp_gpu, 16, 64, None, 1560, True, group_size=64, q_chunk_offset=3)


def test_pool_score_topk_equals_two_step(dev):
    g = torch.Generator().manual_seed(9)
    q = torch.randn(1, 10, 4, 128, generator=g).to(torch.bfloat16).to(dev)
    k = torch.randn(1, 1000, 4, 128, generator=g).to(torch.bfloat16).to(dev)
    idx, kp, sc = _ops().pool_score_topk(q, k, 8, 0.1, 64, 640, 640, False, q_group_size=64, return_scores=True)
    kp2 = _ops().pool_rows(k, 64)
    idx2, sc2 = _ops().topk(q, kp2, 8, 0.1, 64, 640, 640, False, q_group_size=64, return_scores=True)
    assert torch.equal(kp, kp2) and torch.equal(idx, idx2) and torch.equal(sc, sc2)


@pytest.mark.parametrize("case", [
    # M, N, H, D, block, group, topk, chunk, causal, q_off, dtype
    (4680, 32760, 12, 128, 64, 64, 16, 1560, True, 18, torch.bfloat16),    # the Wan layer shape, ragged tails
    (300, 1000, 3, 64, 30, 15, 16, 300, True, 2, torch.bfloat16),          # reference-native 30/15 blocks, D=64
    (130, 64 * 21 + 5, 2, 128, 64, 64, 4, 64, False, 0, torch.float16),    # fp16, 22 key blocks: a short last tile
    (70, 900, 2, 256, 64, 64, 3, 10 ** 6, False, 0, torch.bfloat16),       # D=256
    (64, 64 * 3, 1, 32, 64, 1, 2, 64, True, 2, torch.bfloat16),            # one query per row, three key blocks
])
def test_fused_pool_score_select_equals_the_separate_kernels(dev, case):
    """The fused kernel (keys pooled and scored in one pass) and the whole-selection entry point
    (queries pooled too) against pool_rows + topk: pooled operands, ids and scores bit for bit."""
    M, N, H, D, bs, G, T, chunk, causal, q_off, dtype = case
    g = torch.Generator().manual_seed(M + N)
    q = torch.randn(1, M, H, D, generator=g).to(dtype).to(dev)
    k = torch.randn(1, N, H, D, generator=g).to(dtype).to(dev)
    ops = _ops()
    qp = ops.pool_rows(q, G) if G > 1 else q
    kp = ops.pool_rows(k, bs)
    want_i, want_s = ops.topk(qp, kp, T, D ** -0.5, bs, chunk, chunk, causal, q_chunk_offset=q_off, q_group_size=G,
                              return_scores=True)
    idx, kp2, sc = ops.pool_score_topk(qp, k, T, D ** -0.5, bs, chunk, chunk, causal, q_chunk_offset=q_off,
                                       q_group_size=G, return_scores=True)
    assert torch.equal(kp2, kp), "pooled keys of the fused kernel"
    assert torch.equal(idx, want_i) and torch.equal(sc, want_s)
    idx, qp3, kp3, sc = ops.select_blocks(q, k, T, D ** -0.5, bs, G, chunk, chunk, causal, q_chunk_offset=q_off,
                                          return_scores=True)
    assert torch.equal(qp3, qp) and torch.equal(kp3, kp)
    assert torch.equal(idx, want_i) and torch.equal(sc, want_s)
    # strided keys (a slice of a wider tensor): rows stay 16-byte aligned, no copy is made
    wide = torch.randn(1, N, H, 2 * D, generator=torch.Generator().manual_seed(3)).to(dtype).to(dev)
    wide[..., :D] = k
    idx, _, kp4 = ops.select_blocks(q, wide[..., :D], T, D ** -0.5, bs, G, chunk, chunk, causal, q_chunk_offset=q_off)
    assert torch.equal(kp4, kp) and torch.equal(idx, want_i)


@pytest.mark.parametrize("case", [
    # MG, NC, H, D, topk, dtype, mask fields (block, chunk, chunk_k, G, q_off, ex_win, ex_sink, causal, tf, prog, id_base, id_stride)
    (74, 512, 12, 128, 16, torch.bfloat16, (64, 1560, 1560, 64, 18, 0, 0, 1, 0, 0, 0, 1)),       # the Wan layer shape
    (20, 1000, 3, 128, 32, torch.bfloat16, (64, 4680, 4680, 64, 9, 2, 1, 0, 0, 1, 0, 1)),        # two key rounds, 32 keys per lane
    (9, 700, 2, 64, 64, torch.float16, (30, 300, 300, 15, 40, 3, 0, 1, 0, 1, 0, 1)),             # D=64, fp16, top-64
    (5, 130, 2, 32, 8, torch.bfloat16, (8, 16, 16, 1, 30, 1, 1, 1, 0, 0, 0, 1)),                 # D=32: rows of 4 pieces
    (17, 257, 1, 16, 4, torch.bfloat16, (4, 8, 8, 2, 60, 0, 2, 0, 0, 1, 0, 1)),                  # D=16, a 1-key last tile
    (32, 32, 2, 64, 5, torch.bfloat16, (4, 8, 8, 1, 0, 1, 0, 0, 1, 0, 0, 1)),                    # teacher-forcing layout
    (30, 333, 2, 128, 16, torch.bfloat16, (64, 1560, 1560, 64, 50, 1, 0, 1, 0, 0, 2, 5)),        # shard 2 of 5: global ids
    (8, 1024, 1, 128, 16, torch.bfloat16, (64, 10 ** 6, 10 ** 6, 64, 0, 0, 0, 0, 0, 0, 0, 1)),   # the longest fused row
])
def test_one_kernel_scoring_and_selection_equals_the_two_kernel_path(dev, case):
    """nsa_topk (scores kept in shared memory, one kernel) against nsa_topk_static_scratch (score
    buffer + selection kernel) through the C ABI: ids and scores bit for bit, on every mask mode,
    head dim and tile remainder the one-kernel path serves."""
    import ctypes as C
    from omnimem_b200 import _lib
    MG, NC, H, D, T, dtype, mf = case
    g = torch.Generator().manual_seed(MG * 1000 + NC)
    q = torch.randn(1, MG, H, D, generator=g).to(dtype).to(dev)
    k = torch.randn(1, NC, H, D, generator=g).to(dtype).to(dev)
    k[:, 3::7] = k[:, 2::7][:, :k[:, 3::7].shape[1]]               # exact score ties between neighbours
    m = _lib.TopkMask(*mf)
    code = _lib.NSA_BF16 if dtype == torch.bfloat16 else _lib.NSA_F16
    stream = torch.cuda.current_stream(dev).cuda_stream
    lib = _lib.load()
    ws_bytes = lib.nsa_topk_workspace_bytes(1, MG, H, NC)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
    out = []
    for name in ("nsa_topk", "nsa_topk_static_scratch"):
        idx = torch.full((1, MG, H, T), -7, dtype=torch.int32, device=dev)
        sc = torch.full((1, MG, H, T), 7.0, dtype=torch.float32, device=dev)
        args = [q.data_ptr(), _lib.strides3(q), k.data_ptr(), _lib.strides3(k), 1, MG, H, D, NC, T, D ** -0.5, C.byref(m),
                idx.data_ptr(), sc.data_ptr()]
        args += [ws.data_ptr(), ws_bytes] if name == "nsa_topk" else []
        _lib.call(name, *args, code, stream)
        out.append((idx, sc))
    torch.cuda.synchronize()
    (ia, sa), (ib, sb) = out
    assert (ia != -7).all() and (ib != -7).all()
    assert torch.equal(ia, ib), "block ids"
    assert torch.equal(sa.view(torch.int32), sb.view(torch.int32)), "scores, bit for bit"
    assert (ia >= 0).any()


def test_tf_mask_is_rejected_for_sharded_ids(dev):
    from omnimem_b200 import NSABackendError
    q = torch.randn(1, 8, 2, 64).to(torch.bfloat16).to(dev)
    k = torch.randn(1, 8, 2, 64).to(torch.bfloat16).to(dev)
    with pytest.raises(NSABackendError, match="tf_mask"):
        _ops().topk(q, k, 2, 1.0, 8, 16, 16, True, tf_mask=True, id_base=1, id_stride=3)


def test_head_group_pooling_before_selection(dev):
    """num_kv_head_groups < H: heads are averaged per group first (rounded to the input dtype), the
    queries per group second, and every head of a group receives the group's ids
    (nsa/ops/index_topk.py:108-162)."""
    from omnimem_b200.nsa.ops import parallel_nsa_topk, parallel_nsa_topk_grouped_heads
    g = torch.Generator().manual_seed(13)
    B, M, NC, H, D, G, T, NG = 2, 256, 40, 12, 128, 64, 8, 4
    q = torch.randn(B, M, H, D, generator=g).to(torch.bfloat16)
    k = separated_keys(B, NC, H, D, g)
    idx = parallel_nsa_topk_grouped_heads(q.to(dev), k.to(dev), NG, T, 64, 128, causal=True, group_size=G)
    assert idx.shape == (B, M // G, H, T)
    hpg = H // NG
    qg = q.view(B, M, NG, hpg, D).mean(3)                   # the reference's expressions, on the CPU
    kg = k.view(B, NC, NG, hpg, D).mean(3)
    # the kernel's head means: the reference's values up to the last bit of a 1/3 in fp32
    qg_d = _ops().pool_rows(q.to(dev).reshape(1, B * M * H, 1, D), hpg).view(B, M, NG, D)
    kg_d = _ops().pool_rows(k.to(dev).reshape(1, B * NC * H, 1, D), hpg).view(B, NC, NG, D)
    for a, b in ((qg_d.cpu(), qg), (kg_d.cpu(), kg)):
        assert (a == b).float().mean() > 0.99
        assert ((a.float() - b.float()).abs() <= 2 ** -7 * b.float().abs() + 1e-6).all()
    qg, kg = qg_d.cpu(), kg_d.cpu()
    want = parallel_nsa_topk(qg_d, kg_d, T, 64, None, 128, True, group_size=G)
    assert torch.equal(idx.view(B, M // G, NG, hpg, T), want.unsqueeze(3).expand(-1, -1, -1, hpg, -1))
    qp = O.pool_rows(qg, G)
    s = masked_scores(qp, kg, D ** -0.5, block_size=64, chunk_size=128, chunk_size_k=128, causal=True, q_group_size=G)
    assert_topk_parity(want, s, T)
    # all heads in their own group: the plain path
    same = parallel_nsa_topk_grouped_heads(q.to(dev), k.to(dev), H, T, 64, 128, causal=True, group_size=G)
    assert torch.equal(same, parallel_nsa_topk(q.to(dev), k.to(dev), T, 64, None, 128, True, group_size=G))


@pytest.mark.parametrize("topk,NC,causal", [(32, 9000, False), (100, 9000, False), (16, 16384, True), (16, 1025, True),
                                            (160, 3000, False), (200, 700, False), (129, 1500, True)])   # top-k beyond 128
def test_topk_long_rows(dev, topk, NC, causal):
    """Rows of more than 1024 key blocks: per-segment lists merged in a second stage (top-k up to 64)
    or the block-wide kernel (larger top-k); 9000 keys do not fit the shared-memory key cache."""
    g = torch.Generator().manual_seed(10)
    q = torch.randn(1, 5, 2, 64, generator=g).to(torch.bfloat16)
    k = torch.randn(1, NC, 2, 64, generator=g).to(torch.bfloat16)
    chunk = 64 * 2000 if causal else 10 ** 6                # causal: queries of chunk 3 see the first four key chunks
    got, sc = _ops().topk(q.to(dev), k.to(dev), topk, 0.125, 64, chunk, chunk, causal, q_chunk_offset=3 if causal else 0,
                          q_group_size=64, return_scores=True)
    s = masked_scores(q, k, 0.125, block_size=64, chunk_size=chunk, chunk_size_k=chunk, causal=causal,
                      q_chunk_offset=3 if causal else 0, q_group_size=64)
    assert_topk_parity(got, s, topk)
    picked = torch.gather(s.permute(0, 2, 1, 3), -1, got.cpu().long().clamp_min(0))
    assert torch.allclose(sc.cpu()[got.cpu() >= 0], picked[got.cpu() >= 0], atol=1e-5)


def test_sharded_candidates_merge_to_global_topk(dev):
    g = torch.Generator().manual_seed(11)
    B, MG, NC, H, D, T, R = 1, 9, 203, 3, 128, 16, 4
    q = torch.randn(B, MG, H, D, generator=g).to(torch.bfloat16).to(dev)
    k = separated_keys(B, NC, H, D, g).to(dev)
    full, full_s = _ops().topk(q, k, T, 0.09, 64, 4680, 4680, True, q_chunk_offset=2, q_group_size=64,
                               return_scores=True)
    parts_i, parts_s = [], []
    for r in range(R):
        li, ls = _ops().topk(q, k[:, r::R].contiguous(), T, 0.09, 64, 4680, 4680, True, q_chunk_offset=2,
                             q_group_size=64, id_base=r, id_stride=R, return_scores=True)
        parts_i.append(li)
        parts_s.append(ls)
    mi, ms = _ops().merge_candidates(torch.stack(parts_i), torch.stack(parts_s), T)
    assert torch.equal(mi, full)
    assert torch.equal(ms, full_s)
    oi, _ = O.merge_candidates([p.cpu() for p in parts_i], [p.cpu() for p in parts_s], T)
    assert torch.equal(mi.cpu(), oi)
