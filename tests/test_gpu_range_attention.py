"""Attention over one contiguous range of KV blocks (the layer's compressed and sliding-window
branches) against the CPU oracle and against the selection forward given the same blocks as a list."""
import pytest
import torch

from oracle import nsa_oracle as O
from tests.helpers import assert_close_bf16

pytestmark = pytest.mark.gpu


def _ops():
    from omnimem_b200 import ops
    return ops


def _listed(first, n, B, M, H, G=64):
    ids = torch.arange(first, first + max(n, 1), dtype=torch.int32)
    if n == 0:
        ids = torch.full_like(ids, -1)
    return ids.expand(B, -(-M // G), H, ids.numel()).contiguous()


def _compare(out, lse, o_ref, l_ref, what):
    assert_close_bf16(out, o_ref, f"{what} out")
    fin = torch.isfinite(l_ref)
    assert torch.equal(torch.isfinite(lse.cpu()), fin), f"{what}: -inf pattern of lse"
    assert torch.allclose(lse.cpu()[fin], l_ref[fin], atol=2e-3, rtol=1e-4), f"{what} lse"


@pytest.mark.parametrize("case", [
    # B, M, N, H, first, n
    (1, 256, 1024, 2, 0, 16),       # every block
    (1, 200, 1000, 3, 3, 9),        # ragged rows, a range inside the KV
    (2, 130, 700, 2, 2, 9),         # two batches, partly filled last block
    (1, 64, 300, 2, 1, 40),         # range runs past the end of the KV
    (1, 1560, 64 * 72, 4, 48, 24),  # a sliding window at the rollout's chunk size
    (1, 100, 512, 2, 9, 5),         # range wholly past the end: nothing visible
    (1, 100, 512, 2, 2, 0),         # empty range
], ids=lambda c: "b%d_m%d_n%d_h%d_f%d_n%d" % c)
def test_dense_range_against_oracle_and_listed_blocks(dev, case):
    ops = _ops()
    B, M, N, H, first, n = case
    g = torch.Generator().manual_seed(sum(case))
    q = torch.randn(B, M, H, 128, generator=g).bfloat16()
    k = torch.randn(B, N, H, 128, generator=g).bfloat16()
    v = torch.randn(B, N, H, 128, generator=g).bfloat16()
    scale = 128 ** -0.5
    kv = ops.DenseKV(k.to(dev), v.to(dev))
    out, lse = ops.range_fwd(q.to(dev), kv, first, n, 64, scale)
    ids = _listed(first, n, B, M, H)
    o_ref, l_ref = O.selection_fwd(q.float(), k.float(), v.float(), ids, 64, 1, scale, False, 64)
    _compare(out, lse, o_ref, l_ref, "range vs oracle")
    o_l, l_l = ops.sel_fwd(q.to(dev), kv, ids.to(dev), 64, 1, scale, False, 64)
    assert_close_bf16(out, o_l, "range vs listed blocks", max_abs=1.6e-2, mean_abs=1e-3)
    # same call twice: bit for bit
    out2, lse2 = ops.range_fwd(q.to(dev), kv, first, n, 64, scale)
    assert torch.equal(out, out2) and torch.equal(lse.nan_to_num(neginf=-1e30), lse2.nan_to_num(neginf=-1e30))


def test_paged_range_skips_blocks_without_a_page(dev):
    ops = _ops()
    H, NB, M = 3, 20, 300
    g = torch.Generator().manual_seed(7)
    n_tokens = NB * 64 - 23
    q = torch.randn(1, M, H, 128, generator=g).bfloat16()
    k = torch.randn(1, NB * 64, H, 128, generator=g).bfloat16()
    v = torch.randn(1, NB * 64, H, 128, generator=g).bfloat16()
    # every (head, block) on a page of its own, in a shuffled order; some blocks of the range have none
    pages = torch.randperm(H * NB, generator=g).view(H, NB).to(torch.int32)
    absent = [(0, 6), (1, 9), (1, 10), (2, 19)]
    table = pages.clone()
    for h, b in absent:
        table[h, b] = -1
    k_pool = torch.zeros(H * NB, 64, 128, dtype=torch.bfloat16)
    v_pool = torch.zeros_like(k_pool)
    for h in range(H):
        for b in range(NB):
            k_pool[pages[h, b]] = k[0, b * 64:(b + 1) * 64, h]
            v_pool[pages[h, b]] = v[0, b * 64:(b + 1) * 64, h]
    kv = ops.PagedKV(k_pool.to(dev), v_pool.to(dev), table.to(dev), n_tokens, 64)
    first, n = 4, 16
    scale = 128 ** -0.5
    out, lse = ops.range_fwd(q.to(dev), kv, first, n, 64, scale)
    # oracle: per head, the listed blocks without the absent ones
    ids = _listed(first, n, 1, M, H)
    for h, b in absent:
        ids[:, :, h][ids[:, :, h] == b] = -1
    o_ref, l_ref = O.selection_fwd(q.float(), k[:, :n_tokens].float(), v[:, :n_tokens].float(), ids, 64, 1, scale,
                                   False, 64)
    _compare(out, lse, o_ref, l_ref, "paged range vs oracle")


def test_out_view_and_fallback_shapes(dev):
    """`out` given as a strided view; shapes the range kernel is not built for take the listed route."""
    ops = _ops()
    g = torch.Generator().manual_seed(11)
    q = torch.randn(1, 192, 2, 128, generator=g).bfloat16()
    k = torch.randn(1, 640, 2, 128, generator=g).bfloat16()
    v = torch.randn(1, 640, 2, 128, generator=g).bfloat16()
    scale = 128 ** -0.5
    kv = ops.DenseKV(k.to(dev), v.to(dev))
    buf = torch.zeros(1, 192, 3, 2, 128, dtype=torch.bfloat16, device=dev)
    out, lse = ops.range_fwd(q.to(dev), kv, 2, 6, 64, scale, out=buf[:, :, 1])
    assert out.data_ptr() == buf[:, :, 1].data_ptr()
    ids = _listed(2, 6, 1, 192, 2)
    o_ref, l_ref = O.selection_fwd(q.float(), k.float(), v.float(), ids, 64, 1, scale, False, 64)
    _compare(buf[:, :, 1], lse, o_ref, l_ref, "strided out")
    assert float(buf[:, :, 0].abs().max()) == 0 and float(buf[:, :, 2].abs().max()) == 0
    # fp16 and 32-token blocks: not the range kernel's shapes
    o16, l16 = ops.range_fwd(q.half().to(dev), ops.DenseKV(k.half().to(dev), v.half().to(dev)), 2, 6, 64, scale)
    assert_close_bf16(o16, o_ref, "fp16 fallback")
    ids32 = _listed(3, 7, 1, 192, 2)
    o_ref32, _ = O.selection_fwd(q.float(), k.float(), v.float(), ids32, 32, 1, scale, False, 64)
    o32, _ = ops.range_fwd(q.to(dev), kv, 3, 7, 32, scale)
    assert_close_bf16(o32, o_ref32, "32-token blocks fallback")
    with pytest.raises(ops.NSABackendError):
        ops.range_fwd(q.to(dev), kv, -1, 3, 64, scale)


@pytest.mark.parametrize("splits", [2, 3, 5, 8])
def test_range_cut_into_spans_and_merged(dev, monkeypatch, splits):
    """The range cut into spans on thread blocks of their own and merged, against the oracle and the uncut
    run: more spans than blocks, a partly filled last block, two batches."""
    ops = _ops()
    scale = 128 ** -0.5
    for seed, (B, M, N, H, first, n) in enumerate([(1, 300, 64 * 40 - 17, 3, 2, 38), (2, 130, 700, 2, 1, 10),
                                                   (1, 100, 64 * 4, 2, 1, 3), (1, 100, 512, 2, 9, 5)]):
        g = torch.Generator().manual_seed(100 + seed)
        q = torch.randn(B, M, H, 128, generator=g).bfloat16()
        k = torch.randn(B, N, H, 128, generator=g).bfloat16()
        v = torch.randn(B, N, H, 128, generator=g).bfloat16()
        kv = ops.DenseKV(k.to(dev), v.to(dev))
        monkeypatch.setenv("OMNIMEM_B200_RANGE_SPLITS", "1")
        o1, l1 = ops.range_fwd(q.to(dev), kv, first, n, 64, scale)
        monkeypatch.setenv("OMNIMEM_B200_RANGE_SPLITS", str(splits))
        os_, ls_ = ops.range_fwd(q.to(dev), kv, first, n, 64, scale)
        monkeypatch.delenv("OMNIMEM_B200_RANGE_SPLITS")
        ids = _listed(first, n, B, M, H)
        o_ref, l_ref = O.selection_fwd(q.float(), k.float(), v.float(), ids, 64, 1, scale, False, 64)
        _compare(os_, ls_, o_ref, l_ref, f"{splits} spans vs oracle (case {seed})")
        assert_close_bf16(os_, o1, f"{splits} spans vs uncut (case {seed})", max_abs=1.6e-2, mean_abs=1e-3)


def test_c_entry_refuses_what_it_is_not_built_for(dev):
    """The C entry itself (no Python fallback in front of it): fp16 and 32-token blocks are refused with
    NSA_ERR_UNSUPPORTED and a message, a negative range with NSA_ERR_INVALID; nothing is launched."""
    import ctypes as C
    from omnimem_b200 import _lib
    ops = _ops()
    q = torch.randn(1, 128, 2, 128, device=dev).half()
    k = torch.randn(1, 256, 2, 128, device=dev).half()
    kv = ops.DenseKV(k, k.clone())
    out = torch.empty_like(q)
    lse = torch.empty(1, 2, 128, dtype=torch.float32, device=dev)
    src = kv.struct()
    stream = torch.cuda.current_stream().cuda_stream

    def call(qt, first, n, bs, dtype):
        return _lib.call("nsa_range_fwd", qt.data_ptr(), _lib.strides3(qt), C.byref(src), first, n, out.data_ptr(),
                         _lib.strides3(out), lse.data_ptr(), 1, 128, 2, 128, bs, 128 ** -0.5, None, 0, dtype, stream)

    with pytest.raises(_lib.NSABackendError, match="range_fwd: built for bf16"):
        call(q, 0, 4, 64, _lib.NSA_F16)
    with pytest.raises(_lib.NSABackendError, match="range_fwd: built for bf16"):
        call(q, 0, 4, 32, _lib.NSA_BF16)
    with pytest.raises(_lib.NSABackendError, match="first_block"):
        call(q, -1, 4, 64, _lib.NSA_BF16)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0


def test_full_size_window_properties(dev):
    """The rollout's window at full size (4680 queries x 12 heads over three chunks of pages): the range
    taken whole equals its two halves merged by their log-sum-exps; V -> 2 V doubles the output and leaves
    the log-sum-exp alone; a sample of rows against the oracle."""
    ops = _ops()
    M, H, D = 4680, 12, 128
    N = 3 * M
    nb = -(-N // 64)
    g = torch.Generator(device=dev).manual_seed(31)
    q = torch.randn(1, M, H, D, generator=g, device=dev).bfloat16()
    k = torch.randn(1, N, H, D, generator=g, device=dev).bfloat16()
    v = torch.randn(1, N, H, D, generator=g, device=dev).bfloat16()
    scale = D ** -0.5
    kv = ops.DenseKV(k, v)
    out, lse = ops.range_fwd(q, kv, 0, nb, 64, scale)
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    # halves merged
    cut = 97
    o1, l1 = ops.range_fwd(q, kv, 0, cut, 64, scale)
    o2, l2 = ops.range_fwd(q, kv, cut, nb - cut, 64, scale)
    om, lm = ops.merge_partials(torch.stack([o1, o2]), torch.stack([l1, l2]))
    assert_close_bf16(om, out, "halves merged vs whole", max_abs=4e-3, mean_abs=3e-4)
    assert torch.allclose(lm, lse, atol=1e-4, rtol=1e-5)
    # linear in V
    o_2v, l_2v = ops.range_fwd(q, ops.DenseKV(k, (v.float() * 2).bfloat16()), 0, nb, 64, scale)
    assert torch.equal(l_2v, lse)
    assert torch.equal(o_2v, (out.float() * 2).bfloat16())
    # a sample of rows (first tile, a middle one, the ragged last one) of three heads against the oracle
    rows = torch.cat([torch.arange(0, 64), torch.arange(2304, 2368), torch.arange(M - 72, M)])
    heads = [0, 5, 11]
    qs = q[:, rows][:, :, heads].cpu()
    ks, vs = k[:, :, heads].cpu(), v[:, :, heads].cpu()
    ids = _listed(0, nb, 1, rows.numel(), len(heads))
    o_ref, l_ref = O.selection_fwd(qs.float(), ks.float(), vs.float(), ids, 64, 1, scale, False, 64)
    _compare(out[:, rows][:, :, heads], lse[:, heads][:, :, rows], o_ref, l_ref, "full-size sample vs oracle")
