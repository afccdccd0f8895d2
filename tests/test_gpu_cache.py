"""Block KV cache kernels: append (mid-page starts, pooled-key refresh), selected-block
dedup + LRU touch, eviction to / fetch from the host tier, the reference's K1-K3 contracts."""
import pytest
import torch

from oracle import nsa_oracle as O
from tests.helpers import assert_close_bf16

pytestmark = pytest.mark.gpu


def _mk(dev, H=3, D=128, pages=64, max_blocks=32, pt=64, **kw):
    from omnimem_b200.cache import BlockKVCache
    return BlockKVCache(H, D, pages, max_blocks, pt, torch.bfloat16, dev, **kw)


def _dense_from_cache(cache):
    """Reassemble [n_tokens, H, D] K and V through the block table (resident blocks only)."""
    tab = cache.block_table.cpu()
    kp, vp = cache.k_pool.cpu(), cache.v_pool.cpu()
    K = torch.zeros(cache.n_blocks * cache.page_tokens, cache.H, cache.D, dtype=kp.dtype)
    V = torch.zeros_like(K)
    for h in range(cache.H):
        for b in range(cache.n_blocks):
            p = int(tab[h, b])
            if p >= 0:
                K[b * cache.page_tokens:(b + 1) * cache.page_tokens, h] = kp[p]
                V[b * cache.page_tokens:(b + 1) * cache.page_tokens, h] = vp[p]
    return K[: cache.n_tokens], V[: cache.n_tokens]


def test_append_mid_page_and_pooled_refresh(dev):
    g = torch.Generator().manual_seed(1)
    cache = _mk(dev, host_tier=False)
    H, D = cache.H, cache.D
    chunks = [100, 28, 1, 200, 64, 7]            # starts and ends inside pages
    ks, vs = [], []
    for S in chunks:
        k = torch.randn(S, H, D, generator=g).to(torch.bfloat16)
        v = torch.randn(S, H, D, generator=g).to(torch.bfloat16)
        cache.append(k.to(dev), v.to(dev))
        ks.append(k)
        vs.append(v)
        K, V = torch.cat(ks), torch.cat(vs)
        Kc, Vc = _dense_from_cache(cache)
        assert torch.equal(Kc, K) and torch.equal(Vc, V)
        want = O.pool_rows(K.unsqueeze(0), 64)                       # [1, nb, H, D]
        got = cache.pooled_keys().cpu()
        assert got.shape == want.shape
        assert ((got.float() - want.float()).abs() <= 2 ** -7 * want.float().abs() + 1e-6).all()
        assert (got == want).float().mean() > 0.97
        wantv = O.pool_rows(V.unsqueeze(0), 64)
        assert ((cache.pooled_values().cpu().float() - wantv.float()).abs() <= 2 ** -7 * wantv.float().abs() + 1e-6).all()
    cache.check_status()
    # overwrite the last chunk in place (what each denoising step does)
    k2 = torch.randn(7, H, D, generator=g).to(torch.bfloat16)
    cache.append(k2.to(dev), k2.to(dev), pos0=cache.n_tokens - 7)
    Kc, _ = _dense_from_cache(cache)
    assert torch.equal(Kc[-7:], k2) and torch.equal(Kc[:-7], torch.cat(ks)[:-7])


def test_paged_attention_equals_dense(dev):
    from omnimem_b200 import ops
    g = torch.Generator().manual_seed(2)
    H, D, N, M, G, T = 2, 128, 1000, 200, 64, 5
    cache = _mk(dev, H=H, pages=40, max_blocks=16, host_tier=False)
    k = torch.randn(N, H, D, generator=g).to(torch.bfloat16)
    v = torch.randn(N, H, D, generator=g).to(torch.bfloat16)
    q = torch.randn(1, M, H, D, generator=g).to(torch.bfloat16)
    for a in range(0, N, 300):
        cache.append(k[a:a + 300].to(dev), v[a:a + 300].to(dev))
    ids = O.parallel_nsa_topk(q, cache.pooled_keys().cpu(), T, 64, None, 10 ** 6, False, G)
    out, lse = cache.selection_attention(q.to(dev), ids.to(dev), group_size=G, return_lse=True)
    o_ref, l_ref = O.selection_fwd(q.float(), k.unsqueeze(0).float(), v.unsqueeze(0).float(), ids, 64, 1, None, False, G)
    assert_close_bf16(out, o_ref, "paged out")
    dense, _ = ops.sel_fwd(q.to(dev), ops.DenseKV(k.unsqueeze(0).to(dev), v.unsqueeze(0).to(dev)), ids.to(dev), 64, 1,
                           D ** -0.5, False, G)
    assert torch.equal(out, dense)                       # same kernel, same tiles: bit-identical


def test_pools_start_zero_filled(dev):
    """The kernels read whole pages; rows behind a block's last token must be finite (0 x NaN = NaN in
    P V and dS K), so the pools are zero-filled at allocation even when the allocator hands back
    memory that held non-finite bit patterns."""
    poison = torch.full((64, 64, 128), float("nan"), dtype=torch.bfloat16, device=dev)
    del poison                                            # back to the caching allocator, still NaN
    cache = _mk(dev, H=2, pages=64, max_blocks=16, host_tier=False)
    assert int(torch.count_nonzero(cache.k_pool)) == 0 and int(torch.count_nonzero(cache.v_pool)) == 0
    g = torch.Generator().manual_seed(31)
    k = torch.randn(100, 2, 128, generator=g).to(torch.bfloat16).to(dev)     # second block holds 36 of 64 tokens
    cache.append(k, k)
    assert bool(torch.isfinite(cache.k_pool.float()).all()) and bool(torch.isfinite(cache.v_pool.float()).all())


def test_paged_backward_equals_dense(dev):
    """dQ, dK, dV with K/V read from the page pool through the block table: the same kernels and
    the same tiles as with dense tensors, so the gradients are bit-identical (B = 1, the pool
    has no batch dimension); causal as well, with a ragged last block."""
    from omnimem_b200 import ops
    g = torch.Generator().manual_seed(12)
    H, D, N, M, G, T = 3, 128, 1000, 200, 64, 5
    cache = _mk(dev, H=H, pages=64, max_blocks=16, host_tier=False)     # 3 heads x 16 blocks all resident
    k = torch.randn(N, H, D, generator=g).to(torch.bfloat16)
    v = torch.randn(N, H, D, generator=g).to(torch.bfloat16)
    q = torch.randn(1, M, H, D, generator=g).to(torch.bfloat16).to(dev)
    do = torch.randn(1, M, H, D, generator=g).to(torch.bfloat16).to(dev)
    for a in range(0, N, 250):
        cache.append(k[a:a + 250].to(dev), v[a:a + 250].to(dev))
    dense = ops.DenseKV(k.unsqueeze(0).to(dev), v.unsqueeze(0).to(dev))
    for chunk, causal in ((1, False), (100, True)):
        ids = O.parallel_nsa_topk(q.cpu(), cache.pooled_keys().cpu(), T, 64, None, chunk if causal else 10 ** 6, causal, G).to(dev)
        scale = D ** -0.5
        out, lse = ops.sel_fwd(q, cache.kv_source(), ids, 64, chunk, scale, causal, G)
        got = ops.sel_bwd(q, cache.kv_source(), ids, out, lse, do, 64, chunk, scale, causal, G)
        want = ops.sel_bwd(q, dense, ids, out, lse, do, 64, chunk, scale, causal, G)
        for name, a, b in zip(("dq", "dk", "dv"), got, want):
            assert torch.equal(a, b), f"paged {name} differs from dense (causal={causal})"
        # and against the oracle
        o_ref, l_ref = O.selection_fwd(q.cpu().float(), k.unsqueeze(0).float(), v.unsqueeze(0).float(), ids.cpu(), 64,
                                       chunk, None, causal, G)
        dq_r, dk_r, dv_r = O.selection_bwd(q.cpu().float(), k.unsqueeze(0).float(), v.unsqueeze(0).float(), ids.cpu(),
                                           o_ref, l_ref, do.cpu().float(), 64, chunk, None, causal, G)
        assert_close_bf16(got[0], dq_r, "paged dq")
        assert_close_bf16(got[1], dk_r, "paged dk")
        assert_close_bf16(got[2], dv_r, "paged dv")


def test_dedup_touch_lists(dev):
    g = torch.Generator().manual_seed(3)
    cache = _mk(dev, H=3, pages=30, max_blocks=10, host_tier=False)
    k = torch.randn(640, 3, 128, generator=g).to(torch.bfloat16).to(dev)
    cache.append(k, k)
    ids = torch.randint(-1, 12, (1, 5, 3, 4), generator=g, dtype=torch.int32)
    uniq, miss = cache.touch(ids.to(dev), return_lists=True)
    want = O.dedup_keys(ids, 3, 10)
    n = int(uniq[0])
    assert n == want.numel() and uniq[1:1 + n].cpu().tolist() == want.tolist()
    assert int(miss[0]) == 0
    # touched pages carry the new epoch
    tab = cache.block_table.cpu().view(-1)
    st = cache.page_stamp.cpu()
    for key in want.tolist():
        assert st[tab[key]] == cache.epoch


def test_reference_block_kv_contracts(dev):
    """Smoke vectors of the reference's own warm-up (nsa/cuda_backend/block_kv_ops.py:90-111)."""
    from omnimem_b200 import ops
    for wide in (True, False):
        src = torch.arange(32, dtype=torch.int16, device=dev).view(2, 16) + 1
        dst = torch.zeros(2, 16, dtype=torch.int16, device=dev)
        table = torch.full((4,), -1, dtype=torch.int64, device=dev)
        a = table.data_ptr()
        desc = torch.tensor([src[0].data_ptr(), src[1].data_ptr(), dst[0].data_ptr(), dst[1].data_ptr(),
                             a, a + 8, a + 16, a + 24], dtype=torch.int64, device=dev)
        assert ops.gather_publish_clear(desc, 1, 2, 32, wide, 1) == 2
        assert torch.equal(dst, src)
        assert table.tolist() == [dst[0].data_ptr(), dst[1].data_ptr(), 0, 0]
    assert ops.gather_publish_clear(desc, 0, 0, 32, True, 1) == 0
    tab = torch.zeros(2, 1, 4, dtype=torch.int64, device=dev)
    nv = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.block_range(tab, nv, 0, 4, 4096, 8192, 64, 16, 4, True, True, False)
    assert tab[0, 0].tolist() == [4096 + 16 * j for j in range(4)]
    assert tab[1, 0].tolist() == [8192 + 16 * j for j in range(4)]
    assert nv.item() == 4
    ops.block_range(tab, nv, 1, 2, 0, 0, 0, 0, -1, True, False, True)
    assert tab[0, 0].tolist() == [4096, 0, 0, 4096 + 48] and tab[1, 0, 1].item() == 8192 + 16 and nv.item() == 4
    ids = torch.tensor([0, -1, 3, 3], dtype=torch.int32, device=dev)
    stamp = torch.full((4,), -1, dtype=torch.int32, device=dev)
    out = torch.zeros(1 + 4, dtype=torch.int32, device=dev)
    ops.dedup_run(ids, stamp, out, 1, 4, 1, 4, 4, 4)
    assert out[:3].tolist() == [2, 0, 3]
    # chunked key order (cid*H + h)*bpc + loc with 2 heads, 2 blocks per chunk
    ids = torch.tensor([[3, 0], [2, 3]], dtype=torch.int32, device=dev).view(-1)     # [MG=1,H=2,T=2]
    stamp = torch.zeros(8, dtype=torch.int32, device=dev)
    out = torch.zeros(1 + 8, dtype=torch.int32, device=dev)
    ops.dedup_run(ids, stamp, out, 5, 4, 2, 2, 2, 8)
    # head0: bids 3,0 -> keys (1*2+0)*2+1=5, 0 ; head1: bids 2,3 -> (1*2+1)*2+0=6, 7
    assert out[:5].tolist() == [4, 0, 5, 6, 7]


def test_lru_eviction_and_fetch_follow_the_policy_model(dev):
    g = torch.Generator().manual_seed(4)
    H, D, PT, MB, P = 2, 128, 64, 24, 16                 # 16 pages for up to 48 (head, block) pairs
    cache = _mk(dev, H=H, D=D, pages=P, max_blocks=MB, pt=PT, host_tier=True, protect_blocks=2)
    model = O.EpochLRUPagePool(H, P, MB, PT, protect_blocks=2)
    K = torch.randn(MB * PT, H, D, generator=g).to(torch.bfloat16)
    V = torch.randn(MB * PT, H, D, generator=g).to(torch.bfloat16)
    q = torch.randn(1, 64, H, D, generator=g).to(torch.bfloat16)
    pos = 0
    for step in range(8):
        S = [150, 64, 100, 200, 30, 128, 90, 70][step]
        cache.append(K[pos:pos + S].to(dev), V[pos:pos + S].to(dev))
        model.append(S)
        pos += S
        nb = cache.n_blocks
        ids = torch.stack([torch.randperm(nb, generator=g)[:3] for _ in range(H)]).to(torch.int32).view(1, 1, H, 3)
        uniq, miss = cache.touch(ids.to(dev), return_lists=True)
        mu, mm = model.touch(ids)
        assert uniq[1:1 + int(uniq[0])].cpu().tolist() == mu
        assert miss[1:1 + int(miss[0])].cpu().tolist() == mm
        tab = cache.block_table.cpu().view(-1)
        for key in range(H * MB):
            assert int(tab[key]) == model.table.get(key, -1), f"step {step} key {key}"
        assert cache.page_owner.cpu().tolist() == model.owner
        # every selected block is resident now and holds the right data (fetched from the host tier)
        out, lse = ops_sel(cache, q.to(dev), ids.to(dev))
        o_ref, l_ref = O.selection_fwd(q.float(), K[:pos].unsqueeze(0).float(), V[:pos].unsqueeze(0).float(), ids,
                                       PT, 1, None, False, 64)
        assert_close_bf16(out, o_ref, f"step {step} out after fetch")
    cache.check_status()
    assert model.evicted_any and len(model.host) > 0


def test_block_cache_replays_the_reference_lru_trace(dev, golden):
    """The device cache against the reference itself: the trace of MMCache.lru_touch_per_head
    (models/cache.py:673-699; tests/golden/lru.npz) replayed through BlockKVCache.touch, one
    (head, block) id per call, one pool of `cap` pages per head, every block starting in the host
    tier.  The block each touch evicts, the final LRU order, the hit count and the data that comes
    back from the host tier must be the reference's."""
    d = golden("lru")
    heads, cap, n_ids, n_touch = d["meta"].tolist()
    g = torch.Generator().manual_seed(8)
    caches, data = [], []
    for _ in range(heads):
        c = _mk(dev, H=1, D=128, pages=cap, max_blocks=n_ids, pt=64, host_tier=True)
        K = torch.randn(n_ids * 64, 1, 128, generator=g).to(torch.bfloat16)
        for b in range(n_ids):
            c.append(K[b * 64:(b + 1) * 64].to(dev), K[b * 64:(b + 1) * 64].to(dev))
        c.evict_all()
        c.counters.zero_()
        assert int((c.block_table >= 0).sum()) == 0
        caches.append(c)
        data.append(K)
    for (h, cid), ev in zip(d["trace"].tolist(), d["evicted"].tolist()):
        c = caches[h]
        before = set(torch.nonzero(c.block_table[0] >= 0).view(-1).tolist())
        c.touch(torch.tensor([[[[cid]]]], dtype=torch.int32, device=dev))
        after = set(torch.nonzero(c.block_table[0] >= 0).view(-1).tolist())
        gone = sorted(before - after)
        assert gone == ([ev] if ev >= 0 else []), f"touch ({h}, {cid}) evicted {gone}, the reference evicted {ev}"
        assert cid in after
    hits = 0
    for h, c in enumerate(caches):
        c.check_status()
        order = [x for x in d["final_order"][h].tolist() if x >= 0]
        tab, st = c.block_table[0].cpu(), c.page_stamp.cpu()
        resident = sorted((b for b in range(n_ids) if tab[b] >= 0), key=lambda b: int(st[tab[b]]))
        assert resident == order
        for b in resident:                       # the pages hold what was appended, back from the host
            assert torch.equal(c.k_pool[int(tab[b])].cpu(), data[h][b * 64:(b + 1) * 64, 0])
        s = c.stats()
        hits += s["hits"]
        assert s["pages_fetched"] == s["misses"] and s["bytes_from_host"] == s["misses"] * 2 * 64 * 128 * 2
    assert hits == int(d["hits"][0])


def _block_of(cache, K, h, b):
    """K rows of block b of head h as the cache holds them (the block must be resident)."""
    page = int(cache.block_table[h, b])
    assert page >= 0
    return cache.k_pool[page].cpu()


def test_rewrite_of_an_evicted_partly_filled_block_keeps_its_rows(dev):
    """A tiny pool: the tail block is evicted by a selection, then an append rewrites part of it.
    The block comes back from the host tier first, keeps the rows the append does not cover, is
    not chosen as a victim for the call's own pages, and its pooled key covers every row it holds."""
    g = torch.Generator().manual_seed(21)
    H, D, PT, MB, P = 2, 128, 64, 16, 8
    cache = _mk(dev, H=H, D=D, pages=P, max_blocks=MB, pt=PT, host_tier=True)
    model = O.EpochLRUPagePool(H, P, MB, PT)
    K = torch.randn(MB * PT, H, D, generator=g).to(torch.bfloat16)

    def same_state():
        tab = cache.block_table.cpu().view(-1)
        for key in range(H * MB):
            assert int(tab[key]) == model.table.get(key, -1), f"key {key}"
        assert cache.page_owner.cpu().tolist() == model.owner

    def ids_of(blocks):
        return torch.tensor(blocks, dtype=torch.int32).view(1, 1, 1, -1).expand(1, 1, H, -1).contiguous()

    cache.append(K[:256].to(dev), K[:256].to(dev)); model.append(256)            # blocks 0-3: pool full
    cache.append(K[256:356].to(dev), K[256:356].to(dev)); model.append(100)      # blocks 4, 5 (36 rows): evicts 0, 1
    same_state()
    for blocks in ([0, 2], [0, 1, 3]):                                           # the second one evicts blocks 4 and 5
        cache.touch(ids_of(blocks).to(dev)); model.touch(ids_of(blocks))
        same_state()
    assert int(cache.block_table[0, 5]) < 0 and int(cache.block_table[1, 5]) < 0
    # rewrite tokens 330..379: rows 10..59 of block 5, whose rows 0..9 live in the host tier
    new = torch.randn(50, H, D, generator=g).to(torch.bfloat16)
    cache.append(new.to(dev), new.to(dev), pos0=330); model.append(50, 330)
    same_state()
    cache.check_status()
    want = torch.cat([K[320:330], new])                                          # 60 rows of block 5
    for h in range(H):
        got = _block_of(cache, K, h, 5)
        assert torch.equal(got[:60], want[:, h]), "rows of the rewritten block"
    pooled = O.pool_rows(want.unsqueeze(0), 64)[0, 0]                            # [H, D] mean of the 60 rows
    got = cache.k_pooled[:, 5].cpu()
    assert ((got.float() - pooled.float()).abs() <= 2 ** -7 * pooled.float().abs() + 1e-6).all()
    # a rewrite that ends inside the block leaves the pooled key over all 60 rows
    new2 = torch.randn(5, H, D, generator=g).to(torch.bfloat16)
    cache.append(new2.to(dev), new2.to(dev), pos0=325); model.append(5, 325)
    want[5:10] = new2
    pooled = O.pool_rows(want.unsqueeze(0), 64)[0, 0]
    got = cache.k_pooled[:, 5].cpu()
    assert ((got.float() - pooled.float()).abs() <= 2 ** -7 * pooled.float().abs() + 1e-6).all()
    # every other block still holds its data: bring them back one at a time
    for b in range(5):
        cache.touch(ids_of([b]).to(dev)); model.touch(ids_of([b]))
        for h in range(H):
            assert torch.equal(_block_of(cache, K, h, b), K[b * PT:(b + 1) * PT, h]), f"block {b}"
    same_state()
    cache.check_status()
    s = cache.stats()
    assert (s["hits"], s["misses"], s["pages_evicted"], s["pages_fetched"]) == (
        model.hits, model.misses, model.pages_evicted, model.pages_fetched)


def ops_sel(cache, q, ids):
    from omnimem_b200 import ops
    return ops.sel_fwd(q, cache.kv_source(), ids, cache.page_tokens, 1, q.shape[-1] ** -0.5, False, 64)


@pytest.mark.parametrize("pages,n", [(14040, 888), (28248, 3000), (300, 300), (5000, 1), (70, 90)])
def test_victim_selection_by_radix_select_equals_the_rescanning_kernel(dev, monkeypatch, pages, n):
    """Free pages first, then least recently used, ascending (stamp, page): the radix-select kernel
    (n-th smallest key, gather, sort of the n keys in shared memory) against the kernel that rescans
    the pool per victim, and against a host sort of the same keys."""
    import ctypes as C
    from omnimem_b200 import _lib
    g = torch.Generator().manual_seed(pages + n)
    MB = 1200
    owner = torch.randint(0, 12 * MB, (pages,), generator=g, dtype=torch.int32)
    owner[torch.rand(pages, generator=g) < 0.1] = -1                       # some free pages
    stamp = torch.randint(0, 40, (pages,), generator=g, dtype=torch.int64)
    protect_from, epoch = 1100, 37
    cap = max(n, 1)
    owner_d, stamp_d = owner.to(dev), stamp.to(dev)

    def run():
        victims = torch.full((cap,), -7, dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        _lib.call("nsa_cache_select_victims", owner_d.data_ptr(), stamp_d.data_ptr(), pages, MB, protect_from,
                  epoch, n, None, cap, victims.data_ptr(), status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        return victims.cpu().tolist(), int(status.item())

    fast = run()
    monkeypatch.setenv("OMNIMEM_B200_VICTIMS_KERNEL", "scan")
    slow = run()
    monkeypatch.delenv("OMNIMEM_B200_VICTIMS_KERNEL")
    keys = []
    for pg in range(pages):
        o, st = int(owner[pg]), int(stamp[pg])
        if o < 0:
            keys.append((0, pg))
        elif o % MB < protect_from and st < epoch:
            keys.append((st + 1, pg))
    keys.sort()
    want = [pg for _, pg in keys[:n]] + [-1] * max(0, n - len(keys))
    assert fast[0] == want and slow[0] == want
    assert fast[1] == slow[1] == (_lib.NSA_ERR_EXHAUSTED if len(keys) < n else 0)


def test_pool_exhaustion_sets_status(dev):
    from omnimem_b200 import NSABackendError
    cache = _mk(dev, H=2, pages=4, max_blocks=8, host_tier=False, protect_blocks=8)   # everything protected
    k = torch.randn(128, 2, 128).to(torch.bfloat16).to(dev)
    cache.append(k, k)                      # 2 blocks x 2 heads = 4 pages: full
    cache.check_status()
    cache.append(k[:64], k[:64])            # needs 2 more pages, nothing may be evicted
    with pytest.raises(NSABackendError, match="exhausted"):
        cache.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("pool", [(1, 1, 1), (2, 2, 2)])
def test_append_with_rotary_embedding_matches_rope_then_append(dev, pool):
    """Keys given without RoPE and embedded on the way into the pages == keys embedded by the
    reference's function (oracle restatement, pinned to it by a golden vector) and appended plainly."""
    from omnimem_b200.cache import RopeSpec
    H, D = 3, 128
    f, h, w = 4, 4, 6                                   # 96 tokens per group of two frames
    freqs = torch.cat([O.rope_params(1024, D - 4 * (D // 6)), O.rope_params(1024, 2 * (D // 6)),
                       O.rope_params(1024, 2 * (D // 6))], dim=1)
    g = torch.Generator().manual_seed(4)
    plain = _mk(dev, H=H, D=D, pages=64, max_blocks=16, host_tier=False)
    fused = _mk(dev, H=H, D=D, pages=64, max_blocks=16, host_tier=False)
    # a first chunk of 32 tokens without RoPE so that the embedded chunks start inside a page
    k0 = torch.randn(32, H, D, generator=g).to(torch.bfloat16)
    plain.append(k0.to(dev), k0.to(dev))
    fused.append(k0.to(dev), k0.to(dev))
    start = 0
    for _ in range(2):
        S = f * h * w
        k = torch.randn(S, H, D, generator=g).to(torch.bfloat16)
        v = torch.randn(S, H, D, generator=g).to(torch.bfloat16)
        k_roped = O.reorder_rope_apply(k, (f, h, w), freqs, start, pool)
        # the query-side kernel applies the same embedding to a tensor of its own
        from omnimem_b200.cache import rope_apply
        assert torch.equal(rope_apply(k.to(dev), RopeSpec(freqs, (h, w), start, pool)).cpu(), k_roped)
        plain.append(k_roped.to(dev), v.to(dev))
        fused.append(k.to(dev), v.to(dev), rope=RopeSpec(freqs, (h, w), start, pool))
        start += f
    Kp, Vp = _dense_from_cache(plain)
    Kf, Vf = _dense_from_cache(fused)
    assert torch.equal(Kp, Kf) and torch.equal(Vp, Vf)
    assert torch.equal(plain.pooled_keys(), fused.pooled_keys())
    fused.check_status()
    with pytest.raises(Exception):
        fused.append(k[:50].to(dev), v[:50].to(dev), rope=RopeSpec(freqs, (h, w), start, pool))   # not whole frames


@pytest.mark.parametrize("case", [(90, 5, 64, (5, 6), (1, 1, 1)),      # S not a multiple of the kernel's token group, D = 64
                                  (96, 3, 128, (4, 6), (2, 2, 2)),     # pooled-window token order
                                  (30, 130, 64, (5, 6), (1, 1, 1))],   # more row pieces than a thread block holds
                         ids=["ragged_d64", "pooled_order", "wide"])
def test_query_rotary_embedding_shapes(dev, case):
    """rope_apply bit for bit against the oracle's restatement of the reference function, from a strided view."""
    from omnimem_b200.cache import RopeSpec, rope_apply
    S, H, D, (gh, gw), pool = case
    freqs = torch.cat([O.rope_params(1024, D - 4 * (D // 6)), O.rope_params(1024, 2 * (D // 6)),
                       O.rope_params(1024, 2 * (D // 6))], dim=1)
    g = torch.Generator().manual_seed(S + H)
    wide = torch.randn(S, H, 2 * D, generator=g).to(torch.bfloat16)
    x = wide[:, :, D:]                                                  # row stride 2 D, 16-byte aligned
    f = S // (gh * gw)
    ref = O.reorder_rope_apply(x.contiguous(), (f, gh, gw), freqs, 7, pool)
    got = rope_apply(wide.to(dev)[:, :, D:], RopeSpec(freqs, (gh, gw), 7, pool))
    assert torch.equal(got.cpu(), ref)


def test_rotary_embedding_is_bit_exact_on_a_full_chunk(dev):
    """The rotary embedding must round exactly as the reference's float64 product does: a full chunk of
    random rows (7.2 M elements, a few hundred of which land next to a bf16 rounding boundary, where
    float32 arithmetic would round the other way), rows built to cancel (xr = xi against angles near 45
    degrees, xr = -xi), zeros of both signs, tiny and huge magnitudes, through both kernels."""
    from omnimem_b200.cache import RopeSpec, rope_apply
    H, D, gh, gw, f = 12, 128, 30, 52, 3
    S = f * gh * gw
    freqs = torch.cat([O.rope_params(1024, D - 4 * (D // 6)), O.rope_params(1024, 2 * (D // 6)),
                       O.rope_params(1024, 2 * (D // 6))], dim=1)
    g = torch.Generator().manual_seed(2024)
    x = torch.randn(S, H, D, generator=g)
    # every eighth row: equal / opposite real and imaginary parts, so that real or imaginary results cancel
    x[::8, :, 1::2] = x[::8, :, 0::2]
    x[4::8, :, 1::2] = -x[4::8, :, 0::2]
    x[1::64] *= 2.0 ** -60
    x[2::64] *= 2.0 ** 60
    x[3::64] = 0.0
    x[5::64, :, ::2] = -0.0
    x = x.to(torch.bfloat16)
    for start in (0, 9, 333):
        ref = O.reorder_rope_apply(x, (f, gh, gw), freqs, start, (1, 1, 1))
        got = rope_apply(x.to(dev), RopeSpec(freqs, (gh, gw), start, (1, 1, 1))).cpu()
        same = got.view(torch.int16) == ref.view(torch.int16)
        assert bool(same.all()), f"start {start}: {int((~same).sum())} of {same.numel()} elements differ"
    # the append kernel's copy of the rotation
    cache = _mk(dev, H=H, D=D, pages=H * 80, max_blocks=80, host_tier=False)
    cache.append(x.to(dev), x.to(dev), rope=RopeSpec(freqs, (gh, gw), 9, (1, 1, 1)))
    K, _ = _dense_from_cache(cache)
    ref = O.reorder_rope_apply(x, (f, gh, gw), freqs, 9, (1, 1, 1))
    assert torch.equal(K[:S].view(torch.int16), ref.view(torch.int16))
