"""The rollout harness around the selection path: one NSA layer against the CPU oracle over several
chunks, and a small whole-model rollout whose result must not depend on the cache cap (evicting
blocks to the host tier and fetching them back changes nothing)."""
import pytest
import torch

from oracle import nsa_oracle as O
from tests.helpers import assert_close_bf16

pytestmark = pytest.mark.gpu


def _tiny(frames, cap=None, layers=2):
    from omnimem_b200 import rollout as R
    shape = R.WanShape(dim=256, ffn_dim=512, num_heads=2, num_layers=layers, text_dim=64, text_len=16)
    plan = R.RolloutPlan(latent_frames=frames, latent_h=8, latent_w=16, topk=2, window_chunks=2, exclude_window_chunks=2,
                         cache_cap_frames=cap, timesteps=(1000.0, 500.0))
    return R, shape, plan


def test_nsa_layer_matches_the_oracle_over_four_chunks(dev):
    """Three branches + gates of one layer on chunks 0..3 (96 tokens each: one and a half blocks, so
    chunks start and end inside pages) against the oracle's pooling, top-k, selection attention and
    plain softmax attention on the same projections."""
    R, shape, plan = _tiny(12)
    torch.manual_seed(3)
    layer = R.NSASelfAttention(shape, plan, 0).to(device=dev, dtype=torch.bfloat16).eval()
    torch.nn.init.normal_(layer.g_proj.weight, std=0.5)                 # gates away from 0.5
    cache = R.make_caches(shape, plan, dev)[0]
    hd = shape.dim // shape.num_heads
    freqs = torch.cat([R.rope_table(64, hd - 4 * (hd // 6)), R.rope_table(64, 2 * (hd // 6)), R.rope_table(64, 2 * (hd // 6))], 1)
    gh, gw, S, H = 4, 8, 96, shape.num_heads
    seen = {}
    layer.o.register_forward_pre_hook(lambda m, a: seen.__setitem__("y", a[0].detach()))
    orig = cache.touch
    cache.touch = lambda idx, **kw: (seen.__setitem__("idx", idx.detach().clone()), orig(idx, **kw))[1]
    K_hist, V_hist = [], []
    g = torch.Generator().manual_seed(4)
    with torch.no_grad():
        for chunk in range(4):
            x = torch.randn(1, S, shape.dim, generator=g).to(torch.bfloat16).to(dev)
            start_frame = 3 * chunk
            rope = R.RopeSpec(freqs, (gh, gw), start_frame, (1, 1, 1))
            for _ in range(2):                                          # the second pass rewrites the chunk in place
                layer(x, cache, rope, start_frame * gh * gw)
            q = layer.norm_q(layer.q(x)).view(S, H, hd).cpu()
            k = layer.norm_k(layer.k(x)).view(S, H, hd).cpu()
            v = layer.v(x).view(S, H, hd).cpu()
            gl = layer.g_proj(x).view(1, S, H, 3).cpu()
            qr = O.reorder_rope_apply(q, (3, gh, gw), freqs, start_frame, (1, 1, 1)).unsqueeze(0)
            K_hist.append(O.reorder_rope_apply(k, (3, gh, gw), freqs, start_frame, (1, 1, 1)))
            V_hist.append(v)
            K, V = torch.cat(K_hist).unsqueeze(0), torch.cat(V_hist).unsqueeze(0)
            N = K.shape[1]
            kp, vp = O.pool_rows(K, 64), O.pool_rows(V, 64)
            got_kp = cache.pooled_keys().cpu()                          # fp32 sums in another order: last-bit differences at most
            assert (got_kp == kp).float().mean() > 0.99
            assert ((got_kp.float() - kp.float()).abs() <= 2 ** -7 * kp.float().abs() + 1e-6).all()
            kp, vp = got_kp, cache.pooled_values().cpu()
            scale = hd ** -0.5

            def dense(qq, kk, vv):
                s = torch.einsum("bmhd,bnhd->bhmn", qq.float(), kk.float()) * scale
                return torch.einsum("bhmn,bnhd->bmhd", s.softmax(-1), vv.float())

            o_cmp = dense(qr, kp, vp)
            first_tok = max(0, chunk * S - S) // 64 * 64                # window of two chunks, from its first block on
            o_swa = dense(qr, K[:, first_tok:], V[:, first_tok:])
            idx = seen["idx"].cpu()
            want_idx = O.topk_select(O.pool_rows(qr, 64), kp, 2, scale, block_size=64, chunk_size=S, chunk_size_k=S,
                                     causal=False, ex_win=2, prog_excl=True, q_chunk_offset=chunk, q_group_size=64)
            assert (idx == want_idx).float().mean() >= 0.75             # a near-tie may swap a block
            o_slc, _ = O.selection_fwd(qr.float(), K.float(), V.float(), idx, 64, 1, None, False, 64)
            # the branches reach the gate as bf16, as the kernels deliver them
            y_ref = O.gate_combine(gl, o_cmp.to(torch.bfloat16), o_slc.to(torch.bfloat16), o_swa.to(torch.bfloat16))
            assert_close_bf16(seen["y"].view(1, S, H, hd), y_ref, f"chunk {chunk} gated sum of the three branches")
    cache.check_status()


def test_small_rollout_is_independent_of_the_cache_cap(dev):
    """Fifteen chunks through a two-block model: with every block resident, and with a pool so small
    that the history is evicted to the host tier and fetched back when selected.  Same latents, bit for bit."""
    R, shape, plan = _tiny(45)
    model, caches = R.build(shape, plan, dev, seed=5)
    full = R.rollout(model, caches, plan, dev, keep_latents=True)
    assert full.forwards == 15 * 3 and torch.isfinite(full.latents.float()).all()
    assert full.cache["pages_evicted"] == 0 and full.cache["misses"] == 0 and full.cache["hits"] > 0
    _, _, capped_plan = _tiny(45, cap=6)
    small = R.make_caches(shape, capped_plan, dev)
    assert small[0].num_pages < caches[0].num_pages and small[0].host_k is not None
    capped = R.rollout(model, small, capped_plan, dev, keep_latents=True)
    assert capped.cache["pages_evicted"] > 0 and capped.cache["pages_fetched"] > 0 and capped.cache["misses"] > 0
    assert capped.cache["bytes_from_host"] == capped.cache["pages_fetched"] * 2 * 64 * 128 * 2
    assert torch.equal(capped.latents, full.latents)
    # and a second run over the same (reset) caches reproduces the first
    again = R.rollout(model, small, capped_plan, dev, keep_latents=True)
    assert torch.equal(again.latents, full.latents)
