"""Pointer-path backward (sel_bwd_ptr, selection_bwd.cu:1409-1527): K/V live in per-(head, chunk)
buffers found through address tables, dK/dV go to fp32 scratch found the same way.  Checked
against the dense backward over the same data."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _chunked_cache(H, n_chunks, bpc, bs, D, dev, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    rows = bpc * bs
    k = [[torch.randn(rows, D, generator=g).to(torch.bfloat16).to(dev) for _ in range(n_chunks)] for _ in range(H)]
    v = [[torch.randn(rows, D, generator=g).to(torch.bfloat16).to(dev) for _ in range(n_chunks)] for _ in range(H)]
    dk = [[torch.full((rows, D), 7.0, dtype=torch.float32, device=dev) for _ in range(n_chunks)] for _ in range(H)]
    dv = [[torch.full((rows, D), 7.0, dtype=torch.float32, device=dev) for _ in range(n_chunks)] for _ in range(H)]
    table = lambda bufs: torch.tensor([[t.data_ptr() for t in row] for row in bufs], dtype=torch.int64, device=dev)
    return k, v, dk, dv, table(k), table(v), table(dk), table(dv)


def _dense(bufs, H, n_chunks):
    # [1, N, H, D]
    return torch.stack([torch.cat(bufs[h], 0) for h in range(H)], 1).unsqueeze(0).contiguous()


@pytest.mark.parametrize("bs,G,D,chunked", [(64, 64, 128, True), (32, 16, 64, True), (64, 64, 128, False)])
def test_pointer_backward_matches_dense(bs, G, D, chunked):
    from omnimem_b200 import ops
    import omnimem_b200.torch_ops  # noqa: F401  (registers torch.ops.omnimem_nsa.*)
    dev = torch.device("cuda")
    torch.manual_seed(11)
    H, n_chunks, bpc, T, M = 3, 5, (4 if chunked else 1), (6 if chunked else 4), 4 * G
    NS = n_chunks * bpc
    k, v, dkb, dvb, base_k, base_v, base_dk, base_dv = _chunked_cache(H, n_chunks, bpc, bs, D, dev, 5)
    MG = M // G
    ids = torch.stack([torch.stack([torch.randperm(NS)[:T] for _ in range(H)]) for _ in range(MG)]).unsqueeze(0)
    ids = ids.to(torch.int32).to(dev)                       # [1, MG, H, T]
    ids[0, 1, 0, 2] = -1                                     # an empty slot
    nbph = torch.full((H,), NS, dtype=torch.int32, device=dev)
    nbph[2] = NS - 2                                         # head 2 has fewer valid blocks
    q = torch.randn(1, M, H, D, device=dev, dtype=torch.bfloat16)
    do = torch.randn(1, M, H, D, device=dev, dtype=torch.bfloat16)
    scale = D ** -0.5

    # dense reference over the same data; ids beyond a head's bound are masked out first
    ids_ref = torch.where(ids >= nbph.view(1, 1, H, 1), torch.full_like(ids, -1), ids)
    kd, vd = _dense(k, H, n_chunks), _dense(v, H, n_chunks)
    out, lse = ops.sel_fwd(q, ops.DenseKV(kd, vd), ids_ref, bs, 1 << 30, scale, False, G)
    dq_r, dk_r, dv_r = ops.sel_bwd(q, ops.DenseKV(kd, vd), ids_ref, out, lse, do, bs, 1 << 30, scale, False, G)

    in_chunk = bs * D * 2 if chunked else 0
    # (the per-slot tables are always built chunk-level; one block per chunk is the block-level case)
    ptr_k, ptr_v = ops.build_ptr_table(ids, base_k, base_v, nbph, 0, bpc, bs * D * 2)
    out_p, lse_p = torch.ops.omnimem_nsa.sel_fwd_ptr(q, ptr_k, ptr_v, bs, G, D, 1, scale, "tf32", [])
    assert torch.allclose(out_p.float(), out.float(), atol=2e-2)
    dq, delta = torch.ops.omnimem_nsa.sel_bwd_ptr(
        q, out_p, lse_p, do, ids, ptr_k, ptr_v, base_k, base_v, base_dk, base_dv, nbph, bs, G, 0, 0, D, 1, D, 1,
        bpc if chunked else 0, in_chunk, bs * D * 4 if chunked else 0, scale, "tf32", True, [], [])
    torch.cuda.synchronize()
    assert (dq.float() - dq_r.float()).abs().max().item() <= 4e-2
    assert torch.allclose(delta, (out.float() * do.float()).sum(-1).permute(0, 2, 1), atol=2e-2)
    dk_p = _dense(dkb, H, n_chunks)[0]                      # [N, H, D] fp32 scratch
    dv_p = _dense(dvb, H, n_chunks)[0]
    touched = torch.zeros(NS, H, dtype=torch.bool)
    for g_ in range(MG):
        for h in range(H):
            for t in range(T):
                b_ = int(ids_ref[0, g_, h, t])
                if b_ >= 0:
                    touched[b_, h] = True
    for blk in range(NS):
        for h in range(H):
            sl = slice(blk * bs, (blk + 1) * bs)
            if touched[blk, h]:
                assert (dk_p[sl, h] - dk_r[0, sl, h].float()).abs().max().item() <= 6e-2, (blk, h)
                assert (dv_p[sl, h] - dv_r[0, sl, h].float()).abs().max().item() <= 6e-2, (blk, h)
            else:
                assert (dk_p[sl, h] == 7.0).all() and (dv_p[sl, h] == 7.0).all(), (blk, h)   # scratch left alone


def test_zero_entry_skips_the_block_and_dq_only_mode():
    from omnimem_b200 import ops
    import omnimem_b200.torch_ops  # noqa: F401
    dev = torch.device("cuda")
    torch.manual_seed(3)
    H, n_chunks, bpc, bs, D, G, T = 2, 3, 2, 64, 128, 64, 3
    NS, M = n_chunks * bpc, 128
    k, v, dkb, dvb, base_k, base_v, base_dk, base_dv = _chunked_cache(H, n_chunks, bpc, bs, D, dev, 9)
    base_dk[1, 2] = 0                                        # chunk 2 of head 1 has no gradient scratch
    ids = torch.tensor([[[[0, 3, 5], [4, 1, 5]], [[2, 1, 0], [5, 4, 3]]]], dtype=torch.int32, device=dev)
    nbph = torch.empty(0, dtype=torch.int32, device=dev)
    q = torch.randn(1, M, H, D, device=dev, dtype=torch.bfloat16)
    do = torch.randn(1, M, H, D, device=dev, dtype=torch.bfloat16)
    scale = D ** -0.5
    ptr_k, ptr_v = ops.build_ptr_table(ids, base_k, base_v, torch.full((H,), NS, dtype=torch.int32, device=dev), 0, bpc,
                                       bs * D * 2)
    out, lse = torch.ops.omnimem_nsa.sel_fwd_ptr(q, ptr_k, ptr_v, bs, G, D, 1, scale, "ieee", [])
    args = (q, out, lse, do, ids, ptr_k, ptr_v, base_k, base_v, base_dk, base_dv, nbph, bs, G, 0, 0, D, 1, D, 1, bpc,
            bs * D * 2, bs * D * 4, scale, "ieee")
    dq0, _ = torch.ops.omnimem_nsa.sel_bwd_ptr(*args, False, [], [])
    torch.cuda.synchronize()
    assert all((t == 7.0).all() for row in dkb for t in row)             # dq-only: nothing written
    dq1, _ = torch.ops.omnimem_nsa.sel_bwd_ptr(*args, True, [], [])
    torch.cuda.synchronize()
    assert torch.equal(dq0, dq1)
    assert (dkb[1][2] == 7.0).all() and (dvb[1][2] == 7.0).all()          # all four bases or nothing
    assert not (dkb[0][2] == 7.0).all()
    with pytest.raises(RuntimeError):
        torch.ops.omnimem_nsa.sel_bwd_ptr(*args[:-1], "fp8", True, [], [])
