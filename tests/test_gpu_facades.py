"""The cache-resident selection facades with the reference's signatures
(nsa/ops/selection/padded_ptr: selection_attention_block_store, selection_attention_padded_ptr_fast)
against the dense forward on the same data, and their argument contracts."""
import pytest
import torch

from oracle import nsa_oracle as O
from tests.helpers import assert_close_bf16

pytestmark = pytest.mark.gpu


def test_block_store_facade(dev):
    from omnimem_b200 import ops
    from omnimem_b200.cache import BlockKVStore
    from omnimem_b200.nsa.ops import selection_attention_block_store
    g = torch.Generator().manual_seed(31)
    H, D, N, M, G, T = 3, 128, 900, 192, 64, 4
    store = BlockKVStore(num_layers=2, num_heads=H, head_dim=D, num_pages=H * 16, max_blocks=16, device=dev, host_tier=False)
    k = torch.randn(N, H, D, generator=g).to(torch.bfloat16)
    v = torch.randn(N, H, D, generator=g).to(torch.bfloat16)
    q = torch.randn(1, M, H, D, generator=g).to(torch.bfloat16)
    store.layer(1).append(k.to(dev), v.to(dev))
    ids = O.parallel_nsa_topk(q, store.layer(1).pooled_keys().cpu(), T, 64, None, 10 ** 6, False, G).to(dev)
    with torch.no_grad():
        out, lse = selection_attention_block_store(q.to(dev), ids, 64, G, store, 1, return_lse=True)
        only = selection_attention_block_store(q.to(dev), ids, 64, G, store, 1)
    dense, dl = ops.sel_fwd(q.to(dev), ops.DenseKV(k.unsqueeze(0).to(dev), v.unsqueeze(0).to(dev)), ids, 64, 1, D ** -0.5, False, G)
    assert torch.equal(out, dense) and torch.equal(lse, dl) and torch.equal(only, out)
    o_ref, _ = O.selection_fwd(q.float(), k.unsqueeze(0).float(), v.unsqueeze(0).float(), ids.cpu(), 64, 1, None, False, G)
    assert_close_bf16(out, o_ref, "block-store facade out")
    assert store.stats()["hits"] > 0 and store.stats()["misses"] == 0
    with pytest.raises(AssertionError, match="batch size 1"):
        selection_attention_block_store(q.to(dev).repeat(2, 1, 1, 1), ids, 64, G, store, 1)
    with pytest.raises(AssertionError, match="int32"):
        selection_attention_block_store(q.to(dev), ids.long(), 64, G, store, 1)
    with pytest.raises(AssertionError, match="store geometry"):
        selection_attention_block_store(q.to(dev), ids, 32, G, store, 1)
    with pytest.raises(RuntimeError, match="inference-only"):
        selection_attention_block_store(q.to(dev).requires_grad_(True), ids, 64, G, store, 1)


def test_padded_ptr_fast_facade(dev):
    from omnimem_b200.nsa.ops import selection_attention_padded_ptr_fast
    g = torch.Generator().manual_seed(32)
    H, D, bs, G, T, chunk_len, n_chunks = 2, 128, 64, 64, 3, 256, 3
    N, M = chunk_len * n_chunks, 128
    q = torch.randn(1, M, H, D, generator=g).to(torch.bfloat16)
    # chunk-per-head storage as MMCache keeps it: a [1, chunk_len, D] tensor per (head, chunk)
    kc = [[torch.randn(1, chunk_len, D, generator=g).to(torch.bfloat16).to(dev) for _ in range(n_chunks)] for _ in range(H)]
    vc = [[torch.randn(1, chunk_len, D, generator=g).to(torch.bfloat16).to(dev) for _ in range(n_chunks)] for _ in range(H)]
    k = torch.stack([torch.cat([c[0] for c in kc[h]]) for h in range(H)], 1).unsqueeze(0).cpu()     # [1, N, H, D]
    v = torch.stack([torch.cat([c[0] for c in vc[h]]) for h in range(H)], 1).unsqueeze(0).cpu()
    base_k = torch.tensor([[c.data_ptr() for c in kc[h]] for h in range(H)], dtype=torch.int64, device=dev)
    base_v = torch.tensor([[c.data_ptr() for c in vc[h]] for h in range(H)], dtype=torch.int64, device=dev)
    base_k[1, 2] = 0                                    # a chunk that is not on the device: its blocks are skipped
    base_v[1, 2] = 0
    n_per_head = torch.full((H,), n_chunks, dtype=torch.int32, device=dev)
    strides = dict(batch_stride_bytes=0, token_stride_bytes=D * 2, stride_bn=D, stride_bd=1, chunk_len=chunk_len)
    ids = O.parallel_nsa_topk(q, O.pool_rows(k, bs), T, bs, None, 10 ** 6, False, G).to(torch.int32)
    out, lse = selection_attention_padded_ptr_fast(q.to(dev), ids.to(dev), bs, G, chunk_len, base_k, base_v, n_per_head,
                                                   strides, return_lse=True)
    visible = ids.clone()
    visible[:, :, 1][visible[:, :, 1] >= 2 * (chunk_len // bs)] = -1      # head 1 lost its last chunk
    o_ref, l_ref = O.selection_fwd(q.float(), k.float(), v.float(), visible, bs, 1, None, False, G)
    assert_close_bf16(out, o_ref, "pointer-table facade out")
    fin = torch.isfinite(l_ref)
    assert torch.allclose(lse.cpu()[fin], l_ref[fin], atol=2e-3)
    with pytest.raises(AssertionError, match="multiple of block_size"):
        selection_attention_padded_ptr_fast(q.to(dev), ids.to(dev), bs, G, 100, base_k, base_v, n_per_head, strides)
    with pytest.raises(AssertionError, match="int64"):
        selection_attention_padded_ptr_fast(q.to(dev), ids.to(dev), bs, G, chunk_len, base_k.int(), base_v, n_per_head, strides)
