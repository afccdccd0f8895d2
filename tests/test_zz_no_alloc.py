"""The top-k entry point for callers that cannot allocate device memory
(nsa_topk_static_scratch): called straight through the C ABI, twice in a row, and compared with
the ordinary entry point (nsa_topk, caller-provided workspace) on the same inputs.

Collected last on purpose: if it fails, a run that stops at the first failure has already run
every other test.  It passes on its own in a fresh process as well as after the other tests,
because the entry point looks up its built-in buffer the first time it is used on a device."""
import ctypes as C

import pytest
import torch

from omnimem_b200 import _lib
from omnimem_b200._lib import NSABackendError, TopkMask, call, strides3

pytestmark = pytest.mark.gpu


def _mask(block_size, chunk, causal, q_off, G):
    return TopkMask(block_size, chunk, chunk, G, q_off, 0, 0, int(causal), 0, 0, 0, 1)


def _both(dev, q, k, topk, scale, m):
    """Run the ordinary and the no-allocation entry point on the same device tensors."""
    B, MG, H, D = q.shape
    NC = k.shape[1]
    stream = torch.cuda.current_stream(dev).cuda_stream
    lib = _lib.load()
    ws_bytes = lib.nsa_topk_workspace_bytes(B, MG, H, NC)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
    idx_a = torch.empty(B, MG, H, topk, dtype=torch.int32, device=dev)
    sc_a = torch.empty(B, MG, H, topk, dtype=torch.float32, device=dev)
    call("nsa_topk", q.data_ptr(), strides3(q), k.data_ptr(), strides3(k), B, MG, H, D, NC, topk, scale,
         C.byref(m), idx_a.data_ptr(), sc_a.data_ptr(), ws.data_ptr(), ws_bytes, _lib.NSA_BF16, stream)
    # outputs are allocated by the caller (here: the test); the call itself allocates nothing
    idx_b = torch.full((B, MG, H, topk), -7, dtype=torch.int32, device=dev)
    sc_b = torch.full((B, MG, H, topk), 7.0, dtype=torch.float32, device=dev)
    call("nsa_topk_static_scratch", q.data_ptr(), strides3(q), k.data_ptr(), strides3(k), B, MG, H, D, NC, topk,
         scale, C.byref(m), idx_b.data_ptr(), sc_b.data_ptr(), _lib.NSA_BF16, stream)
    torch.cuda.synchronize()
    return idx_a, sc_a, idx_b, sc_b


def test_static_scratch_topk_matches_the_workspace_entry_point_twice(dev):
    g = torch.Generator().manual_seed(123)
    # first call: the benchmark's geometry (74 pooled query rows, 12 heads, 512 key blocks, top-16)
    q1 = torch.randn(1, 74, 12, 128, generator=g).to(torch.bfloat16).to(dev)
    k1 = torch.randn(1, 512, 12, 128, generator=g).to(torch.bfloat16).to(dev)
    ia, sa, ib, sb = _both(dev, q1, k1, 16, 128 ** -0.5, _mask(64, 1560, True, 18, 64))
    assert torch.equal(ia, ib), "block ids differ between the two entry points (first call)"
    assert torch.equal(torch.isfinite(sa), torch.isfinite(sb))
    fin = torch.isfinite(sa)
    assert torch.allclose(sa[fin], sb[fin], atol=1e-6, rtol=1e-6)
    assert (ib >= 0).all()
    # second call straight after, smaller and with other data: what the first call left in the
    # built-in buffer must not leak into the result
    q2 = torch.randn(2, 9, 3, 64, generator=g).to(torch.bfloat16).to(dev)
    k2 = torch.randn(2, 40, 3, 64, generator=g).to(torch.bfloat16).to(dev)
    ia, sa, ib, sb = _both(dev, q2, k2, 48, 0.125, _mask(16, 64, False, 0, 16))
    assert torch.equal(ia, ib), "block ids differ between the two entry points (second call)"
    fin = torch.isfinite(sa)
    assert torch.equal(fin, torch.isfinite(sb))
    assert torch.allclose(sa[fin], sb[fin], atol=1e-6, rtol=1e-6)
    assert (ib[..., 40:] == -1).all()                     # only 40 blocks exist: the rest is padding


def test_static_scratch_topk_rejects_sizes_beyond_its_buffer(dev):
    lib = _lib.load()
    cap = lib.nsa_topk_static_scratch_max_scores()
    assert cap == 1 << 20
    q = torch.zeros(1, 74, 12, 128, dtype=torch.bfloat16, device=dev)
    k = torch.zeros(1, 16384, 12, 128, dtype=torch.bfloat16, device=dev)   # 74*12*16384 scores > 1 Mi
    idx = torch.full((1, 74, 12, 16), -7, dtype=torch.int32, device=dev)
    m = _mask(64, 1560, False, 0, 64)
    with pytest.raises(NSABackendError, match="exceed the built-in scratch"):
        call("nsa_topk_static_scratch", q.data_ptr(), strides3(q), k.data_ptr(), strides3(k), 1, 74, 12, 128, 16384,
             16, 0.1, C.byref(m), idx.data_ptr(), None, _lib.NSA_BF16, torch.cuda.current_stream(dev).cuda_stream)
    torch.cuda.synchronize()
    assert (idx == -7).all()                              # nothing was launched
