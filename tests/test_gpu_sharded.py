"""Block-sharded selection on real devices: world_size 1 in-process, and NCCL ranks (one child
process per GPU) when the box has at least two GPUs."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import nsa_oracle as O
from tests.helpers import assert_close_bf16

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _case(seed=5, M=200, N=64 * 40 + 20, H=3, D=128):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(1, M, H, D, generator=g).to(torch.bfloat16)
    k = torch.randn(1, N, H, D, generator=g).to(torch.bfloat16)
    v = torch.randn(1, N, H, D, generator=g).to(torch.bfloat16)
    return q, k, v


def _run_rank(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from omnimem_b200 import ops, _lib
        from omnimem_b200.sharded import ShardedSelection, shard_kv
        q, k, v = _case()
        sh = ShardedSelection()
        out, lse, idx = sh.forward(q.to(dev), shard_kv(k, 64, rank, world).to(dev), shard_kv(v, 64, rank, world).to(dev),
                                   8, 64, 64, 100, True, q_chunk_offset=30)
        full = ops.topk(ops.pool_rows(q.to(dev), 64), ops.pool_rows(k.to(dev), 64), 8, 128 ** -0.5, 64, 100, 100, True,
                        q_chunk_offset=30, q_group_size=64)
        o_ref, l_ref = O.selection_fwd(q.float(), k.float(), v.float(), full.cpu(), 64, 1, None, False, 64)
        ok = (bool(torch.equal(idx, full)) and (out.float().cpu() - o_ref).abs().max().item() < 2e-2
              and torch.allclose(lse.cpu(), l_ref, atol=2e-3) and _lib.device_status() == 0)
        flags = [None] * world
        dist.all_gather_object(flags, ok)
        if rank == 0:
            ret.put(flags)
    finally:
        dist.destroy_process_group()


def test_world_size_one(dev):
    port = _free_port()
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1)
    try:
        from omnimem_b200 import ops
        from omnimem_b200.sharded import ShardedSelection
        q, k, v = _case()
        out, lse, idx = ShardedSelection().forward(q.to(dev), k.to(dev), v.to(dev), 8, 64, 64, 100, True, q_chunk_offset=30)
        o_ref, l_ref = O.selection_fwd(q.float(), k.float(), v.float(), idx.cpu(), 64, 1, None, False, 64)
        assert_close_bf16(out, o_ref, "world 1 out")
    finally:
        dist.destroy_process_group()


def test_without_a_process_group(dev):
    """No torch.distributed initialised: one rank, no exchange (the N=1 point of the config-5 leg)."""
    from omnimem_b200 import ops
    from omnimem_b200.sharded import ShardedSelection
    q, k, v = _case(seed=6)
    sh = ShardedSelection()
    assert (sh.rank, sh.world) == (0, 1)
    out, lse, idx = sh.forward(q.to(dev), k.to(dev), v.to(dev), 8, 64, 64, 100, True, q_chunk_offset=30)
    want, _, _ = ops.select_blocks(q.to(dev), k.to(dev), 8, 128 ** -0.5, 64, 64, 100, 100, True, q_chunk_offset=30)
    assert torch.equal(idx, want)
    o_ref, l_ref = O.selection_fwd(q.float(), k.float(), v.float(), idx.cpu(), 64, 1, None, False, 64)
    assert_close_bf16(out, o_ref, "single rank out")


def test_packed_row_merge_equals_the_plain_merge(dev):
    """The merge over packed rows (a token's H x D outputs followed by its H log-sum-exps), which the
    row-split exchange uses, against nsa_merge_partials on the same partials: bit for bit."""
    from omnimem_b200 import ops
    g = torch.Generator().manual_seed(7)
    R, M, H, D = 5, 77, 3, 128
    outs = torch.randn(R, 1, M, H, D, generator=g).to(torch.bfloat16).to(dev)
    lses = torch.randn(R, 1, H, M, generator=g).to(dev)
    lses[1, :, :, ::3] = float("-inf")
    lses[:, :, 1, 5] = float("-inf")                     # a row no part has seen
    want_o, want_l = ops.merge_partials(outs, lses)
    row = ops.packed_row_elems(H, D)
    packed = torch.empty(R, M, row, dtype=torch.bfloat16, device=dev)
    packed[:, :, :H * D] = outs.view(R, M, H * D)
    packed[:, :, H * D:H * D + 2 * H].view(torch.float32).copy_(lses[:, 0].transpose(1, 2))
    merged = ops.merge_packed_rows(packed, H, D)
    assert torch.equal(merged[:, :H * D].view(1, M, H, D), want_o)
    assert torch.equal(merged[:, H * D:H * D + 2 * H].view(torch.float32).t().unsqueeze(0), want_l)


def test_nccl_ranks_match_single_device():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_run_rank, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    assert all(ret.get(timeout=10))


def test_local_block_ids(dev):
    """Global ids -> the ids rank r of R attends itself (block b lives on rank b % R as local block b // R)."""
    from omnimem_b200 import ops
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(-1, 500, (2, 9, 3, 16), generator=g, dtype=torch.int32)
    for R, r in ((1, 0), (2, 1), (5, 3), (8, 0)):
        got = ops.local_block_ids(ids.to(dev), R, r).cpu()
        want = torch.where((ids >= 0) & (ids % R == r), ids // R, torch.full_like(ids, -1))
        assert torch.equal(got, want)
