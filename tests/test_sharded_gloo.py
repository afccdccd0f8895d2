"""Block-sharded selection across ranks: the exchange / merge logic of
``omnimem_b200.sharded.ShardedSelection`` run as world_size-2 and -3 gloo process groups on the
CPU (compute through the oracle stand-in), against the single-device oracle on the whole KV."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import nsa_oracle as O


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, case, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from omnimem_b200.sharded import ShardedSelection, shard_kv
        from tests import oracle_ops
        M, N, H, D, T, bs, G, chunk, causal, q_off = case
        g = torch.Generator().manual_seed(77)
        # bf16 tensors: the partial outputs cross the ranks as packed 16-bit rows
        q = torch.randn(1, M, H, D, generator=g).to(torch.bfloat16)
        k = torch.randn(1, N, H, D, generator=g).to(torch.bfloat16)
        v = torch.randn(1, N, H, D, generator=g).to(torch.bfloat16)
        sh = ShardedSelection(ops=oracle_ops)
        out, lse, idx = sh.forward(q, shard_kv(k, bs, rank, world), shard_kv(v, bs, rank, world), T, bs, G, chunk,
                                   causal, q_chunk_offset=q_off)
        full_idx = O.parallel_nsa_topk(q, O.pool_rows(k, bs), T, bs, None, chunk, causal, G, q_chunk_offset=q_off)
        o_ref, l_ref = O.selection_fwd(q.float(), k.float(), v.float(), full_idx, bs, 1, None, False, G)
        # partials are rounded to bf16 before the merge (2^-9 relative each), the log-sum-exps stay fp32
        ok = (torch.equal(idx, full_idx) and out.shape == o_ref.shape and lse.shape == l_ref.shape
              and torch.allclose(out.float(), o_ref, atol=1.5e-2) and torch.allclose(lse, l_ref, atol=1e-4))
        gathered = [None] * world
        dist.all_gather_object(gathered, (bool(ok), idx.sum().item()))
        if rank == 0:
            ret.put(gathered)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("case", [
    (128, 1000, 2, 32, 6, 64, 64, 128, False, 0),      # ragged last block, no mask
    (200, 1560, 2, 32, 4, 64, 64, 520, True, 2),        # block-causal by chunk, ragged group, offset
])
def test_sharded_forward_matches_single_device(world, case):
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, case, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    results = ret.get(timeout=10)
    assert all(ok for ok, _ in results), results
    assert len({s for _, s in results}) == 1          # every rank holds the same global top-k
