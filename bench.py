"""Benchmark of the NSA selection hot path (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N = 1 and per rank for N > 1): op-level bf16 selection forward + backward at the
Wan2.1-1.3B layer shape - B=1, H=12, D=128, Q = a 3-latent-frame chunk (4680 tokens, frames
18..20), KV = 21 latent frames (32760 tokens) in 64-token blocks, top-16 per 64-query group,
block-causal by frame, Q/K/V/dO ~ N(0,1) from a fixed seed.  One step = block selection (query-group
pooling, key-block pooling fused with scoring, top-k), selection forward, inverted index, dQ, dK/dV.

`value` is executed TFLOP/s (4*D*sum(n_q*n_keys) forward, x2.5 backward) with the inputs
resident in HBM; `e2e` is the same metric with the step's inputs copied from pinned host
memory and its results copied back inside the timed region.  `--impl reference` times the CPU
restatement of the reference's path (oracle/nsa_oracle.py) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CFG = dict(B=1, H=12, D=128, M=4680, N=32760, block=64, group=64, topk=16, frame=1560, q_frame0=18)
METRIC = "nsa_selection_fwd_bwd_tflops"
UNIT = "TFLOP/s"
WORKLOAD = ("config2: bf16 NSA selection fwd+bwd, B=1 H=12 D=128, Q=4680 (3 latent frames), "
            "KV=32760 (21 frames) in 64-token blocks, top-16 per 64-query group")
# kernels of this library launched by one step: pooling (keys and queries), scoring + selection, forward,
# inverted index, dQ, counter reset, dK/dV
LAUNCHES_PER_STEP = 7
# the device-resident figure is the median of this many seconds' worth of back-to-back passes of K steps
TIMED_SECONDS = 2.0


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm=p["hbm_gbs"], tensor=p["bf16_tflops"], tensor_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm=6650.0, tensor=1590.0, tensor_sustained=1400.0, source="fallback")


def make_inputs(seed: int, pin: bool):
    c = CFG
    g = torch.Generator().manual_seed(seed)
    shp_q, shp_k = (c["B"], c["M"], c["H"], c["D"]), (c["B"], c["N"], c["H"], c["D"])
    t = {n: torch.randn(s, generator=g).to(torch.bfloat16) for n, s in
         (("q", shp_q), ("k", shp_k), ("v", shp_k), ("do", shp_q))}
    if pin:
        t = {n: x.pin_memory() for n, x in t.items()}
    return t


def executed_flops_fwd(idx: torch.Tensor) -> int:
    """4*D*sum over (group, head) rows of n_queries * n_valid_selected_tokens."""
    c = CFG
    MG = idx.shape[1]
    g = torch.arange(MG, device=idx.device)
    n_q = torch.clamp(c["M"] - g * c["group"], max=c["group"]).view(1, MG, 1)
    t0 = idx.long() * c["block"]
    n_tok = torch.clamp(c["N"] - t0, min=0, max=c["block"])
    n_keys = torch.where(idx >= 0, n_tok, torch.zeros_like(n_tok)).sum(-1)
    return int(4 * c["D"] * (n_keys * n_q).sum().item())


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.path = gpu_index, None, None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", delete=False, suffix=".csv")
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=f, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------ GPU arm
RECOMPUTE_BACKWARD = False


def gpu_step(ops, d, ev=None, side=None):
    """One pass of the hot path over device tensors; `ev` collects (name, start, stop) events.
    With a `side` stream the inverted index, which depends only on the ids, runs beside the forward."""
    c = CFG
    scale = c["D"] ** -0.5
    cur = torch.cuda.current_stream()

    def timed(name, fn):
        if ev is None:
            return fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        r = fn()
        b.record()
        ev.append((name, a, b))
        return r

    idx, qp, kp = timed("score_topk", lambda: ops.select_blocks(d["q"], d["k"], c["topk"], scale, c["block"], c["group"],
                                                               c["frame"], c["frame"], True, q_chunk_offset=c["q_frame0"]))
    kv = ops.DenseKV(d["k"], d["v"])
    # P and dS are computed once: the dQ kernel stores them (16 KiB per (group, head, slot) pair) and the
    # dK/dV kernel streams them; --recompute-backward runs the two kernels that each compute S and dP
    nbytes = 0 if RECOMPUTE_BACKWARD else ops.stored_probabilities_bytes(d["q"], kv, idx, c["block"], c["group"])
    if nbytes and "pds" not in d:
        d["pds"] = torch.empty(nbytes, dtype=torch.uint8, device=idx.device)
    pds = d.get("pds") if nbytes else None

    def index():
        return ops.inverted_index(idx, -(-c["N"] // c["block"]), c["block"], 1, False, c["group"], with_slots=pds is not None)

    if side is not None:
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            inv = index()
        out, lse = ops.sel_fwd(d["q"], kv, idx, c["block"], 1, scale, False, c["group"])
        cur.wait_stream(side)
    else:
        out, lse = timed("sel_fwd", lambda: ops.sel_fwd(d["q"], kv, idx, c["block"], 1, scale, False, c["group"]))
        inv = timed("inverted_index", index)
    groups, offsets = inv[0], inv[1]
    slots = inv[2] if pds is not None else None
    res = timed("sel_bwd_dq", lambda: ops.sel_bwd_dq(d["q"], kv, idx, out, lse, d["do"], c["block"], 1, scale,
                                                     False, c["group"], pds=pds))
    dq, delta = res[0], res[1]
    if pds is not None and not res[2]:
        slots = pds = None
    dk, dv = timed("sel_bwd_dkv", lambda: ops.sel_bwd_dkv(d["q"], kv, groups, offsets, lse, delta, d["do"],
                                                          c["topk"], c["block"], 1, scale, False, c["group"],
                                                          slots=slots, pds=pds))
    return idx, out, dq, dk, dv


def graph_time_us(fn_list, replays=5):
    """Mean device time per call, in microseconds, of the calls in `fn_list` captured back to back
    in one CUDA graph (no host launch gaps) and replayed `replays` times.  Callers pass calls over
    DIFFERENT tensors whose total size exceeds the L2, so that no call finds its input cached."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            for fn in fn_list:
                fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for fn in fn_list:
            fn()
    g.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(replays):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / (replays * len(fn_list))


def hbm_kernels(ops, dev, d, pk):
    """HBM-bound pieces of the path timed on their own: block selection (pooling + scoring + top-k)
    over three distinct key tensors in rotation, and the block-cache kernels at the rollout's
    chunk size (4680 tokens x 12 heads per append), through the C ABI, inside a CUDA graph."""
    import ctypes as C
    from omnimem_b200 import _lib
    from omnimem_b200.cache import BlockKVCache, RopeSpec
    c = CFG
    scale = c["D"] ** -0.5
    out = {}

    def entry(us, nbytes, peak, unit="GB/s", **kw):
        ach = nbytes / (us * 1e-6) / 1e9
        e = {"us": round(us, 2), "bytes": int(nbytes), "bound": "hbm", "achieved": round(ach, 1), "peak": peak,
             "frac": round(ach / peak, 4), "unit": unit}
        e.update(kw)
        return e

    # ---- block selection: K read once (100.6 MB), raw Q read once (14.4 MB), pooled operands + ids written
    ks = [d["k"]] + [torch.randn_like(d["k"]) for _ in range(2)]
    us = graph_time_us([(lambda kk=kk: ops.select_blocks(d["q"], kk, c["topk"], scale, c["block"], c["group"], c["frame"],
                                                         c["frame"], True, q_chunk_offset=c["q_frame0"])) for kk in ks])
    esz = 2
    MG, NC = -(-c["M"] // c["group"]), -(-c["N"] // c["block"])
    nbytes = (c["N"] + c["M"] + MG + NC) * c["H"] * c["D"] * esz + MG * c["H"] * c["topk"] * 4
    out["score_topk"] = entry(us, nbytes, pk["hbm"], kernels="pool_rows(q) -> pool_score(k) -> select",
                              note="three distinct key tensors in rotation (302 MB > 126 MB L2), calls back to back in one graph")
    del ks

    # ---- cache append at the rollout's chunk size: 8 chunks into 8 distinct page ranges (230 MB in, 230 MB out)
    H, D, S, PT = c["H"], c["D"], 4680, c["block"]
    n_chunks = 8
    max_blocks = -(-S * n_chunks // PT) + 1
    cache = BlockKVCache(H, D, num_pages=H * max_blocks, max_blocks=max_blocks, page_tokens=PT, device=dev, host_tier=False)
    chunks = [(torch.randn(S, H, D, device=dev, dtype=torch.bfloat16), torch.randn(S, H, D, device=dev, dtype=torch.bfloat16))
              for _ in range(n_chunks)]
    for kc, vc in chunks:
        cache.append(kc, vc)                      # pages assigned once; the timed calls rewrite in place
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream

    def raw_append(i, rope=None):
        kc, vc = chunks[i]
        pos0 = i * S
        first, last = pos0 // PT, (pos0 + S - 1) // PT
        args = (kc.data_ptr(), vc.data_ptr(), (C.c_int64 * 3)(kc.stride(0), kc.stride(1), 0), S, pos0, cache.n_tokens, H, D,
                cache.k_pool.data_ptr(), cache.v_pool.data_ptr(), PT, cache.block_table.data_ptr(), cache.max_blocks,
                None, last - first + 1, cache.page_owner.data_ptr(), cache.page_stamp.data_ptr(), 1000 + i,
                cache.k_pooled.data_ptr(), cache.v_pooled.data_ptr(), cache.status.data_ptr(), cache._dtype_code)
        if rope is None:
            _lib.call("nsa_cache_append", *args, stream(dev).cuda_stream)
        else:
            _lib.call("nsa_cache_append_rope", *args, C.byref(rope), stream(dev).cuda_stream)

    app_bytes = 2 * (2 * S * H * D * esz)          # K and V, read and written
    us = graph_time_us([(lambda i=i: raw_append(i)) for i in range(n_chunks)])
    out["cache_append"] = entry(us, app_bytes, pk["hbm"], note="4680 tokens x 12 heads, K and V, pooled keys refreshed; 8 chunks in rotation")
    def rope_table(n, dim):                        # complex128 [n, dim/2], theta 10000 (rope_params, wan_model.py:37-43)
        ang = torch.outer(torch.arange(n, dtype=torch.float64),
                          1.0 / torch.pow(10000.0, torch.arange(0, dim, 2, dtype=torch.float64) / dim))
        return torch.polar(torch.ones_like(ang), ang)

    freqs = torch.cat([rope_table(1024, D - 4 * (D // 6)), rope_table(1024, 2 * (D // 6)), rope_table(1024, 2 * (D // 6))], 1)
    specs = [RopeSpec(freqs, (30, 52), 3 * i, (1, 1, 1)).struct(dev, D) for i in range(n_chunks)]
    us = graph_time_us([(lambda i=i: raw_append(i, specs[i])) for i in range(n_chunks)])
    out["cache_append_rope"] = entry(us, app_bytes, pk["hbm"], note="the same with the rotary embedding applied on the way in (float64 products)")
    # query rotary embedding of one chunk (14.4 MB in, 14.4 MB out), eight chunks in rotation
    q_out = torch.empty(S, H, D, device=dev, dtype=torch.bfloat16)

    def rope_q(i):
        x = chunks[i][0]
        _lib.call("nsa_rope_apply", x.data_ptr(), (C.c_int64 * 3)(x.stride(0), x.stride(1), 0), S, H, D, q_out.data_ptr(),
                  _lib.NSA_BF16, C.byref(specs[i]), stream(dev).cuda_stream)

    us = graph_time_us([(lambda i=i: rope_q(i)) for i in range(n_chunks)])
    out["rope_apply"] = entry(us, 2 * S * H * D * 2, pk["hbm"], note="query rotary embedding of a 4680-token chunk (float64 products)")
    del cache, chunks, q_out

    # ---- LRU machinery at the 48-frame cap: 1170 blocks x 12 heads = 14040 pages, a selection of 888 x 16 ids
    MB = 1170
    cache = BlockKVCache(H, D, num_pages=H * MB, max_blocks=MB + 80, page_tokens=PT, device=dev, host_tier=True)
    cache.n_tokens = MB * PT
    cache.block_table[:, :MB] = torch.arange(H * MB, dtype=torch.int32, device=dev).view(H, MB)
    cache.page_owner.copy_((torch.arange(H, device=dev).view(H, 1) * cache.max_blocks + torch.arange(MB, device=dev)).view(-1))
    cache.page_stamp.copy_(torch.randperm(H * MB, device=dev) % 50)
    cache.epoch = 100
    ids = torch.randint(0, MB, (1, MG, H, c["topk"]), dtype=torch.int32, device=dev)
    cap = ids.numel()
    uniq, miss = (torch.empty(1 + cap, dtype=torch.int32, device=dev) for _ in range(2))
    wsb = _lib.load().nsa_cache_dedup_workspace_bytes(H * cache.max_blocks)
    ws = torch.empty(max(wsb, 1), dtype=torch.uint8, device=dev)
    ep = [200]

    def dedup():
        ep[0] += 1
        _lib.call("nsa_cache_dedup_touch", ids.data_ptr(), ids.numel(), H, c["topk"], cache.max_blocks, cache.max_blocks,
                  cache._stamp32.data_ptr(), ep[0], cache.block_table.data_ptr(), cache.page_stamp.data_ptr(), ep[0],
                  uniq.data_ptr(), miss.data_ptr(), cap, cache.counters.data_ptr(), ws.data_ptr(), wsb, stream(dev).cuda_stream)

    us = graph_time_us([dedup] * 4)
    out["cache_dedup_touch"] = {"us": round(us, 2), "bound": "latency", "note": f"{ids.numel()} selected ids over {H * cache.max_blocks} keys: mark, count, scan, compact"}
    n_vict = 74 * H                                                     # pages a new 4680-token chunk needs
    victims = torch.full((n_vict,), -1, dtype=torch.int32, device=dev)

    def pick():
        _lib.call("nsa_cache_select_victims", cache.page_owner.data_ptr(), cache.page_stamp.data_ptr(), cache.num_pages,
                  cache.max_blocks, MB, 10 ** 6, n_vict, None, n_vict, victims.data_ptr(), cache.status.data_ptr(),
                  stream(dev).cuda_stream)

    us = graph_time_us([pick] * 2)
    out["cache_select_victims"] = {"us": round(us, 2), "bound": "latency", "note": f"{n_vict} least recently used of {cache.num_pages} pages"}
    pick()
    torch.cuda.synchronize()
    keys = torch.cat([torch.tensor([n_vict], dtype=torch.int32, device=dev), cache.page_owner[victims.long()]])

    def move(direction):
        _lib.call("nsa_cache_move_pages", direction, victims.data_ptr(), keys.data_ptr() if direction else None, n_vict, None,
                  n_vict, cache.k_pool.data_ptr(), cache.v_pool.data_ptr(), cache.page_bytes, cache.host_k.data_ptr(),
                  cache.host_v.data_ptr(), cache.block_table.data_ptr(), cache.page_owner.data_ptr(),
                  cache.page_stamp.data_ptr(), 300, cache.counters.data_ptr(), stream(dev).cuda_stream)

    pcie = 55.0                                                          # GB/s per direction, PCIe 5 x16 in practice
    mv_bytes = n_vict * 2 * cache.page_bytes
    us = graph_time_us([lambda: move(0), lambda: move(1)], replays=3) * 2   # one evict + one fetch per pair
    out["cache_evict_fetch"] = {"us_evict_plus_fetch": round(us, 1), "bytes_each_way": int(mv_bytes), "bound": "pcie",
                                "achieved": round(2 * mv_bytes / (us * 1e-6) / 1e9, 1), "peak": 2 * pcie, "unit": "GB/s (both directions summed)",
                                "note": f"{n_vict} pages to the pinned host tier and back (kernel copies through unified addressing)"}
    del cache
    # ---- delivery rooflines of the streaming dK/dV kernel: its copy shape (one block per SM, four stages of
    # three 16 KiB bulk copies) with nothing computed, over an L2-resident and an HBM-resident buffer
    for name, mb in (("bulk_stream_l2_resident", 96), ("bulk_stream_hbm_resident", 1536)):
        buf = torch.empty(mb << 20, dtype=torch.uint8, device=dev)
        buf.view(torch.int32).random_()
        passes = max(1, 3072 // mb)
        run = lambda: _lib.call("nsa_probe_bulk_stream", buf.data_ptr(), buf.numel(), passes, stream().cuda_stream)
        for _ in range(2):
            run()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run()
        e1.record()
        torch.cuda.synchronize()
        moved = (buf.numel() // 49152) * 49152 * passes
        out[name] = {"buffer_mb": mb, "passes": passes, "us": round(e0.elapsed_time(e1) * 1e3, 1),
                     "achieved": round(moved / (e0.elapsed_time(e1) * 1e-3) / 1e9, 1), "unit": "GB/s",
                     "note": "copies only; the rate operands can reach shared memory at in that kernel's shape"}
        del buf
    return out


def range_kernels(ops, dev, pk, replays=20):
    """The range forward (the layer's sliding-window branch) alone, at the rollout's sizes: 4680 queries x
    12 heads over the pages of 1, 2 and 3 chunks, against the selection forward given the same blocks
    as a list.  Inputs (29 - 86 MB of K/V) stay in L2; the kernel is bound by the tensor pipe."""
    M, H, D = 4680, 12, 128
    scale = D ** -0.5
    out = {}

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / replays * 1e3

    g = torch.Generator().manual_seed(77)
    q = torch.randn(1, M, H, D, generator=g).bfloat16().to(dev)
    for chunks in (1, 2, 3):
        N = chunks * M
        nb = -(-N // 64)
        k = torch.randn(1, N, H, D, generator=g).bfloat16().to(dev)
        v = torch.randn(1, N, H, D, generator=g).bfloat16().to(dev)
        kv = ops.DenseKV(k, v)
        ids = torch.arange(nb, dtype=torch.int32, device=dev).expand(1, -(-M // 64), H, nb)
        flops = 4.0 * M * N * H * D
        us_r = timed(lambda: ops.range_fwd(q, kv, 0, nb, 64, scale))
        us_l = timed(lambda: ops.sel_fwd(q, kv, ids, 64, 1, scale, False, 64))
        o_r, _ = ops.range_fwd(q, kv, 0, nb, 64, scale)
        o_l, _ = ops.sel_fwd(q, kv, ids, 64, 1, scale, False, 64)
        out[f"{chunks}_chunks"] = {
            "blocks": nb, "us": round(us_r, 1), "tflops": round(flops / us_r / 1e6, 1),
            "frac": round(flops / us_r / 1e6 / pk["tensor"], 3), "peak": pk["tensor"], "bound": "tensor",
            "us_listed_on_sel_fwd": round(us_l, 1), "max_abs_vs_listed": float((o_r.float() - o_l.float()).abs().max())}
    return out


def run_range_only(args):
    """Only `range_kernels` (the command the ncu capture of the range forward runs)."""
    from omnimem_b200 import ops
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the GPU arm has no CPU fallback)")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    emit({"metric": "range_fwd_tflops", "range_only": True, "kernels": {"range_fwd": range_kernels(ops, dev, peaks())}})


def run_hbm_only(args):
    """Only the isolated HBM / cache kernel timings of `hbm_kernels` (the command the ncu captures of
    those kernels run): one line with their entries."""
    from omnimem_b200 import ops
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the GPU arm has no CPU fallback)")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    d = {n: x.to(dev) for n, x in make_inputs(1234, pin=False).items()}
    emit({"metric": METRIC, "hbm_only": True, "kernels": {"hbm_and_cache": hbm_kernels(ops, dev, d, peaks())}})


def run_gpu(args):
    from omnimem_b200 import ops
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the GPU arm has no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    host = make_inputs(1234 + rank, pin=True)
    d = {n: x.to(dev) for n, x in host.items()}
    c = CFG
    for _ in range(max(args.warmup, 3)):
        idx, out, dq, dk, dv = gpu_step(ops, d)
    torch.cuda.synchronize()
    flops_fwd = executed_flops_fwd(idx)
    # selected (head, block) pairs counted once: ids [1, MG, H, T] -> per head the distinct block ids
    uniq_pairs = sum(int(torch.unique(idx[0, :, h][idx[0, :, h] >= 0]).numel()) for h in range(idx.shape[2]))
    flops_step = int(flops_fwd * 3.5)

    # ---- per-kernel times: eager launches, one pair of events around each.  A spin kernel goes first
    # so that the host has queued the step's launches before the device starts them: the brackets
    # then hold the kernels' own durations, not the host's launch latency.
    ev = []
    for _ in range(args.steps):
        torch.cuda._sleep(3_000_000)
        gpu_step(ops, d, ev)
    torch.cuda.synchronize()

    # ---- device-resident timing: the step's launches replayed as one CUDA graph (launched one by
    # one from Python, the host needs longer per launch than the short kernels run)
    step = None
    if not args.no_graph:
        from omnimem_b200.graph import CapturedStep
        fork = torch.cuda.Stream()
        step = CapturedStep(lambda: gpu_step(ops, d, side=fork))
    run_step = step.replay if step is not None else (lambda: gpu_step(ops, d))
    for _ in range(3):
        run_step()
    if step is not None:
        # the replayed step (forked launches included) must give the eager launches' results bit for bit
        eager = gpu_step(ops, d)
        torch.cuda.synchronize()
        for name, a, b in zip(("idx", "out", "dq", "dk", "dv"), eager, step.outputs):
            if not torch.equal(a, b):
                raise SystemExit(f"bench.py: captured step disagrees with eager launches on {name}")
    # A pass is exactly K steps between two events.  Passes run back to back for about TIMED_SECONDS
    # (K steps alone last milliseconds: too short for a clock sample to fall inside, and the SM clock
    # only settles under seconds of load); the reported time per step is the MEDIAN pass.
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        run_step()
    t1.record()
    torch.cuda.synchronize()
    first_pass_ms = t0.elapsed_time(t1)
    n_pass = args.passes if args.passes > 0 else int(min(2000, max(3, TIMED_SECONDS * 1e3 / max(first_pass_ms, 1e-3))))
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(n_pass + 1)]
    marks[0].record()
    for i in range(n_pass):
        for _ in range(args.steps):
            run_step()
        marks[i + 1].record()
    barrier()
    pass_ms = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(n_pass))
    ms_total = pass_ms[len(pass_ms) // 2]                     # median pass of K steps
    ms_best, ms_all = pass_ms[0], marks[0].elapsed_time(marks[-1])
    clocks_resident = sampler.stop() if rank == 0 else None

    if args.kernels_only:
        if rank == 0:
            emit({"metric": METRIC, "kernels_only": True, "passes": n_pass, "steps": args.steps,
                  "ms_per_step": round(ms_total / args.steps, 4),
                  "value": round(world * flops_step * args.steps / (ms_total * 1e-3) / 1e12, 3)})
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- end to end: pinned host -> device, step, results -> pinned host
    res_host = {n: torch.empty_like(x, device="cpu").pin_memory() for n, x in
                (("out", out), ("dq", dq), ("dk", dk), ("dv", dv))}
    h2d = sum(x.numel() * x.element_size() for x in host.values())
    d2h = sum(x.numel() * x.element_size() for x in res_host.values())

    # Three streams, two slots: while step s computes, step s+1's inputs upload and step s-1's
    # results download (PCIe is full duplex).  Every step still moves its own inputs from pinned
    # host memory and its own results back; the timed region ends when the last download has.
    cur = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    slots = [{n: torch.empty_like(x, device=dev) for n, x in host.items()} for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]
    ev_read = [torch.cuda.Event() for _ in range(2)]
    ev_done = torch.cuda.Event()
    if args.no_graph:
        slot_step = [(lambda sl=sl: gpu_step(ops, slots[sl])) for sl in range(2)]
    else:
        slot_step = [CapturedStep(lambda sl=sl: gpu_step(ops, slots[sl], side=fork)).replay for sl in range(2)]

    def e2e_upload(s):
        sl = s % 2
        with torch.cuda.stream(s_in):
            if s >= 2:
                s_in.wait_event(ev_free[sl])
            for n, x in host.items():
                slots[sl][n].copy_(x, non_blocking=True)
            ev_in[sl].record(s_in)

    def e2e_run(n_steps):
        e2e_upload(0)
        for s in range(n_steps):
            sl = s % 2
            if s + 1 < n_steps:
                e2e_upload(s + 1)
            cur.wait_event(ev_in[sl])
            if s >= 2:
                cur.wait_event(ev_read[sl])          # a captured step reuses its result buffers
            _, o, a, b_, c_ = slot_step[sl]()
            ev_free[sl].record(cur)
            ev_done.record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done)
                for n, x in (("out", o), ("dq", a), ("dk", b_), ("dv", c_)):
                    res_host[n].copy_(x, non_blocking=True)
                    x.record_stream(s_out)
                ev_read[sl].record(s_out)
        cur.wait_stream(s_out)

    e2e_run(3)
    e2e_sampler = ClockSampler(local)
    if rank == 0:
        e2e_sampler.start()
    barrier()
    e2e_pass = []
    for _ in range(3):                                       # three passes of K steps, median
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        e2e_run(args.steps)
        e1.record()
        barrier()
        e2e_pass.append(e0.elapsed_time(e1))
    ms_e2e = sorted(e2e_pass)[1]
    clocks_e2e = e2e_sampler.stop() if rank == 0 else None

    if dist is not None:
        t = torch.tensor([ms_total, ms_e2e, ms_best], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, ms_e2e, ms_best = t.tolist()
    pk = peaks()
    extra = hbm_kernels(ops, dev, d, pk) if (world == 1 and not args.no_extras) else None
    del d, res_host, slots
    torch.cuda.empty_cache()
    sharded = None if args.no_extras else run_sharded(args, dist, dev, rank, world)
    torch.cuda.empty_cache()
    roll = None if args.no_extras else run_rollout(args, dist, dev, rank, world)

    if rank == 0:
        per = {}
        for name, a, b in ev:
            per.setdefault(name, []).append(a.elapsed_time(b))
        per = {n: sum(v) / len(v) for n, v in per.items()}
        work = {"sel_fwd": ("tensor", flops_fwd), "sel_bwd_dq": ("tensor", int(flops_fwd * 1.5)),
                "sel_bwd_dkv": ("tensor", flops_fwd)}
        kernels = {}
        for n, ms in per.items():
            entry = {"ms": round(ms, 5)}
            if n in work:
                bound, amount = work[n]
                ach = amount / (ms * 1e-3) / 1e12
                entry.update(bound=bound, achieved=round(ach, 2), peak=pk["tensor"], frac=round(ach / pk["tensor"], 4),
                             unit="TFLOP/s")
            if n in ("sel_fwd", "sel_bwd_dq"):
                # the other bound of the two tensor-core kernels: what each must move through HBM once.  K / V rows
                # of the selected (head, block) pairs, counted once each; Q, out / dQ rows; for dQ also dO, out
                # (the delta prologue) and, when it stores them, the P / dS tiles
                cc = CFG
                row = cc["H"] * cc["D"] * 2
                nbytes = 2 * uniq_pairs * cc["block"] * cc["D"] * 2 + (2 if n == "sel_fwd" else 4) * cc["M"] * row
                if n == "sel_bwd_dq" and not RECOMPUTE_BACKWARD:
                    nbytes += (-(-cc["M"] // cc["group"])) * cc["H"] * cc["topk"] * 16384
                entry["hbm"] = {"bytes": nbytes, "achieved": round(nbytes / (ms * 1e-3) / 1e9, 1), "peak": pk["hbm"], "unit": "GB/s",
                                "frac": round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm"], 4)}
            if n == "sel_bwd_dkv" and not RECOMPUTE_BACKWARD:
                # the streaming kernel computes nothing twice; what it must move through HBM once: Q and dO rows,
                # the stored P / dS tiles (16 KiB per pair), dK and dV of every token
                cc = CFG
                nbytes = (2 * cc["M"] + 2 * cc["N"]) * cc["H"] * cc["D"] * 2 + (-(-cc["M"] // cc["group"])) * cc["H"] * cc["topk"] * 16384
                entry["hbm"] = {"bytes": nbytes, "achieved": round(nbytes / (ms * 1e-3) / 1e9, 1), "peak": pk["hbm"], "unit": "GB/s",
                                "frac": round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm"], 4),
                                "note": "the bound that is nearer for this kernel: algorithmic bytes over the measured copy rate"}
            kernels[n] = entry
        if extra is not None:
            kernels["hbm_and_cache"] = extra
        dom = max((n for n in per if n in work), key=lambda n: per[n])
        roof = dict(kernels[dom])
        roof.pop("ms")
        # which roof binds: the one whose minimum time for this launch is the longer (tensor work at the measured
        # cuBLAS rate against algorithmic bytes at the measured copy rate); the other one is kept beside it
        hbm_view = roof.pop("hbm", None)
        if hbm_view is not None:
            t_tensor = work[dom][1] / (pk["tensor"] * 1e12)
            t_hbm = hbm_view["bytes"] / (pk["hbm"] * 1e9)
            tensor_view = {k: roof[k] for k in ("achieved", "peak", "frac", "unit")}
            if t_hbm > t_tensor:
                roof.update(bound="hbm", achieved=hbm_view["achieved"], peak=hbm_view["peak"], frac=hbm_view["frac"], unit="GB/s",
                            algorithmic_bytes=hbm_view["bytes"], tensor=tensor_view)
            else:
                roof.update(hbm=hbm_view)
            roof["min_time_us"] = {"tensor": round(t_tensor * 1e6, 1), "hbm": round(t_hbm * 1e6, 1)}
        # dram__bytes_read.sum + dram__bytes_write.sum of one launch at this workload, copied from the
        # committed ncu summaries of these kernels: a record of that capture, not a measurement of this run
        ncu_traffic = {"sel_fwd": 193.0e6 + 10.7e6, "sel_bwd_dq": 257.2e6 + 202.2e6, "sel_bwd_dkv": 262.0e6 + 162.9e6}
        if RECOMPUTE_BACKWARD:
            ncu_traffic.update({"sel_bwd_dq": 222.3e6 + 14.4e6, "sel_bwd_dkv": 206.7e6 + 158.0e6})
        roof.update(kernel=dom, traffic=ncu_traffic.get(dom), traffic_unit="bytes per launch",
                    traffic_source="ncu capture of this kernel at this workload (summary under profiles/), not measured by this run",
                    peak_source=pk["source"] + " (burst)",
                    note="achieved = algorithmic work (bytes for an HBM bound, flops for a tensor bound) of the kernel / mean CUDA-event time of its launches "
                         "(eager pass, launches queued behind a spin kernel so the brackets exclude host latency)")
        value = world * flops_step * args.steps / (ms_total * 1e-3) / 1e12
        e2e_val = world * flops_step * args.steps / (ms_e2e * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": round(value, 3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms_total / args.steps, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "flops_per_step": flops_step, "flops_fwd": flops_fwd,
                       "l2": "inputs (Q,K,V,dO = 230 MB) and outputs (230 MB) exceed the 126 MB L2; no explicit flush",
                       "parallelism": "one independent workload per GPU, no collective" if world > 1 else "1 GPU"},
            "timing": {"passes": n_pass, "steps_per_pass": args.steps, "reported": "median pass",
                       "ms_per_step_best_pass": round(ms_best / args.steps, 4),
                       "ms_per_step_first_pass": round(first_pass_ms / args.steps, 4),
                       "region_seconds": round(ms_all * 1e-3, 3),
                       "fraction_of_sustained_tensor_peak": round(flops_step * args.steps / (ms_total * 1e-3) / 1e12 / pk["tensor_sustained"], 4)},
            "e2e": {"value": round(e2e_val, 3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": round(ms_e2e / args.steps, 4), "passes": 3, "clocks": clocks_e2e,
                    "bound": "PCIe: 230 MB up and 230 MB down per step at the link rate; kernel time hides behind the copies",
                    "overlap": "upload of step s+1 and download of step s-1 run beside the kernels of step s"},
            "gpu_launches": LAUNCHES_PER_STEP * args.steps * n_pass,
            "launch": "eager (one Python call per kernel)" if args.no_graph else
                      "the step's kernels captured once and replayed as one CUDA graph, kernel-to-kernel edges as programmatic dependent launches; `kernels` times are from an eager pass",
            "clocks": clocks_resident, "roofline": roof, "kernels": kernels,
        }
        if sharded is not None:
            line["sharded"] = sharded
        if roll is not None:
            line["rollout"] = roll
        if world == 1 and not args.no_extras:
            line["gpu_baseline"] = gpu_baseline(per)
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(host, steps=1)
        emit(line)
    if dist is not None:
        dist.destroy_process_group()


def gpu_baseline(per):
    """The reference's own CUDA operators (rebuilt for sm_100a, oracle/_ref) timed on this GPU in a
    process of their own, at the divisible stand-in of the workload (M=4672, N=32768, 64/64, top-16):
    a baseline beside the numbers, never part of the measured path."""
    from oracle import ref_cuda_runner as R
    if not R.available():
        return {"unavailable": "oracle/_ref/omnimem_nsa_ref.so is not built (the reference tree exists only in the build container)"}
    with tempfile.TemporaryDirectory() as tmp:
        out = os.path.join(tmp, "t.pt")
        try:
            r = subprocess.run([sys.executable, os.path.join(ROOT, "oracle", "ref_cuda_runner.py"), "--case", "divisible_6464",
                                "--out", out, "--time", "10", "--times-only"], capture_output=True, text=True, timeout=600)
        except subprocess.TimeoutExpired:
            return {"unavailable": "the reference operators did not finish within 600 s"}
        if r.returncode != 0:
            return {"unavailable": "the reference operators failed: " + (r.stderr or r.stdout)[-300:]}
        ms = torch.load(out)["ms"]
    ref_step = ms["pool_q"] + ms["pool_k"] + ms["topk"] + ms["sel_fwd"] + ms["sel_bwd"]
    mine = per.get("score_topk", 0) + per.get("sel_fwd", 0) + per.get("inverted_index", 0) + per.get("sel_bwd_dq", 0) + per.get("sel_bwd_dkv", 0)
    return {"impl": "reference CUDA extension (src/omnimem/nsa/cuda_backend/csrc), TORCH_CUDA_ARCH_LIST=10.0a, eager torch.ops calls",
            "workload": "divisible stand-in: M=4672, N=32768, 64-token blocks, 64-query groups, top-16, bf16",
            "ms": {k: round(v, 4) for k, v in ms.items()}, "ms_per_step": round(ref_step, 4),
            "this_library_ms_per_step_same_brackets": round(mine, 4),
            "speedup_fwd": round(ms["sel_fwd"] / per["sel_fwd"], 2) if per.get("sel_fwd") else None,
            "speedup_bwd": round(ms["sel_bwd"] / (per.get("sel_bwd_dq", 0) + per.get("sel_bwd_dkv", 0) + per.get("inverted_index", 0)), 2)
            if per.get("sel_bwd_dkv") else None,
            "speedup_step": round(ref_step / mine, 2) if mine else None}


def run_sharded(args, dist, dev, rank, world):
    """Config 5: one selection forward (H=12, D=128, 4680 queries) over a 1,048,576-token KV cache
    sharded by block across the ranks (block b on rank b mod R); candidates merged after one
    all-gather, (O, LSE) partials by an all-to-all of row shares and an all-gather of the merged
    rows.  Device-timed, max over ranks.  Rank 0 then rebuilds the whole KV from the ranks' seeds and
    runs the single-device path on it: the parity fields and the strong-scaling baseline."""
    from omnimem_b200 import ops
    from omnimem_b200.sharded import ShardedSelection
    c = CFG
    H, D, bs, G, T = c["H"], c["D"], c["block"], c["group"], c["topk"]
    n_total = 1 << 20
    n_local = n_total // world                      # 16384 / world whole blocks per rank
    scale = D ** -0.5

    def shard(r):
        g = torch.Generator(device=dev).manual_seed(99 + r)
        k = torch.randn(1, n_local, H, D, generator=g, device=dev, dtype=torch.bfloat16)
        v = torch.randn(1, n_local, H, D, generator=g, device=dev, dtype=torch.bfloat16)
        return k, v

    q = torch.randn(1, c["M"], H, D, generator=torch.Generator(device=dev).manual_seed(5), device=dev,
                    dtype=torch.float32).to(torch.bfloat16)
    k, v = shard(rank)
    sh = ShardedSelection()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        for _ in range(3):
            r = fn()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            r = fn()
        b.record()
        barrier()
        ms = torch.tensor([a.elapsed_time(b) / steps], device=dev, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item(), r

    steps = max(5, min(args.steps, 20))
    ms_fly, (out, lse, idx) = timed(lambda: sh.forward(q, k, v, T, bs, G, c["frame"], False), steps)
    kp = ops.pool_rows(k, bs)                        # rollout mode: the cache keeps the pooled keys

    def cached():
        ids, _ = sh.select(q, k, T, bs, G, c["frame"], False, k_pooled_local=kp)
        o, l = sh.attend(q, k, v, ids, bs, G)
        return o, l, ids

    ms_cached, (out_c, _, idx_c) = timed(cached, steps)
    # the same two calls replayed as CUDA graphs (collectives included): what the device needs once
    # the host's launch work is out of the way
    ms_fly_eager, ms_cached_eager, launch = ms_fly, ms_cached, "eager"
    if not args.no_graph:
        try:
            from omnimem_b200.graph import CapturedStep
            cap_fly = CapturedStep(lambda: sh.forward(q, k, v, T, bs, G, c["frame"], False))
            cap_cached = CapturedStep(cached)
            ms_fly, (out, lse, idx) = timed(cap_fly.replay, steps)
            ms_cached, (out_c, _, idx_c) = timed(cap_cached.replay, steps)
            launch = "CUDA graph replay (kernels and collectives of one call captured once)"
        except Exception as e:                       # capture refused: the eager numbers stand
            launch = f"eager (graph capture failed: {type(e).__name__})"
    agree = torch.tensor([float(idx.sum().item())], device=dev, dtype=torch.float64)
    lo, hi = agree.clone(), agree.clone()
    if dist is not None:
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    res = None
    if rank == 0:
        # the whole KV on one device: block b = local block b // R of rank b % R
        kf = torch.empty(1, n_total, H, D, device=dev, dtype=torch.bfloat16)
        vf = torch.empty_like(kf)
        nbl = n_local // bs
        for r in range(world):
            kr, vr = (k, v) if r == 0 else shard(r)
            kf.view(1, nbl, world, bs, H, D)[:, :, r] = kr.view(1, nbl, bs, H, D)
            vf.view(1, nbl, world, bs, H, D)[:, :, r] = vr.view(1, nbl, bs, H, D)
            del kr, vr

        def single():
            ids, _, _ = ops.select_blocks(q, kf, T, scale, bs, G, c["frame"], c["frame"], False)
            o, l = ops.sel_fwd(q, ops.DenseKV(kf, vf), ids, bs, 1, scale, False, G)
            return o, l, ids

        for _ in range(2):
            o1, l1, i1 = single()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(5):
            o1, l1, i1 = single()
        b.record()
        torch.cuda.synchronize()
        ms_single = a.elapsed_time(b) / 5
        fin = torch.isfinite(l1)
        flops = 4 * D * c["M"] * H * T * bs
        esz = 2
        res = {"workload": "config5: selection forward, 4680 queries, 1,048,576-token KV sharded by block (b on rank b mod R), "
                           "top-16 merged after one all-gather, partials by all-to-all of row shares + all-gather of merged rows",
               "ms_per_call": round(ms_fly, 4), "ms_per_call_cached_pooled_keys": round(ms_cached, 4),
               "launch": launch, "ms_per_call_eager": round(ms_fly_eager, 4),
               "ms_per_call_cached_pooled_keys_eager": round(ms_cached_eager, 4),
               "single_device_ms_per_call": round(ms_single, 4),
               "strong_scaling_efficiency": round(ms_single / (world * ms_fly), 4),
               "fwd_tflops": round(flops / (ms_fly * 1e-3) / 1e12, 2),
               "kv_score_gbs_per_gpu": round(n_local * H * D * esz / (ms_fly * 1e-3) / 1e9, 1),
               "ranks_agree_on_topk": bool(lo.item() == hi.item()),
               "topk_equal": bool(torch.equal(idx, i1)) and bool(torch.equal(idx_c, i1)),
               "max_abs_vs_single_device": round((out.float() - o1.float()).abs().max().item(), 5),
               "lse_max_abs_vs_single_device": round((lse[fin] - l1[fin]).abs().max().item(), 6),
               "finite": bool(torch.isfinite(out.float()).all().item()),
               "collectives_per_call": 0 if world == 1 else 3}
        del kf, vf
    barrier()
    return res


def run_rollout(args, dist, dev, rank, world, long_video=False):
    """Configs 3 / 4: the causal rollout of the Wan2.1-1.3B-shaped model (random bf16 weights,
    synthetic conditioning) with every self-attention on the NSA path; one independent rollout per
    GPU.  Latent frames per second = frames / wall time of the denoising loop, max over ranks."""
    from omnimem_b200 import rollout as R
    shape = R.WanShape()
    if long_video:
        plan = R.RolloutPlan(latent_frames=241, cache_cap_frames=48, new_prompt_every=40, seed=rank)
    else:
        plan = R.RolloutPlan(seed=rank)
    if args.rollout_layers:
        shape.num_layers = args.rollout_layers
    model, caches = R.build(shape, plan, dev, seed=1000 + rank)
    warm = R.RolloutPlan(**{**plan.__dict__, "latent_frames": 2 * plan.frames_per_chunk, "new_prompt_every": None})
    R.rollout(model, caches, warm, dev)                                  # warm-up: two chunks
    res = R.rollout(model, caches, plan, dev)
    t = torch.tensor([res.seconds], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    secs = t.item()
    mem = torch.cuda.max_memory_allocated(dev) / 2 ** 30
    # where a forward's time goes: a second, bracketed pass over the last chunks (the brackets cost
    # launches of their own, so the sections add up to more than the timed forward)
    breakdown = None
    if rank == 0 and not long_video:
        tm = R.SectionTimer()
        prof = R.rollout(model, caches, plan, dev, timer=tm)
        breakdown = tm.summary_ms(per=prof.forwards)
    out = {"workload": ("config4: 241 latent frames in 3-frame chunks, block cache capped at 48 frames per layer, "
                        "a fresh conditioning tensor every 40 frames" if long_video else
                        "config3: 21 latent frames (480x832, 81 frames) in 3-frame chunks, 4 denoising steps + 1 cache-write forward per chunk"),
           "model": f"Wan2.1-T2V-1.3B shape, {shape.num_layers} blocks, dim {shape.dim}, {shape.num_heads} heads, ffn {shape.ffn_dim}, random bf16 weights",
           "attention": "cmp + swa on the range forward (128-row tiles), selection (top-16 of 64-token blocks per 64-query group) on the selection forward",
           "latent_frames_per_second": round(world * plan.latent_frames / secs, 3), "seconds": round(secs, 3),
           "forwards": res.forwards, "ms_per_forward": round(secs * 1e3 / res.forwards, 2),
           "rollouts": world, "cache": res.cache, "gpu_mem_gib": round(mem, 1), "device_status_clean": True}
    if breakdown is not None:
        out["ms_per_forward_by_section_bracketed"] = breakdown
        from omnimem_b200 import ops
        out["window_attention_kernel"] = range_kernels(ops, dev, peaks())
    del model, caches
    torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------ CPU reference
def cpu_pass(O, t, groups=None):
    """The oracle's restatement of the same step on host tensors; `groups` limits the pass to a
    sample of query groups (the whole K/V is still pooled and scored)."""
    c = CFG
    q, k, v, do = (t[n].float() for n in ("q", "k", "v", "do"))
    qp = O.pool_rows(t["q"], c["group"])
    kp = O.pool_rows(t["k"], c["block"])
    idx = O.topk_select(qp, kp, c["topk"], block_size=c["block"], chunk_size=c["frame"], chunk_size_k=c["frame"],
                        causal=True, q_chunk_offset=c["q_frame0"], q_group_size=c["group"])
    if groups is not None:
        lo, hi = groups
        m0, m1 = lo * c["group"], min(c["M"], hi * c["group"])
        q, do, idx = q[:, m0:m1], do[:, m0:m1], idx[:, lo:hi]
    out, lse = O.selection_fwd(q, k, v, idx, c["block"], 1, None, False, c["group"])
    O.selection_bwd(q, k, v, idx, out, lse, do, c["block"], 1, None, False, c["group"])
    return O.selection_flops(idx, q.shape[1], c["N"], c["D"], c["block"], 1, False, c["group"]) * 3.5


def cpu_baseline(host, steps: int, groups=None):
    from oracle import nsa_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    t0 = time.perf_counter()
    flops = 0.0
    for _ in range(steps):
        flops += cpu_pass(O, host, groups)
    dt = time.perf_counter() - t0
    n_groups = -(-CFG["M"] // CFG["group"])
    sample = "full workload" if groups is None else f"query groups [{groups[0]}, {groups[1]}) of {n_groups}"
    return {"value": round(flops / dt / 1e12, 5), "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{sample}, {steps} pass(es), {dt:.1f} s, torch CPU ops in fp32", "seconds": round(dt, 2)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import nsa_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    host = make_inputs(1234, pin=False)
    n_groups = -(-CFG["M"] // CFG["group"])
    # size the per-step sample so that warm-up + steps stay near two minutes
    t0 = time.perf_counter()
    cpu_pass(O, host, (0, 8))
    probe = time.perf_counter() - t0
    budget = 120.0 / max(1, args.steps + args.warmup)
    take = int(max(4, min(n_groups, 8 * budget / max(probe, 1e-3))))
    groups = None if take >= n_groups else (n_groups - take, n_groups)
    for _ in range(args.warmup):
        cpu_pass(O, host, groups)
    t0 = time.perf_counter()
    flops = 0.0
    for _ in range(args.steps):
        flops += cpu_pass(O, host, groups)
    dt = time.perf_counter() - t0
    val = round(flops / dt / 1e12, 5)
    sample = "full workload" if groups is None else f"query groups [{groups[0]}, {groups[1]}) of {n_groups}"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample_per_step": sample},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{sample} per step; CPU restatement of the reference's torch path, fp32"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


def run_rollout_only(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the GPU arm has no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    res = run_rollout(args, dist, dev, rank, world, long_video=args.workload == "rollout-long")
    if rank == 0:
        line = {"metric": "wan_causal_rollout_latent_frames_per_second", "value": res["latent_frames_per_second"],
                "unit": "latent frames/s", "n_gpus": world, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic", "config": {"workload": res["workload"], "model": res["model"]},
                "rollout": res, "clocks": sampler.stop()}
        emit(line)
    if dist is not None:
        dist.destroy_process_group()


_LINE_OUT = None


def emit(line):
    out = _LINE_OUT if _LINE_OUT is not None else sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the isolated HBM / cache kernel timings, the config-5 leg and the reference-GPU baseline")
    ap.add_argument("--workload", default="selection", choices=["selection", "rollout", "rollout-long"],
                    help="selection: the op-level step (default, with the rollout of config 3 as an extra); rollout / "
                         "rollout-long: only the rollout of config 3 / config 4, as a line of its own")
    ap.add_argument("--rollout-layers", type=int, default=0, help="fewer transformer blocks than 30 (for quick runs)")
    ap.add_argument("--passes", type=int, default=0, help="passes of K steps in the timed region (default: about 2 s worth)")
    ap.add_argument("--recompute-backward", action="store_true",
                    help="dK/dV kernel that recomputes S and dP instead of streaming the P / dS tiles the dQ kernel stored")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from Python instead of replaying a CUDA graph")
    ap.add_argument("--hbm-only", action="store_true",
                    help="only the isolated timings of the HBM-bound selection and block-cache kernels (the command their ncu captures run)")
    ap.add_argument("--range-only", action="store_true",
                    help="only the isolated timings of the range forward at the rollout's window sizes (the command its ncu capture runs)")
    ap.add_argument("--kernels-only", action="store_true",
                    help="device-resident steps only (no end-to-end leg, no CPU baseline): the command profiled by ncu")
    args = ap.parse_args()
    global RECOMPUTE_BACKWARD
    RECOMPUTE_BACKWARD = args.recompute_backward
    # stdout carries the JSON line and nothing else: libraries that print there (NCCL's version
    # banner, torchrun's notes) are sent to stderr, the line goes to the saved descriptor
    global _LINE_OUT
    sys.stdout.flush()
    _LINE_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference(args)
    elif args.hbm_only:
        run_hbm_only(args)
    elif args.range_only:
        run_range_only(args)
    elif args.workload != "selection":
        run_rollout_only(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
