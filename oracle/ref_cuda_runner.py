"""Runs the reference's own CUDA operators (oracle/_ref/omnimem_nsa_ref.so, built by
oracle/build_ref.py from the reference tree) on seeded inputs, in a process of its own.

Test infrastructure: the second judge of the parity tests and the GPU baseline of bench.py.
It must not share a process with the product, which registers the same operator names
(torch.ops.omnimem_nsa.*) from Python, hence the command-line form:

    python oracle/ref_cuda_runner.py --case divisible_6464 --out /tmp/x.pt [--time 10]

writes a torch file with the operators' outputs for the named case (and, with --time N, the mean
CUDA-event time of N back-to-back launches of each operator after three warm-up launches).

The call sequence is the reference facade's (nsa/ops/index_topk.py:72-105: query-group mean, then
`topk` with the chunk length counted in pooled rows; nsa/cuda_backend/autograd.py:9-43: `sel_fwd`,
`sel_bwd`), with the key pooling of models/transformers/causal_wan_nsa_model.py:408-409.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
NSA_LIB = os.path.join(HERE, "_ref", "omnimem_nsa_ref.so")

# name -> geometry the reference accepts (M % G == 0, chunk % G == 0, chunk % block == 0 when causal)
CASES = {
    # 64-token blocks / 64-query groups at the Wan layer shape on divisible lengths: 73 query groups of
    # chunk 6 against 512 key blocks, block-causal by 4672-token chunk
    "divisible_6464": dict(seed=101, B=1, M=4672, N=32768, H=12, D=128, T=16, bs=64, G=64, chunk=4672, causal=True,
                           ex_win=0, ex_sink=0, prog=False, q_off=6),
    # the reference's native geometry: 30-token blocks, 15-query groups, top-16, window exclusion of 3 chunks,
    # progressive; the rollout call (non-causal, query chunk 6 of 7)
    "native_3015": dict(seed=102, B=1, M=4680, N=32760, H=12, D=128, T=16, bs=30, G=15, chunk=4680, causal=False,
                        ex_win=3, ex_sink=0, prog=True, q_off=6),
    # small cases for quick runs
    "small_6464": dict(seed=103, B=2, M=256, N=2048, H=3, D=128, T=8, bs=64, G=64, chunk=256, causal=True,
                       ex_win=0, ex_sink=0, prog=False, q_off=5),
    # the training layout: queries and keys are the same full sequence, causal by chunk in the top-k AND
    # token-causal inside the attention
    "full_causal_6464": dict(seed=105, B=1, M=1024, N=1024, H=3, D=128, T=6, bs=64, G=64, chunk=256, causal=True,
                             ex_win=0, ex_sink=0, prog=False, q_off=0, attn_causal=True),
    "small_3015": dict(seed=104, B=1, M=240, N=1200, H=2, D=128, T=6, bs=30, G=15, chunk=120, causal=True,
                       ex_win=1, ex_sink=1, prog=True, q_off=3),
}


def make_case(name: str):
    """Seeded bf16 inputs of a case as CPU tensors: (cfg, q, k, v, d_out)."""
    c = CASES[name]
    g = torch.Generator().manual_seed(c["seed"])
    shp_q, shp_k = (c["B"], c["M"], c["H"], c["D"]), (c["B"], c["N"], c["H"], c["D"])
    q, k, v, do = (torch.randn(s, generator=g).to(torch.bfloat16) for s in (shp_q, shp_k, shp_k, shp_q))
    return c, q, k, v, do


def available() -> bool:
    return os.path.exists(NSA_LIB)


def _time(fn, n):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(n):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / n


def run(name: str, n_time: int = 0) -> dict:
    torch.ops.load_library(NSA_LIB)
    ref = torch.ops.omnimem_nsa
    c, q, k, v, do = make_case(name)
    dev = torch.device("cuda:0")
    q, k, v, do = (t.to(dev) for t in (q, k, v, do))
    B, M, N, H, D, T, bs, G = (c[x] for x in ("B", "M", "N", "H", "D", "T", "bs", "G"))
    scale = D ** -0.5
    qp = q.reshape(B, M // G, G, H, D).mean(dim=2)
    kp = k.view(B, N // bs, bs, H, D).mean(2)

    def topk():
        return ref.topk(qp, kp, T, scale, bs, c["chunk"] // G, c["chunk"], c["causal"], c["ex_win"], c["ex_sink"],
                        c["prog"], False, c["q_off"], True)

    idx = topk()
    # the attention runs as the rollout does - every selected block fully visible, the top-k mask has
    # decided - unless the case asks for the training layout's token-causal rule
    a_chunk, a_causal = (c["chunk"], True) if c.get("attn_causal") else (1, False)

    def fwd():
        return ref.sel_fwd(q, k, v, idx, bs, a_chunk, scale, a_causal, G, True)

    out, lse = fwd()

    def bwd():
        return ref.sel_bwd(q, k, v, idx, out, lse, do, bs, a_chunk, scale, a_causal, G, True)

    dq, dk, dv = bwd()
    torch.cuda.synchronize()
    res = dict(case=name, q_pooled=qp.cpu(), k_pooled=kp.cpu(), idx=idx.cpu(), out=out.cpu(), lse=lse.cpu(),
               dq=dq.cpu(), dk=dk.cpu(), dv=dv.cpu(), device=torch.cuda.get_device_name(0))
    if n_time > 0:
        res["ms"] = dict(pool_q=_time(lambda: q.reshape(B, M // G, G, H, D).mean(dim=2), n_time),
                         pool_k=_time(lambda: k.view(B, N // bs, bs, H, D).mean(2), n_time),
                         topk=_time(topk, n_time), sel_fwd=_time(fwd, n_time), sel_bwd=_time(bwd, n_time))
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True, choices=sorted(CASES))
    ap.add_argument("--out", required=True)
    ap.add_argument("--time", type=int, default=0)
    ap.add_argument("--times-only", action="store_true", help="store the timings without the tensors")
    a = ap.parse_args()
    if not available():
        print(f"{NSA_LIB} is missing (python -m oracle.build_ref builds it where the reference tree exists)")
        sys.exit(3)
    res = run(a.case, a.time)
    if a.times_only:
        res = {k: v for k, v in res.items() if not torch.is_tensor(v)}
    torch.save(res, a.out)


if __name__ == "__main__":
    main()
