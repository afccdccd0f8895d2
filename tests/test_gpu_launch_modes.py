"""The step's kernels give the same bits whether they are launched as programmatic dependent
launches (the default) or the ordinary way (OMNIMEM_B200_CHAINED_LAUNCH=0).  The switch is read
once per process, so each mode runs in a child process that prints a digest of its results."""
import hashlib
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

_CHILD = r"""
import hashlib, sys, torch
from omnimem_b200 import ops
dev = torch.device("cuda:0")
g = torch.Generator().manual_seed(77)
B, M, N, H, D, T = 1, 640, 4096, 3, 128, 8
q = torch.randn(B, M, H, D, generator=g).to(torch.bfloat16).to(dev)
k = torch.randn(B, N, H, D, generator=g).to(torch.bfloat16).to(dev)
v = torch.randn(B, N, H, D, generator=g).to(torch.bfloat16).to(dev)
do = torch.randn(B, M, H, D, generator=g).to(torch.bfloat16).to(dev)
scale = D ** -0.5
h = hashlib.sha256()
for _ in range(3):                                  # back-to-back steps: launches of one step follow the previous one's
    qp, kp = ops.pool_rows(q, 64), ops.pool_rows(k, 64)
    idx = ops.topk(qp, kp, T, scale, 64, 320, 320, True, q_group_size=64)
    kv = ops.DenseKV(k, v)
    out, lse = ops.sel_fwd(q, kv, idx, 64, 320, scale, True, 64)
    dq, dk, dv = ops.sel_bwd(q, kv, idx, out, lse, do, 64, 320, scale, True, 64)
    torch.cuda.synchronize()
    for t in (idx, out, lse, dq, dk, dv):
        h.update(t.cpu().contiguous().view(torch.uint8).numpy().tobytes())
print("DIGEST", h.hexdigest())
"""


def _run(mode):
    env = dict(os.environ)
    env["OMNIMEM_B200_CHAINED_LAUNCH"] = mode
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    r = subprocess.run([sys.executable, "-c", _CHILD], env=env, cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("DIGEST ")]
    assert lines, r.stdout[-2000:]
    return lines[-1].split()[1]


def test_chained_and_ordinary_launches_agree_bit_for_bit():
    ordinary = _run("0")
    chained = _run("15")
    assert chained == ordinary
    assert len(chained) == hashlib.sha256().digest_size * 2
