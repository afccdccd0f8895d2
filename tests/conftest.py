import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_terminal_summary(terminalreporter):
    """One line per output / gradient comparison of the run: the measured errors beside the limits."""
    from tests.helpers import PARITY_LOG
    if not PARITY_LOG:
        return
    tr = terminalreporter
    tr.section("measured parity errors (max abs / mean abs vs limit; largest reference magnitude)")
    for what, mx, mean, ref, lim_max, lim_mean in PARITY_LOG:
        tr.write_line(f"PARITY {what}: max_abs {mx:.3e} (limit {lim_max:.1e})  mean_abs {mean:.3e} "
                      f"(limit {lim_mean:.1e})  max|ref| {ref:.3g}")


def load_golden(name):
    """Load tests/golden/<name>.npz; keys ending in _bf16 hold bf16 bit patterns and are
    returned as torch.bfloat16 tensors under the key without the suffix."""
    raw = np.load(os.path.join(GOLDEN_DIR, f"{name}.npz"))
    out = {}
    for key in raw.files:
        arr = raw[key]
        if key.endswith("_bf16"):
            out[key[:-5]] = torch.from_numpy(arr.copy()).view(torch.bfloat16)
        else:
            out[key] = torch.from_numpy(arr.copy())
    return out


@pytest.fixture(scope="session")
def golden():
    return load_golden


def has_cuda():
    return torch.cuda.is_available()


@pytest.fixture(scope="session")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _device_status_is_clean(request):
    """After every GPU test: no kernel gave up on a bounded wait."""
    yield
    if request.node.get_closest_marker("gpu") is not None and torch.cuda.is_available():
        from omnimem_b200 import _lib
        torch.cuda.synchronize()
        assert _lib.device_status() == 0, "a kernel reported a device-side error"
