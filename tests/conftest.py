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
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def load_golden(name):
    """Golden vectors written by tests/golden/make_golden.py, as torch tensors (lengths as a list)."""
    out = {}
    with np.load(os.path.join(GOLDEN_DIR, name + ".npz")) as z:
        for key in z.files:
            arr = z[key]
            if key == "lengths":
                out[key] = [int(x) for x in arr]
            elif arr.dtype == np.int16:          # bf16 bit patterns
                out[key] = torch.from_numpy(arr.copy()).view(torch.bfloat16)
            else:
                out[key] = torch.from_numpy(arr.copy())
    return out


def rel_l2(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


@pytest.fixture(scope="session")
def cuda_device():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
