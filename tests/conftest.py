import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def load_golden(name: str) -> dict:
    """Load ``tests/golden/<name>.npz``; ``__bf16`` / ``__e4m3`` keys come back as torch tensors of that dtype."""
    out = {}
    with np.load(os.path.join(GOLDEN, name + ".npz")) as z:
        for k in z.files:
            a = z[k]
            if k.endswith("__bf16"):
                out[k[:-6]] = torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)
            elif k.endswith("__e4m3"):
                out[k[:-6]] = torch.from_numpy(a.copy()).view(torch.float8_e4m3fn)
            else:
                out[k] = torch.from_numpy(a.copy())
    return out


@pytest.fixture(scope="session")
def cuda_dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)
