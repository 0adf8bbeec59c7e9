"""Shared test set-up: marker registration, import paths, helpers."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "ascend-rsfa_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def golden_cases():
    return sorted(f[:-4] for f in os.listdir(GOLDEN) if f.endswith(".npz"))


def load_golden(name):
    import numpy as np
    import torch

    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    t = {k: torch.from_numpy(z[k]) for k in ("q", "k", "v", "o")}
    t.update(
        causal=bool(z["causal"]), sm_scale=float(z["sm_scale"]),
        block_m=int(z["block_m"]), block_n=int(z["block_n"]),
    )
    return t


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
