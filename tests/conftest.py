import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def golden():
    """Inputs of the two small workloads and the reference's own outputs on them."""
    d = np.load(ROOT / "tests" / "golden" / "walk_golden.npz")
    out = {}
    for k in d.files:
        a = d[k]
        out[k] = a.astype(np.int64) if a.dtype in (np.int16, np.int32) else a
    out["start2"] = np.arange(2708, dtype=np.int64)
    return out


@pytest.fixture(scope="session")
def walklib():
    """The CUDA library, built if needed (nvcc cross-compiles without a GPU)."""
    from mlx_cluster_b200 import _lib, build
    build.build()
    return _lib.lib()


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)
