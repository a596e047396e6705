import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "gemm_golden.npz"))


@pytest.fixture(scope="session")
def built():
    """libo64gemm.so and the oracle, built in-tree if a source changed."""
    sys.path.insert(0, ROOT)
    import __graft_entry__ as ge
    ge.build()
    return True


@pytest.fixture(scope="module")
def eng(built):
    import torch
    import open64_b200 as o
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device: the engine has no CPU fallback")
    e = o.Engine(0)
    yield e
    st, detail = e.last_status()
    e.close()
    assert st == 0, f"device status {st} (detail 0x{detail:x})"
