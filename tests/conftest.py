"""Shared fixtures. Tests marked `gpu` need a B200; everything else runs on CPU."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    """ctypes binding of the C restatement (built on first use)."""
    from oracle import binding
    binding.lib()
    return binding


@pytest.fixture(scope="session")
def have_ref():
    from oracle import binding
    return binding.have_ref()


def load_small(name):
    from litnicelm_b200.formats import ModelDims
    z = np.load(os.path.join(GOLDEN, f"small_{name}.npz"))
    dm = [int(v) for v in z["dims"]]
    return ModelDims(*dm), z


@pytest.fixture(scope="session", params=["c1", "abcdef"])
def small_case(request):
    return (request.param,) + load_small(request.param)
