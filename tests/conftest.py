"""Shared fixtures.  Tests marked ``gpu`` need a B200 and the built libraries
and call the product through its C ABI; everything else runs on a CPU-only
machine (oracle, host logic, symbol exports, gloo multi-process paths)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200) and the built libraries")


def golden(name: str):
    return np.load(os.path.join(GOLDEN, name))


@pytest.fixture(scope="session")
def fast():
    import oracle
    return oracle.fast


@pytest.fixture(scope="session")
def abi():
    """Device C ABI.  Fails (does not skip) when the library or the GPU is missing:
    a GPU test that cannot reach the kernels must not pass."""
    import micrograd_b200
    a = micrograd_b200.load_abi()
    a.mg_init(-1)
    return a


@pytest.fixture(scope="session")
def api(abi):
    """Python mirror of the C++ Tensor API, B200 backend."""
    import micrograd_b200
    return micrograd_b200.load_api()


def rel_err(got, ref):
    """max |got-ref| / |ref| with exact-zero handling (0 vs 0 counts as 0)."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    diff = np.abs(got - ref)
    denom = np.abs(ref)
    out = np.where(denom > 0, diff / np.where(denom > 0, denom, 1.0), diff)
    return float(out.max()) if out.size else 0.0


def norm_err(got, ref):
    """max |got-ref| / max |ref| (normwise)."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    scale = float(np.abs(ref).max()) if ref.size else 0.0
    return float(np.abs(got - ref).max()) / (scale if scale > 0 else 1.0) if ref.size else 0.0
