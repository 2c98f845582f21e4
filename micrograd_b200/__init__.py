"""micrograd_b200 — B200-native (sm_100a) CUDA backend for micrograd's fp64
tensor-op path, behind the reference's own C++ ``Tensor`` API.

The product is two shared libraries built in-tree by ``micrograd_b200.build``:

* ``lib/libmg_cuda.so`` — hand-written CUDA kernels behind the C ABI declared in
  ``include/mg_cuda.h`` (device-resident fp64 storage, elementwise / broadcast /
  reduction / GEMM / fused-loss / SGD kernels, gradient all-reduce over peer
  memory or NCCL);
* ``lib/libmicrograd.so`` — the C++ ``Tensor``/``Linear``/``SGD`` classes
  (``include/micrograd/*.h``) as a thin graph-building layer over that ABI, plus
  the flat C binding ``include/mg_tensor_c.h``.

Python is only the test and benchmark harness: ``load_abi()`` gives ctypes access
to the device C ABI, ``load_api()`` a mirror of the C++ classes.  There is no CPU
fallback: both raise if the libraries are missing, and every device entry
point fails with an error if no CUDA device can be initialised.
"""
from __future__ import annotations

import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_DIR = os.path.join(_HERE, "lib")
CUDA_LIB = os.path.join(LIB_DIR, "libmg_cuda.so")
TENSOR_LIB = os.path.join(LIB_DIR, "libmicrograd.so")

_api = None
_cabi = None


def load_api():
    """Python mirror of the C++ Tensor / Linear / SGD API (B200 backend)."""
    global _api
    if _api is None:
        if not os.path.exists(TENSOR_LIB):
            raise ImportError(f"{TENSOR_LIB} not built: run `python -m micrograd_b200.build`")
        from .tensor_api import bind
        _api = bind(TENSOR_LIB)
    return _api


def load_abi():
    """ctypes view of the device C ABI (include/mg_cuda.h)."""
    global _cabi
    if _cabi is None:
        if not os.path.exists(CUDA_LIB):
            raise ImportError(f"{CUDA_LIB} not built: run `python -m micrograd_b200.build`")
        from .cabi import CudaABI
        _cabi = CudaABI(CUDA_LIB)
    return _cabi
