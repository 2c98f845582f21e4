"""CPU: the C-ABI libraries load and export every symbol their headers declare;
without a GPU the product fails loudly instead of computing on the CPU."""
import ctypes
import os

import pytest

import micrograd_b200
from micrograd_b200 import cabi as K

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header(name):
    with open(os.path.join(ROOT, "include", name)) as f:
        return f.read()


def test_device_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(micrograd_b200.CUDA_LIB)
    names = K.declared_in_header(_header("mg_cuda.h"))
    assert len(names) >= 50
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    assert set(names) == set(K.SIGNATURES), set(names) ^ set(K.SIGNATURES)


def test_tensor_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(micrograd_b200.TENSOR_LIB)
    names = K.declared_in_header(_header("mg_tensor_c.h"))
    assert len(names) >= 45
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def _have_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


@pytest.mark.skipif(_have_gpu(), reason="checks the no-GPU failure mode")
def test_no_cpu_fallback_without_a_gpu():
    abi = micrograd_b200.load_abi()
    with pytest.raises(K.MgError) as e:
        abi.mg_init(-1)
    assert e.value.code == K.ERR_CUDA and "no CPU fallback" in str(e.value)
    api = micrograd_b200.load_api()
    with pytest.raises(RuntimeError, match="no usable CUDA device"):
        api.Tensor([2], [1.0, 2.0])
    # argument validation that needs no device still works
    with pytest.raises(ValueError, match="Tensor and data size mismatch"):
        api.Tensor([2], [1.0, 2.0, 3.0])
    assert api.format_scalar("*", 2.0) == "* 2.00"


def test_product_does_not_import_the_oracle():
    """The checker must never sit on the product path."""
    pkg = os.path.join(ROOT, "micrograd_b200")
    for d, _, files in os.walk(pkg):
        if os.path.basename(d) in ("build", "lib", "__pycache__"):
            continue
        for f in files:
            if f.endswith((".py", ".cpp", ".cu", ".cuh", ".h")):
                text = open(os.path.join(d, f)).read()
                assert "import oracle" not in text and "from oracle" not in text, f
                assert "ref_fast" not in text and "libref_" not in text, f
