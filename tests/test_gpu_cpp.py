"""GPU: C++-level drop-in checks.

``tests/cpp/bin/tensor_test_b200`` is the reference project's own
test/tensor_test.cpp, compiled without modification against this repository's
headers and linked with the B200 backend (built where the reference tree is
mounted).  ``tests/cpp/bin/api_test`` is this repository's own C++ test file.
Both are prebuilt by ``micrograd_b200.build``.
"""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _run(path):
    assert os.path.exists(path), f"{path} not built (python -m micrograd_b200.build)"
    r = subprocess.run([path], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-2000:]
    return r.stdout


def test_reference_test_file_runs_unchanged_on_b200_backend():
    out = _run(os.path.join(ROOT, "tests", "cpp", "bin", "tensor_test_b200"))
    assert "11 tests ran" in out and "[  PASSED  ] 11 tests" in out


def test_cpp_api_tests():
    out = _run(os.path.join(ROOT, "tests", "cpp", "bin", "api_test"))
    assert "[  FAILED  ]" not in out
