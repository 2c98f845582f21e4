"""CPU: the host-side bookkeeping of the data-parallel gradient exchange.

``tests/cpp/bin/buckets_test`` is a C++ test binary over the header-only
``micrograd/detail/GradBuckets.h`` (no CUDA link): how a parameter list is grouped
into all-reduce messages (weight+bias pairs by shape, not by index parity; lists
with all weights first; layers without a bias), that a parameter the backward
sweep never reaches is left for step() to reduce, that stale flags of an earlier
sweep cannot fire a bucket, and that a second sweep after an exchange is refused.
"""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_grad_bucket_logic():
    path = os.path.join(ROOT, "tests", "cpp", "bin", "buckets_test")
    if not os.path.exists(path):
        from micrograd_b200 import build
        build.build_cpp_tests()
    r = subprocess.run([path], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "[  FAILED  ]" not in r.stdout, r.stdout[-3000:] + r.stderr[-1000:]
    assert "8 tests ran" in r.stdout
