"""GPU: the small entry points around the hot path — byte upload with scaling
(the loader's pixel / 255.0), the on-device input generator and its host twin,
the fault-word mirror, and read-only host views that leave the device copy
current."""
import ctypes as C

import numpy as np
import pytest

from micrograd_b200 import cabi as K

pytestmark = pytest.mark.gpu


def test_byte_upload_divides_exactly_like_the_host(abi):
    """dst = byte / 255.0 (src/mnist.cpp:21 of the reference): one IEEE division on
    the device, so all 256 values — and a ragged length — equal numpy's, bit for bit."""
    raw = np.concatenate([np.arange(256, dtype=np.uint8),
                          np.random.default_rng(0).integers(0, 256, 100_003).astype(np.uint8)])
    out = abi.empty(raw.size)
    abi.mg_upload_u8_scaled(out.ptr, raw.ctypes.data, raw.size, 255.0)
    assert np.array_equal(out.numpy(), raw / 255.0)
    with pytest.raises(K.MgError):
        abi.mg_upload_u8_scaled(out.ptr, raw.ctypes.data, raw.size, 0.0)


def test_device_uniform_generator_matches_its_host_formula(abi):
    import bench
    n, seed = 100_003, 20240605
    out = abi.empty(n)
    for first in (0, 7, 784 * 131072):           # a shard starting deep in the stream
        abi.mg_fill_uniform01(out.ptr, n, seed, first)
        got = out.numpy()
        assert np.array_equal(got, bench.uniform01_host(seed, first, n))
        assert got.min() >= 0.0 and got.max() < 1.0
    whole = abi.empty(2 * n)
    abi.mg_fill_uniform01(whole.ptr, 2 * n, seed, 0)
    abi.mg_fill_uniform01(out.ptr, n, seed, n)   # second half generated on its own
    assert np.array_equal(whole.numpy()[n:], out.numpy())
    assert abs(whole.numpy().mean() - 0.5) < 5e-3


def test_fault_word_mirror_reads_without_a_sync(abi):
    st = C.c_int(-1)
    abi.mg_kernel_status_peek(C.byref(st))
    assert st.value == 0                        # nothing mirrored, or a clean word
    abi.mg_kernel_status_mirror()
    abi.mg_sync()
    abi.mg_kernel_status_peek(C.byref(st))
    assert st.value == 0
    abi.mg_check_kernel_status()


def test_reading_values_keeps_the_device_copy_current(api, abi):
    """data()/grad() reads through the flat C API use the read-only views: a
    parameter stays in the optimiser's flat buffers (one-launch SGD step) after
    the host looked at it, and a zero gradient stays logically zero."""
    lin = api.Linear(64, 32)
    W = np.random.default_rng(1).standard_normal((64, 32))
    lin.weights().set_data(W)
    opt = api.SGD([lin.weights(), lin.bias()], 0.5)
    opt.enable_allreduce()                       # single rank: flat buffers, no exchange
    x = api.Tensor([8, 64], np.ones((8, 64)))
    x.set_requires_grad(False)
    assert not lin.weights().grad().any()        # read of a logically-zero gradient
    loss = lin.forward(x).sum()
    opt.zero_grad()
    loss.backward()
    g = lin.weights().grad().reshape(64, 32)     # host read between backward and step
    assert np.array_equal(g, np.full((64, 32), 8.0))
    before = abi.mg_launch_count()
    opt.step()
    assert abi.mg_launch_count() - before == 1   # still the single flat update
    assert np.array_equal(lin.weights().data().reshape(64, 32), W - 0.5 * 8.0)
    assert np.array_equal(lin.bias().data(), np.full(32, -0.5 * 8.0))
