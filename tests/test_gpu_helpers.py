"""GPU: the small entry points around the hot path — byte upload with scaling
(the loader's pixel / 255.0), the on-device input generator and its host twin,
the fault-word mirror, the pool reserve, and read-only host views that leave the device copy
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


def test_pool_reserve_takes_the_memory_once_and_allocations_then_reuse_it(abi):
    """After mg_pool_reserve(n) the pool owns n bytes nobody uses: the device's free
    memory has gone down by the reserve at most once, and an allocation of that size
    afterwards comes out of the pool, not out of the device."""
    def free_bytes():
        free, total = C.c_size_t(), C.c_size_t()
        abi.mg_sync()
        abi.mg_mem_info(C.byref(free), C.byref(total))
        return free.value

    size = 3 << 30
    abi.mg_pool_reserve(0)                              # nothing to do, no error
    before = free_bytes()
    abi.mg_pool_reserve(size)
    after = free_bytes()
    assert before - after <= size + (64 << 20)          # it grew by the reserve at most (or had it)
    abi.mg_pool_reserve(size)                           # already there: no further growth
    assert free_bytes() == after
    block = abi.empty(size // 8)
    assert free_bytes() == after                        # served from the reserve
    del block
    assert free_bytes() == after                        # and handed back to the pool, not the device


def test_prefetch_from_host_refreshes_two_inputs_in_turn(abi, api):
    """Tensor::prefetch_from_host: the copy runs on the copy stream behind the kernels
    already enqueued (which still read the old values) and ahead of the next use.  Two
    input tensors are refreshed in turn, as a double-buffered training loop does, from
    pinned staging buffers; every result equals the one computed from that batch."""
    rows, cols = 4096, 784
    n = rows * cols
    rng = np.random.default_rng(11)
    batches = [rng.random((rows, cols)) for _ in range(5)]
    pinned, views = [], []
    for _ in range(2):
        p = C.c_void_p()
        abi.mg_host_alloc(n * 8, C.byref(p))
        pinned.append(p)
        views.append(np.ctypeslib.as_array(C.cast(p.value, C.POINTER(C.c_double)), shape=(rows, cols)))
    views[0][...] = batches[0]
    views[1][...] = batches[1]
    inputs = [api.from_host([rows, cols], p.value) for p in pinned]
    w = api.Tensor([cols, 8], rng.standard_normal((cols, 8)))
    results = []
    for i, batch in enumerate(batches):
        slot = i % 2
        if i >= 2:
            # the result that read this slot has been downloaded below, so the staging
            # buffer and the device buffer are both free to take the next batch
            views[slot][...] = batch
            inputs[slot].prefetch_from_host(pinned[slot].value)
        out = inputs[slot].matmul(w).relu().sum()
        if i >= 1:
            results[i - 1] = float(results[i - 1].data()[0])   # read one step late, as a loop would
        results.append(out)
    results[-1] = float(results[-1].data()[0])
    wv = np.array(w.data()).reshape(cols, 8)
    for batch, got in zip(batches, results):
        want = np.maximum(batch @ wv, 0.0).sum()
        assert abs(got - want) <= 1e-10 * abs(want)
    assert np.array_equal(np.array(inputs[0].data()).reshape(rows, cols), batches[4])   # host read sees the new values
    assert np.array_equal(np.array(inputs[1].data()).reshape(rows, cols), batches[3])
    small = api.Tensor([2, 2], np.zeros((2, 2)))
    assert api.lib.mgt_prefetch_from_host(small._h, pinned[0], 5) != 0       # size mismatch is refused
    assert b"size mismatch" in api.lib.mgt_last_error()
    assert list(small.data()) == [0.0, 0.0, 0.0, 0.0]
    del inputs
    abi.mg_sync()
    for p in pinned:
        abi.mg_host_free(p.value)
