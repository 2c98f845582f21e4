"""GPU: the benchmark's full sizes, checked through size-independent properties (the
CPU oracle would need minutes to hours at these sizes), plus spot checks of a
few rows against the oracle.

  config 2: 2^28-element elementwise/reduction arrays (2 GiB each)
  config 3: 8192^3 matmul
  config 5: 1,048,576-input batched inference, sharded by rows
"""
import numpy as np
import pytest

from conftest import norm_err
from micrograd_b200 import cabi as K

pytestmark = pytest.mark.gpu


def _filled(abi, n, seed):
    """n doubles on the device, tiled from a 4 Mi-element seeded block."""
    block = np.random.default_rng(seed).standard_normal(1 << 22)
    src = abi.array(block)
    out = abi.empty(n)
    for off in range(0, n, 1 << 22):
        abi.mg_copy(out.offset(off), src.ptr, min(1 << 22, n - off))
    return out, block


def test_elementwise_and_sum_at_2_28(abi, fast):
    n = 1 << 28
    reps = n >> 22
    a, blk_a = _filled(abi, n, 1)
    b, blk_b = _filled(abi, n, 2)
    out, s = abi.empty(n), abi.empty(1)
    # sum of a tiled array = reps * sum(block), up to the reduction tolerance
    abi.mg_sum_all_fwd(a.ptr, s.ptr, n)
    sa = s.numpy()[0]
    scale = reps * np.abs(blk_a).sum()
    assert abs(sa - reps * fast.sum_longdouble(blk_a)) <= 1e-10 * scale
    # linearity: sum(a + b) = sum(a) + sum(b); sum(a - a) = 0 exactly; relu idempotent
    abi.mg_sum_all_fwd(b.ptr, s.ptr, n)
    sb = s.numpy()[0]
    abi.mg_binary_fwd(K.ADD, a.ptr, b.ptr, out.ptr, n)
    abi.mg_sum_all_fwd(out.ptr, s.ptr, n)
    assert abs(s.numpy()[0] - (sa + sb)) <= 1e-10 * (scale + reps * np.abs(blk_b).sum())
    abi.mg_binary_fwd(K.SUB, a.ptr, a.ptr, out.ptr, n)
    abi.mg_sum_all_fwd(out.ptr, s.ptr, n)
    assert s.numpy()[0] == 0.0
    abi.mg_unary_fwd(K.RELU, a.ptr, 0.0, out.ptr, n)
    abi.mg_unary_fwd(K.RELU, out.ptr, 0.0, b.ptr, n)          # b := relu(relu(a))
    abi.mg_binary_fwd(K.SUB, out.ptr, b.ptr, b.ptr, n)
    abi.mg_sum_all_fwd(b.ptr, s.ptr, n)
    assert s.numpy()[0] == 0.0
    # the last 4 Mi elements against the oracle, bit for bit
    tail = np.empty(1 << 22)
    abi.mg_download(tail.ctypes.data, out.offset(n - (1 << 22)), 1 << 22)
    assert np.array_equal(tail, fast.unary_fwd("relu", blk_a))
    # last-axis sum over 16384 x 16384: every row holds the same 16384-element slices
    rows = abi.empty(16384)
    abi.mg_sum_lastaxis_fwd(a.ptr, rows.ptr, 16384, 16384)
    got = rows.numpy()
    ref = fast.sum_lastaxis_fwd(blk_a.reshape(256, 16384))
    assert np.all(np.abs(got[:256] - ref) <= 1e-10 * np.abs(blk_a.reshape(256, 16384)).sum(axis=1))
    assert np.array_equal(got[:256], got[256:512])            # reproducible across identical rows


def test_matmul_8192_cubed(abi, fast):
    n = 8192
    rng = np.random.default_rng(3)
    A = rng.standard_normal((n, n)) / np.sqrt(n)
    dA = abi.array(A)
    eye = abi.array(np.eye(n))
    C = abi.empty(n * n)
    abi.mg_gemm_nn(dA.ptr, eye.ptr, C.ptr, n, n, n, 0, K.EPI_NONE, None)
    assert np.array_equal(C.numpy((n, n)), A)                 # A.I = A exactly
    del eye
    B = rng.standard_normal((n, n)) / np.sqrt(n)
    dB = abi.array(B)
    abi.mg_gemm_nn(dA.ptr, dB.ptr, C.ptr, n, n, n, 0, K.EPI_NONE, None)
    got = C.numpy((n, n))
    rows = rng.integers(0, n, 6)
    assert norm_err(got[rows], fast.matmul_fwd(A[rows], B)) <= 1e-10
    # gradients of loss = sum(C): dA = ones.Bt has identical rows = row sums of B
    ones = abi.array(np.ones(4 * n))                           # 4 rows of ones as a [4, n] G
    gA = abi.empty(4 * n)
    abi.mg_gemm_nt(ones.ptr, dB.ptr, gA.ptr, 4, n, n, 0, K.EPI_NONE, None)
    ref = B.sum(axis=1)
    assert np.all(np.abs(gA.numpy((4, n)) - ref[None, :]) <= 1e-10 * np.abs(B).sum(axis=1)[None, :])
    abi.mg_check_kernel_status()


def test_inference_one_million_inputs_sharded(api, fast):
    """Config 5: ids of the full 1,048,576-row batch equal the ids of its 8 row
    shards (what 8 GPUs compute), and the first 32768 rows equal the oracle's."""
    from test_gpu_mlp import build_mlp, forward
    rng = np.random.default_rng(5)
    sizes = [784, 128, 64, 10]
    params = [(rng.standard_normal((i, o)) / np.sqrt(i), np.zeros(o)) for i, o in zip(sizes[:-1], sizes[1:])]
    layers = build_mlp(api, params)
    total, shard = 1 << 20, 1 << 17
    block = rng.random((shard, 784))
    ids = np.empty(total, dtype=np.int32)
    full = []
    for s in range(total // shard):                           # 8 shards of 131072 rows
        xs = block + 1e-3 * s                                 # distinct inputs per shard
        x = api.Tensor([shard, 784], xs)
        x.set_requires_grad(False)
        ids[s * shard:(s + 1) * shard] = api.argmax_rows(forward(api, layers, x, True))
        full.append(xs if s < 2 else None)
    # two shards at once (a different tiling of the same rows) give the same ids
    x2 = api.Tensor([2 * shard, 784], np.concatenate(full[:2]))
    x2.set_requires_grad(False)
    assert np.array_equal(api.argmax_rows(forward(api, layers, x2, True)), ids[:2 * shard])
    logits, _ = fast.mlp_forward(params, full[0][:32768])
    assert np.array_equal(ids[:32768], fast.argmax_rows(logits))
    assert ids.min() >= 0 and ids.max() <= 9


def test_bounded_waits_report_timeouts_without_touching_the_gpu(abi):
    """Failure detection is host-side: a wait with a deadline returns
    MG_ERR_TIMEOUT while the device is still busy, and MG_OK once it is done."""
    import ctypes as C
    n = 4096
    a, b, c = abi.zeros(n * n), abi.zeros(n * n), abi.empty(n * n)
    ev = C.c_int()
    abi.mg_event_create(C.byref(ev))
    for _ in range(20):                                       # ~80 ms of queued work
        abi.mg_gemm_nn(a.ptr, b.ptr, c.ptr, n, n, n, 0, K.EPI_NONE, None)
    abi.mg_event_record(ev.value)
    with pytest.raises(K.MgError) as e:
        abi.mg_event_wait_bounded(ev.value, 0.001)
    assert e.value.code == K.ERR_TIMEOUT
    abi.mg_event_wait_bounded(ev.value, 30.0)                 # completes well inside the deadline
    abi.mg_comm_wait_bounded(1.0)                             # no communicator: comm stream is idle
    abi.mg_event_destroy(ev.value)
    abi.mg_check_kernel_status()
