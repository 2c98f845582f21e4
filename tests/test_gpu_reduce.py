"""GPU parity: reductions, row broadcast gradients, softmax cross-entropy and
argmax through the device C ABI against the CPU oracle.

Tolerance (the stated parity bar): rel err <= 1e-10 for reductions.  Errors are
measured against the natural scale of the sum (sum of |x|), because the
reference's own left-to-right sum carries a rounding error of that order: with
cancellation |sum| can be far smaller than the error bound of either side.
"""
import numpy as np
import pytest

from conftest import norm_err, rel_err
from micrograd_b200 import cabi as K

pytestmark = pytest.mark.gpu
TOL = 1e-10


@pytest.mark.parametrize("n", [1, 2, 3, 255, 256, 257, 10000, 1 << 20, (1 << 22) + 3])
def test_sum_all(abi, fast, n):
    rng = np.random.default_rng(n)
    x = rng.standard_normal(n)
    dx, out = abi.array(x), abi.empty(1)
    abi.mg_sum_all_fwd(dx.ptr, out.ptr, n)
    got = out.numpy()[0]
    ref = fast.sum(x)
    scale = np.abs(x).sum()
    assert abs(got - ref) <= TOL * scale
    # the device tree sum should be at least as close to the long-double sum
    exact = fast.sum_longdouble(x)
    assert abs(got - exact) <= max(abs(ref - exact), 1e-15 * scale) * 4
    # run-to-run reproducible
    abi.mg_sum_all_fwd(dx.ptr, out.ptr, n)
    assert out.numpy()[0] == got


def test_sum_all_known_answers_and_edges(abi):
    out = abi.empty(1)
    ramp = abi.array(np.arange(1, 10001, dtype=np.float64))
    abi.mg_sum_all_fwd(ramp.ptr, out.ptr, 10000)
    assert out.numpy()[0] == 50005000.0          # reference test: sum 1..10000
    four = abi.array([1.0, 2.0, 3.0, 4.0])
    abi.mg_sum_all_fwd(four.ptr, out.ptr, 4)
    assert out.numpy()[0] == 10.0
    abi.mg_sum_all_fwd(None, out.ptr, 0)          # empty sum is 0.0
    assert out.numpy()[0] == 0.0
    odd = abi.array(np.arange(8, dtype=np.float64))
    abi.mg_sum_all_fwd(odd.offset(1), out.ptr, 7)  # unaligned start
    assert out.numpy()[0] == 28.0


@pytest.mark.parametrize("n", [1, 3, 1000, 65537])
def test_sum_all_backward_bit_exact(abi, fast, n):
    rng = np.random.default_rng(n)
    g0 = rng.standard_normal(n)
    gs = 0.37
    dg, dgx = abi.array([gs]), abi.array(g0)
    abi.mg_sum_all_bwd(dg.ptr, dgx.ptr, n, 0)
    ref = g0.copy()
    fast.sum_bwd(gs, ref)
    assert np.array_equal(dgx.numpy(), ref)
    abi.mg_sum_all_bwd(dg.ptr, dgx.ptr, n, K.ACC_STORE_A)
    assert np.array_equal(dgx.numpy(), np.full(n, gs))


@pytest.mark.parametrize("M,N", [(1, 1), (3, 5), (7, 10), (64, 64), (257, 33), (1024, 1024), (5, 16384)])
def test_sum_lastaxis(abi, fast, M, N):
    rng = np.random.default_rng(M * 7 + N)
    x = rng.standard_normal((M, N))
    dx, out = abi.array(x), abi.empty(M)
    abi.mg_sum_lastaxis_fwd(dx.ptr, out.ptr, M, N)
    ref = fast.sum_lastaxis_fwd(x)
    assert np.all(np.abs(out.numpy() - ref) <= TOL * np.abs(x).sum(axis=1))
    g, g0 = rng.standard_normal(M), rng.standard_normal((M, N))
    dg, dgx = abi.array(g), abi.array(g0)
    abi.mg_sum_lastaxis_bwd(dg.ptr, dgx.ptr, M, N, 0)
    refg = g0.copy()
    fast.sum_lastaxis_bwd(g, refg)
    assert np.array_equal(dgx.numpy((M, N)), refg)
    abi.mg_sum_lastaxis_bwd(dg.ptr, dgx.ptr, M, N, K.ACC_STORE_A)
    assert np.array_equal(dgx.numpy((M, N)), np.repeat(g[:, None], N, axis=1))


@pytest.mark.parametrize("M,N", [(1, 1), (1, 11), (1, 100), (3, 5), (32, 10), (257, 128), (1000, 33),
                                 (4096, 1024), (65536, 10)])
def test_add_row_backward(abi, fast, M, N):
    rng = np.random.default_rng(M + 17 * N)
    g = rng.standard_normal((M, N))
    gx0, gr0 = rng.standard_normal((M, N)), rng.standard_normal(N)
    dg, dgx, dgr = abi.array(g), abi.array(gx0), abi.array(gr0)
    abi.mg_add_row_bwd(dg.ptr, dgx.ptr, dgr.ptr, M, N, 0)
    rx, rr = gx0.copy(), gr0.copy()
    fast.add_row_bwd(g, rx, rr)
    assert np.array_equal(dgx.numpy((M, N)), rx)               # pass-through is exact
    assert np.all(np.abs(dgr.numpy() - rr) <= TOL * (np.abs(g).sum(axis=0) + np.abs(gr0)))
    # bias-gradient form: column sums only, stored
    abi.mg_add_row_bwd(dg.ptr, None, dgr.ptr, M, N, K.ACC_STORE_B)
    z = np.zeros(N)
    fast.add_row_bwd(g, None, z)
    assert np.all(np.abs(dgr.numpy() - z) <= TOL * np.abs(g).sum(axis=0))
    # pass-through only
    abi.mg_add_row_bwd(dg.ptr, dgx.ptr, None, M, N, K.ACC_STORE_A)
    assert np.array_equal(dgx.numpy((M, N)), g)


@pytest.mark.parametrize("M,C", [(1, 10), (32, 10), (1000, 10), (65536, 10), (64, 3), (17, 100)])
def test_softmax_cross_entropy(abi, fast, M, C):
    rng = np.random.default_rng(M * 3 + C)
    z = rng.standard_normal((M, C)) * 3.0
    y = rng.integers(0, C, M).astype(np.int32)
    dz, dy, loss = abi.array(z), abi.int_array(y), abi.empty(1)
    for denom in (float(M), float(4 * M)):       # own mean, and a shard of a larger batch
        abi.mg_softmax_xent_fwd(dz.ptr, dy.ptr, loss.ptr, M, C, denom)
        ref = fast.softmax_xent_fwd(z, y, denom)
        assert abs(loss.numpy()[0] - ref) <= TOL * abs(ref)
        g0 = rng.standard_normal((M, C))
        dg, dgl = abi.array(g0), abi.array([0.5])
        abi.mg_softmax_xent_bwd(dz.ptr, dy.ptr, dgl.ptr, dg.ptr, M, C, denom, 0)
        refg = g0.copy()
        fast.softmax_xent_bwd(z, y, refg, denom, 0.5)
        assert np.max(np.abs(dg.numpy((M, C)) - refg)) <= 1e-12 * max(1.0, np.abs(refg).max())
        abi.mg_softmax_xent_bwd(dz.ptr, dy.ptr, dgl.ptr, dg.ptr, M, C, denom, K.ACC_STORE_A)
        zg = np.zeros((M, C))
        fast.softmax_xent_bwd(z, y, zg, denom, 0.5)
        assert norm_err(dg.numpy((M, C)), zg) <= 1e-12
    abi.mg_check_kernel_status()


def test_softmax_cross_entropy_flags_bad_label(abi):
    z, y = abi.array(np.zeros((2, 3))), abi.int_array([0, 7])
    loss = abi.empty(1)
    abi.mg_softmax_xent_fwd(z.ptr, y.ptr, loss.ptr, 2, 3, 2.0)
    with pytest.raises(K.MgError) as e:
        abi.mg_check_kernel_status()
    assert e.value.code == K.ERR_KERNEL
    abi.mg_check_kernel_status()  # the fault word is cleared once reported


@pytest.mark.parametrize("M,N", [(1, 1), (5, 3), (1000, 10), (65536, 10), (33, 100), (127, 10), (128, 10),
                                 (129, 10), (300, 31), (1000, 32), (1000, 33), (7, 16), (100003, 7),
                                 (1 << 20, 10)])
def test_argmax_rows_bit_exact(abi, fast, M, N):
    rng = np.random.default_rng(M + N)
    x = rng.standard_normal((M, N))
    x[::3] = np.round(x[::3])                    # plenty of exact ties
    dx, out = abi.array(x), abi.int_array(np.zeros(M, dtype=np.int32))
    abi.mg_argmax_rows(dx.ptr, out.ptr, M, N)
    assert np.array_equal(out.numpy(), fast.argmax_rows(x))


def test_argmax_of_narrow_rows_follows_the_reference_loop_on_special_values(abi, fast):
    """Rows of at most 32 columns are walked left to right with `>` like the
    reference's prediction loop: ties and -0.0/+0.0 keep the lower index, a NaN
    never replaces the best so far, and a leading NaN is never replaced."""
    nan, inf = np.nan, np.inf
    rows = np.array([
        [0.0, -0.0, 0.0, -0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0],
        [-0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0],
        [nan, 1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0, 8.0, 9.0],
        [1.0, nan, 2.0, nan, 2.0, 0.0, 0.0, 0.0, 0.0, 0.0],
        [-inf, -inf, -inf, -inf, -inf, -inf, -inf, -inf, -inf, -inf],
        [-inf, -1e308, -inf, -1e308, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0],
        [1.0, 2.0, inf, inf, 3.0, 0.0, 0.0, 0.0, 0.0, 0.0],
        [5e-324, 0.0, 5e-324, 1e-323, 1e-323, 0.0, 0.0, 0.0, 0.0, 0.0],
        [3.0, 3.0, 3.0, 3.0, 3.0, 3.0, 3.0, 3.0, 3.0, np.nextafter(3.0, 4.0)],
    ])
    x = np.tile(rows, (40, 1))                        # 360 rows: three CTAs, a ragged last one
    want = fast.argmax_rows(x)
    assert list(want[:9]) == [0, 0, 0, 2, 0, 4, 2, 3, 9]
    dx, out = abi.array(x), abi.int_array(np.zeros(x.shape[0], dtype=np.int32))
    abi.mg_argmax_rows(dx.ptr, out.ptr, x.shape[0], 10)
    assert np.array_equal(out.numpy(), want)


def test_label_conversion(abi):
    y = np.array([0.0, 9.0, 3.0, 7.0])
    dy, out = abi.array(y), abi.int_array(np.zeros(4, dtype=np.int32))
    abi.mg_f64_to_i32(dy.ptr, out.ptr, 4)
    assert list(out.numpy()) == [0, 9, 3, 7]
