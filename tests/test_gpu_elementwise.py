"""GPU parity: elementwise forward/backward kernels, through the device C ABI,
against the CPU oracle on identical seeded inputs.

Tolerances (the stated parity bar): rel err <= 1e-12 for elementwise ops.  add,
sub, mul, div, relu, the scalar forms, their gradients, fill and the SGD update
use only correctly rounded IEEE operations with no FMA contraction on either
side, so for those the comparison is bit-exact.
"""
import numpy as np
import pytest

from conftest import rel_err
from micrograd_b200 import cabi as K

pytestmark = pytest.mark.gpu

SIZES = [1, 2, 3, 255, 257, 1000, 65537, 1 << 20]
EXACT_UNARY = {"add": K.SADD, "sub": K.SSUB, "mul": K.SMUL, "div": K.SDIV, "relu": K.RELU}
LIBM_UNARY = {"pow": K.POW, "sigmoid": K.SIGMOID, "tanh": K.TANH, "exp": K.EXP}
TOL = 1e-12


def _inputs(n, seed):
    rng = np.random.default_rng(seed)
    a = rng.standard_normal(n)
    b = rng.standard_normal(n)
    b = np.where(np.abs(b) < 0.1, 0.5, b)  # divisors away from zero
    return a, b, rng.standard_normal(n), rng.standard_normal(n), rng.standard_normal(n)


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
def test_binary_forward_backward_bit_exact(abi, fast, op, n):
    a, b, g, ga0, gb0 = _inputs(n, n)
    code = {"add": K.ADD, "sub": K.SUB, "mul": K.MUL, "div": K.DIV}[op]
    da, db, dg = abi.array(a), abi.array(b), abi.array(g)
    out = abi.empty(n)
    abi.mg_binary_fwd(code, da.ptr, db.ptr, out.ptr, n)
    assert np.array_equal(out.numpy(), fast.binary_fwd(op, a, b))
    # accumulate into existing gradients
    dga, dgb = abi.array(ga0), abi.array(gb0)
    abi.mg_binary_bwd(code, da.ptr, db.ptr, dg.ptr, dga.ptr, dgb.ptr, n, 0)
    ga, gb = ga0.copy(), gb0.copy()
    fast.binary_bwd(op, a, b, g, ga, gb)
    assert np.array_equal(dga.numpy(), ga) and np.array_equal(dgb.numpy(), gb)
    # "known zero" destinations: stored, same values as accumulating into zeros
    sga, sgb = abi.empty(n), abi.empty(n)
    abi.mg_binary_bwd(code, da.ptr, db.ptr, dg.ptr, sga.ptr, sgb.ptr, n, K.ACC_STORE_A | K.ACC_STORE_B)
    za, zb = np.zeros(n), np.zeros(n)
    fast.binary_bwd(op, a, b, g, za, zb)
    assert np.array_equal(sga.numpy(), za) and np.array_equal(sgb.numpy(), zb)


@pytest.mark.parametrize("op", ["add", "mul", "div"])
def test_binary_backward_same_tensor_and_skipped_side(abi, fast, op):
    n = 4099
    a, _, g, ga0, _ = _inputs(n, 7)
    a = np.where(np.abs(a) < 0.1, 0.5, a)
    code = {"add": K.ADD, "mul": K.MUL, "div": K.DIV}[op]
    da, dg, dga = abi.array(a), abi.array(g), abi.array(ga0)
    abi.mg_binary_bwd(code, da.ptr, da.ptr, dg.ptr, dga.ptr, dga.ptr, n, 0)  # x op x
    ref = ga0.copy()
    fast.binary_bwd(op, a, a, g, ref, ref)
    assert np.array_equal(dga.numpy(), ref)
    only_b = abi.array(ga0)
    abi.mg_binary_bwd(code, da.ptr, da.ptr, dg.ptr, None, only_b.ptr, n, 0)  # first side skipped
    ra, rb = np.zeros(n), ga0.copy()
    fast.binary_bwd(op, a, a, g, ra, rb)
    assert np.array_equal(only_b.numpy(), rb)


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("op", list(EXACT_UNARY) + list(LIBM_UNARY))
def test_unary_forward_backward(abi, fast, op, n):
    a, _, g, ga0, _ = _inputs(n, 100 + n)
    s = 1.75
    if op == "pow":
        a, s = np.abs(a) + 0.5, 2.5
    if op == "exp":
        a = np.clip(a, -5, 5)
    code = {**EXACT_UNARY, **LIBM_UNARY}[op]
    if op in ("add", "sub", "mul", "div", "pow"):
        ref_out = fast.scalar_fwd(op, a, s)
    else:
        ref_out = fast.unary_fwd(op, a)
    da, dg, out = abi.array(a), abi.array(g), abi.empty(n)
    abi.mg_unary_fwd(code, da.ptr, s, out.ptr, n)
    got = out.numpy()
    ref_g = ga0.copy()
    if op in ("add", "sub", "mul", "div", "pow"):
        fast.scalar_bwd(op, a, s, g, ref_g)
    else:
        fast.unary_bwd(op, a, ref_out, g, ref_g)
    dga = abi.array(ga0)
    # backward consumes the DEVICE forward output, as the Tensor layer does
    abi.mg_unary_bwd(code, da.ptr, out.ptr, s, dg.ptr, dga.ptr, n, 0)
    if op in EXACT_UNARY:
        assert np.array_equal(got, ref_out)
        assert np.array_equal(dga.numpy(), ref_g)
    else:
        assert rel_err(got, ref_out) <= TOL
        # accumulated gradient: error relative to the two terms of the sum
        scale = np.abs(ga0) + np.abs(ref_g - ga0)
        assert np.all(np.abs(dga.numpy() - ref_g) <= TOL * scale + 1e-300)
        st = abi.empty(n)
        abi.mg_unary_bwd(code, da.ptr, out.ptr, s, dg.ptr, st.ptr, n, K.ACC_STORE_A)
        z = np.zeros(n)
        if op == "pow":
            fast.scalar_bwd(op, a, s, g, z)
        else:
            fast.unary_bwd(op, a, ref_out, g, z)
        assert rel_err(st.numpy(), z) <= 1e-11


def test_relu_edge_values(abi):
    x = np.array([0.0, -0.0, np.nan, np.inf, -np.inf, 1e-320, -1e-320, 3.0])
    dx, out = abi.array(x), abi.empty(x.size)
    abi.mg_unary_fwd(K.RELU, dx.ptr, 0.0, out.ptr, x.size)
    got = out.numpy()
    expect = np.array([0.0, 0.0, 0.0, np.inf, 0.0, 1e-320, 0.0, 3.0])  # x > 0 ? x : 0
    assert np.array_equal(got, expect) and not np.signbit(got[1])


def test_tanh_edge_values_and_ulp_bound(abi):
    """The device tanh is a single-path expm1 form: signed zeros, subnormals,
    saturation, infinities and NaN behave like std::tanh, and over a wide range of
    magnitudes the result stays within 4 units in the last place of libm's."""
    x = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1e-320, -1e-320, 5e-324,
                  19.0, -19.5, 20.0, 25.0, 1e300, -1e300, 0.5493061443340549, -0.17328679513998632])
    dx, out = abi.array(x), abi.empty(x.size)
    abi.mg_unary_fwd(K.TANH, dx.ptr, 0.0, out.ptr, x.size)
    got, ref = out.numpy(), np.tanh(x)
    assert np.isnan(got[4])
    assert np.array_equal(np.signbit(got), np.signbit(ref))
    assert np.array_equal(got[:4], ref[:4]) and np.array_equal(got[5:8], ref[5:8])
    finite = ~np.isnan(ref)
    assert np.all(np.abs(got[finite] - ref[finite]) <= 4 * np.spacing(np.abs(ref[finite])))

    rng = np.random.default_rng(77)
    n = 1 << 18
    mags = np.concatenate([rng.standard_normal(n), rng.uniform(-22, 22, n),
                           np.ldexp(rng.uniform(0.5, 1.0, n), -rng.integers(0, 1074, n))
                           * rng.choice([-1.0, 1.0], n)])
    dm, om = abi.array(mags), abi.empty(mags.size)
    abi.mg_unary_fwd(K.TANH, dm.ptr, 0.0, om.ptr, mags.size)
    got, ref = om.numpy(), np.tanh(mags)
    assert np.all(np.abs(got - ref) <= 4 * np.spacing(np.abs(ref)))
    assert np.all(np.abs(got) <= 1.0)


def test_unaligned_pointers_take_scalar_path(abi, fast):
    """Buffers that start 8 bytes off a 16-byte boundary (slices of a larger
    allocation) must give the same bits as aligned ones."""
    n = 1001
    a, b, g, _, _ = _inputs(n + 1, 5)
    da, db, out = abi.array(a), abi.array(b), abi.empty(n + 1)
    abi.mg_binary_fwd(K.MUL, da.offset(1), db.offset(1), out.offset(1), n)
    assert np.array_equal(out.numpy()[1:], fast.binary_fwd("mul", a[1:], b[1:]))
    abi.mg_unary_fwd(K.RELU, da.offset(1), 0.0, out.offset(1), n)
    assert np.array_equal(out.numpy()[1:], fast.unary_fwd("relu", a[1:]))


def test_empty_inputs_are_no_ops(abi):
    abi.mg_binary_fwd(K.ADD, None, None, None, 0)
    abi.mg_unary_fwd(K.RELU, None, 0.0, None, 0)
    abi.mg_fill(None, 1.0, 0)
    abi.mg_sgd_step(None, None, 0.1, 0)
    abi.mg_sync()


def test_invalid_arguments_fail_loudly(abi):
    x = abi.zeros(4)
    with pytest.raises(K.MgError) as e:
        abi.mg_binary_fwd(99, x.ptr, x.ptr, x.ptr, 4)
    assert e.value.code == K.ERR_INVALID and "unknown binary op" in str(e.value)
    with pytest.raises(K.MgError):
        abi.mg_unary_fwd(K.RELU, None, 0.0, x.ptr, 4)


@pytest.mark.parametrize("n", [1, 7, 4096, 109386, 1863690])
def test_sgd_step_and_fill_bit_exact(abi, fast, n):
    rng = np.random.default_rng(n)
    p, g = rng.standard_normal(n), rng.standard_normal(n)
    dp, dg = abi.array(p), abi.array(g)
    abi.mg_sgd_step(dp.ptr, dg.ptr, 0.01, n)
    ref = p.copy()
    fast.sgd_step(ref, g, 0.01)
    assert np.array_equal(dp.numpy(), ref)
    abi.mg_fill(dp.ptr, 1.0, n)
    assert np.array_equal(dp.numpy(), np.ones(n))
    abi.mg_fill(dp.ptr, 0.0, n)
    assert not dp.numpy().any()


@pytest.mark.parametrize("sizes", [[1], [19600, 100, 1000, 10], [7, 0, 4097, 33, 2, 100352, 128, 8192, 64, 640, 10],
                                   [1863690]])
def test_multi_tensor_sgd_step_bit_exact(abi, fast, sizes):
    """One launch per eight parameter tensors; p - (lr*g) with the product rounded
    first, bit for bit like the per-tensor form (slices at odd 8-byte offsets and
    empty tensors included)."""
    import ctypes as C
    rng = np.random.default_rng(len(sizes) * 100 + sizes[0])
    total = sum(sizes) + len(sizes)
    p, g = rng.standard_normal(total), rng.standard_normal(total)
    dp, dg = abi.array(p), abi.array(g)
    offs, o = [], 0
    for i, n in enumerate(sizes):
        offs.append(o)
        o += n + (i % 2)                      # every other tensor starts 8 bytes off a 16-byte boundary
    P = (C.c_void_p * len(sizes))(*[dp.offset(a) for a in offs])
    G = (C.c_void_p * len(sizes))(*[dg.offset(a) for a in offs])
    S = (C.c_size_t * len(sizes))(*sizes)
    abi.mg_sgd_step_multi(P, G, S, len(sizes), 0.01)
    ref = p.copy()
    for a, n in zip(offs, sizes):
        fast.sgd_step(ref[a:a + n], g[a:a + n], 0.01)
    assert np.array_equal(dp.numpy(), ref)


def test_scalar_mirror_returns_the_value_at_enqueue_time(abi):
    """A mirrored scalar is read back without waiting for later work, keeps the
    value it had when the mirror was enqueued, and its ticket expires once the
    256-slot ring has gone round."""
    import ctypes as C
    x = abi.array(np.array([3.25]))
    t = C.c_ulonglong()
    abi.mg_scalar_mirror(x.ptr, C.byref(t))
    abi.mg_fill(x.ptr, 7.0, 1)                              # later write: not seen by the mirror
    big = abi.empty(1 << 24)
    abi.mg_fill(big.ptr, 1.0, 1 << 24)                      # later work the fetch does not wait for
    v, expired = C.c_double(), C.c_int()
    abi.mg_scalar_fetch(t.value, C.byref(v), C.byref(expired))
    assert expired.value == 0 and v.value == 3.25
    assert x.numpy()[0] == 7.0
    first = t.value
    for i in range(256):
        abi.mg_scalar_mirror(x.ptr, C.byref(t))
    abi.mg_scalar_fetch(first, C.byref(v), C.byref(expired))
    assert expired.value == 1
    abi.mg_scalar_fetch(t.value, C.byref(v), C.byref(expired))
    assert expired.value == 0 and v.value == 7.0
    abi.mg_scalar_fetch(0, C.byref(v), C.byref(expired))
    assert expired.value == 1


@pytest.mark.parametrize("M,N", [(1, 1), (3, 5), (32, 10), (257, 128), (1024, 1024), (4099, 33)])
def test_add_row_forward(abi, fast, M, N):
    rng = np.random.default_rng(M * 131 + N)
    x, r = rng.standard_normal((M, N)), rng.standard_normal(N)
    dx, dr, out = abi.array(x), abi.array(r), abi.empty(M * N)
    abi.mg_add_row_fwd(dx.ptr, dr.ptr, out.ptr, M, N)
    assert np.array_equal(out.numpy((M, N)), fast.add_row_fwd(x, r))


def test_elementwise_full_size_properties(abi):
    """2^24 elements (a benchmark sweep size): linearity and idempotence properties
    that need no CPU pass over the data: (a+b)-b == a within one rounding,
    relu(relu(x)) == relu(x) exactly, and x*1 == x exactly."""
    n = 1 << 24
    rng = np.random.default_rng(0)
    a = rng.standard_normal(n)
    da = abi.array(a)
    t1, t2 = abi.empty(n), abi.empty(n)
    abi.mg_unary_fwd(K.RELU, da.ptr, 0.0, t1.ptr, n)
    abi.mg_unary_fwd(K.RELU, t1.ptr, 0.0, t2.ptr, n)
    r1 = t1.numpy()
    assert np.array_equal(r1, t2.numpy()) and np.array_equal(r1, np.maximum(a, 0.0))
    abi.mg_unary_fwd(K.SMUL, da.ptr, 1.0, t1.ptr, n)
    assert np.array_equal(t1.numpy(), a)
    abi.mg_binary_fwd(K.ADD, da.ptr, t2.ptr, t1.ptr, n)
    abi.mg_binary_fwd(K.SUB, t1.ptr, t2.ptr, t1.ptr, n)
    assert np.max(np.abs(t1.numpy() - a)) <= 2 ** -50 * 8
