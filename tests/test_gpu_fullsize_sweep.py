"""GPU parity at the benchmark's full sweep sizes: every config-2 op, forward AND
backward (accumulating into non-zero gradients), at 2^24 and 2^28 elements,
and both matmul gradient products at 4096^3 and 8192^3.

Device arrays of n elements are tiled from seeded 4 Mi-element blocks, so the
CPU oracle runs once on a block (seconds) and EVERY 4 Mi-element tile of the
device result is downloaded and compared with it: first tile, last tile and all
between, which covers the grid-stride tails and the large offsets (the last
tile of a 2^28 array ends at byte 2^31).  A ragged size (2^24 + 4099) runs
too, and one comparison window is laid across tile boundaries.

Bars: bit-exact for add / sub / mul / relu and all their gradients, for the
row-broadcast add and for the two sum gradients; rel err <= 1e-12 for tanh and
exp; <= 1e-10 of the natural bound (sum of |terms|) for sums and matmul.
"""
import ctypes as C

import numpy as np
import pytest

from conftest import rel_err
from micrograd_b200 import cabi as K

pytestmark = pytest.mark.gpu

BLOCK = 1 << 22
SIZES = [1 << 24, (1 << 24) + 4099, 1 << 28]
SQUARE = {1 << 24: 4096, 1 << 28: 16384}


class Tiled:
    """n doubles on the device holding `block` repeated (the last copy cut off)."""

    def __init__(self, abi, block, n):
        self.abi, self.block, self.n = abi, block, n
        src = abi.array(block)
        self.dev = abi.empty(n)
        for off in range(0, n, BLOCK):
            abi.mg_copy(self.dev.offset(off), src.ptr, min(BLOCK, n - off))

    @property
    def ptr(self):
        return self.dev.ptr


class Staging:
    """One pinned 32 MB host buffer; tiles are downloaded through it."""

    def __init__(self, abi):
        self.abi = abi
        self.raw = C.c_void_p()
        abi.mg_host_alloc(BLOCK * 8, C.byref(self.raw))
        self.view = np.ctypeslib.as_array(C.cast(self.raw.value, C.POINTER(C.c_double)), shape=(BLOCK,))

    def tile(self, dev, first, count):
        self.abi.mg_download(self.raw.value, dev.offset(first), count)
        return self.view[:count]

    def close(self):
        self.abi.mg_host_free(self.raw.value)


@pytest.fixture(scope="module")
def staging(abi):
    s = Staging(abi)
    yield s
    s.close()


def _tiles(n):
    return [(off, min(BLOCK, n - off)) for off in range(0, n, BLOCK)]


def assert_tiles_equal(staging, dev, n, ref_block, what):
    """Every tile of the device array equals the oracle's block, bit for bit."""
    for off, cnt in _tiles(n):
        got = staging.tile(dev, off, cnt)
        if not np.array_equal(got, ref_block[:cnt]):
            bad = np.flatnonzero(got != ref_block[:cnt])
            raise AssertionError(f"{what}: {bad.size} elements differ in the tile at {off}, "
                                 f"first at element {off + int(bad[0])}")
    # one window across tile boundaries (starts mid-tile, odd offset)
    if n >= 3 * BLOCK:
        start = n // 2 - BLOCK // 2 + 1
        got = staging.tile(dev, start, BLOCK)
        ref = np.roll(ref_block, -(start % BLOCK))
        assert np.array_equal(got, ref), f"{what}: window at {start} differs"


def assert_tiles_close(staging, dev, n, ref_block, tol, what):
    """Tile 0 within `tol` of the oracle (relative, per element); every other
    tile bit-identical to tile 0 (same inputs, same instruction sequence)."""
    first = staging.tile(dev, 0, min(BLOCK, n)).copy()
    err = rel_err(first, ref_block[:first.size])
    assert err <= tol, f"{what}: rel err {err:.3e}"
    assert_tiles_equal(staging, dev, n, np.resize(first, BLOCK) if first.size < BLOCK else first, what)


def _blocks(seed, count):
    rng = np.random.default_rng(seed)
    return [rng.standard_normal(BLOCK) for _ in range(count)]


@pytest.mark.parametrize("n", SIZES)
def test_binary_ops_forward_backward(abi, fast, staging, n):
    """add, sub, mul (src/ops/Arithmetic.cpp:9-102 of the reference)."""
    ba, bb, bg, bga, bgb = _blocks(n % 1000 + 1, 5)
    a, b, g = Tiled(abi, ba, n), Tiled(abi, bb, n), Tiled(abi, bg, n)
    out = abi.empty(n)
    for op, code in (("add", K.ADD), ("sub", K.SUB), ("mul", K.MUL)):
        abi.mg_binary_fwd(code, a.ptr, b.ptr, out.ptr, n)
        assert_tiles_equal(staging, out, n, fast.binary_fwd(op, ba, bb), f"{op} fwd n={n}")
    del out
    for op, code in (("add", K.ADD), ("sub", K.SUB), ("mul", K.MUL)):
        ga, gb = Tiled(abi, bga, n), Tiled(abi, bgb, n)
        abi.mg_binary_bwd(code, a.ptr, b.ptr, g.ptr, ga.ptr, gb.ptr, n, 0)
        ra, rb = bga.copy(), bgb.copy()
        fast.binary_bwd(op, ba, bb, bg, ra, rb)
        assert_tiles_equal(staging, ga.dev, n, ra, f"{op} bwd ga n={n}")
        assert_tiles_equal(staging, gb.dev, n, rb, f"{op} bwd gb n={n}")
        del ga, gb
    abi.mg_check_kernel_status()


@pytest.mark.parametrize("n", SIZES)
def test_unary_ops_forward_backward(abi, fast, staging, n):
    """relu, tanh, exp (src/ops/Activations.cpp:8-88; exp has no reference form)."""
    bx, bg, bgx = _blocks(n % 1000 + 2, 3)
    bclip = np.clip(bx, -5.0, 5.0)
    g = Tiled(abi, bg, n)
    out = abi.empty(n)
    for op, code, src, tol in (("relu", K.RELU, bx, 0.0), ("tanh", K.TANH, bx, 1e-12),
                               ("exp", K.EXP, bclip, 1e-12)):
        x = Tiled(abi, src, n)
        abi.mg_unary_fwd(code, x.ptr, 0.0, out.ptr, n)
        ref = fast.unary_fwd(op, src)
        if tol == 0.0:
            assert_tiles_equal(staging, out, n, ref, f"{op} fwd n={n}")
        else:
            assert_tiles_close(staging, out, n, ref, tol, f"{op} fwd n={n}")
        # backward from the device's own forward output, into a non-zero gradient
        y_block = staging.tile(out, 0, min(BLOCK, n)).copy()
        y_block = np.resize(y_block, BLOCK) if n < BLOCK else y_block
        gx = Tiled(abi, bgx, n)
        abi.mg_unary_bwd(code, x.ptr, out.ptr, 0.0, g.ptr, gx.ptr, n, 0)
        rg = bgx.copy()
        fast.unary_bwd(op, src, y_block, bg, rg)
        assert_tiles_equal(staging, gx.dev, n, rg, f"{op} bwd n={n}")
        del x, gx
    abi.mg_check_kernel_status()


@pytest.mark.parametrize("n", [1 << 24, 1 << 28])
def test_row_broadcast_forward_backward(abi, fast, staging, n):
    """[M,N] + [N] and its gradients at 4096^2 / 16384^2: gx += g bit-exact, the
    row gradient (column sums over all M rows) against the exact sum."""
    side = SQUARE[n]
    rows_per_block = BLOCK // side
    bx, bg, bgx = _blocks(n % 1000 + 3, 3)
    rng = np.random.default_rng(5)
    row, grow0 = rng.standard_normal(side), rng.standard_normal(side)
    x, g = Tiled(abi, bx, n), Tiled(abi, bg, n)
    drow, out = abi.array(row), abi.empty(n)
    abi.mg_add_row_fwd(x.ptr, drow.ptr, out.ptr, side, side)
    ref = fast.add_row_fwd(bx.reshape(rows_per_block, side), row).reshape(-1)
    assert_tiles_equal(staging, out, n, ref, f"add_row fwd {side}^2")
    del out
    gx, dgrow = Tiled(abi, bgx, n), abi.array(grow0)
    abi.mg_add_row_bwd(g.ptr, gx.ptr, dgrow.ptr, side, side, 0)
    assert_tiles_equal(staging, gx.dev, n, bgx + bg, f"add_row bwd gx {side}^2")
    reps = n // BLOCK
    g2 = bg.reshape(rows_per_block, side).astype(np.longdouble)
    exact = (reps * g2.sum(axis=0)).astype(np.float64) + grow0
    bound = reps * np.abs(bg.reshape(rows_per_block, side)).sum(axis=0) + np.abs(grow0)
    got = dgrow.numpy()
    assert np.all(np.abs(got - exact) <= 1e-10 * bound)
    # the oracle's own ascending-row loop on the first 4 Mi-element slab agrees too
    few = abi.array(grow0)
    abi.mg_add_row_bwd(g.ptr, None, few.ptr, rows_per_block, side, 0)
    rr = grow0.copy()
    fast.add_row_bwd(bg.reshape(rows_per_block, side), None, rr)
    assert np.all(np.abs(few.numpy() - rr) <= 1e-10 * bound)
    abi.mg_check_kernel_status()


@pytest.mark.parametrize("n", SIZES)
def test_full_sum_forward_backward(abi, fast, staging, n):
    """sum() and its gradient broadcast (src/ops/Reduction.cpp:17-30)."""
    bx, bgx = _blocks(n % 1000 + 4, 2)
    x = Tiled(abi, bx, n)
    s = abi.empty(1)
    abi.mg_sum_all_fwd(x.ptr, s.ptr, n)
    full, rest = divmod(n, BLOCK)
    exact = full * fast.sum_longdouble(bx) + fast.sum_longdouble(bx[:rest])
    scale = full * np.abs(bx).sum() + np.abs(bx[:rest]).sum()
    got = s.numpy()[0]
    assert abs(got - exact) <= 1e-10 * scale
    if n <= (1 << 25):                      # the reference's own left-to-right loop, in full
        host = np.resize(bx, n)
        assert abs(got - fast.sum(host)) <= 1e-10 * scale
    gx, g0 = Tiled(abi, bgx, n), abi.array([0.37])
    abi.mg_sum_all_bwd(g0.ptr, gx.ptr, n, 0)
    ref = bgx.copy()
    fast.sum_bwd(0.37, ref)
    assert_tiles_equal(staging, gx.dev, n, ref, f"sum bwd n={n}")
    abi.mg_check_kernel_status()


@pytest.mark.parametrize("n", [1 << 24, 1 << 28])
def test_last_axis_sum_forward_backward(abi, fast, staging, n):
    side = SQUARE[n]
    rows_per_block = BLOCK // side
    bx, bgx = _blocks(n % 1000 + 5, 2)
    x = Tiled(abi, bx, n)
    out = abi.empty(side)
    abi.mg_sum_lastaxis_fwd(x.ptr, out.ptr, side, side)
    ref = fast.sum_lastaxis_fwd(bx.reshape(rows_per_block, side))
    bound = np.abs(bx.reshape(rows_per_block, side)).sum(axis=1)
    got = out.numpy().reshape(-1, rows_per_block)
    assert np.all(np.abs(got - ref[None, :]) <= 1e-10 * bound[None, :])
    assert np.all(got == got[0][None, :])           # identical rows give identical sums
    # backward: gx[i, j] += g[i] with a different g for every row, bit-exact
    gvec = np.random.default_rng(6).standard_normal(side)
    gx, dg = Tiled(abi, bgx, n), abi.array(gvec)
    abi.mg_sum_lastaxis_bwd(dg.ptr, gx.ptr, side, side, 0)
    for t, (off, cnt) in enumerate(_tiles(n)):
        want = bgx.reshape(rows_per_block, side).copy()
        fast.sum_lastaxis_bwd(gvec[t * rows_per_block:(t + 1) * rows_per_block], want)
        assert np.array_equal(staging.tile(gx.dev, off, cnt), want.reshape(-1)), f"tile {t}"
    abi.mg_check_kernel_status()


@pytest.mark.parametrize("n", [4096, 8192])
def test_matmul_gradients_square(abi, fast, n):
    """dA += G.B^T and dB += A^T.G (src/ops/Matmul.cpp:44-58) at 4096^3 / 8192^3 with a
    random G and non-zero initial gradients; 12 rows of dA and 12 rows of dB
    against the oracle's loops (each needs only a slice of the operands)."""
    rng = np.random.default_rng(n)
    A = rng.standard_normal((n, n)) / np.sqrt(n)
    B = rng.standard_normal((n, n)) / np.sqrt(n)
    G = rng.standard_normal((n, n))
    gA0 = rng.standard_normal((n, n))
    gB0 = rng.standard_normal((n, n))
    dA, dB, dG = abi.array(A), abi.array(B), abi.array(G)
    dgA, dgB = abi.array(gA0), abi.array(gB0)
    abi.mg_gemm_nt(dG.ptr, dB.ptr, dgA.ptr, n, n, n, 1, K.EPI_NONE, None)
    abi.mg_gemm_tn(dA.ptr, dG.ptr, dgB.ptr, n, n, n, 1)
    abi.mg_check_kernel_status()
    gotA, gotB = dgA.numpy((n, n)), dgB.numpy((n, n))
    rows = np.unique(np.concatenate([[0, n - 1, 127, 128], rng.integers(0, n, 8)]))
    # dA rows: only those rows of G (and all of B) enter
    refA = gA0[rows].copy()
    fast.matmul_bwd(A[rows], B, G[rows], refA, None)
    boundA = np.abs(G[rows]) @ np.abs(B).T + np.abs(gA0[rows])
    assert np.all(np.abs(gotA[rows] - refA) <= 1e-10 * boundA)
    assert np.abs(gotA[rows] - refA).max() <= 1e-10 * np.abs(refA).max()
    # dB rows k: column k of A (and all of G) enter
    Asub = np.ascontiguousarray(A[:, rows])
    refB = gB0[rows].copy()
    fast.matmul_bwd(Asub, np.ascontiguousarray(B[rows]), G, None, refB)
    boundB = np.abs(Asub).T @ np.abs(G) + np.abs(gB0[rows])
    assert np.all(np.abs(gotB[rows] - refB) <= 1e-10 * boundB)
    assert np.abs(gotB[rows] - refB).max() <= 1e-10 * np.abs(refB).max()
    # rows the oracle did not visit: a second run reproduces them bit for bit, and
    # the stored (beta = 0) form plus the old gradient agrees within rounding
    dgB2 = abi.array(gB0)
    abi.mg_gemm_tn(dA.ptr, dG.ptr, dgB2.ptr, n, n, n, 1)
    assert np.array_equal(dgB2.numpy((n, n)), gotB)
    fresh = abi.empty(n * n)
    abi.mg_gemm_nt(dG.ptr, dB.ptr, fresh.ptr, n, n, n, 0, K.EPI_NONE, None)
    diff = np.abs(fresh.numpy((n, n)) + gA0 - gotA).max()
    assert diff <= 1e-10 * np.abs(gotA).max()
