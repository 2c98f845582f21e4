"""GPU parity: matmul forward and both gradient products through the device C
ABI (mg_gemm_nn / _nt / _tn) against the CPU oracle.

Tolerance (the stated parity bar): rel err <= 1e-10 for matmul.  Element (i,j) is
compared against the natural bound of its dot product, sum_p |a_ip||b_pj|, and
normwise.  The tensor-core kernel uses fused multiply-adds and its own k order,
so it is not bit-identical to the reference's separately rounded ascending-p
sum — except on small-integer inputs, where every intermediate is exact and the
comparison IS bit-exact (this is what catches a wrong fragment layout).
"""
import numpy as np
import pytest

from conftest import golden, norm_err
from micrograd_b200 import cabi as K

pytestmark = pytest.mark.gpu
TOL = 1e-10

# (M, K, N): tiny, odd (fallback kernel), tile-exact, ragged edges, skinny, deep
SHAPES = [(1, 1, 1), (2, 2, 2), (5, 7, 4), (33, 17, 9), (32, 48, 16), (64, 64, 64), (128, 128, 128),
          (256, 256, 256), (200, 136, 72), (130, 18, 258), (1024, 256, 10), (512, 10, 512),
          (300, 784, 128), (96, 1040, 192), (784, 40, 256), (112, 16, 48), (1568, 64, 1024)]
PATHS = [1, 2]  # 1: plain tiled kernel, 2: tensor-core kernel whenever operands allow


def _bound(A, B):
    return np.abs(A) @ np.abs(B)


def _check(got, ref, bound, extra=0.0):
    assert np.all(np.abs(got - ref) <= TOL * (bound + extra) + 1e-300)
    assert norm_err(got, ref) <= TOL


@pytest.fixture(autouse=True)
def _restore_config(abi):
    yield
    abi.mg_gemm_config(0, -1)


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("M,Kd,N", SHAPES)
def test_forward_and_gradients(abi, fast, path, M, Kd, N):
    abi.mg_gemm_config(path, -1)
    rng = np.random.default_rng(M * 1000003 + Kd * 1009 + N)
    A = rng.standard_normal((M, Kd)) / np.sqrt(Kd)
    B = rng.standard_normal((Kd, N)) / np.sqrt(Kd)
    G = rng.standard_normal((M, N))
    gA0, gB0 = rng.standard_normal((M, Kd)), rng.standard_normal((Kd, N))
    dA, dB, dG = abi.array(A), abi.array(B), abi.array(G)
    C = abi.empty(M * N)
    abi.mg_gemm_nn(dA.ptr, dB.ptr, C.ptr, M, N, Kd, 0, K.EPI_NONE, None)
    _check(C.numpy((M, N)), fast.matmul_fwd(A, B), _bound(A, B))
    # gradients, accumulating into existing values (the reference's semantics)
    dgA, dgB = abi.array(gA0), abi.array(gB0)
    abi.mg_gemm_nt(dG.ptr, dB.ptr, dgA.ptr, M, N, Kd, 1, K.EPI_NONE, None)
    abi.mg_gemm_tn(dA.ptr, dG.ptr, dgB.ptr, M, N, Kd, 1)
    rA, rB = gA0.copy(), gB0.copy()
    fast.matmul_bwd(A, B, G, rA, rB)
    _check(dgA.numpy((M, Kd)), rA, _bound(G, B.T), np.abs(gA0))
    _check(dgB.numpy((Kd, N)), rB, _bound(A.T, G), np.abs(gB0))
    # store mode (destination known zero)
    abi.mg_gemm_nt(dG.ptr, dB.ptr, dgA.ptr, M, N, Kd, 0, K.EPI_NONE, None)
    abi.mg_gemm_tn(dA.ptr, dG.ptr, dgB.ptr, M, N, Kd, 0)
    zA, zB = np.zeros((M, Kd)), np.zeros((Kd, N))
    fast.matmul_bwd(A, B, G, zA, zB)
    _check(dgA.numpy((M, Kd)), zA, _bound(G, B.T))
    _check(dgB.numpy((Kd, N)), zB, _bound(A.T, G))
    abi.mg_check_kernel_status()


@pytest.mark.parametrize("shape_id", [0, 1, 2, 3])
@pytest.mark.parametrize("M,Kd,N", [(128, 128, 128), (200, 136, 72), (64, 784, 256)])
def test_integer_inputs_are_bit_exact_for_every_mma_shape(abi, fast, shape_id, M, Kd, N):
    """Small integers: all products and partial sums are exact in fp64, so any k
    order and FMA give the reference's bits.  Run for each mma.sync f64 shape."""
    abi.mg_gemm_config(2, shape_id)
    rng = np.random.default_rng(shape_id * 97 + M)
    A = rng.integers(-8, 9, (M, Kd)).astype(np.float64)
    B = rng.integers(-8, 9, (Kd, N)).astype(np.float64)
    G = rng.integers(-8, 9, (M, N)).astype(np.float64)
    dA, dB, dG = abi.array(A), abi.array(B), abi.array(G)
    C, gA, gB = abi.empty(M * N), abi.empty(M * Kd), abi.empty(Kd * N)
    abi.mg_gemm_nn(dA.ptr, dB.ptr, C.ptr, M, N, Kd, 0, K.EPI_NONE, None)
    abi.mg_gemm_nt(dG.ptr, dB.ptr, gA.ptr, M, N, Kd, 0, K.EPI_NONE, None)
    abi.mg_gemm_tn(dA.ptr, dG.ptr, gB.ptr, M, N, Kd, 0)
    abi.mg_check_kernel_status()
    assert np.array_equal(C.numpy((M, N)), fast.matmul_fwd(A, B))
    zA, zB = np.zeros((M, Kd)), np.zeros((Kd, N))
    fast.matmul_bwd(A, B, G, zA, zB)
    assert np.array_equal(gA.numpy((M, Kd)), zA)
    assert np.array_equal(gB.numpy((Kd, N)), zB)


@pytest.mark.parametrize("path", PATHS)
def test_golden_matmul_vectors(abi, path):
    """Vectors produced by the reference's own code (tests/golden)."""
    abi.mg_gemm_config(path, -1)
    g = golden("matmul_sum.npz")
    for tag in ("small", "odd", "even"):
        A, B, seed = g[f"{tag}_A"], g[f"{tag}_B"], g[f"{tag}_seed"]
        M, Kd = A.shape
        N = B.shape[1]
        dA, dB, dS = abi.array(A), abi.array(B), abi.array(seed)
        C = abi.empty(M * N)
        abi.mg_gemm_nn(dA.ptr, dB.ptr, C.ptr, M, N, Kd, 0, K.EPI_NONE, None)
        _check(C.numpy((M, N)), g[f"{tag}_C"], _bound(A, B))
        gA, gB = abi.array(g[f"{tag}_gA0"]), abi.array(g[f"{tag}_gB0"])
        abi.mg_gemm_nt(dS.ptr, dB.ptr, gA.ptr, M, N, Kd, 1, K.EPI_NONE, None)
        abi.mg_gemm_tn(dA.ptr, dS.ptr, gB.ptr, M, N, Kd, 1)
        _check(gA.numpy((M, Kd)), g[f"{tag}_gA"], _bound(seed, B.T), np.abs(g[f"{tag}_gA0"]))
        _check(gB.numpy((Kd, N)), g[f"{tag}_gB"], _bound(A.T, seed), np.abs(g[f"{tag}_gB0"]))


def test_reference_2x2_known_answer(abi):
    """test/tensor_test.cpp:142-172 / README example."""
    A, B = abi.array([1., 2., 3., 4.]), abi.array([5., 6., 7., 8.])
    ones = abi.array(np.ones(4))
    C, gA, gB = abi.empty(4), abi.empty(4), abi.empty(4)
    abi.mg_gemm_nn(A.ptr, B.ptr, C.ptr, 2, 2, 2, 0, K.EPI_NONE, None)
    abi.mg_gemm_nt(ones.ptr, B.ptr, gA.ptr, 2, 2, 2, 0, K.EPI_NONE, None)
    abi.mg_gemm_tn(A.ptr, ones.ptr, gB.ptr, 2, 2, 2, 0)
    assert list(C.numpy()) == [19., 22., 43., 50.]
    assert list(gA.numpy()) == [11., 15., 11., 15.]
    assert list(gB.numpy()) == [4., 4., 6., 6.]


@pytest.mark.parametrize("path", PATHS)
@pytest.mark.parametrize("M,Kd,N", [(32, 784, 128), (200, 136, 72), (7, 5, 3)])
def test_fused_epilogues(abi, fast, path, M, Kd, N):
    abi.mg_gemm_config(path, -1)
    rng = np.random.default_rng(M + Kd + N)
    A = rng.standard_normal((M, Kd)) / np.sqrt(Kd)
    B = rng.standard_normal((Kd, N)) / np.sqrt(Kd)
    bias = rng.standard_normal(N) * 0.1
    dA, dB, dbias = abi.array(A), abi.array(B), abi.array(bias)
    out = abi.empty(M * N)
    pre = fast.add_row_fwd(fast.matmul_fwd(A, B), bias)
    abi.mg_gemm_nn(dA.ptr, dB.ptr, out.ptr, M, N, Kd, 0, K.EPI_BIAS, dbias.ptr)
    _check(out.numpy((M, N)), pre, _bound(A, B), np.abs(bias)[None, :])
    abi.mg_gemm_nn(dA.ptr, dB.ptr, out.ptr, M, N, Kd, 0, K.EPI_BIAS_RELU, dbias.ptr)
    got = out.numpy((M, N))
    ref = fast.unary_fwd("relu", pre)
    safe = np.abs(pre) > 1e-9          # sign decided identically away from zero
    _check(got[safe], ref[safe], (_bound(A, B) + np.abs(bias)[None, :])[safe])
    assert np.all(got >= 0.0)
    # dA with the ReLU mask of a forward activation fused in
    G = rng.standard_normal((M, N))
    act = rng.standard_normal((M, Kd))
    dG, dact = abi.array(G), abi.array(act)
    g0 = rng.standard_normal((M, Kd))
    dg = abi.array(g0)
    abi.mg_gemm_nt(dG.ptr, dB.ptr, dg.ptr, M, N, Kd, 1, K.EPI_RELU_MASK, dact.ptr)
    full = np.zeros((M, Kd))
    fast.matmul_bwd(A, B, G, full, None)
    ref = g0.copy()
    fast.unary_bwd("relu", act, act, full, ref)
    _check(dg.numpy((M, Kd)), ref, _bound(G, B.T), np.abs(g0))
    abi.mg_check_kernel_status()


def test_split_contraction_is_reproducible_and_correct(abi, fast):
    """Weight-gradient shape: few output tiles, long contraction (the batch) —
    the kernel splits the contraction and folds partial tiles in a fixed order."""
    M, Kd, N = 8192, 256, 128
    rng = np.random.default_rng(42)
    A = rng.standard_normal((M, Kd))
    G = rng.standard_normal((M, N)) / np.sqrt(M)
    dA, dG = abi.array(A), abi.array(G)
    g0 = rng.standard_normal((Kd, N))
    out1, out2 = abi.array(g0), abi.array(g0)
    abi.mg_gemm_tn(dA.ptr, dG.ptr, out1.ptr, M, N, Kd, 1)
    abi.mg_gemm_tn(dA.ptr, dG.ptr, out2.ptr, M, N, Kd, 1)
    got = out1.numpy((Kd, N))
    assert np.array_equal(got, out2.numpy((Kd, N)))
    ref = g0.copy()
    fast.matmul_bwd(A, np.zeros((Kd, N)), G, None, ref)
    _check(got, ref, _bound(A.T, G), np.abs(g0))
    abi.mg_check_kernel_status()


@pytest.mark.parametrize("M,Kd,N", [(4096, 784, 200), (6000, 300, 136), (2048, 1024, 10),
                                     (8192, 200, 1000), (3000, 130, 258)])
def test_split_contraction_ragged_shapes_bit_exact_on_integers(abi, M, Kd, N):
    """Long contractions over few output tiles are cut into per-SM spans whose
    segments cross tile boundaries; partial tiles are packed and folded in k
    order.  Small-integer operands make every partial sum exact, so the result
    must equal the integer product bit for bit, including ragged borders, for the
    weight-gradient (A^T.G), forward (A.B) and input-gradient (G.B^T) layouts."""
    rng = np.random.default_rng(M + Kd + N)
    A = rng.integers(-3, 4, (M, Kd)).astype(np.float64)
    G = rng.integers(-3, 4, (M, N)).astype(np.float64)
    g0 = rng.integers(-5, 6, (Kd, N)).astype(np.float64)
    dA, dG, out = abi.array(A), abi.array(G), abi.array(g0)
    abi.mg_gemm_tn(dA.ptr, dG.ptr, out.ptr, M, N, Kd, 1)          # [Kd, N] += A^T.G, contraction M
    assert np.array_equal(out.numpy((Kd, N)), g0 + A.T @ G)
    # forward layout with the long axis as the contraction: [Kd, M].[M, N]
    At = np.ascontiguousarray(A.T)
    dAt, C = abi.array(At), abi.empty(Kd * N)
    abi.mg_gemm_nn(dAt.ptr, dG.ptr, C.ptr, Kd, N, M, 0, K.EPI_NONE, None)
    assert np.array_equal(C.numpy((Kd, N)), At @ G)
    # input-gradient layout: [Kd, M].[N, M]^T
    Gt = np.ascontiguousarray(G.T)
    dGt, D = abi.array(Gt), abi.array(g0)
    abi.mg_gemm_nt(dAt.ptr, dGt.ptr, D.ptr, Kd, M, N, 1, K.EPI_NONE, None)
    assert np.array_equal(D.numpy((Kd, N)), g0 + At @ Gt.T)
    abi.mg_check_kernel_status()


def _boundary_shapes():
    """Seeded draw of shapes around the tile, k-tile and split boundaries."""
    rng = np.random.default_rng(2024)
    ms = [2, 16, 64, 112, 114, 126, 128, 130, 224, 256, 300, 784, 1000, 2048, 4098]
    # (the 112- and 784-wide outputs take the 128 x 112 tile)
    ns = [2, 8, 10, 16, 18, 32, 34, 64, 66, 112, 128, 130, 200, 258, 784, 1024]
    ks = [2, 10, 16, 18, 32, 100, 112, 512, 784, 1000, 2048, 4098, 9000]
    out = [(256, 784, 64), (300, 112, 34), (4098, 784, 1024)]   # 112-column tile with the staged mask
    for _ in range(48):
        out.append((int(rng.choice(ms)), int(rng.choice(ks)), int(rng.choice(ns))))
    return sorted(set(out))


@pytest.mark.parametrize("M,Kd,N", _boundary_shapes())
def test_boundary_shapes_with_epilogues_bit_exact_on_integers(abi, M, Kd, N):
    """Integer operands, tensor-core path wherever the operands allow it: the three
    products with their fused epilogues (bias+ReLU; ReLU mask with accumulation;
    accumulation) must equal the integer results exactly for shapes that sit on and
    around tile edges, single k-tiles, narrow outputs and split contractions."""
    abi.mg_gemm_config(2, -1)
    rng = np.random.default_rng(M * 7919 + Kd * 31 + N)
    A = rng.integers(-3, 4, (M, Kd)).astype(np.float64)
    B = rng.integers(-3, 4, (Kd, N)).astype(np.float64)
    G = rng.integers(-3, 4, (M, N)).astype(np.float64)
    bias = rng.integers(-4, 5, N).astype(np.float64)
    Hmask = rng.integers(-1, 2, (M, Kd)).astype(np.float64)      # mask source for dA: (> 0)
    gA0 = rng.integers(-5, 6, (M, Kd)).astype(np.float64)
    gB0 = rng.integers(-5, 6, (Kd, N)).astype(np.float64)
    dA, dB, dG, dbias, dH = abi.array(A), abi.array(B), abi.array(G), abi.array(bias), abi.array(Hmask)
    C = abi.empty(M * N)
    abi.mg_gemm_nn(dA.ptr, dB.ptr, C.ptr, M, N, Kd, 0, K.EPI_BIAS_RELU, dbias.ptr)
    assert np.array_equal(C.numpy((M, N)), np.maximum(A @ B + bias, 0.0))
    dgA, dgB = abi.array(gA0), abi.array(gB0)
    abi.mg_gemm_nt(dG.ptr, dB.ptr, dgA.ptr, M, N, Kd, 1, K.EPI_RELU_MASK, dH.ptr)
    assert np.array_equal(dgA.numpy((M, Kd)), gA0 + (G @ B.T) * (Hmask > 0))
    store = abi.empty(M * Kd)
    abi.mg_gemm_nt(dG.ptr, dB.ptr, store.ptr, M, N, Kd, 0, K.EPI_RELU_MASK, dH.ptr)
    assert np.array_equal(store.numpy((M, Kd)), (G @ B.T) * (Hmask > 0))
    abi.mg_gemm_tn(dA.ptr, dG.ptr, dgB.ptr, M, N, Kd, 1)
    assert np.array_equal(dgB.numpy((Kd, N)), gB0 + A.T @ G)
    abi.mg_check_kernel_status()


def test_many_distinct_split_shapes_recycle_the_table_cache(abi):
    """A contraction length that changes on every call (a varying batch) builds a
    new segment table each time; the cache starts over past 256 tables and results
    stay exact before and after."""
    rng = np.random.default_rng(5)
    Kd, N = 128, 128
    for i in range(300):
        M = 512 + 16 * i
        A = rng.integers(-2, 3, (M, Kd)).astype(np.float64)
        G = rng.integers(-2, 3, (M, N)).astype(np.float64)
        dA, dG, out = abi.array(A), abi.array(G), abi.empty(Kd * N)
        abi.mg_gemm_tn(dA.ptr, dG.ptr, out.ptr, M, N, Kd, 0)
        if i % 37 == 0 or i >= 296:
            assert np.array_equal(out.numpy((Kd, N)), A.T @ G)
    abi.mg_check_kernel_status()


def test_empty_dimensions(abi):
    out = abi.array(np.ones(6))
    abi.mg_gemm_nn(None, None, out.ptr, 2, 3, 0, 0, K.EPI_NONE, None)   # K = 0 -> zeros
    assert not out.numpy().any()
    abi.mg_gemm_nn(None, None, None, 0, 3, 4, 0, K.EPI_NONE, None)       # no rows: no-op
    abi.mg_gemm_tn(None, None, out.ptr, 0, 3, 2, 1)                      # empty batch: += 0
    assert not out.numpy().any()


def test_linearity_at_full_size(abi):
    """4096^3 (a benchmark matmul size) without a CPU pass: (A+A').B == A.B + A'.B
    within the dot-product bound, and A.I == A exactly."""
    n = 4096
    rng = np.random.default_rng(1)
    A1 = rng.standard_normal((n, n)) / np.sqrt(n)
    A2 = rng.standard_normal((n, n)) / np.sqrt(n)
    B = rng.standard_normal((n, n)) / np.sqrt(n)
    dA1, dA2, dB = abi.array(A1), abi.array(A2), abi.array(B)
    dS = abi.empty(n * n)
    abi.mg_binary_fwd(K.ADD, dA1.ptr, dA2.ptr, dS.ptr, n * n)
    C1, C2, CS = abi.empty(n * n), abi.empty(n * n), abi.empty(n * n)
    abi.mg_gemm_nn(dA1.ptr, dB.ptr, C1.ptr, n, n, n, 0, K.EPI_NONE, None)
    abi.mg_gemm_nn(dA2.ptr, dB.ptr, C2.ptr, n, n, n, 0, K.EPI_NONE, None)
    abi.mg_gemm_nn(dS.ptr, dB.ptr, CS.ptr, n, n, n, 0, K.EPI_NONE, None)
    abi.mg_check_kernel_status()
    lhs = CS.numpy()
    rhs = C1.numpy() + C2.numpy()
    assert np.max(np.abs(lhs - rhs)) <= 1e-12
    eye = abi.array(np.eye(n))
    abi.mg_gemm_nn(dA1.ptr, eye.ptr, C1.ptr, n, n, n, 0, K.EPI_NONE, None)
    assert np.array_equal(C1.numpy((n, n)), A1)
    # spot-check 8 rows against the oracle
    rows = rng.integers(0, n, 8)
    from oracle import fast
    ref = fast.matmul_fwd(A2[rows], B)
    assert norm_err(C2.numpy((n, n))[rows], ref) <= TOL
