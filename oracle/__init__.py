"""CPU oracle for micrograd's fp64 tensor-op path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product imports this package.  It is the checker used by
``tests/``, by ``__graft_entry__.smoke()`` and by ``bench.py``'s CPU-baseline
and ``--impl reference`` legs.

Two libraries sit behind it (built by ``oracle/Makefile``):

* ``_ref/libref_true.so`` — the reference project's own ``src/core``, ``src/ops``,
  ``src/nn.cpp`` and ``src/Utils.cpp`` compiled unmodified (``-O2
  -ffp-contract=off``), driven through the flat C binding of its public
  ``Tensor`` API.  Single-threaded, as the reference is.  ``ref_true()``.
* ``libref_fast.so`` — ``ref_fast.c``, an order-preserving restatement of the same
  loops on flat arrays with OpenMP across independent outputs.  Bit-identical to
  ``libref_true.so`` on every op both have (asserted in ``tests/test_oracle.py``)
  and fast enough for full-size parity.  ``fast``.

Parity status: pinned for every op the reference implements (against the
reference's own compiled code and its test suite's known answers), and for the
additions that have an exact encoding in reference code: row-broadcast add and
the column sum (``ones[B,1] @ b[1,N]``, ``ones[1,M] @ X``) and the last-axis sum
(``X @ ones[N,1]``), forward and backward.  For ``exp``, softmax cross-entropy
and argmax the reference offers nothing to run; the restatements in
``ref_fast.c`` are the only authority: parity unpinned for those three.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_TRUE_PATH = os.path.join(_HERE, "_ref", "libref_true.so")
REF_FAST_PATH = os.path.join(_HERE, "libref_fast.so")

_dp = C.POINTER(C.c_double)
_ip = C.POINTER(C.c_int)


def build() -> None:
    """Compile the checker libraries (and, where the reference tree is mounted,
    the reference's own sources)."""
    subprocess.run(["make", "-s", "-C", _HERE], check=True)


_ref_true_ns = None


def ref_true():
    """The reference's own compiled code, as a Python mirror of its C++ API."""
    global _ref_true_ns
    if _ref_true_ns is None:
        if not os.path.exists(REF_TRUE_PATH):
            raise FileNotFoundError(
                f"{REF_TRUE_PATH} is missing: run `make -C oracle` where the reference tree is mounted")
        from . import ref_binding
        _ref_true_ns = ref_binding.load(REF_TRUE_PATH)
    return _ref_true_ns


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(_dp)


def _f64(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float64)


class _Fast:
    """numpy front end of ``libref_fast.so`` (see ref_fast.c for citations)."""

    BINARY = {"add": 0, "sub": 1, "mul": 2, "div": 3}
    SCALAR = {"add": 0, "sub": 1, "mul": 2, "div": 3, "pow": 4}
    UNARY = {"relu": 0, "sigmoid": 1, "tanh": 2, "exp": 3}

    def __init__(self):
        self._lib = None

    @property
    def lib(self):
        if self._lib is None:
            if not os.path.exists(REF_FAST_PATH):
                build()
            lib = C.CDLL(REF_FAST_PATH, mode=C.RTLD_LOCAL)
            st = C.c_size_t
            sigs = {
                "rf_num_threads": (C.c_int, []),
                "rf_set_num_threads": (None, [C.c_int]),
                "rf_binary_fwd": (None, [C.c_int, st, _dp, _dp, _dp]),
                "rf_binary_bwd": (None, [C.c_int, st, _dp, _dp, _dp, _dp, _dp]),
                "rf_scalar_fwd": (None, [C.c_int, st, _dp, C.c_double, _dp]),
                "rf_scalar_bwd": (None, [C.c_int, st, _dp, C.c_double, _dp, _dp]),
                "rf_unary_fwd": (None, [C.c_int, st, _dp, _dp]),
                "rf_unary_bwd": (None, [C.c_int, st, _dp, _dp, _dp, _dp]),
                "rf_sum": (C.c_double, [st, _dp]),
                "rf_sum_longdouble": (C.c_double, [st, _dp]),
                "rf_sum_bwd": (None, [st, C.c_double, _dp]),
                "rf_matmul_fwd": (None, [st, st, st, _dp, _dp, _dp]),
                "rf_matmul_bwd": (None, [st, st, st, _dp, _dp, _dp, _dp, _dp]),
                "rf_sgd_step": (None, [st, _dp, _dp, C.c_double]),
                "rf_add_row_fwd": (None, [st, st, _dp, _dp, _dp]),
                "rf_add_row_bwd": (None, [st, st, _dp, _dp, _dp]),
                "rf_sum_lastaxis_fwd": (None, [st, st, _dp, _dp]),
                "rf_sum_lastaxis_bwd": (None, [st, st, _dp, _dp]),
                "rf_softmax_xent_fwd": (C.c_double, [st, st, _dp, _ip, C.c_double]),
                "rf_softmax_xent_bwd": (None, [st, st, _dp, _ip, C.c_double, C.c_double, _dp]),
                "rf_argmax_rows": (None, [st, st, _dp, _ip]),
            }
            for name, (res, args) in sigs.items():
                fn = getattr(lib, name)
                fn.restype, fn.argtypes = res, args
            self._lib = lib
        return self._lib

    def num_threads(self) -> int:
        return int(self.lib.rf_num_threads())

    def set_num_threads(self, n: int) -> None:
        self.lib.rf_set_num_threads(int(n))

    # ---- elementwise ----
    def binary_fwd(self, op: str, a, b) -> np.ndarray:
        a, b = _f64(a), _f64(b)
        out = np.empty_like(a)
        self.lib.rf_binary_fwd(self.BINARY[op], a.size, _ptr(a), _ptr(b), _ptr(out))
        return out

    def binary_bwd(self, op: str, a, b, g, ga: np.ndarray, gb: np.ndarray) -> None:
        """Accumulates into ga and gb in place (they may be the same array)."""
        a, b, g = _f64(a), _f64(b), _f64(g)
        self.lib.rf_binary_bwd(self.BINARY[op], a.size, _ptr(a), _ptr(b), _ptr(g), _ptr(ga), _ptr(gb))

    def scalar_fwd(self, op: str, a, s: float) -> np.ndarray:
        a = _f64(a)
        out = np.empty_like(a)
        self.lib.rf_scalar_fwd(self.SCALAR[op], a.size, _ptr(a), float(s), _ptr(out))
        return out

    def scalar_bwd(self, op: str, a, s: float, g, ga: np.ndarray) -> None:
        a, g = _f64(a), _f64(g)
        self.lib.rf_scalar_bwd(self.SCALAR[op], a.size, _ptr(a), float(s), _ptr(g), _ptr(ga))

    def unary_fwd(self, op: str, a) -> np.ndarray:
        a = _f64(a)
        out = np.empty_like(a)
        self.lib.rf_unary_fwd(self.UNARY[op], a.size, _ptr(a), _ptr(out))
        return out

    def unary_bwd(self, op: str, a, out, g, ga: np.ndarray) -> None:
        a, out, g = _f64(a), _f64(out), _f64(g)
        self.lib.rf_unary_bwd(self.UNARY[op], a.size, _ptr(a), _ptr(out), _ptr(g), _ptr(ga))

    # ---- reductions ----
    def sum(self, a) -> float:
        a = _f64(a)
        return float(self.lib.rf_sum(a.size, _ptr(a)))

    def sum_longdouble(self, a) -> float:
        a = _f64(a)
        return float(self.lib.rf_sum_longdouble(a.size, _ptr(a)))

    def sum_bwd(self, g0: float, ga: np.ndarray) -> None:
        self.lib.rf_sum_bwd(ga.size, float(g0), _ptr(ga))

    def sum_lastaxis_fwd(self, x) -> np.ndarray:
        x = _f64(x)
        M, N = x.shape
        out = np.empty(M, dtype=np.float64)
        self.lib.rf_sum_lastaxis_fwd(M, N, _ptr(x), _ptr(out))
        return out

    def sum_lastaxis_bwd(self, g, gx: np.ndarray) -> None:
        g = _f64(g)
        M, N = gx.shape
        self.lib.rf_sum_lastaxis_bwd(M, N, _ptr(g), _ptr(gx))

    # ---- matmul ----
    def matmul_fwd(self, A, B) -> np.ndarray:
        A, B = _f64(A), _f64(B)
        m, k = A.shape
        k2, n = B.shape
        assert k == k2
        out = np.empty((m, n), dtype=np.float64)
        self.lib.rf_matmul_fwd(m, k, n, _ptr(A), _ptr(B), _ptr(out))
        return out

    def matmul_bwd(self, A, B, gC, gA, gB) -> None:
        """Accumulates into gA / gB in place; either may be None (skipped)."""
        A, B, gC = _f64(A), _f64(B), _f64(gC)
        m, k = A.shape
        n = B.shape[1]
        self.lib.rf_matmul_bwd(m, k, n, _ptr(A), _ptr(B), _ptr(gC),
                               _ptr(gA) if gA is not None else None,
                               _ptr(gB) if gB is not None else None)

    # ---- broadcast ----
    def add_row_fwd(self, x, r) -> np.ndarray:
        x, r = _f64(x), _f64(r).reshape(-1)
        M, N = x.shape
        out = np.empty_like(x)
        self.lib.rf_add_row_fwd(M, N, _ptr(x), _ptr(r), _ptr(out))
        return out

    def add_row_bwd(self, g, gx, gr) -> None:
        g = _f64(g)
        M, N = g.shape
        self.lib.rf_add_row_bwd(M, N, _ptr(g), _ptr(gx) if gx is not None else None,
                                _ptr(gr) if gr is not None else None)

    # ---- loss / argmax / optimiser ----
    def softmax_xent_fwd(self, z, labels, denom=None) -> float:
        z = _f64(z)
        labels = np.ascontiguousarray(labels, dtype=np.int32)
        M, Cn = z.shape
        return float(self.lib.rf_softmax_xent_fwd(M, Cn, _ptr(z), labels.ctypes.data_as(_ip),
                                                  float(denom if denom is not None else M)))

    def softmax_xent_bwd(self, z, labels, gz: np.ndarray, denom=None, gloss: float = 1.0) -> None:
        z = _f64(z)
        labels = np.ascontiguousarray(labels, dtype=np.int32)
        M, Cn = z.shape
        self.lib.rf_softmax_xent_bwd(M, Cn, _ptr(z), labels.ctypes.data_as(_ip),
                                     float(denom if denom is not None else M), float(gloss), _ptr(gz))

    def argmax_rows(self, x) -> np.ndarray:
        x = _f64(x)
        M, N = x.shape
        out = np.empty(M, dtype=np.int32)
        self.lib.rf_argmax_rows(M, N, _ptr(x), out.ctypes.data_as(_ip))
        return out

    def sgd_step(self, p: np.ndarray, g, lr: float) -> None:
        g = _f64(g)
        self.lib.rf_sgd_step(p.size, _ptr(p), _ptr(g), float(lr))

    # ---- MLP built from the pieces above ----
    def mlp_forward(self, params, X):
        """params: [(W[in,out], b[out]), ...].  ReLU between layers, none after
        the last (reference Linear::forward, src/nn.cpp:55-57, with the bias
        broadcast over rows).  Returns (logits, saved activations)."""
        acts = [_f64(X)]
        pre = []
        h = acts[0]
        for li, (W, b) in enumerate(params):
            z = self.add_row_fwd(self.matmul_fwd(h, W), b)
            pre.append(z)
            if li + 1 < len(params):
                h = self.unary_fwd("relu", z)
                acts.append(h)
        return pre[-1], (acts, pre)

    def mlp_train_step(self, params, X, labels, lr: float, denom=None, input_grad: bool = False,
                       apply: bool = True):
        """One SGD step of softmax-cross-entropy training.  Returns (loss, grads,
        grad of X or None).  Gradients start from zero, as after zero_grad()
        (src/nn.cpp:65-69); the update is src/nn.cpp:71-77."""
        logits, (acts, pre) = self.mlp_forward(params, X)
        loss = self.softmax_xent_fwd(logits, labels, denom)
        g = np.zeros_like(logits)
        self.softmax_xent_bwd(logits, labels, g, denom)
        grads = []
        gX = None
        for li in reversed(range(len(params))):
            W, b = params[li]
            gW = np.zeros_like(W)
            gb = np.zeros_like(b)
            gz = g
            # bias-add node: gx += g ; gb += column sums (rows ascending)
            gmm = np.zeros_like(gz)
            self.add_row_bwd(gz, gmm, gb)
            need_in = li > 0 or input_grad
            gin = np.zeros_like(acts[li]) if need_in else None
            self.matmul_bwd(acts[li], W, gmm, gin, gW)
            grads.append((gW, gb))
            if li > 0:
                gpre = np.zeros_like(pre[li - 1])
                self.unary_bwd("relu", pre[li - 1], acts[li], gin, gpre)
                g = gpre
            else:
                gX = gin
        grads.reverse()
        if apply:
            for (W, b), (gW, gb) in zip(params, grads):
                self.sgd_step(W, gW, lr)
                self.sgd_step(b, gb, lr)
        return loss, grads, gX


fast = _Fast()


def mlp_train_step_true(params, X, labels, lr: float, input_grad: bool = True):
    """The same training step run by the reference's own compiled code.

    The reference cannot express a batched bias add or an external loss
    gradient, so two reference-only encodings are used: the bias is broadcast as
    ``ones[B,1] @ b[1,N]`` (exact: 0.0 + 1.0*b), and the softmax-cross-entropy
    gradient G — computed on the host by ``fast.softmax_xent_bwd`` — is injected
    as ``logits.mul(G).sum().backward()``, which leaves exactly G in
    ``logits.grad``.  Everything upstream of the logits (matmul, add, relu,
    their backward closures and the SGD update) is reference code.
    Updates ``params`` in place; returns (loss, grads, grad of X).
    """
    api = ref_true()
    X = _f64(X)
    B = X.shape[0]
    x = api.Tensor(list(X.shape), X)
    ones = api.Tensor([B, 1], np.ones(B))
    Ws = [api.Tensor(list(W.shape), W) for W, _ in params]
    bs = [api.Tensor([1, b.size], b) for _, b in params]
    h = x
    for li in range(len(params)):
        h = h.matmul(Ws[li]).add(ones.matmul(bs[li]))
        if li + 1 < len(params):
            h = h.relu()
    logits = h
    z = logits.data().reshape(B, -1)
    loss = fast.softmax_xent_fwd(z, labels)
    G = np.zeros_like(z)
    fast.softmax_xent_bwd(z, labels, G)
    seed = api.Tensor(list(z.shape), G)
    flat = [t for pair in zip(Ws, bs) for t in pair]
    opt = api.SGD(flat, lr)
    opt.zero_grad()
    logits.mul(seed).sum().backward()
    grads = [(W.grad().reshape(p[0].shape), b.grad().reshape(p[1].shape))
             for W, b, p in zip(Ws, bs, params)]
    gX = x.grad().reshape(X.shape) if input_grad else None
    opt.step()
    for (W, b), Wt, bt in zip(params, Ws, bs):
        W[...] = Wt.data().reshape(W.shape)
        b[...] = bt.data().reshape(b.shape)
    return loss, grads, gX
