"""The checker's own ctypes view of the reference library.  TEST INFRASTRUCTURE ONLY.

``oracle/_ref/libref_true.so`` is the reference project's sources behind the flat
``mgt_*`` C binding (include/mg_tensor_c.h, reference part only).  This module
declares that binding for the checker independently of the product's Python
harness, so a mistake in the product-side binder cannot cancel out in a
comparison of the two libraries.  Only the reference's own interface is bound
(include/micrograd/Tensor.h:15-50 and include/micrograd/nn.h:6-34 of the
reference); the product's additions do not exist on this side.
"""
from __future__ import annotations

import ctypes as C
from types import SimpleNamespace

import numpy as np

_H = C.c_void_p
_DP = C.POINTER(C.c_double)
_SP = C.POINTER(C.c_size_t)

# op codes of mgt_binary / mgt_scalar / mgt_unary
_TENSOR_OPS = ("add", "sub", "mul", "div", "matmul")
_SCALAR_OPS = ("add", "sub", "mul", "div", "pow")
_UNARY_OPS = ("relu", "sigmoid", "tanh", "sum")

_PROTOTYPES = [
    ("mgt_last_error", C.c_char_p), ("mgt_new", _H, _SP, C.c_size_t, _DP, C.c_size_t),
    ("mgt_release", None, _H), ("mgt_ndim", C.c_size_t, _H), ("mgt_shape", None, _H, _SP),
    ("mgt_size", C.c_size_t, _H), ("mgt_get_data", C.c_int, _H, _DP, C.c_size_t),
    ("mgt_get_grad", C.c_int, _H, _DP, C.c_size_t), ("mgt_set_data", C.c_int, _H, _DP, C.c_size_t),
    ("mgt_set_grad", C.c_int, _H, _DP, C.c_size_t), ("mgt_at", C.c_double, _H, _SP, C.c_size_t),
    ("mgt_grad_at", C.c_double, _H, _SP, C.c_size_t),
    ("mgt_set_at", C.c_int, _H, _SP, C.c_size_t, C.c_double), ("mgt_to", C.c_int, _H, C.c_int),
    ("mgt_backend", C.c_int, _H), ("mgt_binary", _H, _H, _H, C.c_int),
    ("mgt_scalar", _H, _H, C.c_double, C.c_int), ("mgt_unary", _H, _H, C.c_int),
    ("mgt_backward", C.c_int, _H), ("mgt_zero_grad", C.c_int, _H), ("mgt_mse_loss", _H, _H, _H),
    ("mgt_avg_pool_2x2", _H, _H), ("mgt_linear_new", _H, C.c_size_t, C.c_size_t),
    ("mgt_linear_release", None, _H), ("mgt_linear_forward", _H, _H, _H),
    ("mgt_linear_weights", _H, _H), ("mgt_linear_bias", _H, _H),
    ("mgt_sgd_new", _H, C.POINTER(_H), C.c_size_t, C.c_double), ("mgt_sgd_release", None, _H),
    ("mgt_sgd_step", C.c_int, _H), ("mgt_sgd_zero_grad", C.c_int, _H),
    ("mgt_save_model", C.c_int, C.c_char_p, _H, _H), ("mgt_load_model", C.c_int, C.c_char_p, _H, _H),
    ("mgt_to_dot", _H, _H), ("mgt_format_scalar", _H, C.c_char_p, C.c_double),
    ("mgt_free_str", None, _H),
]


def load(path: str) -> SimpleNamespace:
    """Open the reference library and return Tensor / Linear / SGD mirrors of it."""
    lib = C.CDLL(path, mode=C.RTLD_LOCAL)
    for name, restype, *argtypes in _PROTOTYPES:
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = restype, list(argtypes)

    def fail():
        text = (lib.mgt_last_error() or b"").decode()
        if text.startswith("invalid_argument: "):
            raise ValueError(text.split(": ", 1)[1])
        raise RuntimeError(text)

    def ok(status):
        if status != 0:
            fail()

    def owned_string(ptr):
        if not ptr:
            fail()
        try:
            return C.string_at(ptr).decode()
        finally:
            lib.mgt_free_str(ptr)

    def flat(values):
        return np.ascontiguousarray(values, dtype=np.float64).ravel()

    def index(indices):
        return (C.c_size_t * len(indices))(*indices), len(indices)

    class Handle:
        """Owns one library object; `free` names its release function."""
        free = None

        def __init__(self, raw):
            if not raw:
                fail()
            self.raw = raw

        def __del__(self):
            raw, self.raw = getattr(self, "raw", None), None
            if raw:
                getattr(lib, self.free)(raw)

    class Tensor(Handle):
        free = "mgt_release"

        def __init__(self, shape, data=None, raw=None):
            if raw is None:
                dims = (C.c_size_t * len(shape))(*map(int, shape))
                if data is None:
                    raw = lib.mgt_new(dims, len(shape), None, 0)
                else:
                    values = flat(data)
                    raw = lib.mgt_new(dims, len(shape), values.ctypes.data_as(_DP), values.size)
            super().__init__(raw)

        @classmethod
        def adopt(cls, raw):
            return cls(None, raw=raw)

        def _with(self, other, op):
            if isinstance(other, Tensor):
                return Tensor.adopt(lib.mgt_binary(self.raw, other.raw, _TENSOR_OPS.index(op)))
            return Tensor.adopt(lib.mgt_scalar(self.raw, float(other), _SCALAR_OPS.index(op)))

        def add(self, other): return self._with(other, "add")
        def sub(self, other): return self._with(other, "sub")
        def mul(self, other): return self._with(other, "mul")
        def div(self, other): return self._with(other, "div")
        def pow(self, exponent): return Tensor.adopt(lib.mgt_scalar(self.raw, float(exponent), 4))
        def matmul(self, other): return self._with(other, "matmul")
        def relu(self): return Tensor.adopt(lib.mgt_unary(self.raw, _UNARY_OPS.index("relu")))
        def sigmoid(self): return Tensor.adopt(lib.mgt_unary(self.raw, _UNARY_OPS.index("sigmoid")))
        def tanh(self): return Tensor.adopt(lib.mgt_unary(self.raw, _UNARY_OPS.index("tanh")))
        def sum(self): return Tensor.adopt(lib.mgt_unary(self.raw, _UNARY_OPS.index("sum")))
        def backward(self): ok(lib.mgt_backward(self.raw))
        def zero_grad(self): ok(lib.mgt_zero_grad(self.raw))

        def shape(self):
            dims = (C.c_size_t * lib.mgt_ndim(self.raw))()
            lib.mgt_shape(self.raw, dims)
            return list(map(int, dims))

        def size(self):
            return int(lib.mgt_size(self.raw))

        def _read(self, getter):
            out = np.empty(self.size())
            ok(getter(self.raw, out.ctypes.data_as(_DP), out.size))
            return out

        def data(self): return self._read(lib.mgt_get_data)
        def grad(self): return self._read(lib.mgt_get_grad)

        def set_data(self, values):
            v = flat(values)
            ok(lib.mgt_set_data(self.raw, v.ctypes.data_as(_DP), v.size))

        def set_grad(self, values):
            v = flat(values)
            ok(lib.mgt_set_grad(self.raw, v.ctypes.data_as(_DP), v.size))

        def at(self, indices): return float(lib.mgt_at(self.raw, *index(indices)))
        def grad_at(self, indices): return float(lib.mgt_grad_at(self.raw, *index(indices)))
        def set_at(self, indices, value): ok(lib.mgt_set_at(self.raw, *index(indices), float(value)))
        def to(self, backend): ok(lib.mgt_to(self.raw, int(backend)))
        def backend(self): return int(lib.mgt_backend(self.raw))
        def to_dot(self): return owned_string(lib.mgt_to_dot(self.raw))

    class Linear(Handle):
        free = "mgt_linear_release"

        def __init__(self, in_features, out_features):
            super().__init__(lib.mgt_linear_new(int(in_features), int(out_features)))

        def forward(self, x): return Tensor.adopt(lib.mgt_linear_forward(self.raw, x.raw))
        def weights(self): return Tensor.adopt(lib.mgt_linear_weights(self.raw))
        def bias(self): return Tensor.adopt(lib.mgt_linear_bias(self.raw))

    class SGD(Handle):
        free = "mgt_sgd_release"

        def __init__(self, parameters, learning_rate):
            raws = (_H * len(parameters))(*[p.raw for p in parameters])
            super().__init__(lib.mgt_sgd_new(raws, len(parameters), float(learning_rate)))

        def step(self): ok(lib.mgt_sgd_step(self.raw))
        def zero_grad(self): ok(lib.mgt_sgd_zero_grad(self.raw))

    return SimpleNamespace(
        lib=lib, extensions=False, Tensor=Tensor, Linear=Linear, SGD=SGD,
        mse_loss=lambda p, t: Tensor.adopt(lib.mgt_mse_loss(p.raw, t.raw)),
        avg_pool_2x2=lambda x: Tensor.adopt(lib.mgt_avg_pool_2x2(x.raw)),
        save_model=lambda path, a, b: ok(lib.mgt_save_model(path.encode(), a.raw, b.raw)),
        load_model=lambda path, a, b: ok(lib.mgt_load_model(path.encode(), a.raw, b.raw)),
        format_scalar=lambda op, s: owned_string(lib.mgt_format_scalar(op.encode(), float(s))),
    )
