"""ctypes binding of ``include/mg_tensor_c.h`` — the flat C view of micrograd's
C++ ``Tensor`` / ``Linear`` / ``SGD`` interface (reference:
include/micrograd/Tensor.h:15-50, include/micrograd/nn.h:6-34).

``bind(path)`` loads one shared library that exports the ``mgt_*`` symbols and
returns a namespace whose classes mirror the C++ API method for method, so a
Python test can be written the way the reference's C++ tests are::

    api = bind(".../libmicrograd.so")
    a = api.Tensor([2, 2], [1, 2, 3, 4]); b = api.Tensor([2, 2], [5, 6, 7, 8])
    loss = a.matmul(b).sum(); loss.backward(); a.grad()   # 11 15 11 15

Errors raised inside the library surface as Python exceptions of the matching
kind: ``invalid_argument`` -> ValueError, anything else -> RuntimeError, with
the original message.
"""
from __future__ import annotations

import ctypes as C
from types import SimpleNamespace

import numpy as np

_c_double_p = C.POINTER(C.c_double)
_c_size_p = C.POINTER(C.c_size_t)
_c_int_p = C.POINTER(C.c_int)

BACKEND_CPU = 0
BACKEND_METAL = 1

_BINARY = {"add": 0, "sub": 1, "mul": 2, "div": 3, "matmul": 4}
_SCALAR = {"add": 0, "sub": 1, "mul": 2, "div": 3, "pow": 4}
_UNARY = {"relu": 0, "sigmoid": 1, "tanh": 2, "sum": 3, "exp": 4}


def _declare(lib, extensions: bool) -> None:
    vp = C.c_void_p
    sigs = {
        "mgt_last_error": (C.c_char_p, []),
        "mgt_new": (vp, [_c_size_p, C.c_size_t, _c_double_p, C.c_size_t]),
        "mgt_release": (None, [vp]),
        "mgt_ndim": (C.c_size_t, [vp]),
        "mgt_shape": (None, [vp, _c_size_p]),
        "mgt_size": (C.c_size_t, [vp]),
        "mgt_get_data": (C.c_int, [vp, _c_double_p, C.c_size_t]),
        "mgt_get_grad": (C.c_int, [vp, _c_double_p, C.c_size_t]),
        "mgt_set_data": (C.c_int, [vp, _c_double_p, C.c_size_t]),
        "mgt_set_grad": (C.c_int, [vp, _c_double_p, C.c_size_t]),
        "mgt_at": (C.c_double, [vp, _c_size_p, C.c_size_t]),
        "mgt_grad_at": (C.c_double, [vp, _c_size_p, C.c_size_t]),
        "mgt_set_at": (C.c_int, [vp, _c_size_p, C.c_size_t, C.c_double]),
        "mgt_to": (C.c_int, [vp, C.c_int]),
        "mgt_backend": (C.c_int, [vp]),
        "mgt_binary": (vp, [vp, vp, C.c_int]),
        "mgt_scalar": (vp, [vp, C.c_double, C.c_int]),
        "mgt_unary": (vp, [vp, C.c_int]),
        "mgt_backward": (C.c_int, [vp]),
        "mgt_zero_grad": (C.c_int, [vp]),
        "mgt_mse_loss": (vp, [vp, vp]),
        "mgt_avg_pool_2x2": (vp, [vp]),
        "mgt_linear_new": (vp, [C.c_size_t, C.c_size_t]),
        "mgt_linear_release": (None, [vp]),
        "mgt_linear_forward": (vp, [vp, vp]),
        "mgt_linear_weights": (vp, [vp]),
        "mgt_linear_bias": (vp, [vp]),
        "mgt_sgd_new": (vp, [C.POINTER(vp), C.c_size_t, C.c_double]),
        "mgt_sgd_release": (None, [vp]),
        "mgt_sgd_step": (C.c_int, [vp]),
        "mgt_sgd_zero_grad": (C.c_int, [vp]),
        "mgt_save_model": (C.c_int, [C.c_char_p, vp, vp]),
        "mgt_load_model": (C.c_int, [C.c_char_p, vp, vp]),
        "mgt_to_dot": (vp, [vp]),
        "mgt_format_scalar": (vp, [C.c_char_p, C.c_double]),
        "mgt_free_str": (None, [vp]),
    }
    if extensions:
        sigs.update({
            "mgt_sum_axis": (vp, [vp, C.c_int]),
            "mgt_softmax_cross_entropy": (vp, [vp, vp, C.c_double]),
            "mgt_softmax_cross_entropy_host": (vp, [vp, _c_int_p, C.c_size_t, C.c_double]),
            "mgt_new_from_host": (vp, [_c_size_p, C.c_size_t, C.c_void_p]),
            "mgt_comm_rank": (C.c_int, []),
            "mgt_comm_world": (C.c_int, []),
            "mgt_argmax_rows": (C.c_int, [vp, _c_int_p, C.c_size_t]),
            "mgt_linear_forward_relu": (vp, [vp, vp]),
            "mgt_set_requires_grad": (C.c_int, [vp, C.c_int]),
            "mgt_sync": (C.c_int, []),
            "mgt_comm_unique_id": (C.c_int, [C.c_char_p]),
            "mgt_comm_init": (C.c_int, [C.c_char_p, C.c_int, C.c_int]),
            "mgt_comm_shutdown": (C.c_int, []),
            "mgt_sgd_enable_allreduce": (C.c_int, [vp]),
            "mgt_copy_from_host": (C.c_int, [vp, _c_double_p, C.c_size_t]),
            "mgt_prefetch_from_host": (C.c_int, [vp, C.c_void_p, C.c_size_t]),
            "mgt_record_begin": (C.c_int, []),
            "mgt_record_end": (C.c_int, []),
            "mgt_record_replay": (C.c_int, []),
            "mgt_record_kernels": (C.c_int, []),
            "mgt_record_abandon": (C.c_int, []),
        })
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args


def bind(path: str) -> SimpleNamespace:
    """Load the library at ``path`` and return its Python mirror of the API."""
    lib = C.CDLL(path, mode=C.RTLD_LOCAL)
    extensions = hasattr(lib, "mgt_sum_axis")
    _declare(lib, extensions)

    def _raise() -> None:
        msg = (lib.mgt_last_error() or b"").decode()
        kind, _, text = msg.partition(": ")
        if kind == "invalid_argument":
            raise ValueError(text)
        raise RuntimeError(msg)

    def _check(rc: int) -> None:
        if rc != 0:
            _raise()

    def _take_str(p) -> str:
        if not p:
            _raise()
        s = C.string_at(p).decode()
        lib.mgt_free_str(p)
        return s

    def _as_f64(values) -> np.ndarray:
        return np.ascontiguousarray(values, dtype=np.float64).reshape(-1)

    class Tensor:
        """Mirror of ``class Tensor`` (reference include/micrograd/Tensor.h:12-50)."""

        __slots__ = ("_h",)

        def __init__(self, shape, data=None, _handle=None):
            if _handle is not None:
                self._h = _handle
                return
            shp = (C.c_size_t * len(shape))(*[int(s) for s in shape])
            if data is None:
                h = lib.mgt_new(shp, len(shape), None, 0)
            else:
                arr = _as_f64(data)
                h = lib.mgt_new(shp, len(shape), arr.ctypes.data_as(_c_double_p), arr.size)
            if not h:
                _raise()
            self._h = h

        def __del__(self):
            h = getattr(self, "_h", None)
            if h:
                lib.mgt_release(h)
                self._h = None

        @staticmethod
        def _wrap(h) -> "Tensor":
            if not h:
                _raise()
            return Tensor(None, _handle=h)

        # -- ops --
        def _bin(self, other, name):
            if isinstance(other, Tensor):
                return Tensor._wrap(lib.mgt_binary(self._h, other._h, _BINARY[name]))
            return Tensor._wrap(lib.mgt_scalar(self._h, float(other), _SCALAR[name]))

        def add(self, other): return self._bin(other, "add")
        def sub(self, other): return self._bin(other, "sub")
        def mul(self, other): return self._bin(other, "mul")
        def div(self, other): return self._bin(other, "div")

        def pow(self, exponent: float):
            return Tensor._wrap(lib.mgt_scalar(self._h, float(exponent), _SCALAR["pow"]))

        def matmul(self, other: "Tensor"):
            return Tensor._wrap(lib.mgt_binary(self._h, other._h, _BINARY["matmul"]))

        def sum(self, axis=None):
            if axis is None:
                return Tensor._wrap(lib.mgt_unary(self._h, _UNARY["sum"]))
            return Tensor._wrap(lib.mgt_sum_axis(self._h, int(axis)))

        def relu(self): return Tensor._wrap(lib.mgt_unary(self._h, _UNARY["relu"]))
        def sigmoid(self): return Tensor._wrap(lib.mgt_unary(self._h, _UNARY["sigmoid"]))
        def tanh(self): return Tensor._wrap(lib.mgt_unary(self._h, _UNARY["tanh"]))
        def exp(self): return Tensor._wrap(lib.mgt_unary(self._h, _UNARY["exp"]))

        # -- autograd --
        def backward(self): _check(lib.mgt_backward(self._h))
        def zero_grad(self): _check(lib.mgt_zero_grad(self._h))

        # -- introspection --
        def shape(self):
            n = lib.mgt_ndim(self._h)
            out = (C.c_size_t * n)()
            lib.mgt_shape(self._h, out)
            return [int(v) for v in out]

        def size(self) -> int:
            return int(lib.mgt_size(self._h))

        def data(self) -> np.ndarray:
            out = np.empty(self.size(), dtype=np.float64)
            _check(lib.mgt_get_data(self._h, out.ctypes.data_as(_c_double_p), out.size))
            return out

        def grad(self) -> np.ndarray:
            out = np.empty(self.size(), dtype=np.float64)
            _check(lib.mgt_get_grad(self._h, out.ctypes.data_as(_c_double_p), out.size))
            return out

        def set_data(self, values) -> None:
            arr = _as_f64(values)
            _check(lib.mgt_set_data(self._h, arr.ctypes.data_as(_c_double_p), arr.size))

        def set_grad(self, values) -> None:
            arr = _as_f64(values)
            _check(lib.mgt_set_grad(self._h, arr.ctypes.data_as(_c_double_p), arr.size))

        def at(self, indices) -> float:
            idx = (C.c_size_t * len(indices))(*indices)
            return float(lib.mgt_at(self._h, idx, len(indices)))

        def grad_at(self, indices) -> float:
            idx = (C.c_size_t * len(indices))(*indices)
            return float(lib.mgt_grad_at(self._h, idx, len(indices)))

        def set_at(self, indices, value: float) -> None:
            idx = (C.c_size_t * len(indices))(*indices)
            _check(lib.mgt_set_at(self._h, idx, len(indices), float(value)))

        def to(self, backend: int) -> None: _check(lib.mgt_to(self._h, int(backend)))
        def backend(self) -> int: return int(lib.mgt_backend(self._h))
        def to_dot(self) -> str: return _take_str(lib.mgt_to_dot(self._h))

        # -- additive API (B200 backend only) --
        def set_requires_grad(self, flag: bool) -> None:
            _check(lib.mgt_set_requires_grad(self._h, 1 if flag else 0))

        def copy_from_host(self, values) -> None:
            """Tensor::copy_from_host: new values into the device buffer the tensor has."""
            arr = _as_f64(values)
            _check(lib.mgt_copy_from_host(self._h, arr.ctypes.data_as(_c_double_p), arr.size))

        def prefetch_from_host(self, pointer: int) -> None:
            """Tensor::prefetch_from_host: size() doubles from a raw host address (e.g.
            pinned memory) into the buffer the tensor has, on the copy stream."""
            _check(lib.mgt_prefetch_from_host(self._h, C.c_void_p(pointer), self.size()))

    class Linear:
        """Mirror of ``class Linear`` (reference include/micrograd/nn.h:10-21)."""

        def __init__(self, in_features: int, out_features: int):
            self._h = lib.mgt_linear_new(in_features, out_features)
            if not self._h:
                _raise()

        def __del__(self):
            if getattr(self, "_h", None):
                lib.mgt_linear_release(self._h)
                self._h = None

        def forward(self, x: Tensor) -> Tensor:
            return Tensor._wrap(lib.mgt_linear_forward(self._h, x._h))

        def forward_relu(self, x: Tensor) -> Tensor:
            return Tensor._wrap(lib.mgt_linear_forward_relu(self._h, x._h))

        def weights(self) -> Tensor: return Tensor._wrap(lib.mgt_linear_weights(self._h))
        def bias(self) -> Tensor: return Tensor._wrap(lib.mgt_linear_bias(self._h))

    class SGD:
        """Mirror of ``class SGD`` (reference include/micrograd/nn.h:23-33)."""

        def __init__(self, parameters, learning_rate: float):
            arr = (C.c_void_p * len(parameters))(*[p._h for p in parameters])
            self._h = lib.mgt_sgd_new(arr, len(parameters), float(learning_rate))
            if not self._h:
                _raise()

        def __del__(self):
            if getattr(self, "_h", None):
                lib.mgt_sgd_release(self._h)
                self._h = None

        def step(self) -> None: _check(lib.mgt_sgd_step(self._h))
        def zero_grad(self) -> None: _check(lib.mgt_sgd_zero_grad(self._h))
        def enable_allreduce(self) -> None: _check(lib.mgt_sgd_enable_allreduce(self._h))

    def mse_loss(prediction: Tensor, target: Tensor) -> Tensor:
        return Tensor._wrap(lib.mgt_mse_loss(prediction._h, target._h))

    def avg_pool_2x2(x: Tensor) -> Tensor:
        return Tensor._wrap(lib.mgt_avg_pool_2x2(x._h))

    def save_model(path: str, l1: Linear, l2: Linear) -> None:
        _check(lib.mgt_save_model(path.encode(), l1._h, l2._h))

    def load_model(path: str, l1: Linear, l2: Linear) -> None:
        _check(lib.mgt_load_model(path.encode(), l1._h, l2._h))

    def format_scalar(op: str, scalar: float) -> str:
        return _take_str(lib.mgt_format_scalar(op.encode(), float(scalar)))

    def softmax_cross_entropy(logits: Tensor, labels, denom: float = 0.0) -> Tensor:
        """labels: a Tensor of class ids (one per row) or a host int array.
        denom: divisor of the mean (0 = rows; a shard passes the global batch)."""
        if isinstance(labels, Tensor):
            return Tensor._wrap(lib.mgt_softmax_cross_entropy(logits._h, labels._h, float(denom)))
        ids = np.ascontiguousarray(labels, dtype=np.int32).reshape(-1)
        return Tensor._wrap(lib.mgt_softmax_cross_entropy_host(
            logits._h, ids.ctypes.data_as(_c_int_p), ids.size, float(denom)))

    def from_host(shape, pointer: int) -> Tensor:
        """Tensor::from_host: upload from a raw host address (e.g. pinned memory)."""
        shp = (C.c_size_t * len(shape))(*[int(s) for s in shape])
        return Tensor._wrap(lib.mgt_new_from_host(shp, len(shape), C.c_void_p(pointer)))

    def argmax_rows(x: Tensor) -> np.ndarray:
        rows = x.shape()[0]
        out = np.empty(rows, dtype=np.int32)
        _check(lib.mgt_argmax_rows(x._h, out.ctypes.data_as(_c_int_p), rows))
        return out

    def synchronize() -> None: _check(lib.mgt_sync())

    def comm_unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        _check(lib.mgt_comm_unique_id(buf))
        return buf.raw

    def comm_init(uid: bytes, rank: int, world: int) -> None:
        _check(lib.mgt_comm_init(uid, rank, world))

    def comm_shutdown() -> None: _check(lib.mgt_comm_shutdown())

    class RecordedStep:
        """micrograd::RecordedStep — record one step of Tensor-API code, replay it
        with a single launch (one recorded step per process through this binding)."""

        def begin(self) -> None: _check(lib.mgt_record_begin())
        def end(self) -> None: _check(lib.mgt_record_end())
        def replay(self) -> None: _check(lib.mgt_record_replay())
        def kernels(self) -> int: return int(lib.mgt_record_kernels())

        def abandon(self) -> None:
            """Destroys the C++ object (as going out of scope would) and makes a new one."""
            _check(lib.mgt_record_abandon())

    return SimpleNamespace(
        lib=lib, extensions=extensions, Tensor=Tensor, Linear=Linear, SGD=SGD,
        mse_loss=mse_loss, avg_pool_2x2=avg_pool_2x2, save_model=save_model,
        load_model=load_model, format_scalar=format_scalar,
        softmax_cross_entropy=softmax_cross_entropy, argmax_rows=argmax_rows, from_host=from_host,
        comm_rank=lambda: int(lib.mgt_comm_rank()), comm_world=lambda: int(lib.mgt_comm_world()),
        synchronize=synchronize, comm_unique_id=comm_unique_id, comm_init=comm_init,
        comm_shutdown=comm_shutdown, RecordedStep=RecordedStep if extensions else None,
    )
