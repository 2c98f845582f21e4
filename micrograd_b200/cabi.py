"""ctypes view of the device C ABI (``include/mg_cuda.h``).

Used by the GPU parity tests and the benchmark to call the kernels exactly as
the C++ ``Tensor`` layer does: plain device pointers and sizes.  ``CudaABI``
declares every entry point of the header; ``DeviceArray`` is a small RAII
wrapper around ``mg_alloc``/``mg_free`` with numpy upload/download.

A non-zero status raises ``MgError`` carrying ``mg_last_error()``; nothing here
falls back to the CPU.
"""
from __future__ import annotations

import ctypes as C
import re

import numpy as np

_dp = C.POINTER(C.c_double)
_ip = C.POINTER(C.c_int)
_sz = C.c_size_t

OK = 0
ERR_INVALID, ERR_OOM, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT, ERR_KERNEL = -1, -2, -3, -4, -5, -6
ACC_STORE_A, ACC_STORE_B = 1, 2
ADD, SUB, MUL, DIV = 0, 1, 2, 3
SADD, SSUB, SMUL, SDIV, POW, RELU, SIGMOID, TANH, EXP = range(9)
EPI_NONE, EPI_BIAS, EPI_BIAS_RELU, EPI_RELU_MASK = 0, 1, 2, 3

# name -> (restype, argtypes); int-returning functions are status codes.
SIGNATURES = {
    "mg_last_error": (C.c_char_p, []),
    "mg_init": (C.c_int, [C.c_int]),
    "mg_shutdown": (C.c_int, []),
    "mg_device": (C.c_int, []),
    "mg_sm_count": (C.c_int, []),
    "mg_sync": (C.c_int, []),
    "mg_check_kernel_status": (C.c_int, []),
    "mg_kernel_status_mirror": (C.c_int, []),
    "mg_kernel_status_peek": (C.c_int, [_ip]),
    "mg_mem_info": (C.c_int, [C.POINTER(_sz), C.POINTER(_sz)]),
    "mg_pool_reserve": (C.c_int, [_sz]),
    "mg_alloc": (C.c_int, [_sz, C.POINTER(C.c_void_p)]),
    "mg_free": (C.c_int, [C.c_void_p]),
    "mg_alloc_i32": (C.c_int, [_sz, C.POINTER(C.c_void_p)]),
    "mg_free_i32": (C.c_int, [C.c_void_p]),
    "mg_upload": (C.c_int, [C.c_void_p, C.c_void_p, _sz]),
    "mg_download": (C.c_int, [C.c_void_p, C.c_void_p, _sz]),
    "mg_upload_async": (C.c_int, [C.c_void_p, C.c_void_p, _sz, _ip]),
    "mg_compute_wait_event": (C.c_int, [C.c_int]),
    "mg_upload_i32": (C.c_int, [C.c_void_p, C.c_void_p, _sz]),
    "mg_download_i32": (C.c_int, [C.c_void_p, C.c_void_p, _sz]),
    "mg_upload_u8_scaled": (C.c_int, [C.c_void_p, C.c_void_p, _sz, C.c_double]),
    "mg_fill": (C.c_int, [C.c_void_p, C.c_double, _sz]),
    "mg_copy": (C.c_int, [C.c_void_p, C.c_void_p, _sz]),
    "mg_host_alloc": (C.c_int, [_sz, C.POINTER(C.c_void_p)]),
    "mg_host_free": (C.c_int, [C.c_void_p]),
    "mg_binary_fwd": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, _sz]),
    "mg_binary_bwd": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                C.c_void_p, _sz, C.c_int]),
    "mg_unary_fwd": (C.c_int, [C.c_int, C.c_void_p, C.c_double, C.c_void_p, _sz]),
    "mg_unary_bwd": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_double, C.c_void_p,
                               C.c_void_p, _sz, C.c_int]),
    "mg_add_row_fwd": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, _sz, _sz]),
    "mg_add_row_bwd": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, _sz, _sz, C.c_int]),
    "mg_colsum_noalloc": (C.c_int, [C.c_void_p, C.c_void_p, _sz, _sz, C.c_int]),
    "mg_sum_all_fwd": (C.c_int, [C.c_void_p, C.c_void_p, _sz]),
    "mg_sum_all_bwd": (C.c_int, [C.c_void_p, C.c_void_p, _sz, C.c_int]),
    "mg_sum_lastaxis_fwd": (C.c_int, [C.c_void_p, C.c_void_p, _sz, _sz]),
    "mg_sum_lastaxis_bwd": (C.c_int, [C.c_void_p, C.c_void_p, _sz, _sz, C.c_int]),
    "mg_gemm_nn": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, _sz, _sz, _sz, C.c_int, C.c_int,
                             C.c_void_p]),
    "mg_gemm_nt": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, _sz, _sz, _sz, C.c_int, C.c_int,
                             C.c_void_p]),
    "mg_gemm_tn": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, _sz, _sz, _sz, C.c_int]),
    "mg_gemm_config": (C.c_int, [C.c_int, C.c_int]),
    "mg_softmax_xent_fwd": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, _sz, _sz, C.c_double]),
    "mg_softmax_xent_bwd": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, _sz, _sz,
                                      C.c_double, C.c_int]),
    "mg_argmax_rows": (C.c_int, [C.c_void_p, C.c_void_p, _sz, _sz]),
    "mg_f64_to_i32": (C.c_int, [C.c_void_p, C.c_void_p, _sz]),
    "mg_avg_pool_28": (C.c_int, [C.c_void_p, C.c_void_p, _sz]),
    "mg_sgd_step": (C.c_int, [C.c_void_p, C.c_void_p, C.c_double, _sz]),
    "mg_graph_begin": (C.c_int, []),
    "mg_graph_end": (C.c_int, [_ip]),
    "mg_graph_launch": (C.c_int, [C.c_int]),
    "mg_graph_kernels": (C.c_int, [C.c_int]),
    "mg_graph_destroy": (C.c_int, [C.c_int]),
    "mg_event_create": (C.c_int, [_ip]),
    "mg_event_record": (C.c_int, [C.c_int]),
    "mg_event_elapsed_ms": (C.c_int, [C.c_int, C.c_int, C.POINTER(C.c_float)]),
    "mg_event_destroy": (C.c_int, [C.c_int]),
    "mg_event_wait_bounded": (C.c_int, [C.c_int, C.c_double]),
    "mg_gemm_plan_describe": (C.c_int, [_sz, _sz, _sz, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int),
                                        C.c_int]),
    "mg_sgd_step_multi": (C.c_int, [C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(_sz), C.c_int,
                                    C.c_double]),
    "mg_scalar_mirror": (C.c_int, [C.c_void_p, C.POINTER(C.c_ulonglong)]),
    "mg_scalar_fetch": (C.c_int, [C.c_ulonglong, C.POINTER(C.c_double), C.POINTER(C.c_int)]),
    "mg_comm_unique_id": (C.c_int, [C.c_char_p]),
    "mg_comm_init": (C.c_int, [C.c_char_p, C.c_int, C.c_int]),
    "mg_comm_destroy": (C.c_int, []),
    "mg_comm_rank": (C.c_int, []),
    "mg_comm_world": (C.c_int, []),
    "mg_allreduce_sum_async": (C.c_int, [C.c_void_p, _sz]),
    "mg_allreduce_sum_async_hint": (C.c_int, [C.c_void_p, _sz, C.c_int]),
    "mg_comm_alloc_shared": (C.c_int, [_sz, C.POINTER(C.c_void_p)]),
    "mg_comm_free_shared": (C.c_int, [C.c_void_p]),
    "mg_comm_peer_path": (C.c_int, [C.c_void_p]),
    "mg_comm_join": (C.c_int, []),
    "mg_comm_trace": (C.c_int, [C.c_int]),
    "mg_comm_trace_summary": (C.c_int, [_dp, _ip, _dp, _ip]),
    "mg_comm_wait_bounded": (C.c_int, [C.c_double]),
    "mg_probe_dmma_tflops": (C.c_int, [C.c_int, C.c_int, _dp]),
    "mg_fill_uniform01": (C.c_int, [C.c_void_p, _sz, C.c_ulonglong, C.c_ulonglong]),
    "mg_flush_l2": (C.c_int, []),
    "mg_launch_count": (C.c_ulonglong, []),
}

# Entry points whose int result is a value, not a status.
_VALUE_INT = {"mg_device", "mg_sm_count", "mg_comm_rank", "mg_comm_world", "mg_comm_peer_path",
              "mg_graph_kernels"}


def declared_in_header(header_text: str) -> list[str]:
    """Names of all functions a C header declares with the ``mg_``/``mgt_`` prefix."""
    return sorted(set(re.findall(r"\b(mgt?_[a-z0-9_]+)\s*\(", header_text)))


class MgError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code


class CudaABI:
    def __init__(self, path: str):
        self.lib = C.CDLL(path, mode=C.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(self.lib, name)
            fn.restype, fn.argtypes = res, args

    def last_error(self) -> str:
        return (self.lib.mg_last_error() or b"").decode()

    def call(self, name: str, *args):
        """Call a status-returning entry point; raise MgError on failure."""
        rc = getattr(self.lib, name)(*args)
        if name not in _VALUE_INT and SIGNATURES[name][0] is C.c_int and rc != OK:
            raise MgError(rc, self.last_error())
        return rc

    def __getattr__(self, name: str):
        if name.startswith("mg_") and name in SIGNATURES:
            return lambda *a: self.call(name, *a)
        raise AttributeError(name)

    # ---- conveniences ----
    def array(self, values) -> "DeviceArray":
        return DeviceArray.from_numpy(self, values)

    def empty(self, n: int) -> "DeviceArray":
        return DeviceArray(self, int(n))

    def zeros(self, n: int) -> "DeviceArray":
        a = DeviceArray(self, int(n))
        self.mg_fill(a.ptr, 0.0, a.n)
        return a

    def int_array(self, values) -> "DeviceInts":
        return DeviceInts.from_numpy(self, values)

    def timed_ms(self, fn, iters: int = 1) -> float:
        """Device time of ``iters`` calls of fn(), by events on the compute stream."""
        e0, e1 = C.c_int(), C.c_int()
        self.mg_event_create(C.byref(e0))
        self.mg_event_create(C.byref(e1))
        self.mg_event_record(e0.value)
        for _ in range(iters):
            fn()
        self.mg_event_record(e1.value)
        ms = C.c_float()
        self.mg_event_elapsed_ms(e0.value, e1.value, C.byref(ms))
        self.mg_event_destroy(e0.value)
        self.mg_event_destroy(e1.value)
        return float(ms.value)


class DeviceArray:
    """fp64 device buffer from mg_alloc (freed on garbage collection)."""

    def __init__(self, abi: CudaABI, n: int):
        self.abi, self.n = abi, int(n)
        p = C.c_void_p()
        abi.mg_alloc(self.n, C.byref(p))
        self.ptr = p.value

    @classmethod
    def from_numpy(cls, abi: CudaABI, values) -> "DeviceArray":
        arr = np.ascontiguousarray(values, dtype=np.float64)
        out = cls(abi, arr.size)
        abi.mg_upload(out.ptr, arr.ctypes.data, arr.size)
        return out

    def numpy(self, shape=None) -> np.ndarray:
        out = np.empty(self.n, dtype=np.float64)
        self.abi.mg_download(out.ctypes.data, self.ptr, self.n)
        return out.reshape(shape) if shape is not None else out

    def offset(self, elems: int) -> int:
        return self.ptr + 8 * int(elems)

    def __del__(self):
        if getattr(self, "ptr", None):
            try:
                self.abi.lib.mg_free(self.ptr)
            except Exception:
                pass
            self.ptr = None


class DeviceInts:
    """int32 device buffer (class ids)."""

    def __init__(self, abi: CudaABI, n: int):
        self.abi, self.n = abi, int(n)
        p = C.c_void_p()
        abi.mg_alloc_i32(self.n, C.byref(p))
        self.ptr = p.value

    @classmethod
    def from_numpy(cls, abi: CudaABI, values) -> "DeviceInts":
        arr = np.ascontiguousarray(values, dtype=np.int32)
        out = cls(abi, arr.size)
        abi.mg_upload_i32(out.ptr, arr.ctypes.data, arr.size)
        return out

    def numpy(self) -> np.ndarray:
        out = np.empty(self.n, dtype=np.int32)
        self.abi.mg_download_i32(out.ctypes.data, self.ptr, self.n)
        return out

    def __del__(self):
        if getattr(self, "ptr", None):
            try:
                self.abi.lib.mg_free_i32(self.ptr)
            except Exception:
                pass
            self.ptr = None
