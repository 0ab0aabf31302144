"""ctypes binding of ``libb200q.so`` (the C ABI declared in ``include/b200q.h``).

The library is the product; this module only loads it and declares signatures.  There is
no CPU fallback: if the shared object is missing or cannot be loaded, importing the
operators fails with an error that says how to build it.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_int, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200q.so")

OK, ERR_INVALID_ARG, ERR_UNSUPPORTED_FORMAT, ERR_BAD_SHAPE, ERR_WORKSPACE_TOO_SMALL, ERR_CUDA, ERR_TIMEOUT, \
    ERR_UNSUPPORTED_DTYPE, ERR_NOT_FUSED = range(9)
DT_F32, DT_BF16, DT_F16, DT_F64 = range(4)
OP_QUANT_MATMUL, OP_QUANT_SWIGLU = 0, 1
STATIC_SCRATCH_BYTES = 8 << 20
TP_HANDLE_BYTES = 64

# every symbol include/b200q.h declares: name -> (restype, argtypes)
SIGNATURES = {
    "b200q_version": (c_int, []),
    "b200q_last_error": (c_char_p, []),
    "b200q_block_size": (c_size_t, [c_int]),
    "b200q_block_bytes": (c_size_t, [c_int]),
    "b200q_storage_bytes": (c_int, [c_int, c_size_t, POINTER(c_size_t)]),
    "b200q_dequantize": (c_int, [c_int, c_void_p, c_size_t, c_void_p, c_int, c_void_p]),
    "b200q_workspace_bytes": (c_size_t, [c_int, c_int, c_size_t, c_size_t, c_size_t]),
    "b200q_quant_matmul": (c_int, [c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_size_t, c_size_t, c_size_t,
                                   c_void_p, c_size_t, c_void_p]),
    "b200q_quant_matmul_batch": (c_int, [c_int, POINTER(c_int), POINTER(c_void_p), POINTER(c_size_t),
                                         POINTER(c_void_p), c_void_p, c_int, c_int, c_size_t, c_size_t, c_void_p,
                                         c_size_t, c_void_p]),
    "b200q_rmsnorm_quant_matmul_batch": (c_int, [c_int, POINTER(c_int), POINTER(c_void_p), POINTER(c_size_t), POINTER(c_void_p),
                                                 c_void_p, c_void_p, ctypes.c_float, c_int, c_int, c_size_t, c_size_t, c_void_p,
                                                 c_size_t, c_void_p]),
    "b200q_quant_swiglu": (c_int, [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_size_t, c_size_t,
                                   c_size_t, c_void_p, c_size_t, c_void_p]),
    "b200q_mlp_workspace_bytes": (c_size_t, [c_int, c_int, c_size_t, c_size_t, c_size_t, c_size_t]),
    "b200q_quant_mlp": (c_int, [c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_size_t, c_size_t,
                                c_size_t, c_size_t, c_void_p, c_size_t, c_void_p]),
    "b200q_prefetch_next": (c_int, [c_int, c_int, POINTER(c_int), POINTER(c_void_p), POINTER(c_size_t), c_size_t]),
    "b200q_quant_matmul_static_scratch": (c_int, [c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_size_t, c_size_t,
                                                  c_size_t, c_void_p]),
    "b200q_shard_pack": (c_int, [c_int, c_void_p, c_size_t, c_size_t, c_int, c_int, c_int, c_void_p, c_size_t]),
    "b200q_check_device_status": (c_int, [c_void_p]),
    "b200q_tp_buffer_bytes": (c_size_t, []),
    "b200q_tp_alloc": (c_int, [POINTER(c_void_p), ctypes.c_char_p]),
    "b200q_tp_open": (c_int, [ctypes.c_char_p, POINTER(c_void_p)]),
    "b200q_tp_close": (c_int, [c_void_p]),
    "b200q_tp_free": (c_int, [c_void_p]),
    "b200q_row_parallel_matmul": (c_int, [c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_size_t, c_size_t, c_size_t,
                                          c_int, c_int, POINTER(c_void_p), c_void_p]),
    "b200q_col_parallel_matmul_gather": (c_int, [c_int, c_void_p, c_int, c_void_p, c_void_p, c_size_t, c_size_t, c_size_t,
                                                 c_int, c_int, POINTER(c_void_p), c_void_p]),
    "b200q_tp_all_reduce": (c_int, [c_void_p, c_size_t, c_int, c_int, POINTER(c_void_p), c_void_p]),
    "b200q_launch_count": (ctypes.c_ulonglong, []),
}

_lib = None


class B200QError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"b200q status {code}: {message}")
        self.code = code
        self.message = message


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m boostr_b200.build` (needs nvcc; no GPU required). "
                "There is no CPU fallback for the quantized-linear path.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(code: int) -> None:
    if code != OK:
        raise B200QError(code, lib().b200q_last_error().decode())
