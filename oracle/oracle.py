"""ctypes front end of the CPU oracle (``boostr_cpu_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by
the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.  The product package
never imports this module.

Every function mirrors one piece of boostr's CPU implementation; the C source cites
the reference file and lines each one follows.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

FMT_Q4_0, FMT_Q5_0, FMT_Q8_0, FMT_Q2_K, FMT_Q3_K, FMT_Q4_K, FMT_Q5_K, FMT_Q6_K = 0, 2, 4, 6, 7, 8, 9, 10
FORMATS = {"Q4_0": FMT_Q4_0, "Q5_0": FMT_Q5_0, "Q8_0": FMT_Q8_0, "Q2_K": FMT_Q2_K, "Q3_K": FMT_Q3_K, "Q4_K": FMT_Q4_K, "Q5_K": FMT_Q5_K, "Q6_K": FMT_Q6_K}
Q8K_BLOCK_BYTES = 292

_libs: dict[str, ctypes.CDLL] = {}


def build(force: bool = False) -> None:
    """Compile the oracle with the Makefile beside this file (gcc only)."""
    target = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "boostr_cpu_oracle.c")
    if force or not os.path.exists(target) or os.path.getmtime(target) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "all"], check=True, capture_output=True)


def _lib(name: str = "liboracle.so") -> ctypes.CDLL:
    if name not in _libs:
        path = os.path.join(_HERE, name)
        if not os.path.exists(path):
            build(force=True)
        lib = ctypes.CDLL(path)
        c = ctypes
        lib.oracle_block_size.argtypes = [c.c_int]
        lib.oracle_block_bytes.argtypes = [c.c_int]
        lib.oracle_f16_to_f32.argtypes = [c.c_uint16]
        lib.oracle_f16_to_f32.restype = c.c_float
        lib.oracle_f32_to_bf16.argtypes = [c.c_float]
        lib.oracle_f32_to_bf16.restype = c.c_uint16
        lib.oracle_f32_to_f16.argtypes = [c.c_float]
        lib.oracle_f32_to_f16.restype = c.c_uint16
        lib.oracle_dequant_f32.argtypes = [c.c_int, c.c_void_p, c.c_size_t, c.c_void_p]
        lib.oracle_dequant_16.argtypes = [c.c_int, c.c_void_p, c.c_size_t, c.c_void_p, c.c_int]
        lib.oracle_quantize_q8k.argtypes = [c.c_void_p, c.c_size_t, c.c_void_p]
        lib.oracle_quantize_q8k.restype = None
        lib.oracle_dot_q8k.argtypes = [c.c_int, c.c_void_p, c.c_void_p, c.c_size_t, c.c_int]
        lib.oracle_dot_q8k.restype = c.c_float
        lib.oracle_dot_f32.argtypes = [c.c_void_p, c.c_void_p, c.c_size_t]
        lib.oracle_dot_f32.restype = c.c_float
        lib.oracle_quant_matmul.argtypes = [c.c_int, c.c_void_p, c.c_void_p, c.c_void_p, c.c_size_t, c.c_size_t,
                                            c.c_size_t, c.c_int, c.c_int]
        lib.oracle_quant_swiglu.argtypes = [c.c_int, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_size_t,
                                            c.c_size_t, c.c_size_t, c.c_int, c.c_int]
        lib.oracle_matmul_exact_f64.argtypes = [c.c_int, c.c_void_p, c.c_void_p, c.c_void_p, c.c_size_t, c.c_size_t,
                                                c.c_size_t]
        _libs[name] = lib
    return _libs[name]


def _fmt(fmt) -> int:
    return FORMATS[fmt] if isinstance(fmt, str) else int(fmt)


def _ptr(a: np.ndarray) -> int:
    return a.ctypes.data


def block_size(fmt) -> int:
    return _lib().oracle_block_size(_fmt(fmt))


def block_bytes(fmt) -> int:
    return _lib().oracle_block_bytes(_fmt(fmt))


def _check_blocks(fmt, blocks: np.ndarray) -> int:
    assert blocks.dtype == np.uint8 and blocks.flags.c_contiguous
    bb = block_bytes(fmt)
    assert bb and blocks.size % bb == 0, "byte count is not a whole number of blocks"
    return blocks.size // bb


def dequantize_f32(fmt, blocks: np.ndarray, lib: str = "liboracle.so") -> np.ndarray:
    """boostr CpuClient::dequantize(.., F32) over a flat run of blocks."""
    nb = _check_blocks(fmt, blocks)
    out = np.empty(nb * block_size(fmt), dtype=np.float32)
    rc = _lib(lib).oracle_dequant_f32(_fmt(fmt), _ptr(blocks), nb, _ptr(out))
    assert rc == 0
    return out


def dequantize_16(fmt, blocks: np.ndarray, kind: str) -> np.ndarray:
    """dequantize to bf16 / f16 bit patterns (uint16).  The cast is numr's: parity unpinned."""
    nb = _check_blocks(fmt, blocks)
    out = np.empty(nb * block_size(fmt), dtype=np.uint16)
    rc = _lib().oracle_dequant_16(_fmt(fmt), _ptr(blocks), nb, _ptr(out), {"bf16": 1, "f16": 2}[kind])
    assert rc == 0
    return out


def quantize_q8k(x: np.ndarray, lib: str = "liboracle.so") -> np.ndarray:
    """boostr quantize_f32_to_q8k (AVX2 semantics) of a flat f32 array, length % 256 == 0."""
    x = np.ascontiguousarray(x, dtype=np.float32).ravel()
    assert x.size % 256 == 0
    out = np.zeros(x.size // 256 * Q8K_BLOCK_BYTES, dtype=np.uint8)
    _lib(lib).oracle_quantize_q8k(_ptr(x), x.size, _ptr(out))
    return out


def dot_q8k(fmt, act_q8k: np.ndarray, wrow: np.ndarray, k: int, simd: bool = False, lib: str = "liboracle.so") -> float:
    return float(_lib(lib).oracle_dot_q8k(_fmt(fmt), _ptr(act_q8k), _ptr(wrow), k, int(simd)))


def dot_f32(a: np.ndarray, b: np.ndarray, lib: str = "liboracle.so") -> float:
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    assert a.size == b.size
    return float(_lib(lib).oracle_dot_f32(_ptr(a), _ptr(b), a.size))


def quant_matmul(fmt, act: np.ndarray, w: np.ndarray, n: int, threads: int = 1, simd: bool = True,
                 lib: str = "liboracle.so") -> np.ndarray:
    """boostr CpuClient::quant_matmul: act [M,K] f32 x packed weight [N,K] -> [M,N] f32."""
    act = np.ascontiguousarray(act, dtype=np.float32)
    m, k = act.shape
    assert w.dtype == np.uint8 and w.flags.c_contiguous
    assert w.size == n * (k // block_size(fmt)) * block_bytes(fmt)
    out = np.empty((m, n), dtype=np.float32)
    rc = _lib(lib).oracle_quant_matmul(_fmt(fmt), _ptr(act), _ptr(w), _ptr(out), m, k, n, threads, int(simd))
    assert rc == 0, rc
    return out


def quant_swiglu(fmt, act: np.ndarray, wg: np.ndarray, wu: np.ndarray, n: int, threads: int = 1) -> np.ndarray:
    act = np.ascontiguousarray(act, dtype=np.float32)
    m, k = act.shape
    out = np.empty((m, n), dtype=np.float32)
    rc = _lib().oracle_quant_swiglu(_fmt(fmt), _ptr(act), _ptr(wg), _ptr(wu), _ptr(out), m, k, n, threads, 1)
    assert rc == 0, rc
    return out


def matmul_exact_f64(fmt, act: np.ndarray, w: np.ndarray, n: int) -> np.ndarray:
    """Diagnostic: exact dequantised weights x f32 activations accumulated in f64."""
    act = np.ascontiguousarray(act, dtype=np.float32)
    m, k = act.shape
    out = np.empty((m, n), dtype=np.float64)
    rc = _lib().oracle_matmul_exact_f64(_fmt(fmt), _ptr(act), _ptr(w), _ptr(out), m, k, n)
    assert rc == 0
    return out


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (vectorised; same rule as the C cast)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)
