"""Host-side checks that need no GPU: the C-ABI library loads and exports every symbol the
header declares, format arithmetic, argument validation that fails before any launch, and the
tensor-parallel shard packer against a numpy restatement."""
import ctypes
import os
import re

import numpy as np
import pytest

from boostr_b200 import _cabi, synth
from boostr_b200.format import QuantError, QuantFormat as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from boostr_b200 import build

    build.build()
    return _cabi.lib()


def test_header_symbols_are_exported(lib):
    hdr = open(os.path.join(ROOT, "include", "b200q.h")).read()
    declared = set(re.findall(r"B200Q_API\s+[\w\s\*]+?\b(b200q_\w+)\s*\(", hdr))
    assert declared, "no declarations found in include/b200q.h"
    assert declared == set(_cabi.SIGNATURES), declared ^ set(_cabi.SIGNATURES)
    for name in declared:
        assert getattr(lib, name) is not None


def test_rust_extern_block_names_the_header_symbols():
    # the Rust -sys crate cannot be compiled here; at least its declarations must cover the header exactly
    hdr = open(os.path.join(ROOT, "include", "b200q.h")).read()
    declared = set(re.findall(r"B200Q_API\s+[\w\s\*]+?\b(b200q_\w+)\s*\(", hdr))
    rs = open(os.path.join(ROOT, "rust", "b200q-sys", "src", "lib.rs")).read()
    bound = set(re.findall(r"pub fn (b200q_\w+)\s*\(", rs))
    assert bound == declared, bound ^ declared


def test_format_tables(lib):
    for f in F:
        assert lib.b200q_block_size(f.format_id) == f.block_size
        assert lib.b200q_block_bytes(f.format_id) == f.block_bytes
        out = ctypes.c_size_t()
        assert lib.b200q_storage_bytes(f.format_id, f.block_size * 7, ctypes.byref(out)) == _cabi.OK
        assert out.value == 7 * f.block_bytes == f.storage_bytes(7 * f.block_size)
        assert lib.b200q_storage_bytes(f.format_id, f.block_size * 7 + 1, ctypes.byref(out)) == _cabi.ERR_BAD_SHAPE
        assert b"not a multiple of block_size" in lib.b200q_last_error()
    assert lib.b200q_block_size(3) == 0
    assert [f.ggml_type_id for f in (F.Q4_0, F.Q8_0, F.Q4_K, F.Q6_K)] == [2, 8, 12, 14]
    assert F.from_ggml_type_id(12) is F.Q4_K
    with pytest.raises(QuantError):
        F.Q4_K.storage_bytes(255)


def test_validation_fails_before_launch(lib):
    # bad arguments are rejected on the host; nothing touches a device
    fake = ctypes.c_void_p(0x1000)
    rc = lib.b200q_quant_matmul(99, fake, 0, fake, fake, 0, 1, 256, 1, None, 0, None)
    assert rc == _cabi.ERR_UNSUPPORTED_FORMAT
    rc = lib.b200q_quant_matmul(F.Q4_K.format_id, fake, 0, fake, fake, 0, 1, 100, 1, None, 0, None)
    assert rc == _cabi.ERR_BAD_SHAPE and b"not a multiple" in lib.b200q_last_error()
    rc = lib.b200q_quant_matmul(F.Q4_K.format_id, fake, 2, fake, fake, 0, 1, 256, 1, None, 0, None)
    assert rc == _cabi.ERR_UNSUPPORTED_DTYPE and b"must be F32" in lib.b200q_last_error()
    rc = lib.b200q_quant_matmul(F.Q4_K.format_id, fake, 0, ctypes.c_void_p(0x1004), fake, 0, 1, 256, 1, None, 0, None)
    assert rc == _cabi.ERR_INVALID_ARG
    rc = lib.b200q_quant_matmul(F.Q4_K.format_id, None, 0, fake, fake, 0, 1, 256, 1, None, 0, None)
    assert rc == _cabi.ERR_INVALID_ARG
    rc = lib.b200q_quant_matmul(F.Q4_K.format_id, fake, 0, fake, fake, 0, 0, 256, 1, None, 0, None)
    assert rc == _cabi.ERR_BAD_SHAPE
    rc = lib.b200q_dequantize(F.Q8_0.format_id, fake, 4, fake, 9, None)
    assert rc == _cabi.ERR_UNSUPPORTED_DTYPE and b"must be float" in lib.b200q_last_error()
    assert lib.b200q_dequantize(F.Q8_0.format_id, fake, 0, fake, 0, None) == _cabi.OK  # empty tensor: nothing to do


def test_prefetch_hint_validation_needs_no_device(lib):
    fm = (ctypes.c_int * 2)(F.Q4_K.format_id, F.Q4_K.format_id)
    wp = (ctypes.c_void_p * 2)(0x1000, 0x2000)
    ns = (ctypes.c_size_t * 2)(512, 512)
    assert lib.b200q_prefetch_next(5, 1, fm, wp, ns, 4096) == _cabi.ERR_INVALID_ARG and b"unknown operation" in lib.b200q_last_error()
    assert lib.b200q_prefetch_next(_cabi.OP_QUANT_MATMUL, 0, fm, wp, ns, 4096) == _cabi.ERR_INVALID_ARG
    assert lib.b200q_prefetch_next(_cabi.OP_QUANT_MATMUL, 2, fm, None, ns, 4096) == _cabi.ERR_INVALID_ARG
    bad = (ctypes.c_int * 1)(3)
    assert lib.b200q_prefetch_next(_cabi.OP_QUANT_MATMUL, 1, bad, wp, ns, 4096) == _cabi.ERR_UNSUPPORTED_FORMAT
    odd = (ctypes.c_void_p * 1)(0x1008)
    assert lib.b200q_prefetch_next(_cabi.OP_QUANT_MATMUL, 1, fm, odd, ns, 4096) == _cabi.ERR_INVALID_ARG
    # a well-formed hint on a machine without a usable device is dropped, not an error: nothing will consume it
    assert lib.b200q_prefetch_next(_cabi.OP_QUANT_SWIGLU, 2, fm, wp, ns, 4096) == _cabi.OK
    # ... and any compute call ends a hint's life: on a machine WITH a device the made-up pointers above must not survive
    assert lib.b200q_dequantize(F.Q8_0.format_id, ctypes.c_void_p(0x1000), 0, ctypes.c_void_p(0x1000), 0, None) == _cabi.OK


@pytest.mark.parametrize("fmt", list(F))
@pytest.mark.parametrize("world", [1, 2, 4])
def test_shard_pack_matches_numpy(lib, fmt, world):
    from boostr_b200.tensor_parallel import shard_bytes

    n, k = 8, fmt.block_size * 8
    rng = synth.rng_for(40, fmt.value + world)
    w = synth.weight_bytes(fmt, rng, n, k)
    rows = w.reshape(n, -1)
    for rank in range(world):
        got0 = shard_bytes(fmt, w, n, k, 0, rank, world)
        assert np.array_equal(got0, rows[rank * n // world:(rank + 1) * n // world].reshape(-1))
        got1 = shard_bytes(fmt, w, n, k, 1, rank, world)
        lb = rows.shape[1] // world
        assert np.array_equal(got1, np.ascontiguousarray(rows[:, rank * lb:(rank + 1) * lb]).reshape(-1))


def test_shard_pack_errors():
    from boostr_b200.tensor_parallel import DistributedError, shard_bytes

    w = synth.weight_bytes(F.Q4_K, synth.rng_for(41), 6, 512)
    with pytest.raises(DistributedError, match="not divisible"):
        shard_bytes(F.Q4_K, w, 6, 512, 0, 0, 4)  # reference reaches this with world_size 3 (tensor_parallel.rs:450-459)
    with pytest.raises(DistributedError, match="block_size"):
        shard_bytes(F.Q4_K, w, 6, 512, 1, 0, 4)  # 128 columns per rank < one 256-block
    with pytest.raises(DistributedError):
        shard_bytes(F.Q4_K, w, 6, 512, 2, 0, 2)


def test_sharded_products_recombine(oracle):
    """Column shards concatenate, row shards add up to the unsharded product (oracle arithmetic):
    with K split on 256-boundaries the Q8_K activation blocks of a shard are those of the full row."""
    from boostr_b200.tensor_parallel import shard_bytes

    rng = synth.rng_for(42)
    m, n, k, p = 3, 16, 2048, 4
    act = synth.activations(rng, m, k)
    for fmt in ("Q4_K", "Q6_K", "Q8_0"):
        w = synth.weight_bytes(fmt, rng, n, k)
        full = oracle.quant_matmul(fmt, act, w, n)
        cols = [oracle.quant_matmul(fmt, act, shard_bytes(fmt, w, n, k, 0, r, p), n // p) for r in range(p)]
        assert np.array_equal(np.concatenate(cols, axis=1), full)
        parts = [oracle.quant_matmul(fmt, np.ascontiguousarray(act[:, r * k // p:(r + 1) * k // p]),
                                     shard_bytes(fmt, w, n, k, 1, r, p), n) for r in range(p)]
        tot = np.sum(np.stack(parts).astype(np.float64), axis=0)
        assert np.abs(tot - full).max() <= 2e-6 * np.abs(full).max()
