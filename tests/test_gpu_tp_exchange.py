"""Fused row-parallel decode product (b200q_row_parallel_matmul) on ONE GPU.

Two exchange buffers are allocated on the same device and the peer's contribution (its partial row,
every element tagged with the epoch) is staged by the host before the launch, so the kernel's wait is
satisfied at once and no kernel ever waits for another launch.  What is checked: the pushed partial
row lands in the peer's buffer under the right parity and tag, the epoch advances, the rank-ordered sum
is bit-identical to the plain sum of the two partial products, over several consecutive calls (both
parities).
"""
import ctypes

import numpy as np
import pytest
import torch

from boostr_b200 import _cabi, synth
from boostr_b200.format import QuantFormat
from boostr_b200.tensor import QuantTensor
from boostr_b200.tensor_parallel import shard_bytes

pytestmark = pytest.mark.gpu

@pytest.fixture(scope="module")
def ops():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from boostr_b200 import ops as o

    return o


INBOX0 = 1024


def _half_bytes():
    """One parity half of the exchange area: 8 rank rows of {f32 bits, epoch} slots."""
    return (_cabi.lib().b200q_tp_buffer_bytes() - INBOX0) // 2


def _row_bytes():
    return _half_bytes() // 8


def _cudart():
    for name in ("libcudart.so.12", "libcudart.so"):
        try:
            return ctypes.CDLL(name)
        except OSError:
            continue
    pytest.skip("libcudart not loadable for raw device copies")


def _h2d(rt, dst, arr):
    assert rt.cudaMemcpy(ctypes.c_void_p(dst), ctypes.c_void_p(arr.ctypes.data), ctypes.c_size_t(arr.nbytes), 1) == 0


def _d2h(rt, src, nbytes):
    out = np.empty(nbytes, dtype=np.uint8)
    assert rt.cudaMemcpy(ctypes.c_void_p(out.ctypes.data), ctypes.c_void_p(src), ctypes.c_size_t(nbytes), 2) == 0
    return out


@pytest.mark.parametrize("fmt,n,k", [("Q4_K", 4096, 4096), ("Q6_K", 4096, 14336), ("Q6_K", 300, 2048), ("Q4_K", 37, 1024)])
def test_row_parallel_exchange_against_staged_peer(ops, fmt, n, k):
    rt = _cudart()
    L = _cabi.lib()
    torch.cuda.synchronize()
    bufs, table = [], (ctypes.c_void_p * 2)()
    for r in range(2):
        b, h = ctypes.c_void_p(), ctypes.create_string_buffer(_cabi.TP_HANDLE_BYTES)
        _cabi.check(L.b200q_tp_alloc(ctypes.byref(b), h))
        bufs.append(b.value)
        table[r] = b.value
    try:
        rng = synth.rng_for(41, n + k)
        full = synth.weight_bytes(fmt, rng, n, k)
        f = QuantFormat.parse(fmt)
        shards = [QuantTensor.from_bytes(shard_bytes(fmt, full, n, k, 1, r, 2), f, (n, k // 2), device="cuda") for r in range(2)]
        for call in range(1, 5):  # epochs 1..4: both parities twice
            act = synth.activations(rng, 1, k)
            a = [torch.from_numpy(np.ascontiguousarray(act[:, r * (k // 2):(r + 1) * (k // 2)])).cuda() for r in range(2)]
            y = [ops.quant_matmul(a[r], shards[r]) for r in range(2)]
            torch.cuda.synchronize()
            # stage rank 1's push into rank 0's buffer: {value bits, epoch} per element
            par = call & 1
            staged = np.empty((n, 2), dtype=np.uint32)
            staged[:, 0] = y[1].cpu().numpy().reshape(-1).view(np.uint32)
            staged[:, 1] = call
            _h2d(rt, bufs[0] + INBOX0 + (par * 8 + 1) * _row_bytes(), staged)
            out = ops.row_parallel_matmul(a[0], shards[0], 0, 2, table)
            assert out is not None
            ops.check_device_status()
            want = (y[0] + y[1]).cpu().numpy()
            assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32)), f"call {call}"
            # what rank 0 left behind: its tagged row in the peer's inbox, its epoch
            pushed = _d2h(rt, bufs[1] + INBOX0 + (par * 8 + 0) * _row_bytes(), n * 8).view(np.uint32).reshape(n, 2)
            assert np.array_equal(pushed[:, 0], y[0].cpu().numpy().reshape(-1).view(np.uint32))
            assert (pushed[:, 1] == call).all()
            ctl = _d2h(rt, bufs[0], 8).view(np.uint32)
            assert ctl[0] == call and ctl[1] == 0
    finally:
        torch.cuda.synchronize()
        for b in bufs:
            L.b200q_tp_free(b)


@pytest.mark.parametrize("fmt,n_local,k", [("Q6_K", 16032, 4096), ("Q4_K", 300, 1024), ("Q6_K", 37, 512)])
def test_col_parallel_gather_against_staged_peer(ops, fmt, n_local, k):
    """Fused column-parallel gather (b200q_col_parallel_matmul_gather) on one GPU: rank 1's slice of the
    assembled row is staged by the host with the right tags before the launch; rank 0 must deliver
    [own slice | peer slice] and leave its own slice, tagged, in the peer's buffer.  The row-parallel exchange
    alternates with it on the same buffers (both kinds share the epoch)."""
    rt = _cudart()
    L = _cabi.lib()
    torch.cuda.synchronize()
    bufs, table = [], (ctypes.c_void_p * 2)()
    for r in range(2):
        b, h = ctypes.c_void_p(), ctypes.create_string_buffer(_cabi.TP_HANDLE_BYTES)
        _cabi.check(L.b200q_tp_alloc(ctypes.byref(b), h))
        bufs.append(b.value)
        table[r] = b.value
    try:
        rng = synth.rng_for(44, n_local + k)
        f = QuantFormat.parse(fmt)
        shards = [QuantTensor.from_bytes(synth.weight_bytes(fmt, rng, n_local, k), f, (n_local, k), device="cuda") for _ in range(2)]
        half_bytes = _half_bytes()
        for call in range(1, 4):
            act = torch.from_numpy(synth.activations(rng, 1, k)).cuda()
            y = [ops.quant_matmul(act, shards[r]) for r in range(2)]
            torch.cuda.synchronize()
            par = call & 1
            staged = np.empty((n_local, 2), dtype=np.uint32)
            staged[:, 0] = y[1].cpu().numpy().reshape(-1).view(np.uint32)
            staged[:, 1] = call
            _h2d(rt, bufs[0] + INBOX0 + par * half_bytes + n_local * 8, staged)   # columns [n_local, 2 n_local)
            full = torch.full((1, 2 * n_local), float("nan"), device="cuda")
            out = ops.col_parallel_matmul_gather(act, shards[0], 0, 2, table, full)
            assert out is not None
            ops.check_device_status()
            want = torch.cat(y, dim=-1)
            assert torch.equal(out.view(torch.int32), want.view(torch.int32)), f"call {call}"
            pushed = _d2h(rt, bufs[1] + INBOX0 + par * half_bytes, n_local * 8).view(np.uint32).reshape(n_local, 2)
            assert np.array_equal(pushed[:, 0], y[0].cpu().numpy().reshape(-1).view(np.uint32)) and (pushed[:, 1] == call).all()
            ctl = _d2h(rt, bufs[0], 8).view(np.uint32)
            assert ctl[0] == call and ctl[1] == 0
        # shapes without a fused gather launch nothing
        before = ops.launch_count()
        big = QuantTensor.from_bytes(synth.weight_bytes("Q4_K", rng, 270000, 256), QuantFormat.Q4_K, (270000, 256), device="cuda")
        a256 = torch.from_numpy(synth.activations(rng, 1, 256)).cuda()
        assert ops.col_parallel_matmul_gather(a256, big, 0, 2, table, torch.empty(1, 540000, device="cuda")) is None
        a2 = torch.from_numpy(synth.activations(rng, 2, k)).cuda()
        assert ops.col_parallel_matmul_gather(a2, shards[0], 0, 2, table, torch.empty(2, 2 * n_local, device="cuda")) is None
        assert ops.launch_count() == before
    finally:
        torch.cuda.synchronize()
        for b in bufs:
            L.b200q_tp_free(b)


def test_row_parallel_shapes_without_fused_path_launch_nothing(ops):
    L = _cabi.lib()
    b, h = ctypes.c_void_p(), ctypes.create_string_buffer(_cabi.TP_HANDLE_BYTES)
    _cabi.check(L.b200q_tp_alloc(ctypes.byref(b), h))
    try:
        table = (ctypes.c_void_p * 2)(b.value, b.value)
        rng = synth.rng_for(42)
        before = ops.launch_count()
        for fmt, m, n, k in [("Q8_0", 1, 64, 256), ("Q4_K", 2, 64, 256), ("Q4_K", 1, 70000, 256), ("Q4_K", 1, 64, 8192)]:
            w = QuantTensor.from_bytes(synth.weight_bytes(fmt, rng, n, k), QuantFormat.parse(fmt), (n, k), device="cuda")
            act = torch.from_numpy(synth.activations(rng, m, k)).cuda()
            assert ops.row_parallel_matmul(act, w, 0, 2, table) is None
        assert ops.launch_count() == before
    finally:
        L.b200q_tp_free(b.value)


@pytest.mark.parametrize("count", [1, 300, 4096, 16 * 4096])
def test_exchange_all_reduce_against_staged_peer(ops, count):
    """b200q_tp_all_reduce on one GPU: the peer's values are staged, tagged, by the host; rank 0 must leave the
    rank-ordered sum in place, its own values tagged in the peer's buffer and the epoch advanced; it alternates with
    the fused row-parallel product on the same buffers."""
    rt = _cudart()
    L = _cabi.lib()
    torch.cuda.synchronize()
    bufs, table = [], (ctypes.c_void_p * 2)()
    for r in range(2):
        b, h = ctypes.c_void_p(), ctypes.create_string_buffer(_cabi.TP_HANDLE_BYTES)
        _cabi.check(L.b200q_tp_alloc(ctypes.byref(b), h))
        bufs.append(b.value)
        table[r] = b.value
    try:
        rng = np.random.default_rng(count)
        for call in range(1, 4):
            mine = rng.standard_normal(count).astype(np.float32)
            peer = rng.standard_normal(count).astype(np.float32)
            par = call & 1
            staged = np.empty((count, 2), dtype=np.uint32)
            staged[:, 0] = peer.view(np.uint32)
            staged[:, 1] = call
            _h2d(rt, bufs[0] + INBOX0 + (par * 8 + 1) * _row_bytes(), staged)
            t = torch.from_numpy(mine.copy()).cuda()
            assert ops.tp_all_reduce(t, 0, 2, table)
            ops.check_device_status()
            want = (mine + peer).astype(np.float32)  # rank order: 0 then 1
            assert np.array_equal(t.cpu().numpy().view(np.uint32), want.view(np.uint32)), f"call {call}"
            pushed = _d2h(rt, bufs[1] + INBOX0 + (par * 8 + 0) * _row_bytes(), count * 8).view(np.uint32).reshape(count, 2)
            assert np.array_equal(pushed[:, 0], mine.view(np.uint32)) and (pushed[:, 1] == call).all()
            ctl = _d2h(rt, bufs[0], 8).view(np.uint32)
            assert ctl[0] == call and ctl[1] == 0
        before = ops.launch_count()
        assert not ops.tp_all_reduce(torch.zeros(70000, device="cuda"), 0, 2, table)  # does not fit: nothing launched
        assert ops.launch_count() == before
    finally:
        torch.cuda.synchronize()
        for b in bufs:
            L.b200q_tp_free(b)
