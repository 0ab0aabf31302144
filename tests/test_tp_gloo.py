"""World-size-2 and -4 collectives of the tensor-parallel layer on CPU ranks (gloo): the
row-major all-gather of column shards and the all-reduce of row-parallel partial products,
with the per-rank products computed by the CPU oracle."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from boostr_b200 import synth
        from boostr_b200.tensor_parallel import all_reduce_tensor, gather_from_ranks, shard_bytes
        from oracle import oracle

        rng = synth.rng_for(43)  # same bytes on every rank
        m, n, k = 3, 8 * world, 1024 * world
        act = synth.activations(rng, m, k)
        ok = True
        for fmt in ("Q4_K", "Q6_K", "Q8_0", "Q4_0"):
            w = synth.weight_bytes(fmt, rng, n, k)
            full = oracle.quant_matmul(fmt, act, w, n)
            # column-parallel: local rows, then all-gather into row-major [M, N]
            loc = oracle.quant_matmul(fmt, act, shard_bytes(fmt, w, n, k, 0, rank, world), n // world)
            got = gather_from_ranks(torch.from_numpy(loc)).numpy()
            ok &= got.shape == (m, n) and np.array_equal(got, full)
            # row-parallel: local K-slice, then all-reduce SUM
            a_loc = np.ascontiguousarray(act[:, rank * k // world:(rank + 1) * k // world])
            part = oracle.quant_matmul(fmt, a_loc, shard_bytes(fmt, w, n, k, 1, rank, world), n)
            red = all_reduce_tensor(torch.from_numpy(part.copy())).numpy()
            ok &= bool(np.abs(red - full).max() <= 3e-6 * np.abs(full).max())
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_gather_and_all_reduce_gloo(world, oracle):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    res = dict(q.get(timeout=5) for _ in range(world))
    assert all(res.values()), res
