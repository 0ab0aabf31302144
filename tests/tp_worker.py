"""One rank of the multi-GPU tensor-parallel check (started by test_gpu_tp_multi.py through
torch.distributed.run).  Row-parallel decode products through the fused peer exchange are compared
with the same products through NCCL's all-reduce, and with the unsharded product."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from boostr_b200 import ops, synth  # noqa: E402
from boostr_b200.tensor import QuantTensor  # noqa: E402
from boostr_b200.format import QuantFormat  # noqa: E402
from boostr_b200.tensor_parallel import PeerExchange, RowParallelQuantLinear  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    ex = PeerExchange()
    worst = 0.0
    for case, (fmt, n, k) in enumerate([("Q4_K", 4096, 4096), ("Q6_K", 4096, 14336 // 8 * 8), ("Q6_K", 512, 2048 * world), ("Q4_K", 100, 1024 * world)]):
        if (k // world) % 256:
            continue
        rng = synth.rng_for(77, case)  # same stream on every rank
        full = synth.weight_bytes(fmt, rng, n, k)
        fused = RowParallelQuantLinear.from_full(fmt, full, n, k, rank, world, exchange=ex)
        plain = RowParallelQuantLinear(fused.weight)
        whole = QuantTensor.from_bytes(full, QuantFormat.parse(fmt), (n, k), device="cuda")
        for it in range(6):
            act = synth.activations(rng, 1, k)
            shard = torch.from_numpy(np.ascontiguousarray(act[:, rank * (k // world):(rank + 1) * (k // world)])).cuda()
            y_fused = fused(shard).clone()
            y_nccl = plain(shard)
            y_one = ops.quant_matmul(torch.from_numpy(act).cuda(), whole)
            ops.check_device_status()
            scale = float(y_one.abs().max())
            e1 = float((y_fused - y_nccl).abs().max()) / scale
            e2 = float((y_fused - y_one).abs().max()) / scale
            worst = max(worst, e1, e2)
            # every rank must hold the same bits
            gathered = [torch.empty_like(y_fused) for _ in range(world)]
            dist.all_gather(gathered, y_fused)
            for g in gathered:
                assert torch.equal(g.view(torch.int32), y_fused.view(torch.int32)), "ranks disagree on the fused sum"
            assert e1 <= 2e-6 and e2 <= 2e-6, (fmt, n, k, it, e1, e2)
    # several rows, and a format without a fused decode kernel: product + the exchange all-reduce kernel against
    # product + NCCL all-reduce; bit-identical on all ranks, equal to NCCL's sum up to the order of additions
    for case, (fmt, m, n, k) in enumerate([("Q4_K", 16, 4096, 4096), ("Q6_K", 5, 512, 2048 * world), ("Q8_0", 1, 300, 1024 * world), ("Q4_K", 64, 1024, 1024 * world)]):
        if (k // world) % 256:
            continue
        rng = synth.rng_for(79, case)
        full = synth.weight_bytes(fmt, rng, n, k)
        viaex = RowParallelQuantLinear.from_full(fmt, full, n, k, rank, world, exchange=ex)
        plain = RowParallelQuantLinear(viaex.weight)
        for it in range(4):
            act = synth.activations(rng, m, k)
            shard = torch.from_numpy(np.ascontiguousarray(act[:, rank * (k // world):(rank + 1) * (k // world)])).cuda()
            before = ops.launch_count()
            y_ex = viaex(shard).clone()
            launched = ops.launch_count() - before
            y_nccl = plain(shard)
            ops.check_device_status()
            assert launched >= 2 and m * n <= 65536, (fmt, m, launched)  # the all-reduce was one of this library's kernels
            scale = float(y_nccl.abs().max())
            assert float((y_ex - y_nccl).abs().max()) / scale <= 2e-6, (fmt, m, it)
            gathered = [torch.empty_like(y_ex) for _ in range(world)]
            dist.all_gather(gathered, y_ex)
            assert all(torch.equal(g, y_ex) for g in gathered), "ranks disagree on the exchange all-reduce"
    # fused column-parallel gather of logits against NCCL all-gather + strided copy (M = 1)
    from boostr_b200.tensor_parallel import ColumnParallelQuantLinear, gather_from_ranks
    for case, (fmt, n, k) in enumerate([("Q6_K", 128256 // 8 * world, 4096), ("Q4_K", 96 * world, 1024)]):
        rng = synth.rng_for(78, case)
        full = synth.weight_bytes(fmt, rng, n, k)
        col = ColumnParallelQuantLinear.from_full(fmt, full, n, k, rank, world)
        whole = QuantTensor.from_bytes(full, QuantFormat.parse(fmt), (n, k), device="cuda")
        for it in range(4):
            act = torch.from_numpy(synth.activations(rng, 1, k)).cuda()
            fused = col.forward_gathered(act, torch.empty(1, n, device="cuda"), ex).clone()
            plain = gather_from_ranks(col(act))
            one = ops.quant_matmul(act, whole)
            ops.check_device_status()
            assert torch.equal(fused, plain), ("fused gather differs from NCCL gather", fmt, it)
            assert torch.equal(fused, one), ("gathered logits differ from the unsharded product", fmt, it)
    # a captured decode step that contains the fused exchange (its epoch lives in device memory) replays to
    # the bits of the eager step, on every rank; M = 1 (fused) and M = 4 (product + exchange all-reduce kernel)
    from boostr_b200.decode_graph import DecodeGraph
    from boostr_b200.decode_stack import DecodeStack

    for m in (1, 4):
        stack = DecodeStack(m, rank, world, layers=3, hidden=1024, kv=256, ffn=2048, vocab=4096, seed=21)
        stack.use_exchange(ex)
        stack.step()  # communicators and lazy set-up outside capture
        torch.cuda.synchronize()
        dist.barrier()
        runner = DecodeGraph(stack.step, {"x": stack.x}, {"logits": stack.logits, "d": stack.d}).capture()
        gen = torch.Generator(device="cuda")
        gen.manual_seed(5)  # the same hidden state on every rank
        for it in range(3):
            x = torch.randn(m, 1024, device="cuda", generator=gen)
            eager = {k: v.clone() for k, v in runner.run_eager(x=x).items()}
            stack.d.zero_()
            out = runner.replay(x=x)
            ops.check_device_status()
            for k in eager:
                assert torch.equal(out[k], eager[k]), ("graph replay differs from eager", m, it, k)
            gathered = [torch.empty_like(out["d"]) for _ in range(world)]
            dist.all_gather(gathered, out["d"])
            assert all(torch.equal(g, out["d"]) for g in gathered), "ranks disagree after a graph replay"
    ex.close()
    if rank == 0:
        print(f"TP_WORKER_OK world={world} worst_rel_err={worst:.3e}", flush=True)
    dist.barrier()
    os._exit(0)


if __name__ == "__main__":
    main()
