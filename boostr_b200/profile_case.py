"""Runs ONE shape of the quantized-linear path a few times, for timing it or profiling it with ncu.

    python -m boostr_b200.profile_case --op matmul  --fmt Q4_K --m 1 --n 14336 --k 4096 --copies 8 --iters 16
    python -m boostr_b200.profile_case --op swiglu  --fmt Q4_K --m 1 --n 14336 --k 4096 --copies 4 --iters 8
    python -m boostr_b200.profile_case --op qkv     --m 1 --k 4096 --copies 8 --iters 16
    python -m boostr_b200.profile_case --op dequant --fmt Q6_K --n 16384 --k 4096 --dtype bf16

The weights are random packed blocks generated on the device (scales drawn as in the synthetic
benchmark inputs); `--copies` distinct weights are used in rotation so that launches stream from HBM
instead of the 126 MB L2.  Without a profiler attached it prints the average device time per call,
measured with CUDA events around `--iters` back-to-back calls after three warm-up calls.
"""
from __future__ import annotations

import argparse
import sys


from .synth import device_weight  # noqa: E402


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--op", choices=["matmul", "swiglu", "qkv", "dequant"], default="matmul")
    ap.add_argument("--fmt", default="Q4_K")
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--n", type=int, default=14336)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--copies", type=int, default=4)
    ap.add_argument("--iters", type=int, default=8)
    ap.add_argument("--dtype", choices=["f32", "bf16"], default="f32", help="activation dtype (dequant: output dtype)")
    a = ap.parse_args(argv)

    import torch

    from . import ops
    from .linear import QuantLinear

    dt = torch.float32 if a.dtype == "f32" else torch.bfloat16
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1)
    act = torch.randn(a.m, a.k, device="cuda", generator=gen).to(dt)
    if a.op == "qkv":  # q, k (Q4_K) and v (Q6_K) of a Llama-3-8B layer share the activation row
        sets = [[QuantLinear(device_weight("Q4_K", 4096, a.k, gen)), QuantLinear(device_weight("Q4_K", 1024, a.k, gen)),
                 QuantLinear(device_weight("Q6_K", 1024, a.k, gen))] for _ in range(a.copies)]
        outs = [torch.empty(a.m, 4096, device="cuda"), torch.empty(a.m, 1024, device="cuda"), torch.empty(a.m, 1024, device="cuda")]
        nbytes = sum(l.weight.storage_bytes() for l in sets[0])
        flops = 0

        def run(j):
            QuantLinear.forward_batch(sets[j], act, outs=outs)
    elif a.op == "dequant":
        ws = [device_weight(a.fmt, a.n, a.k, gen) for _ in range(a.copies)]
        esz = 4 if a.dtype == "f32" else 2
        nbytes = ws[0].storage_bytes() + a.n * a.k * esz
        flops = 0

        def run(j):
            ops.dequantize(ws[j], dt)
    else:
        ws = [device_weight(a.fmt, a.n, a.k, gen) for _ in range(a.copies)]
        ws2 = [device_weight(a.fmt, a.n, a.k, gen) for _ in range(a.copies)] if a.op == "swiglu" else None
        out = torch.empty(a.m, a.n, device="cuda")
        nbytes = ws[0].storage_bytes() * (2 if ws2 else 1)
        flops = 2 * a.m * a.n * a.k * (2 if ws2 else 1)

        def run(j):
            if ws2:
                ops.quant_swiglu(act, ws[j], ws2[j], out=out)
            else:
                ops.quant_matmul(act, ws[j], out=out)

    for i in range(3):
        run(i % a.copies)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.iters):
        run(i % a.copies)
    e1.record()
    torch.cuda.synchronize()
    ops.check_device_status()
    us = e0.elapsed_time(e1) * 1000.0 / a.iters
    msg = f"{a.op} fmt={a.fmt} M={a.m} N={a.n} K={a.k} {a.dtype}: {us:.2f} us/call (stream-ordered, not graphed), {nbytes / us / 1e3:.1f} GB/s"
    if flops and a.m >= 64:
        msg += f", {flops / us / 1e6:.1f} TFLOP/s"
    print(msg)
    return 0


if __name__ == "__main__":
    sys.exit(main())
