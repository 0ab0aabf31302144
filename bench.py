#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path on B200.

Default workload (``--workload c5``): one decode step over the quantized linears of a
Llama-3-8B-shaped stack in a Q4_K_M-style mix (32 layers of q/k/v/o/gate/up/down + lm_head;
Q6_K for v, down and lm_head, Q4_K elsewhere), M tokens per step (``--m``, default 1), synthetic
weights with the block-value distributions of the reference configurations, tensor-parallel over
``--gpus`` ranks (column-parallel q/k/v/gate/up/lm_head, row-parallel o/down with all-reduce,
logits all-gathered).  Metric: decode tokens/s = M * steps/s, whole job.

One JSON line is printed by rank 0.  ``--impl reference`` times the CPU restatement of boostr's
CPU SIMD path (the reference itself is Rust and cannot be built in this environment) on the
host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HIDDEN, KV, FFN, VOCAB, LAYERS = 4096, 1024, 14336, 128256, 32  # the shapes boostr_b200.decode_stack builds
L2_BYTES = 126 * 1024 * 1024


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def fmt_bytes(fmt: str, n: int, k: int) -> int:
    bs, bb = {"Q4_0": (32, 18), "Q8_0": (32, 34), "Q4_K": (256, 144), "Q6_K": (256, 210)}[fmt]
    return n * (k // bs) * bb


# the linears of one layer: (name, format, N, K, parallel split)
LAYER_SPEC = [
    ("q", "Q4_K", HIDDEN, HIDDEN, "col"), ("k", "Q4_K", KV, HIDDEN, "col"), ("v", "Q6_K", KV, HIDDEN, "col"),
    ("o", "Q4_K", HIDDEN, HIDDEN, "row"), ("gate", "Q4_K", FFN, HIDDEN, "col"), ("up", "Q4_K", FFN, HIDDEN, "col"),
    ("down", "Q6_K", HIDDEN, FFN, "row"),
]
STEP_BYTES = LAYERS * sum(fmt_bytes(f, n, k) for _, f, n, k, _ in LAYER_SPEC) + fmt_bytes("Q6_K", VOCAB, HIDDEN)


class ClockSampler:
    """SM clock / throttle-reason samples while the timed region runs.

    Reads NVML directly every 2 ms (a decode step lasts about a millisecond, so `nvidia-smi -lms`
    would miss short regions); falls back to `nvidia-smi -lms 100` when the NVML binding is missing.
    Only reads: no clock, power or mode setting is touched."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    BITS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.stop = threading.Event()
        self.thread = None
        self.handle = None
        try:
            import pynvml
            import torch

            pynvml.nvmlInit()
            try:
                uuid = "GPU-" + str(torch.cuda.get_device_properties(index).uuid)
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.nv = pynvml
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.handle = None

    def _poll(self):
        nv = self.nv
        while not self.stop.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in self.BITS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.handle is not None:
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return self
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=lambda: [self.lines.append(l) for l in self.proc.stdout], daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.thread is not None:
            self.stop.set()
            self.thread.join(timeout=1)
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        if self.thread is not None:
            if not self.samples:
                return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
            return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                    "samples": len(self.samples), "source": "nvml, 2 ms period"}
        sm, mx, reasons = [], [], set()
        for l in self.lines:
            p = [x.strip() for x in l.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1]))
                mx.append(float(p[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm),
                "source": "nvidia-smi -lms 100"}


# --------------------------------------------------------------------------- GPU arm

# DRAM bytes (read + written) of one launch of the dominant kernel at one GPU, from the ncu capture
# summarised in profiles/gemv_m1_q6k_down.md: dram__bytes_read.sum 48.276 MB, dram__bytes_write.sum 0 (the 16 KB of output stay in L2).
# A K-split shard streams proportionally fewer bytes, so the figure is scaled by the shard's packed bytes.
NCU_TRAFFIC_DOWN_1GPU = 48_275_700
NCU_ALGORITHMIC_DOWN_1GPU = 4096 * 56 * 210
REGION_REPEATS = 30


def timed_graph(torch, fn, reps, warm=2):
    """Captures `fn` (a sequence of library calls on distinct weights) in a CUDA graph and returns the
    median / min / max device time of one replay in microseconds over `reps` replays (CUDA events)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1000.0)
    return statistics.median(ts), min(ts), max(ts)


def time_kernel_family(stack, torch, ops):
    """Average device time of the dominant kernel (largest share of the step in the ncu launch list):
    the Q6_K decode GEMV on the down-projection shards of all layers (distinct weights, 1.5 GB in total
    at one GPU, so every launch streams from HBM)."""
    ws = [L["down"].weight for L in stack.layers]
    x = torch.randn(stack.m, ws[0].shape[1], device="cuda")
    outs = torch.empty(stack.m, ws[0].shape[0], device="cuda")

    def run():
        for i, w in enumerate(ws):
            if stack.m == 1:
                ops.prefetch_next([ws[(i + 1) % len(ws)]])  # as in the decode step: each call knows which weights follow
            ops.quant_matmul(x, w, out=outs)

    med, lo, hi = timed_graph(torch, run, reps=20)
    return med / len(ws), ws[0].storage_bytes()


def per_config(torch, ops, pk, world, rank):
    """Device time of every reference configuration that is not the headline workload, each on enough
    distinct weight copies that the rotation exceeds four times the L2 (so every launch streams from HBM),
    replayed as one CUDA graph; median over 10 replays divided by the number of copies.
    At N > 1 only the sharded configurations run (C3: N-split, no communication; C4: N-split + gather)."""
    from boostr_b200 import synth
    from boostr_b200.format import QuantFormat as F
    from boostr_b200.tensor_parallel import gather_from_ranks

    gen = torch.Generator(device="cuda")
    gen.manual_seed(0xC0F + rank)
    out = {}
    l2x4 = 4 * L2_BYTES

    def gemv_case(key, fmt, m, n, k, dt=torch.float32, gather=False):
        f = F.parse(fmt)
        nl = n // world
        wbytes = f.storage_bytes(nl * k)
        copies = max(2, -(-l2x4 // wbytes))
        ws = [synth.device_weight(fmt, nl, k, gen) for _ in range(copies)]
        x = torch.randn(m, k, device="cuda", generator=gen).to(dt)
        y = torch.empty(m, nl, device="cuda")
        full = torch.empty(m, n, device="cuda") if gather and world > 1 else None

        def run():
            for w in ws:
                ops.quant_matmul(x, w, out=y)
                if full is not None:
                    gather_from_ranks(y, out=full)

        med, lo, hi = timed_graph(torch, run, reps=10)
        us = med / copies
        r = {"us": us, "us_min": lo / copies, "us_max": hi / copies, "copies": copies, "rows_per_rank": nl}
        flops = 2.0 * m * nl * k
        if m >= 64:
            r["tflops"] = flops / us / 1e6
            r["frac_measured"] = r["tflops"] / pk["bf16_tflops"]
            r["frac_nominal"] = r["tflops"] / 2250.0
        else:
            r["gbs"] = wbytes / us / 1e3
            r["frac_measured"] = r["gbs"] / pk["hbm_gbs"]
            r["frac_nominal"] = r["gbs"] / 8000.0
        out[key] = r
        del ws

    if world == 1:
        gemv_case("C1 Q4_0 M=1 [4096x4096]", "Q4_0", 1, 4096, 4096)
        for m in (1, 8, 32):
            gemv_case(f"C2 Q8_0 M={m} [11008x4096]", "Q8_0", m, 11008, 4096)
    for m in (1, 16):
        gemv_case(f"C4 Q6_K M={m} [128256x4096] lm-head" + (" + gather" if world > 1 else ""), "Q6_K", m, 128256, 4096, gather=True)
    if world == 1:
        # dequant Q4_K -> bf16: packed bytes in + 2 bytes per element out
        n, k = 14336, 4096
        ws = [synth.device_weight("Q4_K", n, k, gen) for _ in range(4)]

        def run():
            for w in ws:
                ops.dequantize(w, torch.bfloat16)

        med, lo, hi = timed_graph(torch, run, reps=10)
        us = med / len(ws)
        nbytes = ws[0].storage_bytes() + 2 * n * k
        out["dequant Q4_K->bf16 [14336x4096]"] = {"us": us, "gbs": nbytes / us / 1e3, "frac_measured": nbytes / us / 1e3 / pk["hbm_gbs"],
                                                  "frac_nominal": nbytes / us / 1e3 / 8000.0, "bytes_in_plus_out": nbytes}
    # the tensor-core configuration last: seconds of dense MMA lower the SM clock (power) for what is timed right after
    for m in (512, 2048):
        gemv_case(f"C3 Q4_K M={m} [14336x4096] bf16 acts", "Q4_K", m, 14336, 4096, dt=torch.bfloat16)
    return out


def c5_batched(stack, torch, dist, ops, m2, world, steps=5, repeats=5):
    """The same decode stack (same weights) with m2 tokens per step: median ms/step of `repeats` regions of
    `steps` graph replays, max over ranks.  Row-parallel layers with more than one token use the library's
    product followed by the process group's all-reduce."""
    from boostr_b200.decode_graph import DecodeGraph
    from boostr_b200.decode_stack import DecodeStack

    st = DecodeStack(m2, stack.rank, world, weights=stack.layers, lm_head=stack.lm_head)
    st.use_exchange(stack.exchange)
    st.step()
    torch.cuda.synchronize()
    runner = DecodeGraph(st.step, {"x": st.x}, {"logits": st.logits}).capture()
    for _ in range(3):
        runner.graph.replay()
    ts = []
    for _ in range(repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            runner.graph.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) / steps)
    t = torch.tensor(ts, device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = statistics.median(float(v) for v in t.tolist())
    gbs = STEP_BYTES / (ms * 1e-3) / 1e9
    return {"ms_per_step": ms, "tokens_per_s": m2 * 1000.0 / ms, "step_weight_gbs_per_gpu": gbs / world,
            "frac_measured_per_gpu": gbs / world / peaks()["hbm_gbs"], "frac_of_8tbs_per_gpu": gbs / world / 8000.0,
            "tflops": 2.0 * m2 * 7_504_658_432 / (ms * 1e-3) / 1e12}


def log(msg):
    if os.environ.get("BENCH_VERBOSE"):
        sys.stderr.write(f"[bench r{os.environ.get('RANK', '0')} {time.strftime('%H:%M:%S')}] {msg}\n")
        sys.stderr.flush()


def tp_parity(stack, torch, dist, ops, exchange):
    """Cross-GPU correctness of the timed path, outside the timed region: one eager step through the fused
    row-parallel exchange against one through NCCL's all-reduce (last layer's down-projection output and the
    gathered logits), and every rank must hold the same bits of the fused result."""
    world = dist.get_world_size()
    stack.use_exchange(exchange)
    stack.step()
    ops.check_device_status()
    d_f, lg_f = stack.d.clone(), stack.logits.clone()
    stack.use_exchange(None)
    stack.step()
    torch.cuda.synchronize()
    d_n, lg_n = stack.d.clone(), stack.logits.clone()
    stack.use_exchange(exchange)
    rel = max(float((d_f - d_n).abs().max() / d_n.abs().max().clamp_min(1e-30)),
              float((lg_f - lg_n).abs().max() / lg_n.abs().max().clamp_min(1e-30)))
    got = [torch.empty_like(d_f) for _ in range(world)]
    dist.all_gather(got, d_f)
    same = all(torch.equal(g.view(torch.int32), d_f.view(torch.int32)) for g in got)
    got = [torch.empty_like(lg_f) for _ in range(world)]
    dist.all_gather(got, lg_f)
    same = same and all(torch.equal(g.view(torch.int32), lg_f.view(torch.int32)) for g in got)
    finite = bool(torch.isfinite(d_f).all() and torch.isfinite(lg_f).all())
    flag = torch.tensor([rel, 0.0 if (same and finite) else 1.0], device="cuda", dtype=torch.float64)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    return {"max_rel": float(flag[0]), "ranks_bit_identical": bool(flag[1] == 0.0), "compared": "last layer down-projection output "
            "[M,4096] and gathered logits [M,128256]: fused peer exchange vs NCCL all-reduce, eager step"}, d_f


def run_ours(args):
    import torch
    import torch.distributed as dist

    from boostr_b200 import ops
    from boostr_b200.decode_graph import DecodeGraph
    from boostr_b200.decode_stack import DecodeStack

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    torch.cuda.set_device(local_rank)
    m = args.m
    pk = peaks()
    stack = DecodeStack(m, rank, world)
    stack.prefetch = not args.no_prefetch_hint
    torch.cuda.synchronize()
    log("stack built")
    # kernel-family and per-configuration timings run before any process group exists (one-GPU figures on
    # rank 0; the sharded configurations on every rank, no collective inside): a graph capture on one rank
    # while NCCL's watchdog threads are alive and the other ranks sit in a collective can stall
    k_us, k_bytes = time_kernel_family(stack, torch, ops) if rank == 0 else (0.0, 0)
    log("kernel family timed")
    configs = {}
    if not args.no_per_config and world == 1:
        configs = per_config(torch, ops, pk, 1, 0)
        log("per-config timed")
    exchange = None
    parity = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        log("process group up")
        if args.collective == "fused":
            from boostr_b200.tensor_parallel import PeerExchange

            exchange = PeerExchange()
            stack.use_exchange(exchange)
            log("peer exchange mapped")
            parity, d_eager = tp_parity(stack, torch, dist, ops, exchange)
            log(f"tp parity {parity}")
            if parity["max_rel"] > 2e-6 or not parity["ranks_bit_identical"]:
                if rank == 0:
                    print(json.dumps({"error": "tensor-parallel parity check failed", "tp_parity": parity}), flush=True)
                sys.stdout.flush()
                os._exit(3)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # warm-up (also initialises NCCL communicators outside any capture), then capture one step
    launches0 = ops.launch_count()
    stack.step()
    torch.cuda.synchronize()
    launches_per_step = ops.launch_count() - launches0
    log(f"eager step done, {launches_per_step} launches")
    runner = DecodeGraph(stack.step, {"x": stack.x}, {"logits": stack.logits, "d": stack.d})
    graph_ok = False
    if not args.no_graph:
        try:
            runner.capture()
            graph_ok = True
            log("captured")
        except Exception as e:  # capture of a collective can be refused; fall back to eager launches
            sys.stderr.write(f"[bench] CUDA graph capture failed, running eagerly: {e}\n")
            torch.cuda.synchronize()

    def one_step():
        if graph_ok:
            runner.graph.replay()
        else:
            stack.step()

    for _ in range(max(args.warmup, 3)):
        one_step()
    barrier()
    log("warm-up done")
    if parity is not None:
        # the replayed graph (fused exchange included, epoch carried in device memory) must give the eager bits
        parity["graph_replay_bit_identical"] = bool(torch.equal(stack.d.view(torch.int32), d_eager.view(torch.int32)))

    # ---- device-resident timing: the K-step region, CUDA events, max over ranks; the region is repeated
    # REGION_REPEATS times and the median is reported (min / max beside it)
    regions = []
    with ClockSampler(local_rank) as clk:
        for _ in range(REGION_REPEATS):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            barrier()
            ev[0].record()
            for _ in range(args.steps):
                one_step()
            ev[1].record()
            barrier()
            regions.append(ev[0].elapsed_time(ev[1]))
    t = torch.tensor(regions, device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    regions = [float(v) / args.steps for v in t.tolist()]
    ms_per_step = statistics.median(regions)
    ops.check_device_status()
    log(f"timed region done: {ms_per_step:.3f} ms/step")

    # ---- end to end: host activations in, host logits out, every step
    x_host = torch.randn(m, stack.hidden).pin_memory()
    logits_host = torch.empty(m, stack.vocab).pin_memory()

    def e2e_step():
        stack.x.copy_(x_host, non_blocking=True)
        one_step()
        logits_host.copy_(stack.logits, non_blocking=True)

    for _ in range(2):
        e2e_step()
    e2e_regions = []
    for _ in range(REGION_REPEATS):
        ev2 = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        barrier()
        ev2[0].record()
        for _ in range(args.steps):
            e2e_step()
        ev2[1].record()
        barrier()
        e2e_regions.append(ev2[0].elapsed_time(ev2[1]))
    t = torch.tensor(e2e_regions, device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = statistics.median(float(v) / args.steps for v in t.tolist())
    log("e2e done")
    clocks = clk.summary()

    if world > 1 and not args.no_per_config:
        # sharded configurations per rank (C3 N-split; C4 N-split + gather of the logits), after the
        # headline numbers; rank 0 reports its own figures (all ranks do the same work)
        try:
            configs = per_config(torch, ops, pk, world, rank)
        except Exception as e:
            configs = {"error": f"{type(e).__name__}: {e}"}
        barrier()
        log("per-config timed")
    if not args.no_per_config and m == 1:
        for m2 in (16, 64):
            try:
                configs[f"C5 decode step M={m2}"] = c5_batched(stack, torch, dist, ops, m2, world)
            except Exception as e:
                configs[f"C5 decode step M={m2}"] = {"error": f"{type(e).__name__}: {e}"}
            barrier()
        log("batched C5 timed")

    result = None
    if rank == 0:
        achieved = k_bytes / k_us / 1e3  # GB/s
        step_gbs = STEP_BYTES / (ms_per_step * 1e-3) / 1e9
        result = {
            "metric": "decode tokens/s over the quantized linears of a Llama-3-8B-shaped stack (Q4_K_M mix)",
            "value": m * 1000.0 / ms_per_step, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "u8 blocks x int8 (Q8_K) activations, f32 accumulate",
            "data": "synthetic",
            "config": {"workload": f"C5 Llama-3-8B-shaped decode step, 32 layers + lm_head, M={m}",
                       "parallelism": f"tp{world}", "row_parallel_reduce": (args.collective if world > 1 else "none"),
                       "packed_weight_bytes_per_step": STEP_BYTES,
                       "l2": "weights per step per rank exceed L2 (%d MB > 126 MB)" % (stack.bytes_local // 2**20),
                       "cuda_graph": graph_ok},
            "timed_regions": {"repeats": REGION_REPEATS, "steps_each": args.steps, "ms_per_step_median": ms_per_step,
                              "ms_per_step_min": min(regions), "ms_per_step_max": max(regions)},
            "step_weight_gbs": step_gbs, "step_weight_gbs_per_gpu": step_gbs / world,
            "step_frac_of_8tbs_per_gpu": step_gbs / world / 8000.0,
            "e2e": {"value": m * 1000.0 / e2e_ms, "unit": "tokens/s", "h2d_bytes_per_step": m * stack.hidden * 4,
                    "d2h_bytes_per_step": m * stack.vocab * 4},
            "gpu_launches": int(launches_per_step * args.steps),
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "Q6_K decode GEMV, down-projection shard [%d x %d], M=%d" % (
                             stack.hidden, stack.layers[0]["down"].weight.shape[1], m),
                         "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                         "frac_of_8tbs": achieved / 8000.0, "peak_source": pk["source"], "avg_launch_us": k_us,
                         "algorithmic_bytes_per_launch": k_bytes,
                         "traffic": int(NCU_TRAFFIC_DOWN_1GPU * k_bytes / NCU_ALGORITHMIC_DOWN_1GPU),
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch at 1 GPU "
                                           "(profiles/gemv_m1_q6k_down.md), scaled by the shard's packed bytes"},
        }
        if parity is not None:
            result["tp_parity"] = parity
        if configs:
            result["per_config"] = configs
        if world == 1 and not args.no_cpu_baseline:
            result["cpu_baseline"] = cpu_reference(m, budget_s=args.cpu_seconds)
    return result


# --------------------------------------------------------------------------- CPU arm


def cpu_reference(m, budget_s=12.0, steps=None, warmup=1):
    """Times the CPU oracle (C restatement of boostr's CPU SIMD path) on a bounded sample of the
    decode step: whole layers (all seven linears) plus one eighth of the lm_head, all host threads."""
    import numpy as np

    from boostr_b200 import synth
    from oracle import oracle

    oracle.build()
    threads = os.cpu_count() or 1
    rng = synth.rng_for(5, 0)
    nsets = 2  # distinct weight sets so the layer does not sit in the last-level cache
    sets = []
    for _ in range(nsets):
        sets.append([(f, n, k, synth.weight_bytes(f, rng, n, k)) for _, f, n, k, _ in LAYER_SPEC])
    lm_rows = VOCAB // 8
    lm = synth.weight_bytes("Q6_K", rng, lm_rows, HIDDEN)
    acts = {HIDDEN: synth.activations(rng, m, HIDDEN), FFN: synth.activations(rng, m, FFN)}

    def sample(i):
        t0 = time.perf_counter()
        for f, n, k, w in sets[i % nsets]:
            oracle.quant_matmul(f, acts[k], w, n, threads=threads, simd=True)
        t1 = time.perf_counter()
        oracle.quant_matmul("Q6_K", acts[HIDDEN], lm, lm_rows, threads=threads, simd=True)
        t2 = time.perf_counter()
        return t1 - t0, t2 - t1

    for i in range(warmup):
        sample(i)
    lay, head = [], []
    t_start = time.perf_counter()
    i = 0
    while (steps is None and time.perf_counter() - t_start < budget_s) or (steps is not None and i < steps):
        a, b = sample(i)
        lay.append(a)
        head.append(b)
        i += 1
        if steps is not None and time.perf_counter() - t_start > 150:
            break
    t_layer, t_head = statistics.median(lay), statistics.median(head) * 8
    step_s = LAYERS * t_layer + t_head
    return {"value": m / step_s, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"{len(lay)} x (one layer's 7 linears + 1/8 of lm_head), median, scaled to 32 layers + lm_head",
            "ms_per_step": step_s * 1e3,
            "note": "C restatement of boostr's CPU path (AVX2 integer dots, rayon-style column chunks); boostr itself "
                    "is Rust and cannot be built here"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    cb = cpu_reference(args.m, steps=max(args.steps, 1), warmup=max(args.warmup, 1))
    return {
        "impl": "reference",
        "metric": "decode tokens/s over the quantized linears of a Llama-3-8B-shaped stack (Q4_K_M mix)",
        "value": cb["value"], "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": cb["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "u8 blocks x int8 (Q8_K) activations, f32 accumulate", "data": "synthetic",
        "config": {"workload": f"C5 Llama-3-8B-shaped decode step, 32 layers + lm_head, M={args.m}",
                   "parallelism": "host threads"},
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=1, help="tokens per decode step")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--collective", default="fused", choices=["fused", "nccl"],
                    help="row-parallel all-reduce at N > 1: fused into the GEMV kernel over peer memory, or NCCL")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-per-config", action="store_true", help="skip the per-configuration kernel timings")
    ap.add_argument("--no-prefetch-hint", action="store_true",
                    help="decode step without b200q_prefetch_next (each call told which weights follow it); for A/B runs")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    args = ap.parse_args()
    res = run_reference(args) if args.impl == "reference" else run_ours(args)
    if res is not None:
        print(json.dumps(res), flush=True)
    if int(os.environ.get("WORLD_SIZE", "1")) > 1 and args.impl != "reference":
        # Tearing NCCL communicators down while captured graphs still reference them has been seen to
        # stall; every rank has finished its work and rank 0 has printed, so leave without the teardown.
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
