"""CUDA-graph decode loop around a step of quantized linears.

Mirrors the contract of boostr's graph-mode decode (src/inference/decode_graph.rs:1-48,
src/model/llama/model/forward_graph.rs:22-73): every tensor the host touches between replays is allocated
BEFORE capture and keeps its address; per-step values reach the kernels through device memory that is
updated with stream-ordered copies on the compute stream; the captured step allocates nothing.

``DecodeGraph`` owns that discipline for a step function built from this library's operators:

* ``inputs`` / ``outputs``: named, pre-allocated device tensors (stable addresses);
* ``capture()``: warm-up runs on a side stream (lazy set-up such as kernel attributes, the device status
  word and, with tensor parallelism, the communicator must happen outside capture), then one capture;
* ``replay(**new_inputs)``: stream-ordered copies into the stable inputs, then one graph launch;
* ``run_eager(**new_inputs)``: the same step without the graph (the reference for tests).

The fused row-parallel exchange carries its epoch in device memory, so a captured step that contains it
replays without any host-side argument.  ``DeviceScalars`` are the two stream-updated int32 values of the
reference (``seq_len_k``, ``write_pos``); the quantized linears do not read them, attention kernels of a
host model would.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch

from . import ops


class DeviceScalars:
    """Device-resident scalars updated before each replay (src/inference/decode_graph.rs:66-170)."""

    def __init__(self, initial_seq_len: int, device="cuda"):
        self.seq_len_k = torch.full((1,), initial_seq_len, dtype=torch.int32, device=device)
        self.write_pos = torch.full((1,), initial_seq_len, dtype=torch.int32, device=device)

    def seq_len_k_ptr(self) -> int:
        return self.seq_len_k.data_ptr()

    def write_pos_ptr(self) -> int:
        return self.write_pos.data_ptr()

    def update(self, seq_len: int) -> None:
        """write_pos = seq_len, seq_len_k = seq_len + 1; stream-ordered fills, no host pointer involved."""
        self.write_pos.fill_(seq_len)
        self.seq_len_k.fill_(seq_len + 1)


class DecodeGraph:
    def __init__(self, step: Callable[[], object], inputs: Dict[str, torch.Tensor], outputs: Dict[str, torch.Tensor],
                 scalars: Optional[DeviceScalars] = None):
        for name, t in {**inputs, **outputs}.items():
            if not t.is_cuda or not t.is_contiguous():
                raise ValueError(f"'{name}' must be a contiguous CUDA tensor allocated before capture")
        self.step = step
        self.inputs = dict(inputs)
        self.outputs = dict(outputs)
        self.scalars = scalars
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.launches_per_step = 0

    def _stage(self, new_inputs: Dict[str, torch.Tensor]) -> None:
        for name, value in new_inputs.items():
            if name not in self.inputs:
                raise KeyError(f"unknown graph input '{name}'")
            dst = self.inputs[name]
            if tuple(value.shape) != tuple(dst.shape):
                raise ValueError(f"input '{name}' has shape {list(value.shape)}, the captured buffer {list(dst.shape)}")
            dst.copy_(value, non_blocking=True)  # stream-ordered on the compute stream

    def capture(self, warmup: int = 2) -> "DecodeGraph":
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                before = ops.launch_count()
                self.step()
                self.launches_per_step = ops.launch_count() - before
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.step()
        self.graph = g
        return self

    def replay(self, seq_len: Optional[int] = None, **new_inputs: torch.Tensor) -> Dict[str, torch.Tensor]:
        if self.graph is None:
            raise RuntimeError("capture() has not run")
        self._stage(new_inputs)
        if seq_len is not None and self.scalars is not None:
            self.scalars.update(seq_len)
        self.graph.replay()
        return self.outputs

    def run_eager(self, seq_len: Optional[int] = None, **new_inputs: torch.Tensor) -> Dict[str, torch.Tensor]:
        self._stage(new_inputs)
        if seq_len is not None and self.scalars is not None:
            self.scalars.update(seq_len)
        self.step()
        return self.outputs
