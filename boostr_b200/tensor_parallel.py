"""Megatron-style tensor parallelism over packed quantized weights.

boostr's ``ColumnParallelLinear`` / ``RowParallelLinear`` hold dense weights
(src/distributed/tensor_parallel.rs:27-253) and ``QuantTensor`` cannot be sliced; here the
same contract is applied to packed blocks:

* column-parallel (q, k, v, gate, up, lm_head): rank r owns output rows
  ``[r*N/P, (r+1)*N/P)`` — a contiguous byte range of the packed tensor; forward needs no
  communication (tensor_parallel.rs:112-123); ``gather_from_ranks`` assembles full rows.
* row-parallel (o, down): rank r owns input columns ``[r*K/P, (r+1)*K/P)`` of every row,
  repacked tightly (K/P must be a whole number of blocks); forward is the local product
  followed by an all-reduce SUM, then the bias (tensor_parallel.rs:222-244).

One process per GPU; collectives go through ``torch.distributed`` (NCCL on GPUs, gloo in the
CPU tests).  Sharding itself is host-side byte shuffling done by ``b200q_shard_pack``.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from . import _cabi, ops
from .format import QuantError, QuantFormat
from .tensor import QuantTensor


class DistributedError(RuntimeError):
    """Counterpart of ``Error::DistributedError { reason }``."""


def shard_bytes(fmt, packed: np.ndarray, n: int, k: int, dim: int, rank: int, world_size: int) -> np.ndarray:
    """Host-side shard of a packed [N,K] weight (dim 0: rows, dim 1: columns)."""
    fmt = QuantFormat.parse(fmt)
    packed = np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1)
    if packed.size != fmt.storage_bytes(n * k):
        raise QuantError(f"expected {fmt.storage_bytes(n * k)} bytes for {fmt.name} [{n},{k}], got {packed.size}")
    if dim == 0:
        if n % world_size:
            raise DistributedError(f"out_features {n} not divisible by world_size {world_size}")
        out = np.empty(fmt.storage_bytes(n // world_size * k), dtype=np.uint8)
    elif dim == 1:
        if k % world_size:
            raise DistributedError(f"in_features {k} not divisible by world_size {world_size}")
        if (k // world_size) % fmt.block_size:
            raise DistributedError(
                f"in_features per rank {k // world_size} is not a multiple of {fmt.name}'s block_size {fmt.block_size}")
        out = np.empty(fmt.storage_bytes(n * (k // world_size)), dtype=np.uint8)
    else:
        raise DistributedError(f"dim {dim} out of range for 2D tensor")
    _cabi.check(_cabi.lib().b200q_shard_pack(fmt.format_id, packed.ctypes.data, n, k, dim, rank, world_size,
                                             out.ctypes.data, out.size))
    return out


def scatter_to_rank(fmt, packed: np.ndarray, n: int, k: int, dim: int, rank: int, world_size: int,
                    device="cuda") -> QuantTensor:
    """Quantized counterpart of scatter_to_rank (tensor_parallel.rs:258-300): the rank's shard as a QuantTensor."""
    sh = shard_bytes(fmt, packed, n, k, dim, rank, world_size)
    shape = (n // world_size, k) if dim == 0 else (n, k // world_size)
    return QuantTensor.from_bytes(sh, fmt, shape, device=device)


def _world(group) -> int:
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def all_reduce_tensor(t: torch.Tensor, group=None) -> torch.Tensor:
    """In-place SUM all-reduce (src/distributed/comm_utils.rs:15-39)."""
    if _world(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t


def gather_from_ranks(local_shard: torch.Tensor, group=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gather along the LAST dimension into row-major [..., N].

    The reference gathers flat and reshapes (tensor_parallel.rs:302-355), which is only
    layout-correct for a single row; here shard r lands in columns [r*N/P, (r+1)*N/P) of every row.
    """
    p = _world(group)
    if p <= 1:
        return local_shard
    if not local_shard.is_contiguous():
        raise DistributedError("gather_from_ranks requires contiguous tensors")
    lead = local_shard.shape[:-1]
    nl = local_shard.shape[-1]
    staged = torch.empty((p, *lead, nl), dtype=local_shard.dtype, device=local_shard.device)
    if local_shard.is_cuda:
        dist.all_gather_into_tensor(staged.view(-1), local_shard.view(-1), group=group)
    else:  # gloo wants the list form
        dist.all_gather(list(staged.unbind(0)), local_shard, group=group)
    full = out if out is not None else torch.empty((*lead, p * nl), dtype=local_shard.dtype, device=local_shard.device)
    # [P, ..., N/P] -> [..., P, N/P] -> [..., N]
    full.view(*lead, p, nl).copy_(staged.movedim(0, -2))
    return full


class PeerExchange:
    """Exchange buffers for the fused row-parallel decode product (``b200q_row_parallel_matmul``).

    Every rank allocates one buffer in the library, the CUDA IPC handles travel through the process
    group, and each rank maps its peers' buffers.  One PeerExchange serves one stream of calls, issued
    in the same order on all ranks.  With one rank (or no process group) it is inert.
    """

    def __init__(self, group=None):
        self.group = group
        self.world = _world(group)
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self._own = None
        self._peers = {}
        self.table = None
        if self.world <= 1:
            return
        L = _cabi.lib()
        own = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(_cabi.TP_HANDLE_BYTES)
        _cabi.check(L.b200q_tp_alloc(ctypes.byref(own), handle))
        self._own = own.value
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        table = (ctypes.c_void_p * self.world)()
        for r, h in enumerate(handles):
            if r == self.rank:
                table[r] = self._own
            else:
                peer = ctypes.c_void_p()
                _cabi.check(L.b200q_tp_open(ctypes.c_char_p(h), ctypes.byref(peer)))
                self._peers[r] = peer.value
                table[r] = peer.value
        self.table = table
        dist.barrier(group=group)  # nobody pushes before every mapping exists

    def close(self):
        """Unmap the peers and free the own buffer (all ranks, after the last fused call has finished)."""
        if self._own is None:
            return
        torch.cuda.synchronize()
        if dist.is_initialized():
            dist.barrier(group=self.group)
        L = _cabi.lib()
        for ptr in self._peers.values():
            L.b200q_tp_close(ptr)
        self._peers = {}
        if dist.is_initialized():
            dist.barrier(group=self.group)  # a buffer is freed only when nobody maps it any more
        L.b200q_tp_free(self._own)
        self._own = None
        self.table = None


class ColumnParallelQuantLinear:
    """Output features split across ranks; no communication in forward."""

    def __init__(self, local_weight: QuantTensor, bias: Optional[torch.Tensor] = None, group=None):
        self.weight = local_weight
        self.bias = bias
        self.group = group

    @classmethod
    def from_full(cls, fmt, packed: np.ndarray, n: int, k: int, rank: int, world_size: int, device="cuda", group=None):
        return cls(scatter_to_rank(fmt, packed, n, k, 0, rank, world_size, device), None, group)

    def forward(self, input: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        y = ops.quant_matmul(input, self.weight, out=out)
        if self.bias is not None:
            y.add_(self.bias)
        return y

    __call__ = forward

    def forward_gathered(self, input: torch.Tensor, out_full: torch.Tensor, exchange: Optional["PeerExchange"] = None,
                         local: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Local product followed by the gather of every rank's slice into row-major ``out_full``
        [..., world * N/P].  With a ``PeerExchange`` and one activation row the product and the gather are ONE
        kernel (the slice is pushed to all ranks over NVLink); otherwise ``forward`` + ``gather_from_ranks``."""
        if exchange is not None and exchange.table is not None and input.is_cuda and self.bias is None:
            y = ops.col_parallel_matmul_gather(input, self.weight, exchange.rank, exchange.world, exchange.table, out_full)
            if y is not None:
                return y
        return gather_from_ranks(self.forward(input, out=local), self.group, out=out_full)


class RowParallelQuantLinear:
    """Input features split across ranks; forward = local product, all-reduce SUM, then bias.

    With a ``PeerExchange`` the decode case (one activation row, Q4_K/Q6_K) runs as ONE kernel that pushes
    the partial row to all ranks over NVLink and adds the rows in rank order; other results of up to 65536
    values (a few rows) take ``quant_matmul`` + the exchange all-reduce kernel; larger ones ``quant_matmul``
    + the process group's all-reduce."""

    def __init__(self, local_weight: QuantTensor, bias: Optional[torch.Tensor] = None, group=None,
                 exchange: Optional[PeerExchange] = None):
        self.weight = local_weight
        self.bias = bias
        self.group = group
        self.exchange = exchange

    @classmethod
    def from_full(cls, fmt, packed: np.ndarray, n: int, k: int, rank: int, world_size: int, device="cuda", group=None,
                  exchange: Optional[PeerExchange] = None):
        return cls(scatter_to_rank(fmt, packed, n, k, 1, rank, world_size, device), None, group, exchange)

    def forward(self, input_shard: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        ex = self.exchange
        y = None
        if ex is not None and ex.table is not None and input_shard.is_cuda:
            y = ops.row_parallel_matmul(input_shard, self.weight, ex.rank, ex.world, ex.table, out=out)
        if y is None:
            y = ops.quant_matmul(input_shard, self.weight, out=out)
            # small results (a few rows) go through the exchange buffers too: one short kernel instead of a collective
            if not (ex is not None and ex.table is not None and ops.tp_all_reduce(y, ex.rank, ex.world, ex.table)):
                all_reduce_tensor(y, self.group)
        if self.bias is not None:
            y.add_(self.bias)
        return y

    __call__ = forward
