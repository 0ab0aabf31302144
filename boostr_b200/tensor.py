"""``QuantTensor``: packed block storage on a CUDA device.

Mirrors ``QuantTensor<R>`` (src/quant/tensor.rs:23-127): raw little-endian blocks as a U8
buffer, the block format, and the LOGICAL element shape.  Blocks run along the last axis.
"""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from .format import QuantError, QuantFormat


class QuantTensor:
    def __init__(self, storage: torch.Tensor, fmt: QuantFormat, shape: Sequence[int]):
        self._storage = storage
        self._format = fmt
        self._shape = tuple(int(x) for x in shape)

    @classmethod
    def from_bytes(cls, data, fmt, shape: Sequence[int], device="cuda") -> "QuantTensor":
        """src/quant/tensor.rs:44-92 — validates the last dimension and the exact byte count."""
        fmt = QuantFormat.parse(fmt)
        shape = tuple(int(x) for x in shape)
        if len(shape) == 0:
            raise QuantError("QuantTensor shape must be non-empty")
        last = shape[-1]
        if last % fmt.block_size:
            raise QuantError(
                f"last dimension {last} is not a multiple of {fmt.name}'s block_size {fmt.block_size}")
        numel = int(np.prod(shape, dtype=np.int64))
        expected = fmt.storage_bytes(numel)
        if isinstance(data, torch.Tensor):
            t = data.reshape(-1)
            if t.dtype != torch.uint8:
                raise QuantError("QuantTensor storage must be uint8")
        else:
            arr = np.frombuffer(data, dtype=np.uint8) if isinstance(data, (bytes, bytearray, memoryview)) else \
                np.ascontiguousarray(data, dtype=np.uint8).reshape(-1)
            t = torch.from_numpy(arr.copy() if not arr.flags.writeable else arr)
        if t.numel() != expected:
            raise QuantError(
                f"expected {expected} bytes for {fmt.name} with {numel} elements, got {t.numel()} bytes")
        t = t.to(device).contiguous()
        if t.data_ptr() % 16:  # torch's allocator hands out 512-byte aligned blocks; views may not be
            t = t.clone()
        return cls(t, fmt, shape)

    # accessors: src/quant/tensor.rs:95-127
    @property
    def format(self) -> QuantFormat:
        return self._format

    @property
    def shape(self) -> tuple:
        return self._shape

    def numel(self) -> int:
        return int(np.prod(self._shape, dtype=np.int64))

    def num_blocks(self) -> int:
        return self.numel() // self._format.block_size

    def storage_bytes(self) -> int:
        return self.num_blocks() * self._format.block_bytes

    @property
    def device(self) -> torch.device:
        return self._storage.device

    @property
    def storage(self) -> torch.Tensor:
        return self._storage
