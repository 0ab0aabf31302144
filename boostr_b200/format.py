"""Block formats of the quantized-linear path.

Mirrors ``QuantFormat`` (src/quant/format.rs:23-230) for the GGUF formats this library
implements: Q4_0, Q5_0, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K and Q6_K.  Blocks are packed along the last (K) axis of a row-major tensor and
rows carry no padding (src/quant/format.rs:5-20).
"""
from __future__ import annotations

import enum


class QuantError(ValueError):
    """Counterpart of ``Error::QuantError { reason }`` (src/error.rs:22-27)."""


class QuantFormat(enum.Enum):
    # value = QuantFormat::format_id (src/quant/format.rs:204-230); it is also the id the C ABI takes
    Q4_0 = 0
    Q5_0 = 2
    Q8_0 = 4
    Q2_K = 6
    Q3_K = 7
    Q4_K = 8
    Q5_K = 9
    Q6_K = 10

    @property
    def block_size(self) -> int:  # src/quant/format.rs:81-108
        return 32 if self in (QuantFormat.Q4_0, QuantFormat.Q5_0, QuantFormat.Q8_0) else 256

    @property
    def block_bytes(self) -> int:  # src/quant/format.rs:110-140
        return {QuantFormat.Q4_0: 18, QuantFormat.Q5_0: 22, QuantFormat.Q8_0: 34, QuantFormat.Q2_K: 84, QuantFormat.Q3_K: 110, QuantFormat.Q4_K: 144, QuantFormat.Q5_K: 176, QuantFormat.Q6_K: 210}[self]

    @property
    def ggml_type_id(self) -> int:  # src/quant/format.rs:174-200
        return {QuantFormat.Q4_0: 2, QuantFormat.Q5_0: 6, QuantFormat.Q8_0: 8, QuantFormat.Q2_K: 10, QuantFormat.Q3_K: 11, QuantFormat.Q4_K: 12, QuantFormat.Q5_K: 13, QuantFormat.Q6_K: 14}[self]

    @property
    def format_id(self) -> int:
        return self.value

    def storage_bytes(self, numel: int) -> int:  # src/quant/format.rs:142-157
        if numel % self.block_size:
            raise QuantError(f"{self.name}: element count {numel} is not a multiple of block_size {self.block_size}")
        return numel // self.block_size * self.block_bytes

    def num_blocks(self, numel: int) -> int:  # src/quant/format.rs:159-172
        if numel % self.block_size:
            raise QuantError(f"{self.name}: element count {numel} is not a multiple of block_size {self.block_size}")
        return numel // self.block_size

    @classmethod
    def from_ggml_type_id(cls, type_id: int) -> "QuantFormat":  # src/quant/format.rs:232-260
        for f in cls:
            if f.ggml_type_id == type_id:
                return f
        raise QuantError(f"unsupported GGML type id {type_id}")

    @classmethod
    def parse(cls, x) -> "QuantFormat":
        if isinstance(x, cls):
            return x
        if isinstance(x, str):
            key = x.upper().replace("Q2K", "Q2_K").replace("Q3K", "Q3_K").replace("Q4K", "Q4_K").replace("Q5K", "Q5_K").replace("Q6K", "Q6_K")
            return cls[key]
        return cls(int(x))
