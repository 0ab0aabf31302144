"""Quantized linear modules: the callers of the quantized ops.

Mirrors ``QuantLinear`` and the quantized arm of ``MaybeQuantLinear`` (src/nn/linear.rs:60-179):
``forward`` is ``quant_matmul(input, weight)`` plus an optional bias add, ``forward_batch`` uses
``quant_matmul_batch`` when every layer is quantized and bias-free.  Inference only.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from . import ops
from .tensor import QuantTensor


class QuantLinear:
    def __init__(self, weight: QuantTensor, bias: Optional[torch.Tensor] = None):
        if len(weight.shape) != 2:
            raise ValueError(f"QuantLinear weight must be 2D [out_features, in_features], got {list(weight.shape)}")
        self._weight = weight
        self._bias = bias

    @property
    def weight(self) -> QuantTensor:
        return self._weight

    @property
    def bias(self) -> Optional[torch.Tensor]:
        return self._bias

    @property
    def out_features(self) -> int:
        return self._weight.shape[0]

    @property
    def in_features(self) -> int:
        return self._weight.shape[1]

    def forward(self, input: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """input [..., in_features] -> [..., out_features] (src/nn/linear.rs:73-82)."""
        y = ops.quant_matmul(input, self._weight, out=out)
        if self._bias is not None:
            y.add_(self._bias)
        return y

    __call__ = forward

    @staticmethod
    def forward_batch(layers: Sequence["QuantLinear"], input: torch.Tensor,
                      outs: Optional[Sequence[torch.Tensor]] = None) -> List[torch.Tensor]:
        """Several projections of one input (src/nn/linear.rs:145-179)."""
        if all(l.bias is None for l in layers):
            return ops.quant_matmul_batch(input, [l.weight for l in layers], outs=outs)
        return [l.forward(input, None if outs is None else outs[i]) for i, l in enumerate(layers)]


class MaybeQuantLinear:
    """A linear that holds either a dense weight or a quantized one (src/nn/linear.rs:98-179).

    ``Quantized`` forwards through ``QuantLinear``; ``Standard`` is a plain ``x @ W^T + b`` on a dense
    tensor (norm-free layers a GGUF file keeps in F32/F16; torch's matmul, not part of the quantized path).
    ``forward_batch`` takes the one-launch batch path only when every layer is quantized and bias-free,
    as the reference does (:160-174); otherwise each layer runs by itself."""

    def __init__(self, quantized: Optional[QuantLinear] = None, weight: Optional[torch.Tensor] = None,
                 bias: Optional[torch.Tensor] = None):
        if (quantized is None) == (weight is None):
            raise ValueError("MaybeQuantLinear holds exactly one of a QuantLinear or a dense weight")
        self.quantized = quantized
        self.dense_weight = weight
        self.dense_bias = bias

    @classmethod
    def from_weight(cls, weight, bias: Optional[torch.Tensor] = None) -> "MaybeQuantLinear":
        if isinstance(weight, QuantTensor):
            return cls(quantized=QuantLinear(weight, bias))
        return cls.standard(weight, bias)

    @classmethod
    def standard(cls, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> "MaybeQuantLinear":
        if weight.dim() != 2:
            raise ValueError(f"Linear weight must be 2D [out_features, in_features], got {list(weight.shape)}")
        return cls(weight=weight, bias=bias)

    @property
    def is_quantized(self) -> bool:
        return self.quantized is not None

    def forward(self, input: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.quantized is not None:
            return self.quantized.forward(input, out)
        y = torch.nn.functional.linear(input.to(self.dense_weight.dtype), self.dense_weight,
                                       None if self.dense_bias is None else self.dense_bias.to(self.dense_weight.dtype))
        if out is not None:
            out.copy_(y)
            return out
        return y

    __call__ = forward

    @staticmethod
    def forward_batch(layers: Sequence["MaybeQuantLinear"], input: torch.Tensor,
                      outs: Optional[Sequence[torch.Tensor]] = None) -> List[torch.Tensor]:
        if all(l.quantized is not None and l.quantized.bias is None for l in layers):
            return ops.quant_matmul_batch(input, [l.quantized.weight for l in layers], outs=outs)
        return [l.forward(input, None if outs is None else outs[i]) for i, l in enumerate(layers)]
