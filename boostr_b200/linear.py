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
