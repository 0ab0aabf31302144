"""The quantized linears of a LLaMA-shaped decoder, composed the way boostr's tensor-parallel LLaMA
composes them (src/model/llama/model_tp.rs:321-359, block_tp.rs:72-102, 299-304): q/k/v as one batched
column-parallel projection, o row-parallel, gate/up through ``quant_swiglu``, down row-parallel, and a
column-parallel lm_head whose logits are gathered.  Attention, normalisation and the residual stream are
not part of the quantized-linear path and are left out: o_proj consumes the q projection, and every layer
starts again from the step input so magnitudes stay finite.

Used by ``bench.py`` (Llama-3-8B shapes, Q4_K_M mix) and by the graph-replay tests (small shapes).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from . import ops, synth
from .linear import QuantLinear
from .tensor_parallel import ColumnParallelQuantLinear, PeerExchange, RowParallelQuantLinear

# (name, format, N, K, parallel split) of one layer of a Llama-3-8B-shaped model in a Q4_K_M-style mix
HIDDEN, KV, FFN, VOCAB, LAYERS = 4096, 1024, 14336, 128256, 32


def layer_spec(hidden: int = HIDDEN, kv: int = KV, ffn: int = FFN) -> List[Tuple[str, str, int, int, str]]:
    return [
        ("q", "Q4_K", hidden, hidden, "col"), ("k", "Q4_K", kv, hidden, "col"), ("v", "Q6_K", kv, hidden, "col"),
        ("o", "Q4_K", hidden, hidden, "row"), ("gate", "Q4_K", ffn, hidden, "col"), ("up", "Q4_K", ffn, hidden, "col"),
        ("down", "Q6_K", hidden, ffn, "row"),
    ]


class DecodeStack:
    """``layers`` blocks + lm_head, sharded for rank ``rank`` of ``world``; all activations pre-allocated,
    so ``step()`` allocates nothing and can be captured in a CUDA graph."""

    def __init__(self, m: int, rank: int = 0, world: int = 1, layers: int = LAYERS, hidden: int = HIDDEN, kv: int = KV,
                 ffn: int = FFN, vocab: int = VOCAB, seed: int = 0xB200, same_weights_on_all_ranks: bool = False,
                 weights: Optional[Sequence[dict]] = None, lm_head=None):
        self.m, self.rank, self.world = m, rank, world
        self.spec = layer_spec(hidden, kv, ffn)
        self.hidden, self.kv, self.ffn, self.vocab = hidden, kv, ffn, vocab
        gen = torch.Generator(device="cuda")
        gen.manual_seed(seed + (0 if same_weights_on_all_ranks else rank))
        p = world
        self.layers = []
        for li in range(layers):
            L = {}
            for name, fmt, n, k, split in self.spec:
                if weights is not None:
                    L[name] = weights[li][name]
                elif split == "col":
                    L[name] = ColumnParallelQuantLinear(synth.device_weight(fmt, n // p, k, gen))
                else:
                    L[name] = RowParallelQuantLinear(synth.device_weight(fmt, n, k // p, gen))
            L["qkv"] = [QuantLinear(L["q"].weight), QuantLinear(L["k"].weight), QuantLinear(L["v"].weight)]
            self.layers.append(L)
        self.lm_head = lm_head if lm_head is not None else ColumnParallelQuantLinear(synth.device_weight("Q6_K", vocab // p, hidden, gen))
        f32 = dict(dtype=torch.float32, device="cuda")
        self.x = torch.randn(m, hidden, generator=gen, **f32)           # step input (hidden state)
        self.q = torch.empty(m, hidden // p, **f32)
        self.k = torch.empty(m, kv // p, **f32)
        self.v = torch.empty(m, kv // p, **f32)
        self.o = torch.empty(m, hidden, **f32)
        self.h = torch.empty(m, ffn // p, **f32)
        self.d = torch.empty(m, hidden, **f32)
        self.logits_local = torch.empty(m, vocab // p, **f32)
        self.logits = torch.empty(m, vocab, **f32) if p > 1 else self.logits_local
        self.exchange: Optional[PeerExchange] = None
        self.prefetch = True  # tell each call which weights follow it (ops.prefetch_next)
        self.bytes_local = sum(L[n].weight.storage_bytes() for L in self.layers for n, *_ in self.spec) + \
            self.lm_head.weight.storage_bytes()

    def use_exchange(self, exchange: Optional[PeerExchange]) -> None:
        """Row-parallel layers run fused with their all-reduce over peer memory (None: NCCL all-reduce)."""
        self.exchange = exchange
        for L in self.layers:
            L["o"].exchange = exchange
            L["down"].exchange = exchange

    def step(self) -> torch.Tensor:
        # single-row decode: every call is told which weights come after it, so its launch ends by pulling their head
        # into L2 (a hint only; it is baked into a captured graph like any other argument)
        hint = ops.prefetch_next if self.m == 1 and self.prefetch else (lambda *a, **k: None)
        for i, L in enumerate(self.layers):
            hint([L["o"].weight])
            QuantLinear.forward_batch(L["qkv"], self.x, outs=[self.q, self.k, self.v])   # column-parallel
            hint([L["gate"].weight, L["up"].weight], swiglu=True)
            L["o"].forward(self.q, out=self.o)                      # row-parallel: all-reduce inside
            hint([L["down"].weight])
            ops.quant_swiglu(self.o, L["gate"].weight, L["up"].weight, out=self.h)
            hint([l.weight for l in self.layers[i + 1]["qkv"]] if i + 1 < len(self.layers) else [self.lm_head.weight])
            L["down"].forward(self.h, out=self.d)                   # row-parallel: all-reduce inside
        hint([l.weight for l in self.layers[0]["qkv"]])             # the next step starts there
        if self.world > 1:
            self.lm_head.forward_gathered(self.x, self.logits, self.exchange, local=self.logits_local)
        else:
            self.lm_head.forward(self.x, out=self.logits_local)
        return self.logits
