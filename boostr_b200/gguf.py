"""GGUF files -> device ``QuantTensor``s and quantized linears, with tensor-parallel sharding at load.

Mirrors the part of boostr's GGUF reader that feeds the quantized-linear path:
``Gguf::open`` / ``from_bytes`` / ``parse_header`` (src/format/gguf/reader.rs:53-140: magic, version 1-3,
tensor and key/value counts, ``general.alignment``, tensor infos, aligned data offset),
``load_tensor_quantized`` (reader.rs:473-503: GGML-order shape reversed to row-major, bytes handed to
``QuantTensor::from_bytes``), the GGML type ids (src/format/gguf/types.rs:108-125), the GGUF -> HuggingFace
tensor names (src/format/gguf/name_map.rs:17-69) and ``VarBuilder::take_maybe_quant_linear``
(src/nn/var_builder.rs:137-153).

What the reference does not have, because its ``QuantTensor`` cannot be sliced: the rank's shard is cut
while loading.  Column-parallel tensors (split along N) are a contiguous byte range of the file, so only
that range is read; row-parallel tensors (split along K) are read whole and repacked on the host by
``b200q_shard_pack``.  The file format itself is the published GGUF layout; the parser below is written
against that layout, not against the reference's code.
"""
from __future__ import annotations

import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

from .format import QuantError, QuantFormat
from .tensor import QuantTensor

GGUF_MAGIC = 0x46554747  # "GGUF", little endian
GGUF_DEFAULT_ALIGNMENT = 32

# GGML tensor types: id -> (name, block_size, block_bytes)  (src/format/gguf/types.rs)
GGML_TYPES = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22),
    7: ("Q5_1", 32, 24), 8: ("Q8_0", 32, 34), 9: ("Q8_1", 32, 36), 10: ("Q2_K", 256, 84), 11: ("Q3_K", 256, 110),
    12: ("Q4_K", 256, 144), 13: ("Q5_K", 256, 176), 14: ("Q6_K", 256, 210), 15: ("Q8_K", 256, 292),
    24: ("I8", 1, 1), 25: ("I16", 1, 2), 26: ("I32", 1, 4), 27: ("I64", 1, 8), 28: ("F64", 1, 8), 30: ("BF16", 1, 2),
}
_DENSE = {0: torch.float32, 1: torch.float16, 30: torch.bfloat16, 28: torch.float64}

# metadata value types of the GGUF key/value section
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_T_STRING, _T_ARRAY = 8, 9


class GgufError(RuntimeError):
    """Counterpart of ``Error::ModelError { reason }`` raised by the reference's reader."""


@dataclass
class GgufTensorInfo:
    """src/format/gguf/tensor_info.rs: ``shape`` is in GGML order (innermost dimension first)."""
    name: str
    shape: Tuple[int, ...]
    ggml_type: int
    offset: int

    @property
    def type_name(self) -> str:
        return GGML_TYPES.get(self.ggml_type, (f"type{self.ggml_type}", 1, 0))[0]

    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n

    def size_bytes(self) -> int:
        _, bs, bb = GGML_TYPES[self.ggml_type]
        return -(-self.numel() // bs) * bb

    def row_major_shape(self) -> Tuple[int, ...]:
        return tuple(reversed(self.shape))


class _Cursor:
    def __init__(self, buf, version_hint: int = 3):
        self.buf, self.pos, self.version = buf, 0, version_hint

    def take(self, fmt: str):
        size = struct.calcsize(fmt)
        if self.pos + size > len(self.buf):
            raise GgufError("unexpected end of GGUF header")
        v = struct.unpack_from(fmt, self.buf, self.pos)[0]
        self.pos += size
        return v

    def length(self) -> int:  # v1 files use 32-bit counts and lengths
        return self.take("<I") if self.version == 1 else self.take("<Q")

    def string(self) -> str:
        n = self.length()
        if self.pos + n > len(self.buf):
            raise GgufError("unexpected end of GGUF header")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8", errors="replace")
        self.pos += n
        return s

    def value(self, vtype: int):
        if vtype in _SCALARS:
            return self.take(_SCALARS[vtype])
        if vtype == _T_STRING:
            return self.string()
        if vtype == _T_ARRAY:
            item = self.take("<I")
            n = self.length()
            return [self.value(item) for _ in range(n)]
        raise GgufError(f"unknown GGUF metadata value type {vtype}")


def gguf_to_hf_name(name: str) -> str:
    """GGUF tensor name -> HuggingFace name (src/format/gguf/name_map.rs:17-69); unknown names pass through."""
    glob = {"token_embd.weight": "model.embed_tokens.weight", "output_norm.weight": "model.norm.weight",
            "output.weight": "lm_head.weight"}
    if name in glob:
        return glob[name]
    if name.startswith("blk."):
        rest = name[4:]
        layer, dot, suffix = rest.partition(".")
        if dot and layer.isdigit():
            if suffix in _LAYER_SUFFIX:
                return f"model.layers.{layer}.{_LAYER_SUFFIX[suffix]}"
            parts = suffix.split(".", 2)  # MoE experts: ffn_{gate,up,down}.E.weight
            if len(parts) == 3 and parts[1].isdigit() and parts[0] in _MOE_PROJ:
                return f"model.layers.{layer}.block_sparse_moe.experts.{parts[1]}.{_MOE_PROJ[parts[0]]}.{parts[2]}"
    return name


_MOE_PROJ = {"ffn_gate": "gate_proj", "ffn_up": "up_proj", "ffn_down": "down_proj"}
_LAYER_SUFFIX = {
    "attn_q.weight": "self_attn.q_proj.weight", "attn_k.weight": "self_attn.k_proj.weight",
    "attn_v.weight": "self_attn.v_proj.weight", "attn_output.weight": "self_attn.o_proj.weight",
    "attn_q.bias": "self_attn.q_proj.bias", "attn_k.bias": "self_attn.k_proj.bias",
    "attn_v.bias": "self_attn.v_proj.bias", "attn_output.bias": "self_attn.o_proj.bias",
    "ffn_gate.weight": "mlp.gate_proj.weight", "ffn_up.weight": "mlp.up_proj.weight",
    "ffn_down.weight": "mlp.down_proj.weight",
    "attn_norm.weight": "input_layernorm.weight", "ffn_norm.weight": "post_attention_layernorm.weight",
}

# Megatron plan of a LLaMA block (src/model/llama/model_tp.rs, src/distributed/tensor_parallel.rs:27-253):
# output features split for q/k/v/gate/up and the lm_head, input features split for o/down.
_COLUMN = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj", "lm_head")
_ROW = ("o_proj", "down_proj")


def parallel_dim(hf_name: str) -> Optional[int]:
    """0 = column-parallel (split N), 1 = row-parallel (split K), None = replicated."""
    stem = hf_name.rsplit(".", 1)[0].rsplit(".", 1)[-1] if "." in hf_name else hf_name
    if stem in _COLUMN:
        return 0
    if stem in _ROW:
        return 1
    return None


class Gguf:
    """A parsed GGUF file: metadata, tensor directory, and tensor reads (whole or one rank's shard)."""

    def __init__(self, data, version: int, metadata: Dict[str, object], tensors: Dict[str, GgufTensorInfo], data_offset: int,
                 keep=None):
        self._data = data          # bytes-like covering the whole file
        self._keep = keep          # (file object, mmap) kept alive while tensors are read
        self.version = version
        self.metadata = metadata
        self.tensors = tensors
        self.data_offset = data_offset

    # -- construction ---------------------------------------------------------------------------
    @classmethod
    def open(cls, path: str) -> "Gguf":
        f = open(path, "rb")
        try:
            mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        except (ValueError, OSError):
            data = f.read()
            f.close()
            return cls.from_bytes(data)
        g = cls.from_bytes(mm)
        g._keep = (f, mm)
        return g

    @classmethod
    def from_bytes(cls, data) -> "Gguf":
        c = _Cursor(data)
        if len(data) < 8 or c.take("<I") != GGUF_MAGIC:
            magic = struct.unpack_from("<I", data, 0)[0] if len(data) >= 4 else 0
            raise GgufError(f"invalid GGUF magic: 0x{magic:08x}")
        version = c.take("<I")
        if not 1 <= version <= 3:
            raise GgufError(f"unsupported GGUF version: {version}")
        c.version = version
        tensor_count = c.length()
        kv_count = c.length()
        metadata: Dict[str, object] = {}
        for _ in range(kv_count):
            key = c.string()
            metadata[key] = c.value(c.take("<I"))
        alignment = int(metadata.get("general.alignment", GGUF_DEFAULT_ALIGNMENT))
        tensors: Dict[str, GgufTensorInfo] = {}
        for _ in range(tensor_count):
            name = c.string()
            n_dims = c.take("<I")
            shape = tuple(c.length() for _ in range(n_dims))
            ggml_type = c.take("<I")
            offset = c.take("<Q")
            tensors[name] = GgufTensorInfo(name, shape, ggml_type, offset)
        data_offset = (c.pos + alignment - 1) // alignment * alignment
        return cls(data, version, metadata, tensors, data_offset)

    def close(self) -> None:
        if self._keep is not None:
            f, mm = self._keep
            self._data = b""
            mm.close()
            f.close()
            self._keep = None

    # -- reads ------------------------------------------------------------------------------------
    def _info(self, name: str) -> GgufTensorInfo:
        if name not in self.tensors:
            raise GgufError(f"GGUF tensor not found: {name}")
        return self.tensors[name]

    def tensor_names(self) -> List[str]:
        return list(self.tensors)

    def _range(self, info: GgufTensorInfo, begin: int, nbytes: int) -> np.ndarray:
        start = self.data_offset + info.offset + begin
        if start + nbytes > len(self._data):
            raise GgufError(f"tensor '{info.name}' extends past the end of the file")
        return np.frombuffer(self._data, dtype=np.uint8, count=nbytes, offset=start)

    def read_tensor_bytes(self, name: str) -> np.ndarray:
        info = self._info(name)
        if info.ggml_type not in GGML_TYPES:
            raise GgufError(f"tensor '{name}' has unknown GGML type id {info.ggml_type}")
        return self._range(info, 0, info.size_bytes())

    def quant_format(self, name: str) -> QuantFormat:
        info = self._info(name)
        try:
            return QuantFormat.from_ggml_type_id(info.ggml_type)
        except QuantError:
            raise GgufError(f"tensor '{name}' type {info.type_name} is not a quantized format of this library") from None

    def load_tensor_quantized(self, name: str, device="cuda", rank: int = 0, world: int = 1,
                              dim: Optional[int] = None) -> QuantTensor:
        """The tensor (or rank ``rank``'s shard of it along ``dim``) as a device ``QuantTensor``.

        dim 0 reads only the rank's rows from the file; dim 1 repacks the rank's K range of every row."""
        info = self._info(name)
        fmt = self.quant_format(name)
        shape = info.row_major_shape()
        if world <= 1 or dim is None:
            return QuantTensor.from_bytes(self.read_tensor_bytes(name), fmt, shape, device=device)
        if len(shape) != 2:
            raise GgufError(f"tensor '{name}' is not 2-D: cannot be sharded")
        n, k = shape
        if dim == 0:
            from .tensor_parallel import DistributedError

            if n % world:
                raise DistributedError(f"out_features {n} not divisible by world_size {world}")
            rows = n // world
            row_bytes = fmt.storage_bytes(k)
            return QuantTensor.from_bytes(self._range(info, rank * rows * row_bytes, rows * row_bytes), fmt, (rows, k), device=device)
        from .tensor_parallel import scatter_to_rank

        return scatter_to_rank(fmt, self.read_tensor_bytes(name), n, k, 1, rank, world, device=device)

    def load_tensor_dense(self, name: str, device="cuda") -> torch.Tensor:
        """F32 / F16 / BF16 / F64 tensors (norm weights, biases) as torch tensors in row-major shape."""
        info = self._info(name)
        if info.ggml_type not in _DENSE:
            raise GgufError(f"tensor '{name}' type {info.type_name} is not a dense float type")
        dt = _DENSE[info.ggml_type]
        raw = torch.from_numpy(self.read_tensor_bytes(name).copy())
        return raw.view(dt).reshape(info.row_major_shape()).to(device)


class GgufVarMap:
    """HF-named view of a GGUF file from which modules take their weights once
    (``VarMap::from_gguf`` + ``VarBuilder``, src/nn/var_builder.rs:137-153)."""

    def __init__(self, gguf: Gguf, device="cuda", rank: int = 0, world: int = 1):
        self.gguf, self.device, self.rank, self.world = gguf, device, rank, world
        self._names = {gguf_to_hf_name(n): n for n in gguf.tensor_names()}

    def contains(self, hf_name: str) -> bool:
        return hf_name in self._names

    def names(self) -> List[str]:
        return sorted(self._names)

    def _take(self, hf_name: str) -> str:
        if hf_name not in self._names:
            raise GgufError(f"tensor not found: {hf_name}")
        return self._names.pop(hf_name)

    def take_quant_tensor(self, hf_name: str, dim: Optional[int] = None) -> QuantTensor:
        return self.gguf.load_tensor_quantized(self._take(hf_name), self.device, self.rank, self.world, dim)

    def take_tensor(self, hf_name: str) -> torch.Tensor:
        return self.gguf.load_tensor_dense(self._take(hf_name), self.device)

    def take_maybe_quant_linear(self, hf_name: str, bias_name: Optional[str] = None, group=None, exchange=None):
        """The linear behind ``hf_name``: quantized types give a ``QuantLinear`` (one rank) or its
        column-/row-parallel form (several ranks, by the Megatron plan of ``parallel_dim``); dense float
        types give a ``MaybeQuantLinear`` holding a plain tensor."""
        from .linear import MaybeQuantLinear, QuantLinear
        from .tensor_parallel import ColumnParallelQuantLinear, RowParallelQuantLinear

        gname = self._names.get(hf_name)
        if gname is None:
            raise GgufError(f"tensor not found: {hf_name}")
        bias = None
        if bias_name is not None and self.contains(bias_name):
            bias = self.take_tensor(bias_name).float()
        if self.gguf.tensors[gname].ggml_type in _DENSE:
            return MaybeQuantLinear.standard(self.take_tensor(hf_name), bias)
        dim = parallel_dim(hf_name) if self.world > 1 else None
        qt = self.take_quant_tensor(hf_name, dim)
        if dim == 0:
            if bias is not None:  # the bias of a column-parallel layer is split like its rows
                bias = bias.chunk(self.world)[self.rank].contiguous()
            return ColumnParallelQuantLinear(qt, bias, group)
        if dim == 1:
            return RowParallelQuantLinear(qt, bias, group, exchange)
        return QuantLinear(qt, bias)


def load_llama_linears(path_or_gguf, device="cuda", rank: int = 0, world: int = 1, group=None, exchange=None) -> Dict[str, object]:
    """Every ``*_proj`` / ``lm_head`` linear of a LLaMA-style GGUF file, keyed by its HF module name
    (``model.layers.3.mlp.down_proj``), sharded for this rank."""
    g = path_or_gguf if isinstance(path_or_gguf, Gguf) else Gguf.open(os.fspath(path_or_gguf))
    vm = GgufVarMap(g, device, rank, world)
    out: Dict[str, object] = {}
    for name in vm.names():
        if not name.endswith(".weight"):
            continue
        stem = name[:-len(".weight")]
        if stem.endswith("_proj") or stem == "lm_head":
            out[stem] = vm.take_maybe_quant_linear(name, stem + ".bias", group, exchange)
    return out
