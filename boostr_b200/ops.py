"""Host-side mirror of boostr's quantized ops, bound to the sm_100a library.

``dequantize`` ~ DequantOps::dequantize (src/quant/traits/dequant.rs:15),
``quant_matmul`` / ``quant_matmul_batch`` / ``quant_swiglu`` ~ QuantMatmulOps
(src/quant/traits/quant_matmul.rs:22-39,122-127).  Same argument meaning, same shape rules
and the same error texts as the reference's CUDA implementation
(src/quant/cuda/quant_matmul/impl_ops.rs:112-172, src/quant/cuda/dequant.rs:74-146).  The
calls enqueue on torch's current stream and do not synchronise.  torch supplies device
memory and the stream handle only; all arithmetic happens in ``libb200q.so``.
"""
from __future__ import annotations

import ctypes
from typing import List, Sequence

import torch

from . import _cabi
from .format import QuantError
from .tensor import QuantTensor

_DT = {torch.float32: _cabi.DT_F32, torch.bfloat16: _cabi.DT_BF16, torch.float16: _cabi.DT_F16,
       torch.float64: _cabi.DT_F64}

_workspaces: dict = {}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise QuantError(f"{what} must live on a CUDA device: this library has no CPU path")


def workspace(nbytes: int, device) -> torch.Tensor:
    """Scratch buffer reused across calls on one device (grown on demand, never shrunk)."""
    key = (torch.device(device).index, torch.cuda.current_stream().cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def dequantize(qt: QuantTensor, target_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    if target_dtype not in _DT:
        raise QuantError(f"dequantize target must be float, got {target_dtype}")
    _require_cuda(qt.storage, "QuantTensor")
    out = torch.empty(qt.shape, dtype=target_dtype, device=qt.device)
    with torch.cuda.device(qt.device):
        _cabi.check(_cabi.lib().b200q_dequantize(qt.format.format_id, qt.storage.data_ptr(), qt.num_blocks(),
                                                 out.data_ptr(), _DT[target_dtype], _stream()))
    return out


def _check_act(op: str, activation: torch.Tensor, weight: QuantTensor, allow_bf16: bool):
    ok = (torch.float32, torch.bfloat16) if allow_bf16 else (torch.float32,)
    if activation.dtype not in ok:
        raise QuantError(f"{op} activation must be F32, got {activation.dtype}")
    if len(weight.shape) != 2:
        raise QuantError(f"{op} weight must be 2D [N, K], got {list(weight.shape)}")
    n, k = weight.shape
    if activation.dim() == 0:
        raise QuantError(f"{op} activation must be at least 1D")
    if activation.shape[-1] != k:
        raise QuantError(f"{op} dimension mismatch: activation K={activation.shape[-1]}, weight K={k}")
    _require_cuda(activation, "activation")
    _require_cuda(weight.storage, "QuantTensor")
    act = activation.contiguous()
    if act.data_ptr() % 16:
        act = act.clone()
    m = act.numel() // k
    return act, m, k, n


def _out_buffer(out, shape, dtype, device):
    if out is None:
        return torch.empty(shape, dtype=dtype, device=device)
    if tuple(out.shape) != tuple(shape) or out.dtype != dtype or not out.is_contiguous() or out.device != device:
        raise QuantError(f"out must be a contiguous {dtype} tensor of shape {list(shape)} on {device}")
    return out


def quant_matmul(activation: torch.Tensor, weight: QuantTensor, out_dtype: torch.dtype = torch.float32,
                 allow_bf16_activation: bool = True, out: torch.Tensor = None) -> torch.Tensor:
    """activation [..., M, K] x weight [N, K] -> [..., M, N] (F32 unless out_dtype says otherwise).

    ``out`` lets the caller supply the result buffer (as boostr's CUDA backend allocates the
    output before the launch); with it the call allocates nothing, which CUDA-graph capture needs."""
    act, m, k, n = _check_act("quant_matmul", activation, weight, allow_bf16_activation)
    out = _out_buffer(out, (*activation.shape[:-1], n), out_dtype, act.device)
    if m == 0:
        return out
    L = _cabi.lib()
    with torch.cuda.device(act.device):
        need = L.b200q_workspace_bytes(_cabi.OP_QUANT_MATMUL, weight.format.format_id, m, k, n)
        ws = workspace(need, act.device) if need else None
        _cabi.check(L.b200q_quant_matmul(weight.format.format_id, act.data_ptr(), _DT[act.dtype],
                                         weight.storage.data_ptr(), out.data_ptr(), _DT[out_dtype], m, k, n,
                                         ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
                                         _stream()))
    return out


def row_parallel_matmul(activation: torch.Tensor, weight: QuantTensor, rank: int, world: int, table,
                        out: torch.Tensor = None):
    """Local product of a row-parallel shard fused with the all-reduce over peer memory
    (``b200q_row_parallel_matmul``).  Returns None, having launched nothing, when the shape has no fused
    path; the caller then runs ``quant_matmul`` and a collective."""
    act, m, k, n = _check_act("row_parallel_matmul", activation, weight, True)
    if m != 1:
        return None
    out = _out_buffer(out, (*activation.shape[:-1], n), torch.float32, act.device)
    L = _cabi.lib()
    with torch.cuda.device(act.device):
        rc = L.b200q_row_parallel_matmul(weight.format.format_id, act.data_ptr(), _DT[act.dtype], weight.storage.data_ptr(),
                                         out.data_ptr(), _cabi.DT_F32, m, k, n, rank, world, table, _stream())
    if rc == _cabi.ERR_NOT_FUSED:
        return None
    _cabi.check(rc)
    return out


def col_parallel_matmul_gather(activation: torch.Tensor, weight: QuantTensor, rank: int, world: int, table,
                               out_full: torch.Tensor):
    """Local product of a column-parallel shard fused with the gather of all ranks' slices into
    ``out_full`` [..., world * n_local] (``b200q_col_parallel_matmul_gather``).  Returns None, having
    launched nothing, when the shape has no fused path."""
    act, m, k, n = _check_act("col_parallel_matmul_gather", activation, weight, True)
    if m != 1:
        return None
    out_full = _out_buffer(out_full, (*activation.shape[:-1], n * world), torch.float32, act.device)
    L = _cabi.lib()
    with torch.cuda.device(act.device):
        rc = L.b200q_col_parallel_matmul_gather(weight.format.format_id, act.data_ptr(), _DT[act.dtype], weight.storage.data_ptr(),
                                                out_full.data_ptr(), m, k, n, rank, world, table, _stream())
    if rc == _cabi.ERR_NOT_FUSED:
        return None
    _cabi.check(rc)
    return out_full


def tp_all_reduce(tensor: torch.Tensor, rank: int, world: int, table) -> bool:
    """In-place sum of a small contiguous f32 CUDA tensor over the exchange buffers (``b200q_tp_all_reduce``).
    Returns False, having launched nothing, when the tensor does not fit (use the process group instead)."""
    if not tensor.is_cuda or tensor.dtype != torch.float32 or not tensor.is_contiguous():
        return False
    L = _cabi.lib()
    with torch.cuda.device(tensor.device):
        rc = L.b200q_tp_all_reduce(tensor.data_ptr(), tensor.numel(), rank, world, table, _stream())
    if rc == _cabi.ERR_NOT_FUSED:
        return False
    _cabi.check(rc)
    return True


def quant_matmul_batch(activation: torch.Tensor, weights: Sequence[QuantTensor],
                       out_dtype: torch.dtype = torch.float32, outs: Sequence[torch.Tensor] = None) -> List[torch.Tensor]:
    """One activation against several weights sharing K (q/k/v, gate/up)."""
    if not weights:
        return []
    acts = [_check_act("quant_matmul", activation, w, True) for w in weights]
    act, m, k, _ = acts[0]
    outs = [_out_buffer(None if outs is None else outs[i], (*activation.shape[:-1], a[3]), out_dtype, act.device)
            for i, a in enumerate(acts)]
    if m == 0:
        return outs
    L = _cabi.lib()
    nw = len(weights)
    fmts = (ctypes.c_int * nw)(*[w.format.format_id for w in weights])
    wptr = (ctypes.c_void_p * nw)(*[w.storage.data_ptr() for w in weights])
    ns = (ctypes.c_size_t * nw)(*[a[3] for a in acts])
    optr = (ctypes.c_void_p * nw)(*[o.data_ptr() for o in outs])
    with torch.cuda.device(act.device):
        need = max(L.b200q_workspace_bytes(_cabi.OP_QUANT_MATMUL, w.format.format_id, m, k, a[3])
                   for w, a in zip(weights, acts))
        ws = workspace(need, act.device) if need else None
        _cabi.check(L.b200q_quant_matmul_batch(nw, fmts, wptr, ns, optr, act.data_ptr(), _DT[act.dtype],
                                               _DT[out_dtype], m, k, ws.data_ptr() if ws is not None else None,
                                               ws.numel() if ws is not None else 0, _stream()))
    return outs


def rmsnorm_quant_matmul_batch(activation: torch.Tensor, norm_weight: torch.Tensor, eps: float, weights: Sequence[QuantTensor],
                               out_dtype: torch.dtype = torch.float32, outs: Sequence[torch.Tensor] = None) -> List[torch.Tensor]:
    """RMSNorm(activation) against several weights sharing K: the attention block's input_layernorm + q/k/v
    projections as one operator (``b200q_rmsnorm_quant_matmul_batch``).  With one activation row and Q4_K / Q6_K weights
    the normalisation happens inside the decode kernel."""
    if not weights:
        return []
    acts = [_check_act("rmsnorm_quant_matmul", activation, w, True) for w in weights]
    act, m, k, _ = acts[0]
    if norm_weight.dtype != torch.float32 or norm_weight.numel() != k or not norm_weight.is_cuda or not norm_weight.is_contiguous():
        raise QuantError(f"norm weight must be a contiguous F32 CUDA tensor of {k} elements")
    outs = [_out_buffer(None if outs is None else outs[i], (*activation.shape[:-1], a[3]), out_dtype, act.device)
            for i, a in enumerate(acts)]
    if m == 0:
        return outs
    L = _cabi.lib()
    nw = len(weights)
    fmts = (ctypes.c_int * nw)(*[w.format.format_id for w in weights])
    wptr = (ctypes.c_void_p * nw)(*[w.storage.data_ptr() for w in weights])
    ns = (ctypes.c_size_t * nw)(*[a[3] for a in acts])
    optr = (ctypes.c_void_p * nw)(*[o.data_ptr() for o in outs])
    with torch.cuda.device(act.device):
        need = max(L.b200q_workspace_bytes(_cabi.OP_QUANT_MATMUL, w.format.format_id, m, k, a[3]) for w, a in zip(weights, acts))
        need += (m * k * 4 + 255) // 256 * 256
        ws = workspace(need, act.device)
        _cabi.check(L.b200q_rmsnorm_quant_matmul_batch(nw, fmts, wptr, ns, optr, act.data_ptr(), norm_weight.data_ptr(), float(eps),
                                                       _DT[act.dtype], _DT[out_dtype], m, k, ws.data_ptr(), ws.numel(), _stream()))
    return outs


def quant_swiglu(activation: torch.Tensor, gate_weight: QuantTensor, up_weight: QuantTensor,
                 out_dtype: torch.dtype = torch.float32, out: torch.Tensor = None) -> torch.Tensor:
    """silu(activation x gate^T) * (activation x up^T); gate and up share N, K and format."""
    if gate_weight.format != up_weight.format or tuple(gate_weight.shape) != tuple(up_weight.shape):
        raise QuantError("quant_swiglu: gate and up weights must have the same format and shape")
    act, m, k, n = _check_act("quant_swiglu", activation, gate_weight, True)
    out = _out_buffer(out, (*activation.shape[:-1], n), out_dtype, act.device)
    if m == 0:
        return out
    L = _cabi.lib()
    with torch.cuda.device(act.device):
        need = L.b200q_workspace_bytes(_cabi.OP_QUANT_SWIGLU, gate_weight.format.format_id, m, k, n)
        ws = workspace(need, act.device) if need else None
        _cabi.check(L.b200q_quant_swiglu(gate_weight.format.format_id, act.data_ptr(), _DT[act.dtype],
                                         gate_weight.storage.data_ptr(), up_weight.storage.data_ptr(), out.data_ptr(),
                                         _DT[out_dtype], m, k, n, ws.data_ptr() if ws is not None else None,
                                         ws.numel() if ws is not None else 0, _stream()))
    return out


def prefetch_next(weights: Sequence[QuantTensor], swiglu: bool = False) -> None:
    """Hint for a single-row decode loop (``b200q_prefetch_next``): ``weights`` are those of the operation AFTER the next
    call — several weights sharing one activation row, or ``[gate, up]`` with ``swiglu=True``.  The next call pulls the
    head of those weights into L2 while it drains.  Purely a performance hint; results never depend on it."""
    if not weights:
        return
    nw = len(weights)
    k = weights[0].shape[-1]
    fmts = (ctypes.c_int * nw)(*[w.format.format_id for w in weights])
    wptr = (ctypes.c_void_p * nw)(*[w.storage.data_ptr() for w in weights])
    ns = (ctypes.c_size_t * nw)(*[w.shape[0] for w in weights])
    with torch.cuda.device(weights[0].storage.device):
        _cabi.check(_cabi.lib().b200q_prefetch_next(_cabi.OP_QUANT_SWIGLU if swiglu else _cabi.OP_QUANT_MATMUL, nw, fmts, wptr, ns, k))


def quant_mlp(activation: torch.Tensor, gate_weight: QuantTensor, up_weight: QuantTensor, down_weight: QuantTensor,
              out_dtype: torch.dtype = torch.float32, out: torch.Tensor = None) -> torch.Tensor:
    """down(silu(activation x gate^T) * (activation x up^T)): the feed-forward block of a quantized layer
    (src/model/llama/model/blocks_mlp.rs:38-46) as one call; the hidden state stays in scratch."""
    if gate_weight.format != up_weight.format or tuple(gate_weight.shape) != tuple(up_weight.shape):
        raise QuantError("quant_mlp: gate and up weights must have the same format and shape")
    act, m, k, n_ff = _check_act("quant_mlp", activation, gate_weight, True)
    if len(down_weight.shape) != 2 or down_weight.shape[1] != n_ff:
        raise QuantError(f"quant_mlp: down weight {tuple(down_weight.shape)} does not take a hidden state of {n_ff}")
    n_out = down_weight.shape[0]
    out = _out_buffer(out, (*activation.shape[:-1], n_out), out_dtype, act.device)
    if m == 0:
        return out
    L = _cabi.lib()
    with torch.cuda.device(act.device):
        need = L.b200q_mlp_workspace_bytes(gate_weight.format.format_id, down_weight.format.format_id, m, k, n_ff, n_out)
        ws = workspace(need, act.device)
        _cabi.check(L.b200q_quant_mlp(gate_weight.format.format_id, gate_weight.storage.data_ptr(), up_weight.storage.data_ptr(),
                                      down_weight.format.format_id, down_weight.storage.data_ptr(), act.data_ptr(), _DT[act.dtype],
                                      out.data_ptr(), _DT[out_dtype], m, k, n_ff, n_out, ws.data_ptr(), ws.numel(), _stream()))
    return out


def launch_count() -> int:
    """Kernel launches issued by the library so far in this process."""
    return int(_cabi.lib().b200q_launch_count())


def check_device_status() -> None:
    """Synchronises the current stream and raises if a kernel gave up on a bounded wait."""
    _cabi.check(_cabi.lib().b200q_check_device_status(_stream()))
