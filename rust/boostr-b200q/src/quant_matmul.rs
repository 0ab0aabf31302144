//! `QuantMatmulOps::{quant_matmul, quant_matmul_batch, quant_swiglu}` for `CudaClient`
//! (replaces the bodies at `src/quant/cuda/quant_matmul/impl_ops.rs:112-172, 174-335, 337-441`).
//! The M <= 64 / M > 64 dispatch, the Q8_1 activation-quantise launch (`helpers.rs:33-77`) and the PTX
//! module cache are not needed for these formats: the library picks the kernel family from the shape.
use std::os::raw::{c_int, c_void};

use boostr::error::{Error, Result};
use boostr::quant::QuantTensor;
use numr::dtype::DType;
use numr::runtime::cuda::{CudaClient, CudaRuntime};
use numr::tensor::Tensor;

use crate::{check, format_id, ptr_or_null, scratch, stream_of};

/// dtype / shape rules of `quant_matmul` (impl_ops.rs:117-150): returns (m, k, n, output shape).
fn validate(op: &str, activation: &Tensor<CudaRuntime>, weight: &QuantTensor<CudaRuntime>) -> Result<(usize, usize, usize, Vec<usize>)> {
    if activation.dtype() != DType::F32 {
        return Err(Error::QuantError { reason: format!("{op} activation must be F32, got {:?}", activation.dtype()) });
    }
    let w_shape = weight.shape();
    if w_shape.len() != 2 {
        return Err(Error::QuantError { reason: format!("{op} weight must be 2D [N, K], got {:?}", w_shape) });
    }
    let (n, k) = (w_shape[0], w_shape[1]);
    let a_shape = activation.shape();
    if a_shape.is_empty() {
        return Err(Error::QuantError { reason: format!("{op} activation must be at least 1D") });
    }
    let a_k = a_shape[a_shape.len() - 1];
    if a_k != k {
        return Err(Error::QuantError { reason: format!("{op} dimension mismatch: activation K={a_k}, weight K={k}") });
    }
    let m = a_shape.iter().product::<usize>() / k;
    let mut out_shape = a_shape[..a_shape.len() - 1].to_vec();
    out_shape.push(n);
    Ok((m, k, n, out_shape))
}

pub fn quant_matmul(client: &CudaClient, activation: &Tensor<CudaRuntime>, weight: &QuantTensor<CudaRuntime>) -> Result<Tensor<CudaRuntime>> {
    let (m, k, n, out_shape) = validate("quant_matmul", activation, weight)?;
    let Some(fmt) = format_id(weight.format()) else {
        return boostr::quant::cuda::quant_matmul::quant_matmul_ptx(client, activation, weight);
    };
    let act = activation.contiguous()?;
    let out = Tensor::<CudaRuntime>::empty(&out_shape, DType::F32, activation.device());
    let ws_bytes = unsafe { b200q_sys::b200q_workspace_bytes(b200q_sys::B200Q_OP_QUANT_MATMUL, fmt, m, k, n) };
    let ws = scratch(ws_bytes, activation);
    check(unsafe {
        b200q_sys::b200q_quant_matmul(fmt, act.ptr() as *const c_void, b200q_sys::B200Q_F32, weight.storage().ptr() as *const c_void,
                                      out.ptr() as *mut c_void, b200q_sys::B200Q_F32, m, k, n, ptr_or_null(&ws), ws_bytes,
                                      stream_of(client))
    })?;
    Ok(out)
}

pub fn quant_matmul_batch(client: &CudaClient, activation: &Tensor<CudaRuntime>, weights: &[&QuantTensor<CudaRuntime>]) -> Result<Vec<Tensor<CudaRuntime>>> {
    if weights.is_empty() {
        return Ok(Vec::new());
    }
    // a format the library does not implement anywhere in the batch: the trait's default loop (quant_matmul.rs:30-39)
    if weights.iter().any(|w| format_id(w.format()).is_none()) {
        return weights.iter().map(|w| quant_matmul(client, activation, w)).collect();
    }
    let mut shapes = Vec::with_capacity(weights.len());
    for w in weights {
        shapes.push(validate("quant_matmul", activation, w)?);
    }
    let (m, k) = (shapes[0].0, shapes[0].1);
    let act = activation.contiguous()?;
    let outs: Vec<Tensor<CudaRuntime>> = shapes.iter().map(|s| Tensor::<CudaRuntime>::empty(&s.3, DType::F32, activation.device())).collect();
    let formats: Vec<c_int> = weights.iter().map(|w| format_id(w.format()).unwrap()).collect();
    let w_ptrs: Vec<*const c_void> = weights.iter().map(|w| w.storage().ptr() as *const c_void).collect();
    let ns: Vec<usize> = shapes.iter().map(|s| s.2).collect();
    let out_ptrs: Vec<*mut c_void> = outs.iter().map(|t| t.ptr() as *mut c_void).collect();
    let ws_bytes = formats.iter().zip(&ns)
        .map(|(&f, &n)| unsafe { b200q_sys::b200q_workspace_bytes(b200q_sys::B200Q_OP_QUANT_MATMUL, f, m, k, n) })
        .max().unwrap_or(0);
    let ws = scratch(ws_bytes, activation);
    check(unsafe {
        b200q_sys::b200q_quant_matmul_batch(weights.len() as c_int, formats.as_ptr(), w_ptrs.as_ptr(), ns.as_ptr(), out_ptrs.as_ptr(),
                                            act.ptr() as *const c_void, b200q_sys::B200Q_F32, b200q_sys::B200Q_F32, m, k,
                                            ptr_or_null(&ws), ws_bytes, stream_of(client))
    })?;
    Ok(outs)
}

pub fn quant_swiglu(client: &CudaClient, activation: &Tensor<CudaRuntime>, gate: &QuantTensor<CudaRuntime>, up: &QuantTensor<CudaRuntime>) -> Result<Tensor<CudaRuntime>> {
    if gate.format() != up.format() || gate.shape() != up.shape() {
        return Err(Error::QuantError { reason: "quant_swiglu: gate and up weights must have the same format and shape".into() });
    }
    let (m, k, n, out_shape) = validate("quant_swiglu", activation, gate)?;
    let Some(fmt) = format_id(gate.format()) else {
        return boostr::quant::cuda::quant_matmul::quant_swiglu_ptx(client, activation, gate, up);
    };
    let act = activation.contiguous()?;
    let out = Tensor::<CudaRuntime>::empty(&out_shape, DType::F32, activation.device());
    let ws_bytes = unsafe { b200q_sys::b200q_workspace_bytes(b200q_sys::B200Q_OP_QUANT_SWIGLU, fmt, m, k, n) };
    let ws = scratch(ws_bytes, activation);
    check(unsafe {
        b200q_sys::b200q_quant_swiglu(fmt, act.ptr() as *const c_void, b200q_sys::B200Q_F32, gate.storage().ptr() as *const c_void,
                                      up.storage().ptr() as *const c_void, out.ptr() as *mut c_void, b200q_sys::B200Q_F32, m, k, n,
                                      ptr_or_null(&ws), ws_bytes, stream_of(client))
    })?;
    Ok(out)
}

/// The feed-forward block `down(silu(gate x) * (up x))` of `src/model/llama/model/blocks_mlp.rs:38-46` as one call
/// (the hidden state stays in the library's scratch).  Falls back to the two separate ops for formats libb200q does not serve.
pub fn quant_mlp(client: &CudaClient, activation: &Tensor<CudaRuntime>, gate: &QuantTensor<CudaRuntime>, up: &QuantTensor<CudaRuntime>,
                 down: &QuantTensor<CudaRuntime>) -> Result<Tensor<CudaRuntime>> {
    if gate.format() != up.format() || gate.shape() != up.shape() {
        return Err(Error::QuantError { reason: "quant_mlp: gate and up weights must have the same format and shape".into() });
    }
    let (m, k, n_ff, _) = validate("quant_mlp", activation, gate)?;
    let dshape = down.shape();
    if dshape.len() != 2 || dshape[1] != n_ff {
        return Err(Error::QuantError { reason: format!("quant_mlp: down weight {:?} does not take a hidden state of {}", dshape, n_ff) });
    }
    let (Some(fgu), Some(fd)) = (format_id(gate.format()), format_id(down.format())) else {
        let h = quant_swiglu(client, activation, gate, up)?;
        return quant_matmul(client, &h, down);
    };
    let n_out = dshape[0];
    let act = activation.contiguous()?;
    let mut out_shape = activation.shape().to_vec();
    *out_shape.last_mut().unwrap() = n_out;
    let out = Tensor::<CudaRuntime>::empty(&out_shape, DType::F32, activation.device());
    let ws_bytes = unsafe { b200q_sys::b200q_mlp_workspace_bytes(fgu, fd, m, k, n_ff, n_out) };
    let ws = scratch(ws_bytes, activation);
    check(unsafe {
        b200q_sys::b200q_quant_mlp(fgu, gate.storage().ptr() as *const c_void, up.storage().ptr() as *const c_void, fd,
                                   down.storage().ptr() as *const c_void, act.ptr() as *const c_void, b200q_sys::B200Q_F32,
                                   out.ptr() as *mut c_void, b200q_sys::B200Q_F32, m, k, n_ff, n_out, ptr_or_null(&ws), ws_bytes,
                                   stream_of(client))
    })?;
    Ok(out)
}

/// Decode-loop hint (`b200q_prefetch_next`): `weights` are those of the operation AFTER the next call made by this thread:
/// several weights sharing one activation row, or `[gate, up]` with `swiglu`.  The next call, when it is a single-row
/// product, pulls the head of those weights into L2 while it drains.  A hint only: results never depend on it, and a
/// weight of a format libb200q does not serve simply drops it.  The weights must outlive the call that consumes the hint.
pub fn prefetch_next(weights: &[&QuantTensor<CudaRuntime>], swiglu: bool) -> Result<()> {
    if weights.is_empty() {
        return Ok(());
    }
    let mut formats = Vec::with_capacity(weights.len());
    for w in weights {
        let Some(f) = format_id(w.format()) else { return Ok(()) };
        formats.push(f);
    }
    let ptrs: Vec<*const c_void> = weights.iter().map(|w| w.storage().ptr() as *const c_void).collect();
    let ns: Vec<usize> = weights.iter().map(|w| w.shape()[0]).collect();
    let k = *weights[0].shape().last().unwrap();
    let op = if swiglu { b200q_sys::B200Q_OP_QUANT_SWIGLU } else { b200q_sys::B200Q_OP_QUANT_MATMUL };
    check(unsafe { b200q_sys::b200q_prefetch_next(op, weights.len() as c_int, formats.as_ptr(), ptrs.as_ptr(), ns.as_ptr(), k) })
}

/// For a host that must not allocate at the call site (see `b200q_quant_matmul_static_scratch` in the header):
/// same result as `quant_matmul`, scratch inside the library, calls on one device must not overlap.
pub fn quant_matmul_no_alloc(client: &CudaClient, activation: &Tensor<CudaRuntime>, weight: &QuantTensor<CudaRuntime>,
                             out: &Tensor<CudaRuntime>) -> Result<()> {
    let (m, k, n, _) = validate("quant_matmul", activation, weight)?;
    let fmt = format_id(weight.format()).ok_or_else(|| Error::QuantError { reason: "format not served by libb200q".into() })?;
    check(unsafe {
        b200q_sys::b200q_quant_matmul_static_scratch(fmt, activation.ptr() as *const c_void, b200q_sys::B200Q_F32,
                                                     weight.storage().ptr() as *const c_void, out.ptr() as *mut c_void,
                                                     b200q_sys::B200Q_F32, m, k, n, stream_of(client))
    })
}
