//! boostr's quantized-linear traits for `CudaClient`, served by `libb200q.so`.
//!
//! NOT COMPILED in the environment this was written in (no Rust toolchain; numr is not vendored).
//! The modules are written to be moved into boostr (`src/quant/cuda/`, `src/distributed/`) as they are.
pub mod dequant;
pub mod quant_matmul;
pub mod tensor_parallel;

use std::os::raw::{c_int, c_void};

use boostr::error::{Error, Result};
use boostr::quant::QuantFormat;
use numr::dtype::DType;
use numr::runtime::cuda::{CudaClient, CudaRuntime};
use numr::tensor::Tensor;

/// Status code -> `Error::QuantError { reason }` with the library's message for this thread.
pub(crate) fn check(rc: c_int) -> Result<()> {
    if rc == b200q_sys::B200Q_OK {
        return Ok(());
    }
    let reason = unsafe { std::ffi::CStr::from_ptr(b200q_sys::b200q_last_error()) }.to_string_lossy().into_owned();
    Err(Error::QuantError { reason })
}

/// The four formats the library implements; everything else stays on boostr's own kernels.
pub(crate) fn format_id(format: QuantFormat) -> Option<c_int> {
    match format {
        QuantFormat::Q4_0 | QuantFormat::Q8_0 | QuantFormat::Q4K | QuantFormat::Q6K => Some(format.format_id() as c_int),
        _ => None,
    }
}

pub(crate) fn dtype_id(dtype: DType) -> Option<c_int> {
    match dtype {
        DType::F32 => Some(b200q_sys::B200Q_F32),
        DType::BF16 => Some(b200q_sys::B200Q_BF16),
        DType::F16 => Some(b200q_sys::B200Q_F16),
        DType::F64 => Some(b200q_sys::B200Q_F64),
        _ => None,
    }
}

pub(crate) fn stream_of(client: &CudaClient) -> *mut c_void {
    client.stream().cu_stream() as *mut c_void
}

/// Scratch for one call: a U8 tensor from numr's stream-ordered allocator, dropped after the launch like the
/// Q8_1 activation buffer of boostr's own path (`src/quant/cuda/quant_matmul/helpers.rs:44`).
pub(crate) fn scratch(bytes: usize, like: &Tensor<CudaRuntime>) -> Option<Tensor<CudaRuntime>> {
    (bytes > 0).then(|| Tensor::<CudaRuntime>::empty(&[bytes], DType::U8, like.device()))
}

pub(crate) fn ptr_or_null(t: &Option<Tensor<CudaRuntime>>) -> *mut c_void {
    t.as_ref().map_or(std::ptr::null_mut(), |t| t.ptr() as *mut c_void)
}
