//! `DequantOps::dequantize` for `CudaClient` (replaces `src/quant/cuda/dequant.rs:74-146` for the four formats):
//! one launch that writes the target dtype directly — no f32 intermediate, no `cast` pass.
use std::os::raw::c_void;

use boostr::error::{Error, Result};
use boostr::quant::QuantTensor;
use numr::dtype::DType;
use numr::runtime::cuda::{CudaClient, CudaRuntime};
use numr::tensor::Tensor;

use crate::{check, dtype_id, format_id, stream_of};

pub fn dequantize(client: &CudaClient, qt: &QuantTensor<CudaRuntime>, target_dtype: DType) -> Result<Tensor<CudaRuntime>> {
    let dt = match target_dtype {
        DType::F32 | DType::F16 | DType::BF16 | DType::F64 => dtype_id(target_dtype).unwrap(),
        _ => {
            return Err(Error::QuantError { reason: format!("dequantize target must be float, got {:?}", target_dtype) });
        }
    };
    let Some(fmt) = format_id(qt.format()) else {
        // other formats: boostr's existing kernels (dequant_generic.cu)
        return boostr::quant::cuda::dequant::dequantize_ptx(client, qt, target_dtype);
    };
    let out = Tensor::<CudaRuntime>::empty(qt.shape(), target_dtype, qt.device());
    check(unsafe {
        b200q_sys::b200q_dequantize(fmt, qt.storage().ptr() as *const c_void, qt.num_blocks(), out.ptr() as *mut c_void, dt,
                                    stream_of(client))
    })?;
    Ok(out)
}
