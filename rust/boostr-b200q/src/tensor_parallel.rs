//! Quantized counterparts of `ColumnParallelLinear` / `RowParallelLinear`
//! (`src/distributed/tensor_parallel.rs:27-253`, which hold dense `Var` weights; `QuantTensor` cannot be sliced,
//! so the shard is cut from the packed bytes on the host with `b200q_shard_pack`) and the hand-shake of the
//! fused peer exchange over boostr's `Communicator`.
use std::os::raw::{c_int, c_void};
use std::sync::Arc;

use boostr::distributed::comm_utils::all_reduce_tensor;
use boostr::error::{Error, Result};
use boostr::quant::{QuantFormat, QuantTensor};
use numr::dtype::DType;
use numr::ops::BinaryOps;
use numr::runtime::cuda::{CudaClient, CudaRuntime};
use numr::runtime::{Communicator, ReduceOp};
use numr::tensor::Tensor;

use crate::quant_matmul::quant_matmul;
use crate::{check, format_id, stream_of};

/// Rank `rank`'s shard of a packed `[n, k]` weight held in HOST memory: dim 0 = rows `[rank*n/world, ..)`
/// (column-parallel), dim 1 = columns `[rank*k/world, ..)` of every row (row-parallel; `k/world` must be whole blocks).
pub fn shard_packed(format: QuantFormat, packed: &[u8], n: usize, k: usize, dim: usize, rank: usize, world: usize) -> Result<Vec<u8>> {
    let fmt = format_id(format).ok_or_else(|| Error::QuantError { reason: format!("{:?} is not served by libb200q", format) })?;
    let numel = if dim == 0 { n / world.max(1) * k } else { n * (k / world.max(1)) };
    let mut bytes = 0usize;
    check(unsafe { b200q_sys::b200q_storage_bytes(fmt, numel, &mut bytes) })?;
    let mut dst = vec![0u8; bytes];
    check(unsafe {
        b200q_sys::b200q_shard_pack(fmt, packed.as_ptr() as *const c_void, n, k, dim as c_int, rank as c_int, world as c_int,
                                    dst.as_mut_ptr() as *mut c_void, dst.len())
    }).map_err(|e| match e {
        Error::QuantError { reason } => Error::DistributedError { reason },
        other => other,
    })?;
    Ok(dst)
}

/// Peer-mapped exchange buffers of one tensor-parallel group (`b200q_tp_*`).  One per stream of fused calls.
pub struct PeerExchange {
    own: *mut c_void,
    table: Vec<*mut c_void>,  // table[r] = rank r's buffer as seen from this process
    rank: usize,
}
unsafe impl Send for PeerExchange {}

impl PeerExchange {
    /// Every rank allocates its buffer, the 64-byte CUDA IPC handles travel through `Communicator::all_gather`
    /// (as U8), and each rank maps its peers.  Ends with a `sync` so nobody pushes before every mapping exists.
    pub fn new(comm: &dyn Communicator, device: &numr::runtime::cuda::CudaDevice) -> Result<Self> {
        let (rank, world) = (comm.rank(), comm.world_size());
        let mut own: *mut c_void = std::ptr::null_mut();
        let mut handle = [0u8; b200q_sys::B200Q_TP_HANDLE_BYTES];
        check(unsafe { b200q_sys::b200q_tp_alloc(&mut own, handle.as_mut_ptr()) })?;
        let send = Tensor::<CudaRuntime>::from_slice(&handle, &[handle.len()], device);
        let recv = Tensor::<CudaRuntime>::empty(&[world * handle.len()], DType::U8, device);
        unsafe { comm.all_gather(send.ptr(), recv.ptr(), handle.len(), DType::U8) }
            .map_err(|e| Error::DistributedError { reason: format!("all_gather of exchange handles failed: {e}") })?;
        comm.sync().map_err(|e| Error::DistributedError { reason: format!("sync failed: {e}") })?;
        let all: Vec<u8> = recv.to_vec();
        let mut table = vec![std::ptr::null_mut(); world];
        for r in 0..world {
            if r == rank {
                table[r] = own;
            } else {
                check(unsafe { b200q_sys::b200q_tp_open(all[r * handle.len()..].as_ptr(), &mut table[r]) })?;
            }
        }
        comm.barrier().map_err(|e| Error::DistributedError { reason: format!("barrier failed: {e}") })?;
        Ok(Self { own, table, rank })
    }
}

impl Drop for PeerExchange {
    fn drop(&mut self) {
        // the owner of the group synchronises the stream and barriers before dropping (a buffer is freed
        // only when no peer maps it any more)
        for (r, p) in self.table.iter().enumerate() {
            if r != self.rank && !p.is_null() {
                unsafe { b200q_sys::b200q_tp_close(*p) };
            }
        }
        unsafe { b200q_sys::b200q_tp_free(self.own) };
    }
}

/// Output features split across ranks; forward needs no communication (tensor_parallel.rs:112-123).
pub struct ColumnParallelQuantLinear {
    weight: QuantTensor<CudaRuntime>,
    bias: Option<Tensor<CudaRuntime>>,
}

impl ColumnParallelQuantLinear {
    pub fn from_shard(weight: QuantTensor<CudaRuntime>, bias: Option<Tensor<CudaRuntime>>) -> Self {
        Self { weight, bias }
    }
    pub fn forward(&self, client: &CudaClient, input: &Tensor<CudaRuntime>) -> Result<Tensor<CudaRuntime>> {
        let y = quant_matmul(client, input, &self.weight)?;
        match &self.bias {
            Some(b) => client.add(&y, b).map_err(Error::Numr),
            None => Ok(y),
        }
    }
}

/// Input features split across ranks; forward = local product, all-reduce SUM, then bias (tensor_parallel.rs:222-244).
pub struct RowParallelQuantLinear {
    weight: QuantTensor<CudaRuntime>,
    bias: Option<Tensor<CudaRuntime>>,
    comm: Arc<dyn Communicator>,
    exchange: Option<Arc<PeerExchange>>,
}

impl RowParallelQuantLinear {
    pub fn from_shard(weight: QuantTensor<CudaRuntime>, bias: Option<Tensor<CudaRuntime>>, comm: Arc<dyn Communicator>,
                      exchange: Option<Arc<PeerExchange>>) -> Self {
        Self { weight, bias, comm, exchange }
    }

    pub fn forward(&self, client: &CudaClient, input_shard: &Tensor<CudaRuntime>) -> Result<Tensor<CudaRuntime>> {
        let world = self.comm.world_size();
        let mut fused: Option<Tensor<CudaRuntime>> = None;
        if let (Some(ex), Some(fmt)) = (&self.exchange, format_id(self.weight.format())) {
            if world > 1 && input_shard.dtype() == DType::F32 {
                let (n, k) = (self.weight.shape()[0], self.weight.shape()[1]);
                let m = input_shard.numel() / k;
                let act = input_shard.contiguous()?;
                let mut shape = input_shard.shape()[..input_shard.shape().len() - 1].to_vec();
                shape.push(n);
                let out = Tensor::<CudaRuntime>::empty(&shape, DType::F32, input_shard.device());
                let rc = unsafe {
                    b200q_sys::b200q_row_parallel_matmul(fmt, act.ptr() as *const c_void, b200q_sys::B200Q_F32,
                                                         self.weight.storage().ptr() as *const c_void, out.ptr() as *mut c_void,
                                                         b200q_sys::B200Q_F32, m, k, n, ex.rank as c_int, world as c_int,
                                                         ex.table.as_ptr(), stream_of(client))
                };
                // NOT_FUSED: nothing was launched; take the pair of calls below
                if rc != b200q_sys::B200Q_ERR_NOT_FUSED {
                    check(rc)?;
                    fused = Some(out);
                }
            }
        }
        let y = match fused {
            Some(y) => y,
            None => {
                let y = quant_matmul(client, input_shard, &self.weight)?;
                if world > 1 {
                    all_reduce_tensor(self.comm.as_ref(), &y, ReduceOp::Sum)?;
                    self.comm.sync().map_err(|e| Error::DistributedError { reason: format!("sync after all_reduce failed: {e}") })?;
                }
                y
            }
        };
        match &self.bias {
            Some(b) => client.add(&y, b).map_err(Error::Numr),
            None => Ok(y),
        }
    }
}
