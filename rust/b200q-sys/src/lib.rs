//! Raw bindings of `libb200q.so` — one declaration per entry point of `include/b200q.h`, in the header's order.
//!
//! NOT COMPILED in the environment this file was written in (it has no Rust toolchain); the same entry
//! points are exercised through Python `ctypes` by the repository's parity tests, and
//! `tests/test_cabi_host.py` checks that this block names every symbol the header declares.
//!
//! Conventions (see the header): every `*const c_void` / `*mut c_void` named `w`, `act`, `out`, `ws` is a
//! DEVICE pointer (`Tensor::ptr()` / `Storage::ptr()` as `u64` in boostr); `stream` is a `CUstream`; calls
//! enqueue and return; the library allocates nothing.  Every function returns a `b200q_status`.
#![allow(non_camel_case_types)]

use std::os::raw::{c_char, c_int, c_ulonglong, c_void};

pub const B200Q_OK: c_int = 0;
pub const B200Q_ERR_INVALID_ARG: c_int = 1;
pub const B200Q_ERR_UNSUPPORTED_FORMAT: c_int = 2;
pub const B200Q_ERR_BAD_SHAPE: c_int = 3;
pub const B200Q_ERR_WORKSPACE_TOO_SMALL: c_int = 4;
pub const B200Q_ERR_CUDA: c_int = 5;
pub const B200Q_ERR_TIMEOUT: c_int = 6;
pub const B200Q_ERR_UNSUPPORTED_DTYPE: c_int = 7;
pub const B200Q_ERR_NOT_FUSED: c_int = 8;

/// `QuantFormat::format_id()` of the formats the library implements.
pub const B200Q_Q4_0: c_int = 0;
pub const B200Q_Q8_0: c_int = 4;
pub const B200Q_Q4_K: c_int = 8;
pub const B200Q_Q6_K: c_int = 10;

pub const B200Q_F32: c_int = 0;
pub const B200Q_BF16: c_int = 1;
pub const B200Q_F16: c_int = 2;
pub const B200Q_F64: c_int = 3;

pub const B200Q_OP_QUANT_MATMUL: c_int = 0;
pub const B200Q_OP_QUANT_SWIGLU: c_int = 1;

pub const B200Q_STATIC_SCRATCH_BYTES: usize = 8 << 20;
pub const B200Q_TP_HANDLE_BYTES: usize = 64;

#[link(name = "b200q")]
extern "C" {
    pub fn b200q_version() -> c_int;
    pub fn b200q_last_error() -> *const c_char;
    pub fn b200q_block_size(format: c_int) -> usize;
    pub fn b200q_block_bytes(format: c_int) -> usize;
    pub fn b200q_storage_bytes(format: c_int, numel: usize, out_bytes: *mut usize) -> c_int;
    pub fn b200q_dequantize(format: c_int, w: *const c_void, nblocks: usize, out: *mut c_void, out_dtype: c_int,
                            stream: *mut c_void) -> c_int;
    pub fn b200q_workspace_bytes(op: c_int, format: c_int, m: usize, k: usize, n: usize) -> usize;
    pub fn b200q_quant_matmul(format: c_int, act: *const c_void, act_dtype: c_int, w: *const c_void, out: *mut c_void,
                              out_dtype: c_int, m: usize, k: usize, n: usize, ws: *mut c_void, ws_bytes: usize,
                              stream: *mut c_void) -> c_int;
    pub fn b200q_quant_matmul_batch(n_weights: c_int, formats: *const c_int, w: *const *const c_void, n: *const usize,
                                    out: *const *mut c_void, act: *const c_void, act_dtype: c_int, out_dtype: c_int,
                                    m: usize, k: usize, ws: *mut c_void, ws_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn b200q_rmsnorm_quant_matmul_batch(n_weights: c_int, formats: *const c_int, w: *const *const c_void, n: *const usize,
                                            out: *const *mut c_void, act: *const c_void, norm_weight: *const f32, eps: f32,
                                            act_dtype: c_int, out_dtype: c_int, m: usize, k: usize, ws: *mut c_void,
                                            ws_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn b200q_quant_swiglu(format: c_int, act: *const c_void, act_dtype: c_int, w_gate: *const c_void,
                              w_up: *const c_void, out: *mut c_void, out_dtype: c_int, m: usize, k: usize, n: usize,
                              ws: *mut c_void, ws_bytes: usize, stream: *mut c_void) -> c_int;
    pub fn b200q_mlp_workspace_bytes(format_gate_up: c_int, format_down: c_int, m: usize, k: usize, n_ff: usize,
                                     n_out: usize) -> usize;
    pub fn b200q_quant_mlp(format_gate_up: c_int, w_gate: *const c_void, w_up: *const c_void, format_down: c_int,
                           w_down: *const c_void, act: *const c_void, act_dtype: c_int, out: *mut c_void, out_dtype: c_int,
                           m: usize, k: usize, n_ff: usize, n_out: usize, ws: *mut c_void, ws_bytes: usize,
                           stream: *mut c_void) -> c_int;
    /// Decode-loop hint: describes the operation AFTER the next call (its weights' head goes to L2 while that call drains).
    pub fn b200q_prefetch_next(op: c_int, n_weights: c_int, formats: *const c_int, w: *const *const c_void, n: *const usize,
                               k: usize) -> c_int;
    pub fn b200q_quant_matmul_static_scratch(format: c_int, act: *const c_void, act_dtype: c_int, w: *const c_void,
                                             out: *mut c_void, out_dtype: c_int, m: usize, k: usize, n: usize,
                                             stream: *mut c_void) -> c_int;
    /// HOST memory to HOST memory.
    pub fn b200q_shard_pack(format: c_int, src: *const c_void, n: usize, k: usize, dim: c_int, rank: c_int, world: c_int,
                            dst: *mut c_void, dst_bytes: usize) -> c_int;
    pub fn b200q_check_device_status(stream: *mut c_void) -> c_int;
    pub fn b200q_launch_count() -> c_ulonglong;
    pub fn b200q_tp_buffer_bytes() -> usize;
    pub fn b200q_tp_alloc(buf: *mut *mut c_void, handle: *mut u8 /* B200Q_TP_HANDLE_BYTES */) -> c_int;
    pub fn b200q_tp_open(handle: *const u8, peer_buf: *mut *mut c_void) -> c_int;
    pub fn b200q_tp_close(peer_buf: *mut c_void) -> c_int;
    pub fn b200q_tp_free(buf: *mut c_void) -> c_int;
    pub fn b200q_row_parallel_matmul(format: c_int, act: *const c_void, act_dtype: c_int, w: *const c_void,
                                     out: *mut c_void, out_dtype: c_int, m: usize, k: usize, n: usize, rank: c_int,
                                     world: c_int, bufs: *const *mut c_void, stream: *mut c_void) -> c_int;
    pub fn b200q_col_parallel_matmul_gather(format: c_int, act: *const c_void, act_dtype: c_int, w: *const c_void,
                                            out_full: *mut c_void, m: usize, k: usize, n_local: usize, rank: c_int,
                                            world: c_int, bufs: *const *mut c_void, stream: *mut c_void) -> c_int;
    pub fn b200q_tp_all_reduce(data: *mut c_void, count: usize, rank: c_int, world: c_int, bufs: *const *mut c_void,
                               stream: *mut c_void) -> c_int;
}
