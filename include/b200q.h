/*
 * b200q — C ABI of the B200 (sm_100a) quantized-linear library.
 *
 * This is the boundary a boostr maintainer binds from Rust (`extern "C"`) in place of
 * the PTX modules boostr's CUDA backend loads today.  Every entry point names the
 * boostr interface it stands in for (paths are relative to the boostr repository).
 *
 * Conventions (same as boostr's CUDA backend, src/quant/cuda/quant_matmul/impl_ops.rs:112-172):
 *   - all `const void* w / act`, `void* out / ws` arguments are DEVICE pointers
 *     (boostr passes `Tensor::ptr()` / `Storage::ptr()` as u64);
 *   - the caller allocates outputs and scratch; the library never allocates or frees;
 *   - work is enqueued on `stream` (a CUstream / cudaStream_t, may be NULL for the
 *     default stream) and the call returns without synchronising;
 *   - weights are packed blocks, row-major [N, K] with blocks along K and no row
 *     padding (src/quant/format.rs:5-20); `w` must be 16-byte aligned;
 *   - activations are contiguous row-major [M, K]; outputs are row-major [M, N];
 *   - every function returns a b200q_status; on failure `b200q_last_error()` gives the
 *     reason for the calling thread (the counterpart of Error::QuantError { reason },
 *     src/error.rs:22-27).  Nothing aborts, traps or throws.
 */
#ifndef B200Q_H
#define B200Q_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define B200Q_API
#else
#define B200Q_API __attribute__((visibility("default")))
#endif

typedef enum b200q_status {
    B200Q_OK = 0,
    B200Q_ERR_INVALID_ARG = 1,
    B200Q_ERR_UNSUPPORTED_FORMAT = 2,
    B200Q_ERR_BAD_SHAPE = 3,
    B200Q_ERR_WORKSPACE_TOO_SMALL = 4,
    B200Q_ERR_CUDA = 5,
    B200Q_ERR_TIMEOUT = 6,
    B200Q_ERR_UNSUPPORTED_DTYPE = 7,
    B200Q_ERR_NOT_FUSED = 8 /* b200q_row_parallel_matmul has no fused exchange for this shape */
} b200q_status;

/* Block formats; values are QuantFormat::format_id (src/quant/format.rs:204-230). */
typedef enum b200q_format {
    B200Q_Q4_0 = 0,
    B200Q_Q5_0 = 2, /* 22-byte blocks (src/quant/format.rs:114); all row counts through the small-M kernel and, from 64 rows, the tensor-core path */
    B200Q_Q8_0 = 4,
    B200Q_Q2_K = 6, /* dequantize at full speed; matmul through a generic integer-dot kernel (exact CPU numerics, not tuned) */
    B200Q_Q3_K = 7, /* as Q2_K */
    B200Q_Q4_K = 8,
    B200Q_Q5_K = 9, /* decode shapes run through the small-M kernel; no fused row-/column-parallel exchange */
    B200Q_Q6_K = 10
} b200q_format;

/* Element types of activations / outputs (numr DType subset). */
typedef enum b200q_dtype {
    B200Q_F32 = 0,
    B200Q_BF16 = 1,
    B200Q_F16 = 2,
    B200Q_F64 = 3 /* dequantize target only */
} b200q_dtype;

/* Operations that may need scratch memory; argument of b200q_workspace_bytes. */
typedef enum b200q_op {
    B200Q_OP_QUANT_MATMUL = 0,
    B200Q_OP_QUANT_SWIGLU = 1
} b200q_op;

/* Library version: major * 10000 + minor * 100 + patch. */
B200Q_API int b200q_version(void);

/* Message of the last failed call made by this thread ("" if none). */
B200Q_API const char* b200q_last_error(void);

/* QuantFormat::block_size / block_bytes (src/quant/format.rs:81-140); 0 for an unknown format. */
B200Q_API size_t b200q_block_size(int format);
B200Q_API size_t b200q_block_bytes(int format);

/* QuantFormat::storage_bytes (src/quant/format.rs:142-157): bytes of `numel` elements;
 * B200Q_ERR_BAD_SHAPE when numel is not a multiple of the block size. */
B200Q_API int b200q_storage_bytes(int format, size_t numel, size_t* out_bytes);

/*
 * DequantOps::dequantize (src/quant/traits/dequant.rs:15; CUDA impl
 * src/quant/cuda/dequant.rs:74-146, kernels src/quant/cuda/kernels/dequant.cu:18-206).
 * Decodes `nblocks` packed blocks at `w` into nblocks * block_size elements of
 * `out_dtype` at `out` (F32, BF16, F16 or F64).  16-bit targets are one
 * round-to-nearest-even rounding of the exact f32 value; there is no intermediate
 * f32 tensor and no second cast pass.
 */
B200Q_API int b200q_dequantize(int format, const void* w, size_t nblocks, void* out, int out_dtype, void* stream);

/*
 * Scratch bytes b200q_quant_matmul / b200q_quant_swiglu need for this shape with F32 activations:
 * 0 for the decode shapes (one activation row); the prepared activation image for 2 <= M < 64 (a few
 * hundred KB; the integer tensor-core kernels for Q4_K / Q8_0 add up to ~5 MB of f32 pieces of tiles cut
 * along K) and for the bf16 tensor-core path (2 bytes per activation), plus split-K partial sums when K
 * is long.  `ws` must be 16-byte aligned.  Scratch contents need no initialisation and carry nothing
 * between calls, but calls that may overlap on the GPU must not share one scratch buffer.
 * Returns 0 as well when the arguments are invalid; the op itself reports the error.
 */
B200Q_API size_t b200q_workspace_bytes(int op, int format, size_t M, size_t K, size_t N);

/*
 * QuantMatmulOps::quant_matmul (src/quant/traits/quant_matmul.rs:23; CUDA impl
 * src/quant/cuda/quant_matmul/impl_ops.rs:112-172, kernels
 * src/quant/cuda/kernels/quant_gemv.cu and quant_matmul.cu):
 *     out[M,N] = act[M,K] x dequant(w[N,K])^T
 * act_dtype: F32 (what boostr accepts) or BF16 (extension); out_dtype: F32 (what boostr
 * returns), BF16 or F16.  Requires M, K, N > 0 and K a multiple of the block size.
 * Q4_K / Q6_K follow boostr's CPU numerics: each 256-wide run of an activation row is
 * quantised to int8 with one f32 scale (Q8_K) and the dot products are integer
 * (src/quant/cpu/kernels/quant_matmul.rs:107-158); Q4_0 / Q8_0 keep the activation
 * precision (f32 there, :193-209).
 */
B200Q_API int b200q_quant_matmul(int format, const void* act, int act_dtype, const void* w, void* out, int out_dtype,
                                 size_t M, size_t K, size_t N, void* ws, size_t ws_bytes, void* stream);

/*
 * QuantMatmulOps::quant_matmul_batch (src/quant/traits/quant_matmul.rs:30-39; CUDA impl
 * src/quant/cuda/quant_matmul/impl_ops.rs:174-335): one activation against `n_weights`
 * weights that share K.  formats[i], w[i], N[i], out[i] describe weight i; out[i] is [M, N[i]].
 * `ws` must hold the largest b200q_workspace_bytes over the weights.
 */
B200Q_API int b200q_quant_matmul_batch(int n_weights, const int* formats, const void* const* w, const size_t* N,
                                       void* const* out, const void* act, int act_dtype, int out_dtype, size_t M,
                                       size_t K, void* ws, size_t ws_bytes, void* stream);

/*
 * RMSNorm fused in front of quant_matmul_batch: what a LLaMA attention block does with its input,
 * `input_layernorm` followed by the batched q/k/v projections (src/model/llama/model/blocks_attention.rs:95-99 after
 * RmsNorm::forward, src/nn/rmsnorm.rs:40):
 *     x' = act * (1 / sqrt(mean(act^2) + eps)) * norm_weight      (per row, f32)
 *     out[i] = x' x dequant(w[i])^T
 * With one activation row and Q4_K / Q6_K weights the decode kernels normalise the row while they quantise it (no extra
 * launch, no round trip of the normalised row through memory); other shapes run one stand-alone normalisation launch
 * into the front of `ws`, which must then hold M * K * 4 bytes (rounded up to 256) in addition to
 * b200q_workspace_bytes.  norm_weight: K f32 values on the device, 16-byte aligned.
 */
B200Q_API int b200q_rmsnorm_quant_matmul_batch(int n_weights, const int* formats, const void* const* w, const size_t* N,
                                               void* const* out, const void* act, const float* norm_weight, float eps,
                                               int act_dtype, int out_dtype, size_t M, size_t K, void* ws, size_t ws_bytes,
                                               void* stream);

/*
 * QuantMatmulOps::quant_swiglu (src/quant/traits/quant_matmul.rs:122-127; CUDA impl
 * src/quant/cuda/quant_matmul/impl_ops.rs:337-441):
 *     out[M,N] = silu(act x Wg^T) * (act x Wu^T),   silu(x) = x / (1 + exp(-x))
 * Wg and Wu share format, N and K.
 */
B200Q_API int b200q_quant_swiglu(int format, const void* act, int act_dtype, const void* w_gate, const void* w_up,
                                 void* out, int out_dtype, size_t M, size_t K, size_t N, void* ws, size_t ws_bytes,
                                 void* stream);

/*
 * The feed-forward block of a quantized layer, down(silu(gate x) * (up x))
 * (src/model/llama/model/blocks_mlp.rs:38-46: `quant_swiglu` followed by the down projection's
 * `forward`), as ONE call: activation [M, K] -> hidden [M, n_ff] (f32, kept in `ws`) -> out [M, n_out].
 * The gate and up weights are [n_ff, K] of `format_gate_up`, the down weight [n_out, n_ff] of
 * `format_down` (a Q4_K_M file mixes them: Q4_K gate/up, Q6_K or Q4_K down).  The two products run
 * back to back under programmatic dependent launch (the second streams its weights while the first
 * drains); the hidden state never goes back to the caller.  Results are those of b200q_quant_swiglu
 * followed by b200q_quant_matmul, bit for bit.  b200q_mlp_workspace_bytes gives the scratch for F32
 * activations: the hidden state plus what the two products need.
 */
B200Q_API size_t b200q_mlp_workspace_bytes(int format_gate_up, int format_down, size_t M, size_t K, size_t n_ff, size_t n_out);
B200Q_API int b200q_quant_mlp(int format_gate_up, const void* w_gate, const void* w_up, int format_down, const void* w_down,
                              const void* act, int act_dtype, void* out, int out_dtype, size_t M, size_t K, size_t n_ff,
                              size_t n_out, void* ws, size_t ws_bytes, void* stream);

/*
 * Optional hint for a decode loop (single activation row), where every launch is short and the time
 * between the last byte of one weight and the first byte of the next is a visible share of the step.
 * (No counterpart in boostr, whose decode step launches its kernels back to back,
 * src/model/llama/model/forward_graph.rs:22-73; results never depend on the hint.)
 *
 * The call describes the operation that will FOLLOW the next call this thread makes:
 * B200Q_OP_QUANT_MATMUL with `n_weights` weights [N[i], K] that share one activation row (as in
 * b200q_quant_matmul / b200q_quant_matmul_batch), or B200Q_OP_QUANT_SWIGLU with w[0] = gate and
 * w[1] = up, both [N[0], K].  The next call, when it is a single-row product of a format with a
 * streaming decode kernel (Q4_K, Q6_K), then spends its last microseconds pulling the first ~100 KB
 * that each SM of the following launch will read into L2, so that launch starts from L2 instead of
 * from idle HBM.  The hint lives for exactly one call (any b200q compute call consumes or drops it)
 * and is dropped at once when the described operation has no such kernel, or when the consuming
 * call runs on another device than the one current at the time of the hint.  The weight pointers
 * must stay valid device memory until the call that consumed the hint has finished on its stream;
 * under stream capture the hint is baked into the captured launch, so the same holds for every replay.
 * b200q_quant_mlp places the hint for its own down-projection itself.
 */
B200Q_API int b200q_prefetch_next(int op, int n_weights, const int* formats, const void* const* w, const size_t* N, size_t K);

/*
 * quant_matmul for callers that cannot hand over scratch memory.  (No counterpart in boostr:
 * its CUDA backend always has numr's allocator at hand.)
 *
 * Some hosts reach this library with nothing but the pointers of their inputs and outputs:
 * an FFI caller whose tensor runtime has reserved all device memory for its own pool, or a
 * code path where a cudaMalloc — which can synchronise the whole device — is not acceptable.
 * For them everything b200q_quant_matmul keeps in `ws` — split-K partial sums, and the prepared
 * activation image (Q8_K codes / bf16) that the small-M and tensor-core kernels read — lives in a
 * fixed B200Q_STATIC_SCRATCH_BYTES array inside the library's device image instead (every GPU
 * that loads the library holds that array until the process exits).  The call allocates nothing:
 * no cudaMalloc, no cudaFree, no allocating library routine.
 *
 *   - Same arguments, results and errors as b200q_quant_matmul, minus ws / ws_bytes.  A shape
 *     whose scratch need (for its activation type) exceeds B200Q_STATIC_SCRATCH_BYTES is refused
 *     with B200Q_ERR_WORKSPACE_TOO_SMALL and a message naming both sizes.
 *   - The first call on a device resolves the array's device address (once per device, with
 *     that device current; a failed look-up is tried again by the next call).  Make that first
 *     call before starting any stream capture.  The address belongs to the device's primary context.
 *   - All calls on a device share the one array and it keeps the previous call's contents.
 *     Nothing in it has to start at zero: every byte a kernel reads is written earlier in the same call.
 *     Two calls that may run on the GPU at the same time (different streams) race on it;
 *     keep such calls on one stream or order them yourself.
 */
#define B200Q_STATIC_SCRATCH_BYTES (8u << 20)
B200Q_API int b200q_quant_matmul_static_scratch(int format, const void* act, int act_dtype, const void* w, void* out,
                                                int out_dtype, size_t M, size_t K, size_t N, void* stream);

/*
 * Tensor-parallel shard extraction, HOST memory to HOST memory.  boostr shards dense
 * weights with scatter_to_rank (src/distributed/tensor_parallel.rs:258-300) and has no
 * quantised counterpart; this cuts rank `rank` of `world` out of a packed [N,K] weight:
 *   dim 0 (column-parallel): rows [rank*N/world, (rank+1)*N/world) — a contiguous byte range;
 *   dim 1 (row-parallel):   columns [rank*K/world, ...) of every row, repacked tightly;
 *                           K/world must be a multiple of the block size.
 * `dst` receives (N/world)*K or N*(K/world) elements' worth of blocks.
 */
B200Q_API int b200q_shard_pack(int format, const void* src, size_t N, size_t K, int dim, int rank, int world,
                               void* dst, size_t dst_bytes);

/*
 * Waits for `stream` and reports whether any kernel of this library gave up on a
 * bounded wait since the last call (B200Q_ERR_TIMEOUT) — the library never spins
 * without a limit.  Diagnostic; not needed in normal operation.
 */
B200Q_API int b200q_check_device_status(void* stream);

/*
 * Number of kernel launches this library has issued in the calling process (all threads,
 * all devices).  Launches recorded while a stream is being captured count once, at capture.
 * Diagnostic: lets a harness state how many of this library's kernels ran in a timed region.
 */
B200Q_API unsigned long long b200q_launch_count(void);

/*
 * Tensor-parallel exchange over peer memory (one process per GPU, GPUs of one NVLink domain).
 *
 * Replaces, for decode (M = 1), the pair "local quant_matmul, then Communicator::all_reduce(Sum) and
 * sync" of RowParallelLinear::forward (src/distributed/tensor_parallel.rs:230-238, all_reduce_tensor in
 * src/distributed/comm_utils.rs:15-39) by ONE kernel: it pushes every element of the local partial row
 * into every rank's exchange buffer as one 8-byte store {value, epoch} over NVLink, and each CTA then
 * collects the partial values of its own rows from all ranks (waiting at most 1 s for an element whose
 * epoch has not arrived, then B200Q_ERR_TIMEOUT is reported by b200q_check_device_status) and adds them
 * in rank order, so all ranks store bit-identical sums.
 *
 * Set-up, once per process: b200q_tp_alloc creates this rank's exchange buffer (cudaMalloc, zeroed) and
 * its 64-byte CUDA IPC handle; the handles are exchanged by whatever the host uses (boostr: its
 * Communicator's broadcast/all_gather of bytes); b200q_tp_open maps a peer's buffer.  `bufs[r]` is rank
 * r's buffer as seen from this process (own buffer at bufs[rank]).  All ranks must issue the same
 * sequence of b200q_row_parallel_matmul calls.  The buffers carry the exchange state (the epoch), so
 * one set of buffers serves one stream of calls.
 *
 * Shapes without a fused path (M > 1, formats other than Q4_K/Q6_K, N > 65536, non-f32 output) return
 * B200Q_ERR_NOT_FUSED without launching anything: run b200q_quant_matmul and the communicator's
 * all_reduce instead.
 */
#define B200Q_TP_HANDLE_BYTES 64
B200Q_API size_t b200q_tp_buffer_bytes(void);
B200Q_API int b200q_tp_alloc(void** buf, unsigned char* handle /* B200Q_TP_HANDLE_BYTES */);
B200Q_API int b200q_tp_open(const unsigned char* handle, void** peer_buf);
B200Q_API int b200q_tp_close(void* peer_buf);
B200Q_API int b200q_tp_free(void* buf);
B200Q_API int b200q_row_parallel_matmul(int format, const void* act, int act_dtype, const void* w, void* out, int out_dtype,
                                        size_t M, size_t K, size_t N, int rank, int world, void* const* bufs, void* stream);

/*
 * Column-parallel counterpart: the local product of a row shard [n_local, K] fused with the all-gather of
 * the logits (gather_from_ranks, src/distributed/tensor_parallel.rs:302-355, used after a column-parallel
 * lm_head).  Every element of the local result is pushed, tagged, into column rank * n_local + i of every
 * rank's exchange buffer; each rank then copies the assembled row [world * n_local] into `out_full`
 * (row-major, shard r in columns [r * n_local, (r + 1) * n_local): the layout the reference's flat gather
 * only gives for one row).  Same set-up, ordering rules and bounded waits as b200q_row_parallel_matmul;
 * the two may alternate on one set of buffers.  M = 1, Q4_K / Q6_K, world * n_local <= 524288, f32 output;
 * anything else returns B200Q_ERR_NOT_FUSED without launching.
 */
B200Q_API int b200q_col_parallel_matmul_gather(int format, const void* act, int act_dtype, const void* w, void* out_full,
                                               size_t M, size_t K, size_t n_local, int rank, int world, void* const* bufs,
                                               void* stream);

/*
 * All-reduce (sum) of `count` f32 values in place over the same exchange buffers: the small-message stand-in for
 * all_reduce_tensor + sync (src/distributed/comm_utils.rs:15-39) behind a row-parallel product that has no exchange
 * inside its kernel (2 <= M rows, Q4_0 / Q8_0).  One kernel: tagged 8-byte stores to every rank, then each rank adds
 * the ranks' values in rank order (bit-identical on all ranks), every wait bounded as above.  Same ordering rules;
 * may alternate with the two calls above on one set of buffers.  count <= 65536, else B200Q_ERR_NOT_FUSED (nothing
 * launched: use the communicator).
 */
B200Q_API int b200q_tp_all_reduce(void* data, size_t count, int rank, int world, void* const* bufs, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H */
