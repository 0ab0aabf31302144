// C ABI of the library (declared in include/b200q.h): argument validation with the same rules
// as boostr's QuantTensor::from_bytes / quant_matmul checks, kernel-family dispatch, and a
// thread-local error string in place of Error::QuantError { reason }.
#include <cstdarg>
#include <cstdio>
#include <atomic>
#include <cstring>
#include <mutex>

#include "../../include/b200q.h"
#include "common.cuh"
#include "tmap.cuh"

namespace b200q {
cudaError_t launch_dequant(int fmt, const void* w, size_t nblocks, void* out, int out_dtype, cudaStream_t st, int sm_count,
                           unsigned int* status);
cudaError_t launch_gemv(int fmt, const void* act, int act_dtype, const void* w0, const void* w1, void* out, int out_dtype,
                        size_t M, size_t K, size_t N, void* ws, size_t ws_bytes, bool swiglu, int sm_count, cudaStream_t st,
                        unsigned int* status, bool* ws_too_small, bool image_ready = false);
size_t gemv_workspace_bytes(int fmt, size_t M, size_t K, size_t N, bool swiglu, int sm_count);
bool gemv_m1_supported(int fmt, size_t M, size_t K, size_t N, bool swiglu);
bool m1_next_set(bool swiglu, int n_weights, const int* formats, const void* const* w, const size_t* N, size_t K, int sm_count);
void m1_next_clear();
void m1_next_stash();
void m1_next_unstash();
cudaError_t launch_gemv_m1(int fmt, const void* act, int act_dtype, const void* w, const void* w_up, void* out,
                           int out_dtype, size_t K, size_t N, int sm_count, cudaStream_t st, unsigned int* status,
                           const float* norm_w = nullptr, float norm_eps = 0.f);
cudaError_t launch_gemv_m1_mixed(const void* act, int act_dtype, int nseg, const void* const* w, const size_t* n,
                                 void* const* out, const void* w6, size_t n6, void* out6, int out_dtype, size_t K, int sm_count,
                                 cudaStream_t st, unsigned int* status, const float* norm_w = nullptr, float norm_eps = 0.f);
cudaError_t launch_gemv_m1_batch(const void* act, int act_dtype, int nseg, const void* const* w, const size_t* n,
                                 void* const* out, const void* w_up, int out_dtype, size_t K, int sm_count, cudaStream_t st,
                                 unsigned int* status, const float* norm_w = nullptr, float norm_eps = 0.f);
cudaError_t launch_rmsnorm(const void* act, int act_dtype, const float* norm_w, float eps, float* out, size_t M, size_t K, cudaStream_t st);
cudaError_t launch_tp_all_reduce(float* data, size_t count, const PeerComm& comm, int sm_count, cudaStream_t st, unsigned int* status);
cudaError_t launch_gemv_m1_rowpar(int fmt, const void* act, int act_dtype, const void* w, void* out, size_t K, size_t N,
                                  int sm_count, cudaStream_t st, unsigned int* status, const PeerComm& comm);
bool gemv_m1_f32_supported(int fmt, size_t M, size_t K, size_t N);
cudaError_t launch_gemv_m1_f32(int fmt, const void* act, int act_dtype, const void* w, void* out, int out_dtype, size_t K,
                               size_t N, int sm_count, cudaStream_t st, unsigned int* status);
bool prefill_supported(int fmt, size_t M, size_t K, size_t N);
size_t prefill_workspace_bytes(int fmt, int act_dtype, size_t M, size_t K, size_t N, int sm_count);
cudaError_t launch_prefill(int fmt, const void* act, int act_dtype, const void* w, void* out, int out_dtype, size_t M,
                           size_t K, size_t N, void* ws, size_t ws_bytes, int sm_count, cudaStream_t st,
                           unsigned int* status, bool* ws_too_small, char* err, size_t err_len, bool acts_prepared);
bool kq_generic_supported(int fmt, size_t M, size_t K, size_t N);
size_t kq_generic_workspace_bytes(size_t M, size_t K);
cudaError_t launch_kq_generic(int fmt, const void* act, int act_dtype, const void* w, void* out, int out_dtype, size_t M, size_t K,
                              size_t N, void* ws, size_t ws_bytes, int sm_count, cudaStream_t st, bool* ws_too_small);
cudaError_t launch_swiglu_gate(const float* gate, const float* up, void* out, int out_dtype, size_t n, int sm_count,
                               cudaStream_t st);
bool smallm_i8_supported(int fmt, size_t M, size_t K, size_t N);
bool smallm_i8_preferred(int fmt, size_t M, size_t K, size_t N, int sm_count);
size_t smallm_i8_workspace_bytes(int fmt, size_t M, size_t K, size_t N, int sm_count);
cudaError_t launch_smallm_i8(int fmt, const void* act, int act_dtype, const void* w, void* out, int out_dtype, size_t M, size_t K,
                             size_t N, void* ws, size_t ws_bytes, int sm_count, cudaStream_t st, unsigned int* status,
                             bool* ws_too_small, char* err, size_t err_len, bool acts_prepared);
}  // namespace b200q

using namespace b200q;

namespace {
std::atomic<unsigned long long> g_launches{0};
}
namespace b200q {
void note_launch(unsigned n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}
}  // namespace b200q

// One status word per device image of this library; kernels receive its address.
__device__ unsigned int g_status_word = 0;

namespace {

// Device address of g_status_word on the current device.  (The symbol's name in host code is only a
// handle; kernels need the address.)  Only a successful lookup is cached, so a failure (for instance a
// first call made while a stream is being captured) is retried by the next call.  The address belongs
// to the device's primary context.
unsigned int* status_ptr_current() {
    static std::atomic<unsigned int*> cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    unsigned int* p = cached[dev].load(std::memory_order_acquire);
    if (p) return p;
    void* q = nullptr;
    if (cudaGetSymbolAddress(&q, g_status_word) != cudaSuccess || !q) {
        cudaGetLastError();  // the failed lookup must not poison the next launch check
        return nullptr;
    }
    cached[dev].store(static_cast<unsigned int*>(q), std::memory_order_release);
    return static_cast<unsigned int*>(q);
}

thread_local char t_err[512] = "";

struct NextScope {
    ~NextScope() { m1_next_clear(); }
};

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_err, sizeof(t_err), fmt, ap);
    va_end(ap);
    return code;
}

bool known_format(int f) { return f == FMT_Q4_0 || f == FMT_Q5_0 || f == FMT_Q8_0 || f == FMT_Q2_K || f == FMT_Q3_K || f == FMT_Q4_K || f == FMT_Q5_K || f == FMT_Q6_K; }
const char* format_name(int f) {
    switch (f) {
    case FMT_Q4_0: return "Q4_0";
    case FMT_Q8_0: return "Q8_0";
    case FMT_Q4_K: return "Q4_K";
    case FMT_Q2_K: return "Q2_K";
    case FMT_Q3_K: return "Q3_K";
    case FMT_Q5_0: return "Q5_0";
    case FMT_Q5_K: return "Q5_K";
    case FMT_Q6_K: return "Q6_K";
    default: return "?";
    }
}

// SM count of the current device, looked up once per device.
int sm_count_current() {
    static int cached[64];
    static std::once_flag once[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::call_once(once[dev], [dev] {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    });
    return cached[dev];
}

int check_matmul_args(const char* op, int format, const void* act, int act_dtype, const void* w, const void* out,
                      int out_dtype, size_t M, size_t K, size_t N) {
    if (!known_format(format)) return fail(B200Q_ERR_UNSUPPORTED_FORMAT, "%s: unsupported format id %d", op, format);
    if (act_dtype != DT_F32 && act_dtype != DT_BF16)
        return fail(B200Q_ERR_UNSUPPORTED_DTYPE, "%s activation must be F32 (or BF16), got dtype id %d", op, act_dtype);
    if (out_dtype != DT_F32 && out_dtype != DT_BF16 && out_dtype != DT_F16)
        return fail(B200Q_ERR_UNSUPPORTED_DTYPE, "%s output must be F32, BF16 or F16, got dtype id %d", op, out_dtype);
    if (M == 0 || K == 0 || N == 0) return fail(B200Q_ERR_BAD_SHAPE, "%s: M, K, N must be positive (M=%zu K=%zu N=%zu)", op, M, K, N);
    if (K % fmt_block_size(format))
        return fail(B200Q_ERR_BAD_SHAPE, "last dimension %zu is not a multiple of %s's block_size %d", K, format_name(format),
                    fmt_block_size(format));
    if (M > 0x7FFFFFFFull / 2 || K > 0x7FFFFFFFull / 2 || N > 0x7FFFFFFFull / 2 ||
        (K / fmt_block_size(format)) * (size_t)fmt_block_bytes(format) > 0x7FFFFFFFull)
        return fail(B200Q_ERR_BAD_SHAPE, "%s: dimension too large (M=%zu K=%zu N=%zu)", op, M, K, N);
    if (!act || !w || !out) return fail(B200Q_ERR_INVALID_ARG, "%s: null pointer", op);
    if (reinterpret_cast<uintptr_t>(w) & 15) return fail(B200Q_ERR_INVALID_ARG, "%s: weight pointer must be 16-byte aligned", op);
    if (reinterpret_cast<uintptr_t>(act) & 15) return fail(B200Q_ERR_INVALID_ARG, "%s: activation pointer must be 16-byte aligned", op);
    if (reinterpret_cast<uintptr_t>(out) & 3) return fail(B200Q_ERR_INVALID_ARG, "%s: output pointer must be 4-byte aligned", op);
    return B200Q_OK;
}

bool i8_in_passes(int format, size_t M, size_t K, size_t N);

// Scratch bytes of one call with activations of `act_dtype` (the public query assumes F32).
size_t workspace_need(int op, int format, int act_dtype, size_t M, size_t K, size_t N) {
    if (!known_format(format) || M == 0 || K == 0 || N == 0 || K % fmt_block_size(format)) return 0;
    const bool swiglu = op == B200Q_OP_QUANT_SWIGLU;
    if (kq_generic_supported(format, M, K, N))  // formats without a tuned kernel: the Q8_K image (+ gate and up for SwiGLU)
        return kq_generic_workspace_bytes(M, K) + (swiglu ? 2 * ((M * N * sizeof(float) + 255) & ~(size_t)255) : 0);
    if (prefill_supported(format, M, K, N)) {
        size_t a = prefill_workspace_bytes(format, act_dtype, M, K, N, sm_count_current());
        // large-M SwiGLU = two prefill GEMMs into scratch, then the gate
        if (swiglu) a += 2 * ((M * N * sizeof(float) + 255) & ~(size_t)255);
        return a;
    }
    // the decode kernels (one activation row) quantise the row inside the kernel and need no scratch
    if (gemv_m1_supported(format, M, K, N, swiglu)) return 0;
    if (!swiglu && gemv_m1_f32_supported(format, M, K, N)) return 0;
    // small-M kernel: the activation image, plus split-K partial sums when K is long
    if (smallm_i8_preferred(format, M, K, N, sm_count_current()))  // integer tensor-core kernel (+ gate and up for SwiGLU)
        return smallm_i8_workspace_bytes(format, M, K, N, sm_count_current()) + (swiglu ? 2 * ((M * N * sizeof(float) + 255) & ~(size_t)255) : 0);
    if (!swiglu && i8_in_passes(format, M, K, N)) {  // passes of 32 rows; a last pass of one row uses the mma.sync kernel's scratch
        const size_t a = smallm_i8_workspace_bytes(format, 32, K, N, sm_count_current()), b = gemv_workspace_bytes(format, 1, K, N, false, sm_count_current());
        return a > b ? a : b;
    }
    return gemv_workspace_bytes(format, M, K, N, swiglu, sm_count_current());
}

}  // namespace

namespace {
// 33..63 activation rows that do not take the bf16 tensor-core path go through the integer tensor-core kernels in passes of
// up to 32 rows (the mma.sync kernel would take passes of 16).
bool i8_in_passes(int format, size_t M, size_t K, size_t N) {
    return M > 32 && M < 64 && !prefill_supported(format, M, K, N) && smallm_i8_preferred(format, 32, K, N, sm_count_current());
}
size_t dtype_bytes(int dt) { return dt == DT_F32 ? 4 : dt == DT_F64 ? 8 : 2; }
cudaError_t launch_i8_passes(int format, const void* act, int act_dtype, const void* w, void* out, int out_dtype, size_t M, size_t K, size_t N,
                             void* ws, size_t ws_bytes, cudaStream_t st, unsigned int* status, bool* small, char* msg, size_t msg_len) {
    cudaError_t e = cudaSuccess;
    for (size_t m0 = 0; m0 < M && e == cudaSuccess && !*small; m0 += 32) {
        const size_t rows = M - m0 < 32 ? M - m0 : 32;
        const void* a = static_cast<const uint8_t*>(act) + m0 * K * dtype_bytes(act_dtype);
        void* o = static_cast<uint8_t*>(out) + m0 * N * dtype_bytes(out_dtype);
        if (rows >= 2 && smallm_i8_supported(format, rows, K, N))
            e = launch_smallm_i8(format, a, act_dtype, w, o, out_dtype, rows, K, N, ws, ws_bytes, sm_count_current(), st, status, small, msg, msg_len,
                                 false);
        else  // a last pass of one row (or of a row count the kernels do not take): the mma.sync kernel
            e = launch_gemv(format, a, act_dtype, w, nullptr, o, out_dtype, rows, K, N, ws, ws_bytes, false, sm_count_current(), st, status, small);
    }
    return e;
}

// Which prepared form of the activations (in scratch) a product reads; -1: none that another weight of a batch could
// share.  The bf16 tensor-core path prepares one form per class of formats (K-quants: Q8_K round trip; others: bf16);
// the mma.sync small-M kernel one image per format (Q5_K reads Q4_K's).
int prepared_class(int format, size_t M, size_t K, size_t N) {
    if (kq_generic_supported(format, M, K, N)) return -1;
    if (prefill_supported(format, M, K, N)) return (format == FMT_Q4_K || format == FMT_Q5_K || format == FMT_Q6_K) ? 101 : 100;
    if (gemv_m1_supported(format, M, K, N, false) || gemv_m1_f32_supported(format, M, K, N)) return -1;
    if (smallm_i8_preferred(format, M, K, N, sm_count_current()) || i8_in_passes(format, M, K, N)) return -1;
    return 200 + (format == FMT_Q5_K ? FMT_Q4_K : format);
}

// acts_prepared: the scratch already holds this activation matrix in the form this product reads (prepared_class): a
// previous weight of the same batch left it there
int quant_matmul_impl(int format, const void* act, int act_dtype, const void* w, void* out, int out_dtype, size_t M,
                      size_t K, size_t N, void* ws, size_t ws_bytes, void* stream, bool acts_prepared) {
    int rc = check_matmul_args("quant_matmul", format, act, act_dtype, w, out, out_dtype, M, K, N);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned int* status = status_ptr_current();
    if (!status) return fail(B200Q_ERR_CUDA, "quant_matmul: cannot resolve the device status word");
    bool small = false;
    cudaError_t e;
    if (kq_generic_supported(format, M, K, N)) {
        e = launch_kq_generic(format, act, act_dtype, w, out, out_dtype, M, K, N, ws, ws_bytes, sm_count_current(), st, &small);
    } else if (prefill_supported(format, M, K, N)) {
        char msg[256] = "";
        e = launch_prefill(format, act, act_dtype, w, out, out_dtype, M, K, N, ws, ws_bytes, sm_count_current(), st,
                           status, &small, msg, sizeof(msg), acts_prepared);
        if (e != cudaSuccess && msg[0]) return fail(B200Q_ERR_CUDA, "quant_matmul: %s", msg);
    } else if (gemv_m1_supported(format, M, K, N, false)) {
        e = launch_gemv_m1(format, act, act_dtype, w, nullptr, out, out_dtype, K, N, sm_count_current(), st, status);
    } else if (gemv_m1_f32_supported(format, M, K, N)) {
        e = launch_gemv_m1_f32(format, act, act_dtype, w, out, out_dtype, K, N, sm_count_current(), st, status);
    } else if (smallm_i8_preferred(format, M, K, N, sm_count_current())) {
        char msg[256] = "";
        e = launch_smallm_i8(format, act, act_dtype, w, out, out_dtype, M, K, N, ws, ws_bytes, sm_count_current(), st, status, &small, msg,
                             sizeof(msg), false);
        if (e != cudaSuccess && msg[0]) return fail(B200Q_ERR_CUDA, "quant_matmul: %s", msg);
    } else if (i8_in_passes(format, M, K, N)) {
        char msg[256] = "";
        e = launch_i8_passes(format, act, act_dtype, w, out, out_dtype, M, K, N, ws, ws_bytes, st, status, &small, msg, sizeof(msg));
        if (e != cudaSuccess && msg[0]) return fail(B200Q_ERR_CUDA, "quant_matmul: %s", msg);
    } else {
        e = launch_gemv(format, act, act_dtype, w, nullptr, out, out_dtype, M, K, N, ws, ws_bytes, false, sm_count_current(),
                        st, status, &small, acts_prepared);
    }
    if (small)
        return fail(B200Q_ERR_WORKSPACE_TOO_SMALL, "quant_matmul: workspace of %zu bytes is too small, need %zu", ws_bytes,
                    b200q_workspace_bytes(B200Q_OP_QUANT_MATMUL, format, M, K, N));
    if (e != cudaSuccess) return fail(B200Q_ERR_CUDA, "CUDA quant_matmul kernel launch failed: %s", cudaGetErrorString(e));
    return B200Q_OK;
}

}  // namespace

extern "C" {

int b200q_version(void) { return 100; }

const char* b200q_last_error(void) { return t_err; }

size_t b200q_block_size(int format) { return known_format(format) ? (size_t)fmt_block_size(format) : 0; }
size_t b200q_block_bytes(int format) { return known_format(format) ? (size_t)fmt_block_bytes(format) : 0; }

int b200q_storage_bytes(int format, size_t numel, size_t* out_bytes) {
    if (!known_format(format)) return fail(B200Q_ERR_UNSUPPORTED_FORMAT, "unsupported format id %d", format);
    if (!out_bytes) return fail(B200Q_ERR_INVALID_ARG, "out_bytes is null");
    size_t bs = fmt_block_size(format);
    if (numel % bs)
        return fail(B200Q_ERR_BAD_SHAPE, "%s: element count %zu is not a multiple of block_size %zu", format_name(format), numel, bs);
    *out_bytes = numel / bs * fmt_block_bytes(format);
    return B200Q_OK;
}

int b200q_dequantize(int format, const void* w, size_t nblocks, void* out, int out_dtype, void* stream) {
    NextScope next_scope;  // a hint about the following launch lives for one call
    if (!known_format(format)) return fail(B200Q_ERR_UNSUPPORTED_FORMAT, "dequantize: unsupported format id %d", format);
    if (out_dtype != DT_F32 && out_dtype != DT_BF16 && out_dtype != DT_F16 && out_dtype != DT_F64)
        return fail(B200Q_ERR_UNSUPPORTED_DTYPE, "dequantize target must be float, got dtype id %d", out_dtype);
    if (nblocks == 0) return B200Q_OK;
    if (!w || !out) return fail(B200Q_ERR_INVALID_ARG, "dequantize: null pointer");
    if (reinterpret_cast<uintptr_t>(w) & 15) return fail(B200Q_ERR_INVALID_ARG, "dequantize: weight pointer must be 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(out) & 15) return fail(B200Q_ERR_INVALID_ARG, "dequantize: output pointer must be 16-byte aligned");
    unsigned int* status = status_ptr_current();
    if (!status) return fail(B200Q_ERR_CUDA, "dequantize: cannot resolve the device status word");
    cudaError_t e = launch_dequant(format, w, nblocks, out, out_dtype, static_cast<cudaStream_t>(stream), sm_count_current(), status);
    if (e != cudaSuccess) return fail(B200Q_ERR_CUDA, "CUDA dequant kernel launch failed: %s", cudaGetErrorString(e));
    return B200Q_OK;
}

size_t b200q_workspace_bytes(int op, int format, size_t M, size_t K, size_t N) {
    // F32 activations need the most scratch (the bf16 / Q8_K activation image of the tensor-core path)
    return workspace_need(op, format, DT_F32, M, K, N);
}

int b200q_quant_matmul(int format, const void* act, int act_dtype, const void* w, void* out, int out_dtype, size_t M,
                       size_t K, size_t N, void* ws, size_t ws_bytes, void* stream) {
    NextScope next_scope;  // a hint about the following launch lives for one call
    return quant_matmul_impl(format, act, act_dtype, w, out, out_dtype, M, K, N, ws, ws_bytes, stream, false);
}

}  // extern "C" (reopened below)

namespace {
// quant_matmul_batch with an optional RMSNorm prologue (norm_w == nullptr: none)
int matmul_batch_impl(const char* op, int n_weights, const int* formats, const void* const* w, const size_t* N, void* const* out,
                      const void* act, int act_dtype, int out_dtype, size_t M, size_t K, void* ws, size_t ws_bytes, void* stream,
                      const float* norm_w, float eps) {
    if (n_weights < 0) return fail(B200Q_ERR_INVALID_ARG, "%s: negative weight count", op);
    if (n_weights == 0) return B200Q_OK;
    if (!formats || !w || !N || !out) return fail(B200Q_ERR_INVALID_ARG, "%s: null array", op);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // The decode kernels (M = 1, Q4_K / Q6_K) normalise the row themselves while they quantise it.  Every other shape
    // gets the normalised activations from one stand-alone launch into the front of the scratch buffer.
    bool all_fused = norm_w != nullptr;
    for (int i = 0; i < n_weights && all_fused; ++i) all_fused = known_format(formats[i]) && gemv_m1_supported(formats[i], M, K, N[i], false);
    if (norm_w && !all_fused) {
        const size_t nbytes = (M * K * sizeof(float) + 255) & ~(size_t)255;
        if (act_dtype != DT_F32 && act_dtype != DT_BF16) return fail(B200Q_ERR_UNSUPPORTED_DTYPE, "%s activation must be F32 (or BF16), got dtype id %d", op, act_dtype);
        if (M == 0 || K == 0 || K % 8) return fail(B200Q_ERR_BAD_SHAPE, "%s: M and K must be positive and K a multiple of 8 (M=%zu K=%zu)", op, M, K);
        if (!act || (reinterpret_cast<uintptr_t>(act) & 15)) return fail(B200Q_ERR_INVALID_ARG, "%s: activation pointer must be non-null and 16-byte aligned", op);
        if (!ws || ws_bytes < nbytes || (reinterpret_cast<uintptr_t>(ws) & 15))
            return fail(B200Q_ERR_WORKSPACE_TOO_SMALL, "%s: workspace of %zu bytes is too small for the normalised activations (%zu bytes)", op, ws_bytes, nbytes);
        cudaError_t e = launch_rmsnorm(act, act_dtype, norm_w, eps, static_cast<float*>(ws), M, K, st);
        if (e != cudaSuccess) return fail(B200Q_ERR_CUDA, "CUDA rmsnorm kernel launch failed: %s", cudaGetErrorString(e));
        act = ws;
        act_dtype = DT_F32;
        ws = static_cast<uint8_t*>(ws) + nbytes;
        ws_bytes -= nbytes;
        norm_w = nullptr;
    }
    int prepared_cls = -1;
    for (int i = 0; i < n_weights;) {
        // decode (M = 1): runs of up to three Q4_K weights, optionally followed by one Q6_K weight (the
        // q/k/v projections of a Q4_K_M model), go out as ONE launch that streams them side by side
        int run = 1;
        bool mixed = false;
        if (formats[i] == FMT_Q4_K && gemv_m1_supported(FMT_Q4_K, M, K, N[i], false)) {
            while (run < 3 && i + run < n_weights && formats[i + run] == FMT_Q4_K) ++run;
            mixed = i + run < n_weights && formats[i + run] == FMT_Q6_K && gemv_m1_supported(FMT_Q6_K, M, K, N[i + run], false);
        }
        const int total = run + (mixed ? 1 : 0);
        if (total > 1 || norm_w) {
            for (int j = 0; j < total; ++j) {
                int rc = check_matmul_args(op, formats[i + j], act, act_dtype, w[i + j], out[i + j], out_dtype, M, K, N[i + j]);
                if (rc) return rc;
            }
            unsigned int* status = status_ptr_current();
            if (!status) return fail(B200Q_ERR_CUDA, "%s: cannot resolve the device status word", op);
            cudaError_t e;
            if (mixed)
                e = launch_gemv_m1_mixed(act, act_dtype, run, w + i, N + i, out + i, w[i + run], N[i + run], out[i + run], out_dtype, K,
                                         sm_count_current(), st, status, norm_w, eps);
            else if (formats[i] == FMT_Q4_K)
                e = launch_gemv_m1_batch(act, act_dtype, run, w + i, N + i, out + i, nullptr, out_dtype, K, sm_count_current(), st, status,
                                         norm_w, eps);
            else  // a single fused-prologue weight of another format (Q6_K)
                e = launch_gemv_m1(formats[i], act, act_dtype, w[i], nullptr, out[i], out_dtype, K, N[i], sm_count_current(), st, status,
                                   norm_w, eps);
            if (e != cudaSuccess) return fail(B200Q_ERR_CUDA, "CUDA %s kernel launch failed: %s", op, cudaGetErrorString(e));
        } else {
            // the weights of a batch share the prepared activations where consecutive ones read the same form of them
            const int cls = prepared_class(formats[i], M, K, N[i]);
            int rc = quant_matmul_impl(formats[i], act, act_dtype, w[i], out[i], out_dtype, M, K, N[i], ws, ws_bytes, stream,
                                       cls >= 0 && prepared_cls == cls);
            if (rc) return rc;
            prepared_cls = cls;  // -1: another kernel family may have used the scratch for something else
        }
        i += total;
    }
    return B200Q_OK;
}
}  // namespace

extern "C" {

int b200q_quant_matmul_batch(int n_weights, const int* formats, const void* const* w, const size_t* N, void* const* out,
                             const void* act, int act_dtype, int out_dtype, size_t M, size_t K, void* ws, size_t ws_bytes,
                             void* stream) {
    NextScope next_scope;  // a hint about the following launch lives for one call
    return matmul_batch_impl("quant_matmul_batch", n_weights, formats, w, N, out, act, act_dtype, out_dtype, M, K, ws, ws_bytes, stream,
                             nullptr, 0.f);
}

int b200q_rmsnorm_quant_matmul_batch(int n_weights, const int* formats, const void* const* w, const size_t* N, void* const* out,
                                     const void* act, const float* norm_weight, float eps, int act_dtype, int out_dtype, size_t M,
                                     size_t K, void* ws, size_t ws_bytes, void* stream) {
    NextScope next_scope;  // a hint about the following launch lives for one call
    if (!norm_weight) return fail(B200Q_ERR_INVALID_ARG, "rmsnorm_quant_matmul_batch: null norm weight");
    if (reinterpret_cast<uintptr_t>(norm_weight) & 15) return fail(B200Q_ERR_INVALID_ARG, "rmsnorm_quant_matmul_batch: norm weight must be 16-byte aligned");
    return matmul_batch_impl("rmsnorm_quant_matmul_batch", n_weights, formats, w, N, out, act, act_dtype, out_dtype, M, K, ws, ws_bytes,
                             stream, norm_weight, eps);
}

int b200q_quant_swiglu(int format, const void* act, int act_dtype, const void* w_gate, const void* w_up, void* out,
                       int out_dtype, size_t M, size_t K, size_t N, void* ws, size_t ws_bytes, void* stream) {
    NextScope next_scope;  // a hint about the following launch lives for one call
    int rc = check_matmul_args("quant_swiglu", format, act, act_dtype, w_gate, out, out_dtype, M, K, N);
    if (rc) return rc;
    if (!w_up) return fail(B200Q_ERR_INVALID_ARG, "quant_swiglu: null pointer");
    if (reinterpret_cast<uintptr_t>(w_up) & 15) return fail(B200Q_ERR_INVALID_ARG, "quant_swiglu: weight pointer must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned int* status = status_ptr_current();
    if (!status) return fail(B200Q_ERR_CUDA, "quant_swiglu: cannot resolve the device status word");
    const size_t need = b200q_workspace_bytes(B200Q_OP_QUANT_SWIGLU, format, M, K, N);
    if (need > ws_bytes || (need && !ws))
        return fail(B200Q_ERR_WORKSPACE_TOO_SMALL, "quant_swiglu: workspace of %zu bytes is too small, need %zu", ws_bytes, need);
    bool small = false;
    cudaError_t e;
    if (kq_generic_supported(format, M, K, N)) {
        // two products into f32 scratch (the second finds the Q8_K image again, it is rebuilt: same bytes), then the gate
        const size_t mn = (M * N * sizeof(float) + 255) & ~(size_t)255;
        float* g = static_cast<float*>(ws);
        float* u = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + mn);
        uint8_t* rest = static_cast<uint8_t*>(ws) + 2 * mn;
        const size_t rest_bytes = ws_bytes - 2 * mn;
        e = launch_kq_generic(format, act, act_dtype, w_gate, g, DT_F32, M, K, N, rest, rest_bytes, sm_count_current(), st, &small);
        if (e == cudaSuccess && !small)
            e = launch_kq_generic(format, act, act_dtype, w_up, u, DT_F32, M, K, N, rest, rest_bytes, sm_count_current(), st, &small);
        if (e == cudaSuccess && !small) e = launch_swiglu_gate(g, u, out, out_dtype, M * N, sm_count_current(), st);
    } else if (prefill_supported(format, M, K, N)) {
        // two tensor-core GEMMs into f32 scratch, then silu(gate) * up
        const size_t mn = (M * N * sizeof(float) + 255) & ~(size_t)255;
        float* g = static_cast<float*>(ws);
        float* u = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + mn);
        uint8_t* rest = static_cast<uint8_t*>(ws) + 2 * mn;
        const size_t rest_bytes = ws_bytes - 2 * mn;
        char msg[256] = "";
        e = launch_prefill(format, act, act_dtype, w_gate, g, DT_F32, M, K, N, rest, rest_bytes, sm_count_current(), st, status,
                           &small, msg, sizeof(msg), false);
        if (e == cudaSuccess && !small)  // the prepared activations of the first product are still in `rest`
            e = launch_prefill(format, act, act_dtype, w_up, u, DT_F32, M, K, N, rest, rest_bytes, sm_count_current(), st,
                               status, &small, msg, sizeof(msg), true);
        if (e != cudaSuccess && msg[0]) return fail(B200Q_ERR_CUDA, "quant_swiglu: %s", msg);
        if (e == cudaSuccess && !small) e = launch_swiglu_gate(g, u, out, out_dtype, M * N, sm_count_current(), st);
    } else if (gemv_m1_supported(format, M, K, N, true)) {
        e = launch_gemv_m1(format, act, act_dtype, w_gate, w_up, out, out_dtype, K, N, sm_count_current(), st, status);
    } else if (smallm_i8_preferred(format, M, K, N, sm_count_current())) {
        // two integer tensor-core products into f32 scratch (the second reuses the quantised activations), then the gate
        const size_t mn = (M * N * sizeof(float) + 255) & ~(size_t)255;
        float* g = static_cast<float*>(ws);
        float* u = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + mn);
        uint8_t* rest = static_cast<uint8_t*>(ws) + 2 * mn;
        const size_t rest_bytes = ws_bytes - 2 * mn;
        char msg[256] = "";
        e = launch_smallm_i8(format, act, act_dtype, w_gate, g, DT_F32, M, K, N, rest, rest_bytes, sm_count_current(), st, status, &small, msg,
                             sizeof(msg), false);
        if (e == cudaSuccess && !small)
            e = launch_smallm_i8(format, act, act_dtype, w_up, u, DT_F32, M, K, N, rest, rest_bytes, sm_count_current(), st, status, &small, msg,
                                 sizeof(msg), true);
        if (e != cudaSuccess && msg[0]) return fail(B200Q_ERR_CUDA, "quant_swiglu: %s", msg);
        if (e == cudaSuccess && !small) e = launch_swiglu_gate(g, u, out, out_dtype, M * N, sm_count_current(), st);
    } else {
        e = launch_gemv(format, act, act_dtype, w_gate, w_up, out, out_dtype, M, K, N, ws, ws_bytes, true, sm_count_current(),
                        st, status, &small);
    }
    if (small) return fail(B200Q_ERR_WORKSPACE_TOO_SMALL, "quant_swiglu: workspace of %zu bytes is too small, need %zu", ws_bytes, need);
    if (e != cudaSuccess) return fail(B200Q_ERR_CUDA, "CUDA quant_swiglu kernel launch failed: %s", cudaGetErrorString(e));
    return B200Q_OK;
}

size_t b200q_mlp_workspace_bytes(int format_gate_up, int format_down, size_t M, size_t K, size_t n_ff, size_t n_out) {
    const size_t a = workspace_need(B200Q_OP_QUANT_SWIGLU, format_gate_up, DT_F32, M, K, n_ff);
    const size_t b = workspace_need(B200Q_OP_QUANT_MATMUL, format_down, DT_F32, M, n_ff, n_out);
    return ((M * n_ff * sizeof(float) + 255) & ~(size_t)255) + (a > b ? a : b);
}

int b200q_quant_mlp(int format_gate_up, const void* w_gate, const void* w_up, int format_down, const void* w_down, const void* act,
                    int act_dtype, void* out, int out_dtype, size_t M, size_t K, size_t n_ff, size_t n_out, void* ws, size_t ws_bytes,
                    void* stream) {
    NextScope next_scope;  // a hint about the following launch lives for one call
    const size_t hid = (M * n_ff * sizeof(float) + 255) & ~(size_t)255;
    if (!ws || ws_bytes < hid || (reinterpret_cast<uintptr_t>(ws) & 15))
        return fail(B200Q_ERR_WORKSPACE_TOO_SMALL, "quant_mlp: workspace of %zu bytes is too small, need %zu", ws_bytes,
                    b200q_mlp_workspace_bytes(format_gate_up, format_down, M, K, n_ff, n_out));
    float* h = static_cast<float*>(ws);
    uint8_t* rest = static_cast<uint8_t*>(ws) + hid;
    const size_t rest_bytes = ws_bytes - hid;
    // the gate/up launch pulls the head of the down-projection into L2 while it drains; the caller's own hint is for the
    // launch after the down-projection
    m1_next_stash();
    if (M == 1) m1_next_set(false, 1, &format_down, &w_down, &n_out, n_ff, sm_count_current());
    int rc = b200q_quant_swiglu(format_gate_up, act, act_dtype, w_gate, w_up, h, DT_F32, M, K, n_ff, rest, rest_bytes, stream);
    m1_next_unstash();
    if (rc) return rc;
    return quant_matmul_impl(format_down, h, DT_F32, w_down, out, out_dtype, M, n_ff, n_out, rest, rest_bytes, stream, false);
}

int b200q_prefetch_next(int op, int n_weights, const int* formats, const void* const* w, const size_t* N, size_t K) {
    m1_next_clear();
    if (op != B200Q_OP_QUANT_MATMUL && op != B200Q_OP_QUANT_SWIGLU) return fail(B200Q_ERR_INVALID_ARG, "prefetch_next: unknown operation %d", op);
    if (n_weights < 1 || !formats || !w || !N) return fail(B200Q_ERR_INVALID_ARG, "prefetch_next: null array or no weights");
    for (int i = 0; i < n_weights; ++i) {
        if (!known_format(formats[i])) return fail(B200Q_ERR_UNSUPPORTED_FORMAT, "prefetch_next: unsupported format id %d", formats[i]);
        if (!w[i] || (reinterpret_cast<uintptr_t>(w[i]) & 15)) return fail(B200Q_ERR_INVALID_ARG, "prefetch_next: weight pointer must be non-null and 16-byte aligned");
    }
    m1_next_set(op == B200Q_OP_QUANT_SWIGLU, n_weights, formats, w, N, K, sm_count_current());  // false: no kernel would use it
    return B200Q_OK;
}

int b200q_shard_pack(int format, const void* src, size_t N, size_t K, int dim, int rank, int world, void* dst,
                     size_t dst_bytes) {
    if (!known_format(format)) return fail(B200Q_ERR_UNSUPPORTED_FORMAT, "shard_pack: unsupported format id %d", format);
    if (!src || !dst) return fail(B200Q_ERR_INVALID_ARG, "shard_pack: null pointer");
    if (world <= 0 || rank < 0 || rank >= world) return fail(B200Q_ERR_INVALID_ARG, "shard_pack: rank %d out of range for world size %d", rank, world);
    const size_t bs = fmt_block_size(format), bb = fmt_block_bytes(format);
    if (K % bs) return fail(B200Q_ERR_BAD_SHAPE, "last dimension %zu is not a multiple of %s's block_size %zu", K, format_name(format), bs);
    const size_t row_bytes = K / bs * bb;
    const uint8_t* s = static_cast<const uint8_t*>(src);
    uint8_t* d = static_cast<uint8_t*>(dst);
    if (dim == 0) {
        if (N % (size_t)world) return fail(B200Q_ERR_BAD_SHAPE, "out_features %zu not divisible by world_size %d", N, world);
        const size_t rows = N / world, bytes = rows * row_bytes;
        if (dst_bytes < bytes) return fail(B200Q_ERR_INVALID_ARG, "shard_pack: destination holds %zu bytes, need %zu", dst_bytes, bytes);
        memcpy(d, s + (size_t)rank * bytes, bytes);
        return B200Q_OK;
    }
    if (dim == 1) {
        if (K % (size_t)world) return fail(B200Q_ERR_BAD_SHAPE, "in_features %zu not divisible by world_size %d", K, world);
        const size_t kl = K / world;
        if (kl % bs) return fail(B200Q_ERR_BAD_SHAPE, "in_features per rank %zu is not a multiple of %s's block_size %zu", kl, format_name(format), bs);
        const size_t lrow = kl / bs * bb, bytes = N * lrow;
        if (dst_bytes < bytes) return fail(B200Q_ERR_INVALID_ARG, "shard_pack: destination holds %zu bytes, need %zu", dst_bytes, bytes);
        for (size_t r = 0; r < N; ++r) memcpy(d + r * lrow, s + r * row_bytes + (size_t)rank * lrow, lrow);
        return B200Q_OK;
    }
    return fail(B200Q_ERR_INVALID_ARG, "shard_pack: dim must be 0 or 1, got %d", dim);
}

}  // extern "C" (reopened below)

// Scratch of b200q_quant_matmul_static_scratch.  In host code this name is only a handle of the
// symbol; the address kernels can use comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[B200Q_STATIC_SCRATCH_BYTES];

namespace {
// Device address of g_static_scratch on the current device; resolved on the first call made with
// that device current.  Returns nullptr (and sets *err) when the lookup fails; only a successful
// lookup is remembered, so the next call tries again.  The address belongs to the device's primary
// context.
void* static_scratch_current(cudaError_t* err) {
    static std::atomic<void*> cached[64];
    int dev = 0;
    *err = cudaGetDevice(&dev);
    if (*err != cudaSuccess) return nullptr;
    if (dev < 0 || dev >= 64) {
        *err = cudaErrorInvalidDevice;
        return nullptr;
    }
    void* p = cached[dev].load(std::memory_order_acquire);
    if (p) return p;
    *err = cudaGetSymbolAddress(&p, g_static_scratch);
    if (*err != cudaSuccess || !p) {
        cudaGetLastError();
        if (*err == cudaSuccess) *err = cudaErrorInvalidSymbol;
        return nullptr;
    }
    cached[dev].store(p, std::memory_order_release);
    return p;
}
}  // namespace

extern "C" {

int b200q_quant_matmul_static_scratch(int format, const void* act, int act_dtype, const void* w, void* out, int out_dtype,
                                      size_t M, size_t K, size_t N, void* stream) {
    NextScope next_scope;  // a hint about the following launch lives for one call
    int rc = check_matmul_args("quant_matmul_static_scratch", format, act, act_dtype, w, out, out_dtype, M, K, N);
    if (rc) return rc;
    const size_t need = workspace_need(B200Q_OP_QUANT_MATMUL, format, act_dtype, M, K, N);
    if (need > B200Q_STATIC_SCRATCH_BYTES)
        return fail(B200Q_ERR_WORKSPACE_TOO_SMALL,
                    "quant_matmul_static_scratch: this shape (M=%zu K=%zu N=%zu) needs %zu bytes of scratch, the built-in "
                    "array holds %u; use b200q_quant_matmul with caller-provided scratch",
                    M, K, N, need, (unsigned)B200Q_STATIC_SCRATCH_BYTES);
    cudaError_t e = cudaSuccess;
    void* scratch = static_scratch_current(&e);
    if (!scratch)
        return fail(B200Q_ERR_CUDA, "quant_matmul_static_scratch: cannot resolve the scratch array: %s", cudaGetErrorString(e));
    return b200q_quant_matmul(format, act, act_dtype, w, out, out_dtype, M, K, N, scratch, B200Q_STATIC_SCRATCH_BYTES, stream);
}

unsigned long long b200q_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

size_t b200q_tp_buffer_bytes(void) { return TP_BUF_BYTES; }

int b200q_tp_alloc(void** buf, unsigned char* handle) {
    if (!buf || !handle) return fail(B200Q_ERR_INVALID_ARG, "tp_alloc: null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == B200Q_TP_HANDLE_BYTES, "IPC handle size");
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, TP_BUF_BYTES);
    if (e == cudaSuccess) e = cudaMemset(p, 0, TP_BUF_BYTES);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        if (p) cudaFree(p);
        return fail(B200Q_ERR_CUDA, "tp_alloc: %s", cudaGetErrorString(e));
    }
    memcpy(handle, &h, sizeof(h));
    *buf = p;
    return B200Q_OK;
}

int b200q_tp_open(const unsigned char* handle, void** peer_buf) {
    if (!handle || !peer_buf) return fail(B200Q_ERR_INVALID_ARG, "tp_open: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(B200Q_ERR_CUDA, "tp_open: %s", cudaGetErrorString(e));
    *peer_buf = p;
    return B200Q_OK;
}

int b200q_tp_close(void* peer_buf) {
    cudaError_t e = cudaIpcCloseMemHandle(peer_buf);
    return e == cudaSuccess ? B200Q_OK : fail(B200Q_ERR_CUDA, "tp_close: %s", cudaGetErrorString(e));
}

int b200q_tp_free(void* buf) {
    cudaError_t e = cudaFree(buf);
    return e == cudaSuccess ? B200Q_OK : fail(B200Q_ERR_CUDA, "tp_free: %s", cudaGetErrorString(e));
}

int b200q_row_parallel_matmul(int format, const void* act, int act_dtype, const void* w, void* out, int out_dtype, size_t M,
                              size_t K, size_t N, int rank, int world, void* const* bufs, void* stream) {
    NextScope next_scope;  // a hint about the following launch lives for one call
    int rc = check_matmul_args("row_parallel_matmul", format, act, act_dtype, w, out, out_dtype, M, K, N);
    if (rc) return rc;
    if (world < 1 || world > (int)TP_MAX_WORLD || rank < 0 || rank >= world)
        return fail(B200Q_ERR_INVALID_ARG, "row_parallel_matmul: rank %d of world %d (at most %u ranks)", rank, world, TP_MAX_WORLD);
    if (!bufs) return fail(B200Q_ERR_INVALID_ARG, "row_parallel_matmul: null buffer table");
    if (M != 1 || out_dtype != DT_F32 || N > TP_MAX_N || !gemv_m1_supported(format, M, K, N, false))
        return fail(B200Q_ERR_NOT_FUSED, "row_parallel_matmul: no fused exchange for %s M=%zu K=%zu N=%zu; use quant_matmul + all-reduce",
                    format_name(format), M, K, N);
    PeerComm comm{};
    comm.world = (uint32_t)world;
    comm.rank = (uint32_t)rank;
    for (int r = 0; r < world; ++r) {
        if (!bufs[r]) return fail(B200Q_ERR_INVALID_ARG, "row_parallel_matmul: null exchange buffer of rank %d", r);
        comm.buf[r] = static_cast<uint8_t*>(bufs[r]);
    }
    unsigned int* status = status_ptr_current();
    if (!status) return fail(B200Q_ERR_CUDA, "row_parallel_matmul: cannot resolve the device status word");
    cudaError_t e = launch_gemv_m1_rowpar(format, act, act_dtype, w, out, K, N, sm_count_current(), static_cast<cudaStream_t>(stream),
                                          status, comm);
    if (e != cudaSuccess) return fail(B200Q_ERR_CUDA, "CUDA row_parallel_matmul kernel launch failed: %s", cudaGetErrorString(e));
    return B200Q_OK;
}

int b200q_col_parallel_matmul_gather(int format, const void* act, int act_dtype, const void* w, void* out_full, size_t M, size_t K,
                                     size_t n_local, int rank, int world, void* const* bufs, void* stream) {
    NextScope next_scope;  // a hint about the following launch lives for one call
    int rc = check_matmul_args("col_parallel_matmul_gather", format, act, act_dtype, w, out_full, DT_F32, M, K, n_local);
    if (rc) return rc;
    if (world < 1 || world > (int)TP_MAX_WORLD || rank < 0 || rank >= world)
        return fail(B200Q_ERR_INVALID_ARG, "col_parallel_matmul_gather: rank %d of world %d (at most %u ranks)", rank, world, TP_MAX_WORLD);
    if (!bufs) return fail(B200Q_ERR_INVALID_ARG, "col_parallel_matmul_gather: null buffer table");
    const size_t n_total = n_local * (size_t)world;
    if (M != 1 || n_total > (size_t)TP_MAX_WORLD * TP_MAX_N || !gemv_m1_supported(format, M, K, n_local, false))
        return fail(B200Q_ERR_NOT_FUSED,
                    "col_parallel_matmul_gather: no fused gather for %s M=%zu K=%zu N=%zu x %d ranks; use quant_matmul + all-gather",
                    format_name(format), M, K, n_local, world);
    PeerComm comm{};
    comm.world = (uint32_t)world;
    comm.rank = (uint32_t)rank;
    comm.gather = 1;
    comm.n_total = (uint32_t)n_total;
    for (int r = 0; r < world; ++r) {
        if (!bufs[r]) return fail(B200Q_ERR_INVALID_ARG, "col_parallel_matmul_gather: null exchange buffer of rank %d", r);
        comm.buf[r] = static_cast<uint8_t*>(bufs[r]);
    }
    unsigned int* status = status_ptr_current();
    if (!status) return fail(B200Q_ERR_CUDA, "col_parallel_matmul_gather: cannot resolve the device status word");
    cudaError_t e = launch_gemv_m1_rowpar(format, act, act_dtype, w, out_full, K, n_local, sm_count_current(),
                                          static_cast<cudaStream_t>(stream), status, comm);
    if (e != cudaSuccess) return fail(B200Q_ERR_CUDA, "CUDA col_parallel_matmul_gather kernel launch failed: %s", cudaGetErrorString(e));
    return B200Q_OK;
}

int b200q_tp_all_reduce(void* data, size_t count, int rank, int world, void* const* bufs, void* stream) {
    NextScope next_scope;  // a hint about the following launch lives for one call
    if (!data || (reinterpret_cast<uintptr_t>(data) & 3)) return fail(B200Q_ERR_INVALID_ARG, "tp_all_reduce: data must be a 4-byte aligned device pointer");
    if (world < 1 || world > (int)TP_MAX_WORLD || rank < 0 || rank >= world)
        return fail(B200Q_ERR_INVALID_ARG, "tp_all_reduce: rank %d of world %d (at most %u ranks)", rank, world, TP_MAX_WORLD);
    if (!bufs) return fail(B200Q_ERR_INVALID_ARG, "tp_all_reduce: null buffer table");
    if (count == 0) return B200Q_OK;
    if (count > TP_MAX_N)
        return fail(B200Q_ERR_NOT_FUSED, "tp_all_reduce: %zu values exceed the exchange buffer (%u); use the communicator's all-reduce", count, TP_MAX_N);
    PeerComm comm{};
    comm.world = (uint32_t)world;
    comm.rank = (uint32_t)rank;
    for (int r = 0; r < world; ++r) {
        if (!bufs[r]) return fail(B200Q_ERR_INVALID_ARG, "tp_all_reduce: null exchange buffer of rank %d", r);
        comm.buf[r] = static_cast<uint8_t*>(bufs[r]);
    }
    unsigned int* status = status_ptr_current();
    if (!status) return fail(B200Q_ERR_CUDA, "tp_all_reduce: cannot resolve the device status word");
    cudaError_t e = launch_tp_all_reduce(static_cast<float*>(data), count, comm, sm_count_current(), static_cast<cudaStream_t>(stream), status);
    if (e != cudaSuccess) return fail(B200Q_ERR_CUDA, "CUDA tp_all_reduce kernel launch failed: %s", cudaGetErrorString(e));
    return B200Q_OK;
}

int b200q_check_device_status(void* stream) {
    cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(B200Q_ERR_CUDA, "stream synchronize failed: %s", cudaGetErrorString(e));
    unsigned int word = 0, zero = 0;
    e = cudaMemcpyFromSymbol(&word, g_status_word, sizeof(word));
    if (e != cudaSuccess) return fail(B200Q_ERR_CUDA, "status read failed: %s", cudaGetErrorString(e));
    if (word) {
        cudaMemcpyToSymbol(g_status_word, &zero, sizeof(zero));
        return fail(B200Q_ERR_TIMEOUT, "a kernel gave up on a bounded wait (status 0x%x)", word);
    }
    return B200Q_OK;
}

}  // extern "C"
