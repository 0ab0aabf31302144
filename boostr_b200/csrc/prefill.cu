// Tensor-core prefill GEMM (M >= 64): placeholder translation unit until the tcgen05 kernel lands.
#include "common.cuh"

namespace b200q {

bool prefill_supported(int, size_t, size_t, size_t) { return false; }
size_t prefill_workspace_bytes(int, int, size_t, size_t, size_t) { return 0; }
cudaError_t launch_prefill(int, const void*, int, const void*, void*, int, size_t, size_t, size_t, void*, size_t, int,
                           cudaStream_t, unsigned int*, bool* ws_too_small, char*, size_t) {
    *ws_too_small = false;
    return cudaErrorNotSupported;
}

namespace {
__global__ void __launch_bounds__(256) swiglu_gate_kernel(const float* __restrict__ g, const float* __restrict__ u, void* out,
                                                          int out_dtype, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float x = g[i];
        float v = x / (1.0f + expf(-x)) * u[i];
        if (out_dtype == DT_F32) static_cast<float*>(out)[i] = v;
        else if (out_dtype == DT_BF16) static_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
        else static_cast<__half*>(out)[i] = __float2half_rn(v);
    }
}
}  // namespace

cudaError_t launch_swiglu_gate(const float* gate, const float* up, void* out, int out_dtype, size_t n, int sm_count,
                               cudaStream_t st) {
    size_t want = (n + 255) / 256;
    int grid = (int)(want < (size_t)sm_count * 8 ? want : (size_t)sm_count * 8);
    if (grid < 1) grid = 1;
    swiglu_gate_kernel<<<grid, 256, 0, st>>>(gate, up, out, out_dtype, n);
    note_launch();
    return cudaGetLastError();
}

}  // namespace b200q
