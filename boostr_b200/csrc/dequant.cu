// Dequantise packed GGUF blocks (Q4_0, Q8_0, Q4_K, Q6_K) straight to f32 / bf16 / f16 / f64.
//
// Stands in for boostr's dequant_*_f32 kernels (src/quant/cuda/kernels/dequant.cu:18-206, one
// thread per block, scalar stores) plus the separate cast pass of CudaClient::dequantize
// (src/quant/cuda/dequant.rs:141-145).  Here one warp owns 256 consecutive elements, each lane
// decodes 8 consecutive elements and writes them with 16-byte stores, so a warp writes 512 B
// (bf16) or 1 KiB (f32) contiguously and the output is produced in a single pass.  The kernel is
// bound by HBM writes: 2 or 4 bytes written per element against 0.56-1.06 bytes read.
//
// Every dequantised value is exactly representable in f32 (block scales are fp16, codes have at
// most 8 bits), so the f32 result is independent of evaluation order; Q4_K's final
// d*sc*q - dmin*m is one rounding of an exact product, written without FMA contraction.
#include "common.cuh"

namespace b200q {

namespace {

__device__ __forceinline__ uint32_t ldg_u16(const uint8_t* p) { return __ldg(reinterpret_cast<const unsigned short*>(p)); }

// 4 bytes at a 2-byte-aligned global address
__device__ __forceinline__ uint32_t ldg_w(const uint8_t* p) {
    if ((reinterpret_cast<uintptr_t>(p) & 3u) == 0) return __ldg(reinterpret_cast<const uint32_t*>(p));
    return ldg_u16(p) | (ldg_u16(p + 2) << 16);
}

template <typename T>
__device__ __forceinline__ void store8(T* out, const float (&v)[8]);

template <>
__device__ __forceinline__ void store8<float>(float* out, const float (&v)[8]) {
    reinterpret_cast<float4*>(out)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(out)[1] = make_float4(v[4], v[5], v[6], v[7]);
}
template <>
__device__ __forceinline__ void store8<double>(double* out, const float (&v)[8]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) reinterpret_cast<double2*>(out)[i] = make_double2((double)v[2 * i], (double)v[2 * i + 1]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* out, const float (&v)[8]) {
    uint4 r;
    __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0], v[1]), p1 = __floats2bfloat162_rn(v[2], v[3]);
    __nv_bfloat162 p2 = __floats2bfloat162_rn(v[4], v[5]), p3 = __floats2bfloat162_rn(v[6], v[7]);
    r.x = *reinterpret_cast<uint32_t*>(&p0);
    r.y = *reinterpret_cast<uint32_t*>(&p1);
    r.z = *reinterpret_cast<uint32_t*>(&p2);
    r.w = *reinterpret_cast<uint32_t*>(&p3);
    *reinterpret_cast<uint4*>(out) = r;
}
template <>
__device__ __forceinline__ void store8<__half>(__half* out, const float (&v)[8]) {
    uint4 r;
    __half2 p0 = __floats2half2_rn(v[0], v[1]), p1 = __floats2half2_rn(v[2], v[3]);
    __half2 p2 = __floats2half2_rn(v[4], v[5]), p3 = __floats2half2_rn(v[6], v[7]);
    r.x = *reinterpret_cast<uint32_t*>(&p0);
    r.y = *reinterpret_cast<uint32_t*>(&p1);
    r.z = *reinterpret_cast<uint32_t*>(&p2);
    r.w = *reinterpret_cast<uint32_t*>(&p3);
    *reinterpret_cast<uint4*>(out) = r;
}

// float value of byte `I` of x (0..255) without an integer-to-float conversion instruction
template <int I>
__device__ __forceinline__ float byte_to_float(uint32_t x) {
    return __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7650 | I)) - 8388608.0f;
}

// Decode the 8 consecutive elements [8*lane, 8*lane+8) of one 256-element run starting at `u`.
template <int FMT>
__device__ __forceinline__ void decode8(const uint8_t* u, int lane, float (&v)[8]) {
    if constexpr (FMT == FMT_Q4_0) {
        // block = f16 d | 16 B nibbles; byte i -> elements 2i (low), 2i+1 (high)
        // (src/quant/cpu/kernels/dequant_simple.rs:11-32)
        const uint8_t* blk = u + (lane >> 2) * 18;
        float d = f16bits_to_f32(ldg_u16(blk));
        const uint32_t w = ldg_w(blk + 2 + 4 * (lane & 3));
        const uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
        v[0] = (byte_to_float<0>(lo) - 8.0f) * d; v[1] = (byte_to_float<0>(hi) - 8.0f) * d;
        v[2] = (byte_to_float<1>(lo) - 8.0f) * d; v[3] = (byte_to_float<1>(hi) - 8.0f) * d;
        v[4] = (byte_to_float<2>(lo) - 8.0f) * d; v[5] = (byte_to_float<2>(hi) - 8.0f) * d;
        v[6] = (byte_to_float<3>(lo) - 8.0f) * d; v[7] = (byte_to_float<3>(hi) - 8.0f) * d;
    } else if constexpr (FMT == FMT_Q8_0) {
        // block = f16 d | 32 x i8 (dequant_simple.rs:137-155)
        const uint8_t* blk = u + (lane >> 2) * 34;
        float d = f16bits_to_f32(ldg_u16(blk));
        const uint8_t* q = blk + 2 + 8 * (lane & 3);
        const uint32_t w0 = ldg_w(q) ^ 0x80808080u, w1 = ldg_w(q + 4) ^ 0x80808080u;  // q + 128 as unsigned bytes
        v[0] = (byte_to_float<0>(w0) - 128.0f) * d; v[1] = (byte_to_float<1>(w0) - 128.0f) * d;
        v[2] = (byte_to_float<2>(w0) - 128.0f) * d; v[3] = (byte_to_float<3>(w0) - 128.0f) * d;
        v[4] = (byte_to_float<0>(w1) - 128.0f) * d; v[5] = (byte_to_float<1>(w1) - 128.0f) * d;
        v[6] = (byte_to_float<2>(w1) - 128.0f) * d; v[7] = (byte_to_float<3>(w1) - 128.0f) * d;
    } else if constexpr (FMT == FMT_Q4_K) {
        // block = f16 d | f16 dmin | 12 B packed 6-bit scales/mins | 128 B nibbles
        // (src/quant/cpu/kernels/dequant_k_quants/q4k_q5k.rs:10-47, :108-122)
        const int j = lane >> 2;  // 32-element sub-block
        const uint32_t* hd = reinterpret_cast<const uint32_t*>(u);
        const uint32_t dm = __ldg(hd), h1 = __ldg(hd + 1), h2 = __ldg(hd + 2), h3 = __ldg(hd + 3);
        const float d = f16bits_to_f32(dm & 0xFFFF), dmin = f16bits_to_f32(dm >> 16);
        // the four 6-bit scales / mins of sub-blocks 0-3 or 4-7 as packed bytes
        const uint32_t scw = j < 4 ? (h1 & 0x3F3F3F3Fu) : ((h3 & 0x0F0F0F0Fu) | ((h1 >> 2) & 0x30303030u));
        const uint32_t mnw = j < 4 ? (h2 & 0x3F3F3F3Fu) : (((h3 >> 4) & 0x0F0F0F0Fu) | ((h2 >> 2) & 0x30303030u));
        const int sh8 = 8 * (j & 3);
        // d * sc and dmin * m are exact (11 x 6 bits), and so is (d * sc) * q: the fused multiply-add below
        // rounds once, exactly like the multiply-then-subtract of the reference
        const float dl = d * (float)((scw >> sh8) & 0xFF), nml = -(dmin * (float)((mnw >> sh8) & 0xFF));
        const uint2 w = __ldg(reinterpret_cast<const uint2*>(u + 16 + (j >> 1) * 32 + 8 * (lane & 3)));
        const int sh = (j & 1) * 4;
        const uint32_t q0 = (w.x >> sh) & 0x0F0F0F0Fu, q1 = (w.y >> sh) & 0x0F0F0F0Fu;
        v[0] = fmaf(dl, byte_to_float<0>(q0), nml); v[1] = fmaf(dl, byte_to_float<1>(q0), nml);
        v[2] = fmaf(dl, byte_to_float<2>(q0), nml); v[3] = fmaf(dl, byte_to_float<3>(q0), nml);
        v[4] = fmaf(dl, byte_to_float<0>(q1), nml); v[5] = fmaf(dl, byte_to_float<1>(q1), nml);
        v[6] = fmaf(dl, byte_to_float<2>(q1), nml); v[7] = fmaf(dl, byte_to_float<3>(q1), nml);
    } else {
        // Q6_K block = 128 B ql | 64 B qh | 16 x i8 scales | f16 d
        // (src/quant/cpu/kernels/dequant_k_quants/q6k_q8k.rs:10-56)
        int n = lane >> 4, gq = (lane >> 2) & 3, l0 = 8 * (lane & 3);
        float d = f16bits_to_f32(ldg_u16(u + 208));
        int sc = (int)(signed char)__ldg(u + 192 + 8 * n + 2 * gq + (l0 >> 4));
        float ds = d * (float)sc;
        const uint8_t* ql = u + 64 * n + 32 * (gq & 1) + l0;
        const uint8_t* qh = u + 128 + 32 * n + l0;
        uint32_t l_0 = ldg_w(ql), l_1 = ldg_w(ql + 4), h_0 = ldg_w(qh), h_1 = ldg_w(qh + 4);
        const int lsh = (gq >> 1) * 4, hsh = 2 * gq;
        // four 6-bit values per word; (float)q - 32 and its product with d * sc round exactly as d * sc * (q - 32)
        const uint32_t qa = ((l_0 >> lsh) & 0x0F0F0F0Fu) | (((h_0 >> hsh) & 0x03030303u) << 4);
        const uint32_t qb = ((l_1 >> lsh) & 0x0F0F0F0Fu) | (((h_1 >> hsh) & 0x03030303u) << 4);
        v[0] = ds * (byte_to_float<0>(qa) - 32.0f); v[1] = ds * (byte_to_float<1>(qa) - 32.0f);
        v[2] = ds * (byte_to_float<2>(qa) - 32.0f); v[3] = ds * (byte_to_float<3>(qa) - 32.0f);
        v[4] = ds * (byte_to_float<0>(qb) - 32.0f); v[5] = ds * (byte_to_float<1>(qb) - 32.0f);
        v[6] = ds * (byte_to_float<2>(qb) - 32.0f); v[7] = ds * (byte_to_float<3>(qb) - 32.0f);
    }
}

template <int FMT, typename OutT>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ w, OutT* __restrict__ out, size_t nunits,
                                                      int tail_elems) {
    // unit = 256 elements.  The last unit of a Q4_0/Q8_0 tensor may be partial (tail_elems of 256).
    const int lane = threadIdx.x & 31;
    size_t warp = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const size_t nwarps = (size_t)gridDim.x * (blockDim.x >> 5);
    constexpr int UB = fmt_slice_bytes(FMT);
    // two runs per trip: the loads of both are in flight before either is decoded
    for (size_t unit = warp; unit < nunits; unit += 2 * nwarps) {
        const size_t unit2 = unit + nwarps;
        const bool has2 = unit2 < nunits;
        const int valid = (unit + 1 == nunits && tail_elems) ? tail_elems : 256;
        const int valid2 = !has2 ? 0 : (unit2 + 1 == nunits && tail_elems) ? tail_elems : 256;
        // elements come in whole 32-blocks, so 8-lane groups are all-or-nothing
        float v[8], v2[8];
        if (8 * lane < valid) decode8<FMT>(w + unit * UB, lane, v);
        if (8 * lane < valid2) decode8<FMT>(w + unit2 * UB, lane, v2);
        if (8 * lane < valid) store8<OutT>(out + unit * 256 + 8 * lane, v);
        if (8 * lane < valid2) store8<OutT>(out + unit2 * 256 + 8 * lane, v2);
    }
}

template <int FMT>
cudaError_t launch_dequant_fmt(const void* w, size_t nblocks, void* out, int out_dtype, cudaStream_t st, int sm_count) {
    constexpr int per_unit = 256 / fmt_block_size(FMT);
    size_t nunits = (nblocks + per_unit - 1) / per_unit;
    int tail = (int)(nblocks % per_unit) * fmt_block_size(FMT);
    size_t want = (nunits + 7) / 8;
    size_t cap = (size_t)sm_count * 8;  // 8 CTAs of 256 threads per SM keep 64 warps resident
    int grid = (int)(want < cap ? want : cap);
    if (grid < 1) grid = 1;
    const uint8_t* wp = static_cast<const uint8_t*>(w);
    switch (out_dtype) {
    case DT_F32: dequant_kernel<FMT, float><<<grid, 256, 0, st>>>(wp, static_cast<float*>(out), nunits, tail); break;
    case DT_BF16: dequant_kernel<FMT, __nv_bfloat16><<<grid, 256, 0, st>>>(wp, static_cast<__nv_bfloat16*>(out), nunits, tail); break;
    case DT_F16: dequant_kernel<FMT, __half><<<grid, 256, 0, st>>>(wp, static_cast<__half*>(out), nunits, tail); break;
    case DT_F64: dequant_kernel<FMT, double><<<grid, 256, 0, st>>>(wp, static_cast<double*>(out), nunits, tail); break;
    default: return cudaErrorInvalidValue;
    }
    note_launch();
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_dequant(int fmt, const void* w, size_t nblocks, void* out, int out_dtype, cudaStream_t st, int sm_count) {
    switch (fmt) {
    case FMT_Q4_0: return launch_dequant_fmt<FMT_Q4_0>(w, nblocks, out, out_dtype, st, sm_count);
    case FMT_Q8_0: return launch_dequant_fmt<FMT_Q8_0>(w, nblocks, out, out_dtype, st, sm_count);
    case FMT_Q4_K: return launch_dequant_fmt<FMT_Q4_K>(w, nblocks, out, out_dtype, st, sm_count);
    case FMT_Q6_K: return launch_dequant_fmt<FMT_Q6_K>(w, nblocks, out, out_dtype, st, sm_count);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace b200q
