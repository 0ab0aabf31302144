// Quantized matmul for the K-quant formats that have no tuned kernel yet (Q2_K, Q3_K): correct on every shape, not fast.
//
// boostr's CPU path for these formats (src/quant/cpu/kernels/quant_matmul.rs:107-135) quantises each activation row to
// Q8_K (src/quant/cpu/kernels/simd/quantize_act_q8k.rs:26-98) and takes an integer dot product per 256-block
// (src/quant/cpu/kernels/simd/fused_q2k_q8k_dot.rs:152-214, fused_q3k_q8k_dot.rs:33-205 in the form x86-64 runs):
// sumf += (d * d8) * isum - (dmin * d8) * summs (Q3_K: no min term).  The
// integer sums are exact and the blocks are added in K order without FMA contraction, so the result has the CPU's bits.
//
//   * kq_act_prep_kernel: one warp per (activation row, 256-block) writes the Q8_K block in the CPU's own layout
//     (f32 d8 | 256 codes | 16 sums of 16) into caller scratch;
//   * kq_generic_kernel<FMT>: one warp per weight row; a lane owns 8 consecutive elements of every block (codes
//     through two dp4a), block sums leave through warp-wide integer reductions, eight activation rows per pass.
// No barriers, no waits.
#include "common.cuh"

namespace b200q {

namespace {

constexpr uint32_t Q8K_BYTES = 292;  // f32 d8 | 256 x i8 | 16 x i16

template <typename InT>
__global__ void __launch_bounds__(256) kq_act_prep_kernel(const InT* __restrict__ act, uint8_t* __restrict__ img, size_t nruns) {
    const int lane = threadIdx.x & 31;
    for (size_t run = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5); run < nruns; run += (size_t)gridDim.x * 8) {
        float v[8];
        const size_t base = run * 256 + 8 * lane;
        if constexpr (sizeof(InT) == 4) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(act + base)), b = __ldg(reinterpret_cast<const float4*>(act + base) + 1);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
            const uint4 r = __ldg(reinterpret_cast<const uint4*>(act + base));
            v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xFFFF0000u);
            v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xFFFF0000u);
            v[4] = __uint_as_float(r.z << 16); v[5] = __uint_as_float(r.z & 0xFFFF0000u);
            v[6] = __uint_as_float(r.w << 16); v[7] = __uint_as_float(r.w & 0xFFFF0000u);
        }
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
        const float id = amax != 0.f ? __fdiv_rn(127.0f, amax) : 0.f;
        int c[8], s = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            c[i] = max(-128, min(127, __float2int_rn(__fmul_rn(v[i], id))));  // round half to even, as the AVX2 quantiser
            s += c[i];
        }
        uint8_t* blk = img + run * Q8K_BYTES;
        uint32_t w0 = 0, w1 = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            w0 |= (uint32_t)(c[i] & 0xFF) << (8 * i);
            w1 |= (uint32_t)(c[4 + i] & 0xFF) << (8 * i);
        }
        *reinterpret_cast<uint32_t*>(blk + 4 + 8 * lane) = w0;
        *reinterpret_cast<uint32_t*>(blk + 8 + 8 * lane) = w1;
        s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);  // 16 elements = two lanes
        if ((lane & 1) == 0) *reinterpret_cast<short*>(blk + 260 + lane) = (short)s;
        if (lane == 0) *reinterpret_cast<float*>(blk) = __fdiv_rn(amax, 127.0f);
    }
}

struct KqParams {
    const uint8_t* w;
    const uint8_t* img;  // [M][K / 256] Q8_K blocks
    void* out;
    uint32_t M, K, N;
    int out_dtype;
};

// What a lane holds of one weight block: its 8 codes as two words of unsigned bytes, the integer scale and min of
// its 16-wide sub-block, and the block's two f32 scales.
struct LaneBlk {
    uint32_t q0, q1;
    int sc, mn;
    float d, dmin;
};

template <int FMT>
__device__ __forceinline__ LaneBlk load_lane_blk(const uint8_t* blk, int lane);

// Q2_K (src/quant/cpu/kernels/dequant_k_quants/q2k_q3k.rs:13-58): element e = 128 n + 32 g + 16 h + l takes bits
// 2g..2g+1 of byte 32 n + 16 h + l; scale byte e / 16 = low nibble scale, high nibble min.  Blocks are 4-byte aligned
// (84 bytes, rows of whole blocks, 16-byte aligned tensor).
template <>
__device__ __forceinline__ LaneBlk load_lane_blk<FMT_Q2_K>(const uint8_t* blk, int lane) {
    LaneBlk r;
    const int n = lane >> 4, g = (lane >> 2) & 3, h = (lane >> 1) & 1;
    const uint32_t* w = reinterpret_cast<const uint32_t*>(blk + 16 + 32 * n + 16 * h + 8 * (lane & 1));
    r.q0 = (__ldg(w) >> (2 * g)) & 0x03030303u;
    r.q1 = (__ldg(w + 1) >> (2 * g)) & 0x03030303u;
    const uint32_t sc = __ldg(blk + (lane >> 1));
    r.sc = (int)(sc & 15u);
    r.mn = (int)(sc >> 4);
    const uint32_t dm = __ldg(reinterpret_cast<const uint32_t*>(blk + 80));
    r.d = f16bits_to_f32(dm & 0xFFFF);
    r.dmin = f16bits_to_f32(dm >> 16);
    return r;
}

// Q3_K (q2k_q3k.rs:64-144): low two bits as Q2_K from the 64 code bytes at offset 32, the high bit 4 n + g of
// hmask[16 h + l], a clear high bit subtracts 4; sixteen 6-bit scales minus 32, no min term.  Blocks (110 bytes) are only
// 2-byte aligned.  The codes minus 4 leave as signed bytes.
template <>
__device__ __forceinline__ LaneBlk load_lane_blk<FMT_Q3_K>(const uint8_t* blk, int lane) {
    LaneBlk r;
    const int n = lane >> 4, g = (lane >> 2) & 3, h = (lane >> 1) & 1, j = lane >> 1;
    auto w32 = [](const uint8_t* p) {
        const unsigned short* q = reinterpret_cast<const unsigned short*>(p);
        return (uint32_t)__ldg(q) | ((uint32_t)__ldg(q + 1) << 16);
    };
    const uint8_t* qp = blk + 32 + 32 * n + 16 * h + 8 * (lane & 1);
    const uint8_t* hp = blk + 16 * h + 8 * (lane & 1);
    const uint32_t c0 = ((w32(qp) >> (2 * g)) & 0x03030303u) | (((w32(hp) >> (4 * n + g)) & 0x01010101u) << 2);
    const uint32_t c1 = ((w32(qp + 4) >> (2 * g)) & 0x03030303u) | (((w32(hp + 4) >> (4 * n + g)) & 0x01010101u) << 2);
    // per byte c - 4 in two's complement: the set top bit keeps the subtraction inside its byte
    r.q0 = ((c0 | 0x80808080u) - 0x04040404u) ^ 0x80808080u;
    r.q1 = ((c1 | 0x80808080u) - 0x04040404u) ^ 0x80808080u;
    const uint32_t low4 = ((uint32_t)__ldg(blk + 96 + (j & 7)) >> (4 * (j >> 3))) & 15u;
    const uint32_t high2 = ((uint32_t)__ldg(blk + 104 + (j & 3)) >> (2 * (j >> 2))) & 3u;
    r.sc = (int)(low4 | (high2 << 4)) - 32;
    r.mn = 0;
    r.d = f16bits_to_f32(__ldg(reinterpret_cast<const unsigned short*>(blk + 108)));
    r.dmin = 0.f;
    return r;
}

constexpr int KQ_MC = 8;  // activation rows per pass

template <int FMT>
__global__ void __launch_bounds__(256) kq_generic_kernel(const KqParams p) {
    constexpr uint32_t BB = fmt_block_bytes(FMT);
    const int lane = threadIdx.x & 31;
    const uint32_t nblk = p.K / 256;
    const size_t row_bytes = (size_t)nblk * BB;
    const uint32_t warps = gridDim.x * (blockDim.x >> 5);
    for (uint32_t n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); n < p.N; n += warps) {
        const uint8_t* wrow = p.w + (size_t)n * row_bytes;
        for (uint32_t m0 = 0; m0 < p.M; m0 += KQ_MC) {
            float sumf[KQ_MC];
#pragma unroll
            for (int i = 0; i < KQ_MC; ++i) sumf[i] = 0.f;
            for (uint32_t b = 0; b < nblk; ++b) {
                const LaneBlk wb = load_lane_blk<FMT>(wrow + (size_t)b * BB, lane);
#pragma unroll
                for (int i = 0; i < KQ_MC; ++i) {
                    if (m0 + i < p.M) {  // warp-uniform
                        const uint8_t* a = p.img + ((size_t)(m0 + i) * nblk + b) * Q8K_BYTES;
                        const int a0 = (int)__ldg(reinterpret_cast<const uint32_t*>(a + 4 + 8 * lane));
                        const int a1 = (int)__ldg(reinterpret_cast<const uint32_t*>(a + 8 + 8 * lane));
                        const int isuml = __dp4a((int)wb.q1, a1, __dp4a((int)wb.q0, a0, 0));  // codes 0..3 read the same as signed bytes
                        int part = wb.sc * isuml;
                        // the sub-block's sum of 16 activation codes, counted once per sub-block (even lanes)
                        int mpart = (lane & 1) ? 0 : wb.mn * (int)__ldg(reinterpret_cast<const short*>(a + 260 + lane));
                        const int isum = __reduce_add_sync(0xFFFFFFFFu, part);
                        const int summs = __reduce_add_sync(0xFFFFFFFFu, mpart);
                        const float d8 = __ldg(reinterpret_cast<const float*>(a));
                        const float t = __fsub_rn(__fmul_rn(__fmul_rn(wb.d, d8), (float)isum), __fmul_rn(__fmul_rn(wb.dmin, d8), (float)summs));
                        sumf[i] = __fadd_rn(sumf[i], t);
                    }
                }
            }
            if (lane == 0) {
#pragma unroll
                for (int i = 0; i < KQ_MC; ++i) {
                    if (m0 + i < p.M) {
                        const size_t idx = (size_t)(m0 + i) * p.N + n;
                        if (p.out_dtype == DT_F32) static_cast<float*>(p.out)[idx] = sumf[i];
                        else if (p.out_dtype == DT_BF16) static_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(sumf[i]);
                        else static_cast<__half*>(p.out)[idx] = __float2half_rn(sumf[i]);
                    }
                }
            }
        }
    }
}

}  // namespace

bool kq_generic_supported(int fmt, size_t M, size_t K, size_t N) { return (fmt == FMT_Q2_K || fmt == FMT_Q3_K) && M >= 1 && N >= 1 && K % 256 == 0; }

size_t kq_generic_workspace_bytes(size_t M, size_t K) { return (M * (K / 256) * Q8K_BYTES + 255) & ~(size_t)255; }

cudaError_t launch_kq_generic(int fmt, const void* act, int act_dtype, const void* w, void* out, int out_dtype, size_t M, size_t K,
                              size_t N, void* ws, size_t ws_bytes, int sm_count, cudaStream_t st, bool* ws_too_small) {
    *ws_too_small = false;
    const size_t need = kq_generic_workspace_bytes(M, K);
    if (!ws || ws_bytes < need || (reinterpret_cast<uintptr_t>(ws) & 15)) {
        *ws_too_small = true;
        return cudaSuccess;
    }
    const size_t nruns = M * (K / 256);
    int grid = (int)((nruns + 7) / 8);
    if (grid > sm_count * 8) grid = sm_count * 8;
    if (act_dtype == DT_F32) kq_act_prep_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(act), static_cast<uint8_t*>(ws), nruns);
    else kq_act_prep_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(act), static_cast<uint8_t*>(ws), nruns);
    note_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    KqParams p{};
    p.w = static_cast<const uint8_t*>(w);
    p.img = static_cast<const uint8_t*>(ws);
    p.out = out;
    p.M = (uint32_t)M; p.K = (uint32_t)K; p.N = (uint32_t)N;
    p.out_dtype = out_dtype;
    size_t g2 = (N + 7) / 8;
    if (g2 > (size_t)sm_count * 8) g2 = (size_t)sm_count * 8;
    if (fmt == FMT_Q2_K) kq_generic_kernel<FMT_Q2_K><<<(unsigned)g2, 256, 0, st>>>(p);
    else if (fmt == FMT_Q3_K) kq_generic_kernel<FMT_Q3_K><<<(unsigned)g2, 256, 0, st>>>(p);
    else return cudaErrorInvalidValue;
    note_launch();
    return cudaGetLastError();
}

}  // namespace b200q
