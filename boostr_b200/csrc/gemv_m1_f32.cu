// Decode GEMV (M = 1) for Q8_0 and Q4_0: y[n] = sum_k x[k] * W[n,k] with the activation row kept in f32.
//
// boostr's CPU path for these two formats dequantises a weight row and takes an f32 dot product with
// the f32 activations (src/quant/cpu/quant_matmul.rs, dot_f32 in kernels/simd/dot_f32.rs); nothing is
// quantised on the activation side, so the GPU kernel multiplies in f32 too:
//   y = sum_b d_b * sum_{k in b} (q_k - z) * x_k,
// where (q_k - z) is produced exactly from the unsigned byte (q + 128 for Q8_0, the nibble for Q4_0) by one
// byte-permute (byte -> float bit pattern 2^23 + byte, no conversion instruction) and one subtraction of
// 2^23 + 128 (or + 8); an element then costs permute + FADD + FFMA, a block one f16 conversion and one FFMA more.
// The result differs from the CPU loop only in the order of f32 additions.
//
// Streaming structure as in the K-quant decode kernels: persistent CTA per SM, 4 groups of 4 warps,
// group g consumes fills g, g + 4, ... of a ring of small fills (whole rows, contiguous in memory: one
// bulk copy each, rows of any 2-byte alignment), two fills ahead of the grid dependency and the rest
// after the activation loads; a warp takes `rpw` rows of a fill one after the other, lane l the blocks
// l, l + 32, ... of the row.  The activation image in shared memory gives every block 36 floats (32 + 4 of
// padding), so that the lanes' 128-bit reads of different blocks fall into different banks with constant
// offsets.  All waits are bounded.
#include "common.cuh"

namespace b200q {

struct GemvM1F32Params {
    const uint8_t* w;
    const void* act;
    void* out;
    uint32_t K, N;
    uint32_t nblk;          // K / 32
    uint32_t row_bytes;     // nblk * 34 (Q8_0) or nblk * 18 (Q4_0)
    uint32_t rows_per_cta;
    uint32_t rpw;           // rows a warp takes per fill; a fill is 4 * rpw rows
    uint32_t stage_bytes, nstages;
    uint32_t x_off, stage_off;
    uint32_t part_off;      // int8-piece kernel: table of quarter sums, [nstages][rows per fill][4] floats
    int act_dtype, out_dtype;
    unsigned int* status;
};

namespace {

// (byte I of x) - Z as a float, exactly: the permute builds the bit pattern of 2^23 + byte
template <int I>
__device__ __forceinline__ float byte_minus(uint32_t x, float magic_plus_z) {
    return __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7650 | I)) - magic_plus_z;
}

// sum over one 32-element block of (code - Z) * x, and the block's scale.  `blk` is 2-byte aligned in shared
// memory; `xb` points at the block's 32 activations.
template <int FMT>
__device__ __forceinline__ float block_dot(const uint8_t* blk, const float* xb, float& d) {
    constexpr float MZ = 8388608.0f + (FMT == FMT_Q8_0 ? 128.0f : 8.0f);
    // aligned words covering the block: scale in the low or the high half of A[0], data words either
    // aligned from A[1] on (block at 2 mod 4) or straddling A[i], A[i+1] (block at 0 mod 4)
    const uint32_t odd = (uint32_t)(reinterpret_cast<uintptr_t>(blk) & 2);
    const uint32_t* A = reinterpret_cast<const uint32_t*>(blk - odd);
    const uint32_t dsel = odd ? 0x7654u : 0x5432u;  // data word i = bytes of (A[i], A[i+1]) selected by dsel
    uint32_t prev = A[0];
    d = f16bits_to_f32((odd ? prev >> 16 : prev) & 0xFFFFu);
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;  // four independent chains hide the FFMA latency
    if constexpr (FMT == FMT_Q8_0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t next = A[i + 1];
            const uint32_t q = __byte_perm(prev, next, dsel) ^ 0x80808080u;  // q + 128 as unsigned bytes
            prev = next;
            const float4 x = *reinterpret_cast<const float4*>(xb + 4 * i);
            a0 = fmaf(byte_minus<0>(q, MZ), x.x, a0);
            a1 = fmaf(byte_minus<1>(q, MZ), x.y, a1);
            a2 = fmaf(byte_minus<2>(q, MZ), x.z, a2);
            a3 = fmaf(byte_minus<3>(q, MZ), x.w, a3);
        }
    } else {  // Q4_0: byte j holds elements 2 j (low nibble) and 2 j + 1 (high nibble)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t next = A[i + 1];
            const uint32_t w = __byte_perm(prev, next, dsel);
            prev = next;
            const uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
            const float4 x0 = *reinterpret_cast<const float4*>(xb + 8 * i);
            const float4 x1 = *reinterpret_cast<const float4*>(xb + 8 * i + 4);
            a0 = fmaf(byte_minus<0>(lo, MZ), x0.x, a0);
            a1 = fmaf(byte_minus<0>(hi, MZ), x0.y, a1);
            a2 = fmaf(byte_minus<1>(lo, MZ), x0.z, a2);
            a3 = fmaf(byte_minus<1>(hi, MZ), x0.w, a3);
            a0 = fmaf(byte_minus<2>(lo, MZ), x1.x, a0);
            a1 = fmaf(byte_minus<2>(hi, MZ), x1.y, a1);
            a2 = fmaf(byte_minus<3>(lo, MZ), x1.z, a2);
            a3 = fmaf(byte_minus<3>(hi, MZ), x1.w, a3);
        }
    }
    return (a0 + a1) + (a2 + a3);
}

template <int FMT>
__global__ void __launch_bounds__(512, 1) gemv_m1_f32_kernel(const __grid_constant__ GemvM1F32Params p) {
    constexpr uint32_t BB = FMT == FMT_Q8_0 ? 34 : 18;
    constexpr uint32_t XSTRIDE = 36;
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_full = smem_u32(smem), bar_empty = bar_full + 128;
    float* xim = reinterpret_cast<float*>(smem + p.x_off);  // activation image, 36 floats per block
    const uint32_t stage0 = smem_u32(smem + p.stage_off);
    const uint32_t FR = 4 * p.rpw;

    const uint32_t row_begin = blockIdx.x * p.rows_per_cta;
    const uint32_t row_end = min(p.N, row_begin + p.rows_per_cta);
    const uint32_t nfill = row_end > row_begin ? (row_end - row_begin + FR - 1) / FR : 0;

    auto issue_fill = [&](uint32_t f, uint32_t slot) {  // one lane
        const uint32_t r0 = row_begin + f * FR;
        const uint32_t nrows = min(FR, row_end - r0);
        fill_contiguous(stage0 + slot * p.stage_bytes, smem + p.stage_off + slot * p.stage_bytes, p.w + (size_t)r0 * p.row_bytes,
                        nrows * p.row_bytes, p.w + (size_t)p.N * p.row_bytes, bar_full + 8 * slot);
    };

    if (warp == 15 && (uint32_t)lane < p.nstages) {
        mbar_init(bar_full + 8 * lane, 1);
        mbar_init(bar_empty + 8 * lane, 4);
        mbar_fence_init();
    }
    __syncthreads();
    if (warp == 15 && lane < 2 && (uint32_t)lane < nfill) issue_fill(lane, lane);
    grid_dep_launch();
    grid_dep_wait();

    // activation image: thread t takes 8 consecutive values at a time = two chunks of one block
    for (uint32_t e = 8 * threadIdx.x; e < p.K; e += 8 * blockDim.x) {
        float4 a, b;
        if (p.act_dtype == DT_F32) {
            const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(p.act) + e);
            a = __ldg(src);
            b = __ldg(src + 1);
        } else {
            const uint4 r = __ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.act) + e));
            a = make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xFFFF0000u), __uint_as_float(r.y << 16), __uint_as_float(r.y & 0xFFFF0000u));
            b = make_float4(__uint_as_float(r.z << 16), __uint_as_float(r.z & 0xFFFF0000u), __uint_as_float(r.w << 16), __uint_as_float(r.w & 0xFFFF0000u));
        }
        if (e == 8 * threadIdx.x) {  // first trip: the rest of the ring leaves right behind the activation loads
            const uint32_t f1 = 2 + (uint32_t)warp;
            if (lane == 0 && f1 < p.nstages && f1 < nfill) issue_fill(f1, f1);
        }
        float* xb = xim + XSTRIDE * (e >> 5) + (e & 31);
        *reinterpret_cast<float4*>(xb) = a;
        *reinterpret_cast<float4*>(xb + 4) = b;
    }
    if (p.K < 8 * blockDim.x && 8 * threadIdx.x >= p.K) {  // threads without a trip still issue their fill
        const uint32_t f1 = 2 + (uint32_t)warp;
        if (lane == 0 && f1 < p.nstages && f1 < nfill) issue_fill(f1, f1);
    }
    __syncthreads();

    const uint32_t grp = (uint32_t)warp >> 2, wi = (uint32_t)warp & 3;
    bool dead = false;
    uint32_t slot = grp, par = 0;
    for (uint32_t f = grp; f < nfill; f += 4) {
        if (!dead && !mbar_wait(bar_full + 8 * slot, par)) {
            dead = true;
            atomicOr(p.status, STATUS_TIMEOUT_FULL);
        }
        const uint32_t r0 = row_begin + f * FR;
        const uint32_t nrows = min(FR, row_end - r0);
        const uint32_t phase = (uint32_t)((reinterpret_cast<uintptr_t>(p.w) + (size_t)r0 * p.row_bytes) & 15);
        const uint8_t* base = smem + p.stage_off + slot * p.stage_bytes + phase;
        for (uint32_t j = 0; j < p.rpw; ++j) {
            const uint32_t rr = wi * p.rpw + j;
            if (rr >= nrows || dead) break;  // warp-uniform
            const uint8_t* row = base + rr * p.row_bytes;
            float tot = 0.f;
            for (uint32_t b = lane; b < p.nblk; b += 32) {
                float d;
                const float acc = block_dot<FMT>(row + b * BB, xim + XSTRIDE * b, d);
                tot = fmaf(d, acc, tot);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xFFFFFFFFu, tot, o);
            if (lane == 0) {
                const size_t idx = r0 + rr;
                if (p.out_dtype == DT_F32) static_cast<float*>(p.out)[idx] = tot;
                else if (p.out_dtype == DT_BF16) static_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(tot);
                else static_cast<__half*>(p.out)[idx] = __float2half_rn(tot);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + 8 * slot);
        if (f + p.nstages < nfill && ((f >> 2) & 3) == wi) {
            if (!dead && !mbar_wait(bar_empty + 8 * slot, par)) {
                dead = true;
                atomicOr(p.status, STATUS_TIMEOUT_EMPTY);
            }
            if (!dead && lane == 0) issue_fill(f + p.nstages, slot);
        }
        slot += 4;
        if (slot >= p.nstages) {
            slot -= p.nstages;
            par ^= 1;
        }
    }
}


// ------------------------------------------------------------------------------------------------------------------
// The same product with the activation row split into int8 PIECES, for K a multiple of 256: per 256-run of K
//   x = (amax / 127) * (a1 + a2 / 254 + a3 / 254^2),  a_i int8 (relative error ~1e-7 of the run's amax),
// so a block costs 24 dp4a on the weights' own int8 codes instead of 32 x (permute + FADD + FFMA): about half the
// issue slots per weight.  Within 1e-5 of the f32 dot of the CPU path (src/quant/cpu/kernels/quant_matmul.rs:193-209),
// the same bar as the f32 kernel above, which stays for rows that are not whole 256-runs.
constexpr uint32_t XB_I8 = 112;  // bytes per 32-block of the image: 3 pieces x 32 codes, 3 block sums; 7 x 16 B keeps lanes' 16-byte reads conflict-free

// The aligned words covering one 32-block of a row (2-byte aligned in shared memory): loaded first for several rows,
// so that their latencies overlap, then multiplied.
template <int FMT>
struct RawBlk {
    uint32_t a[FMT == FMT_Q8_0 ? 9 : 5];
    uint32_t odd;
};
template <int FMT>
__device__ __forceinline__ void load_blk(const uint8_t* blk, RawBlk<FMT>& r) {
    r.odd = (uint32_t)(reinterpret_cast<uintptr_t>(blk) & 2);
    const uint32_t* A = reinterpret_cast<const uint32_t*>(blk - r.odd);
#pragma unroll
    for (int i = 0; i < (FMT == FMT_Q8_0 ? 9 : 5); ++i) r.a[i] = A[i];
}
// One 32-block against the lane's own activation block held in registers: x[6] = three pieces of 32 codes (Q4_0: even
// elements then odd elements within a piece), bs = the pieces' block sums.
template <int FMT>
__device__ __forceinline__ float block_dot_i8(const RawBlk<FMT>& r, const uint4 (&x)[6], const uint4& bs, float xs) {
    const uint32_t dsel = r.odd ? 0x7654u : 0x5432u;
    const float d = f16bits_to_f32((r.odd ? r.a[0] >> 16 : r.a[0]) & 0xFFFFu);
    int s0, s1, s2;
    auto dot4 = [](const uint32_t* w, const uint4& a, int acc) {
        acc = __dp4a((int)w[0], (int)a.x, acc);
        acc = __dp4a((int)w[1], (int)a.y, acc);
        acc = __dp4a((int)w[2], (int)a.z, acc);
        return __dp4a((int)w[3], (int)a.w, acc);
    };
    if constexpr (FMT == FMT_Q8_0) {
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = __byte_perm(r.a[i], r.a[i + 1], dsel);
        // two chains of four per piece, so six independent dp4a chains
        s0 = dot4(w, x[0], 0) + dot4(w + 4, x[1], 0);
        s1 = dot4(w, x[2], 0) + dot4(w + 4, x[3], 0);
        s2 = dot4(w, x[4], 0) + dot4(w + 4, x[5], 0);
    } else {
        // Q4_0: byte j = elements 2 j (low nibble), 2 j + 1 (high): low-nibble words meet the even codes of a piece,
        // high-nibble words the odd ones; q - 8 through the block sums of the pieces
        uint32_t lo[4], hi[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t w = __byte_perm(r.a[i], r.a[i + 1], dsel);
            lo[i] = w & 0x0F0F0F0Fu;
            hi[i] = (w >> 4) & 0x0F0F0F0Fu;
        }
        s0 = dot4(lo, x[0], 0) + dot4(hi, x[1], 0) - 8 * (int)bs.x;
        s1 = dot4(lo, x[2], 0) + dot4(hi, x[3], 0) - 8 * (int)bs.y;
        s2 = dot4(lo, x[4], 0) + dot4(hi, x[5], 0) - 8 * (int)bs.z;
    }
    constexpr float C1 = 1.0f / 254.0f;
    const float f = fmaf(fmaf((float)s2, C1, (float)s1), C1, (float)s0);
    return __fmul_rn(d, xs) * f;
}

// NB: blocks of its quarter of the row a lane holds (1 up to K = 4096, 2 up to 8192)
template <int FMT, int NB>
__global__ void __launch_bounds__(512, 1) gemv_m1_i8_kernel(const __grid_constant__ GemvM1F32Params p) {
    constexpr uint32_t BB = FMT == FMT_Q8_0 ? 34 : 18;
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_full = smem_u32(smem), bar_empty = bar_full + 128;
    float* xscale = reinterpret_cast<float*>(smem + p.x_off);                  // one scale per 256-run
    uint8_t* xim = smem + p.x_off + ((p.K / 256 * 4 + 15) & ~15u);             // the piece image, XB_I8 bytes per block
    const uint32_t stage0 = smem_u32(smem + p.stage_off);
    const uint32_t FR = 4 * p.rpw;

    const uint32_t row_begin = blockIdx.x * p.rows_per_cta;
    const uint32_t row_end = min(p.N, row_begin + p.rows_per_cta);
    const uint32_t nfill = row_end > row_begin ? (row_end - row_begin + FR - 1) / FR : 0;

    auto issue_fill = [&](uint32_t f, uint32_t slot) {  // one lane
        const uint32_t r0 = row_begin + f * FR;
        const uint32_t nrows = min(FR, row_end - r0);
        fill_contiguous(stage0 + slot * p.stage_bytes, smem + p.stage_off + slot * p.stage_bytes, p.w + (size_t)r0 * p.row_bytes,
                        nrows * p.row_bytes, p.w + (size_t)p.N * p.row_bytes, bar_full + 8 * slot);
    };

    if (warp == 15 && (uint32_t)lane < p.nstages) {
        mbar_init(bar_full + 8 * lane, 1);
        mbar_init(bar_empty + 8 * lane, 4);
        mbar_fence_init();
    }
    __syncthreads();
    if (warp == 15 && lane < 2 && (uint32_t)lane < nfill) issue_fill(lane, lane);
    grid_dep_launch();
    grid_dep_wait();

    // the piece image: a warp takes one 256-run per trip (8 values per lane), so the run's amax is a warp reduction
    for (uint32_t e = 8 * threadIdx.x; e < p.K; e += 8 * blockDim.x) {
        float v[8];
        if (p.act_dtype == DT_F32) {
            const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(p.act) + e);
            const float4 a = __ldg(src), b = __ldg(src + 1);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
            const uint4 r = __ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.act) + e));
            v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xFFFF0000u);
            v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xFFFF0000u);
            v[4] = __uint_as_float(r.z << 16); v[5] = __uint_as_float(r.z & 0xFFFF0000u);
            v[6] = __uint_as_float(r.w << 16); v[7] = __uint_as_float(r.w & 0xFFFF0000u);
        }
        if (e == 8 * threadIdx.x) {  // first trip: the rest of the ring leaves right behind the activation loads
            const uint32_t f1 = 2 + (uint32_t)warp;
            if (lane == 0 && f1 < p.nstages && f1 < nfill) issue_fill(f1, f1);
        }
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
        const float id = amax != 0.f ? __fdiv_rn(127.0f, amax) : 0.f;
        int c[3][8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float r = __fmul_rn(v[i], id);
#pragma unroll
            for (int pc = 0; pc < 3; ++pc) {
                c[pc][i] = max(-127, min(127, (int)rintf(r)));
                r = __fmul_rn(__fsub_rn(r, (float)c[pc][i]), 254.0f);  // remainder in [-0.5, 0.5] -> [-127, 127]
            }
        }
        uint8_t* blk = xim + XB_I8 * (e >> 5);
        const uint32_t off = e & 31;  // 0, 8, 16 or 24
        int bsum[3];
#pragma unroll
        for (int pc = 0; pc < 3; ++pc) {
            auto pk = [&](int a, int b, int cc, int dd) {
                return (uint32_t)(c[pc][a] & 0xFF) | ((uint32_t)(c[pc][b] & 0xFF) << 8) | ((uint32_t)(c[pc][cc] & 0xFF) << 16) | ((uint32_t)(c[pc][dd] & 0xFF) << 24);
            };
            if constexpr (FMT == FMT_Q8_0) {
                *reinterpret_cast<uint2*>(blk + 32 * pc + off) = make_uint2(pk(0, 1, 2, 3), pk(4, 5, 6, 7));
            } else {
                *reinterpret_cast<uint32_t*>(blk + 32 * pc + off / 2) = pk(0, 2, 4, 6);
                *reinterpret_cast<uint32_t*>(blk + 32 * pc + 16 + off / 2) = pk(1, 3, 5, 7);
            }
            int t = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) t += c[pc][i];
            t += __shfl_xor_sync(0xFFFFFFFFu, t, 1);
            t += __shfl_xor_sync(0xFFFFFFFFu, t, 2);
            bsum[pc] = t;
        }
        if ((lane & 3) == 0) *reinterpret_cast<uint4*>(blk + 96) = make_uint4((uint32_t)bsum[0], (uint32_t)bsum[1], (uint32_t)bsum[2], 0u);
        if (lane == 0) xscale[e >> 8] = __fdiv_rn(amax, 127.0f);
    }
    if (p.K < 8 * blockDim.x && 8 * threadIdx.x >= p.K) {  // threads without a trip still issue their fill
        const uint32_t f1 = 2 + (uint32_t)warp;
        if (lane == 0 && f1 < p.nstages && f1 < nfill) issue_fill(f1, f1);
    }
    __syncthreads();

    // The four warps of a group share every row of a fill: warp wi takes the wi-th quarter of the row's blocks, a lane
    // the same block positions of every row, so its activation pieces stay in registers for the whole launch (with
    // the image read from shared memory per block, the kernel was bound by shared-memory bandwidth: 96 bytes of
    // activations per 34 bytes of weights).  Quarter sums meet in a small table; the warp that refills the slot adds them.
    const uint32_t grp = (uint32_t)warp >> 2, wi = (uint32_t)warp & 3;
    const uint32_t cb = p.nblk / 4;  // blocks per quarter (K is a multiple of 256, so nblk is a multiple of 8)
    uint4 xr[NB][6], xbs[NB];
    float xsc[NB];
    bool have[NB];
#pragma unroll
    for (int j = 0; j < NB; ++j) {
        const uint32_t bl = (uint32_t)lane + 32 * j;
        have[j] = bl < cb;
        const uint32_t b = wi * cb + (have[j] ? bl : 0);
        const uint4* X = reinterpret_cast<const uint4*>(xim + XB_I8 * b);
#pragma unroll
        for (int i = 0; i < 6; ++i) xr[j][i] = X[i];
        xbs[j] = X[6];
        xsc[j] = xscale[b >> 3];
    }
    float* part = reinterpret_cast<float*>(smem + p.part_off);  // [slot][row of the fill][quarter]
    bool dead = false;
    uint32_t slot = grp, par = 0;
    for (uint32_t f = grp; f < nfill; f += 4) {
        if (!dead && !mbar_wait(bar_full + 8 * slot, par)) {
            dead = true;
            atomicOr(p.status, STATUS_TIMEOUT_FULL);
        }
        const uint32_t r0 = row_begin + f * FR;
        const uint32_t nrows = min(FR, row_end - r0);
        const uint32_t phase = (uint32_t)((reinterpret_cast<uintptr_t>(p.w) + (size_t)r0 * p.row_bytes) & 15);
        const uint8_t* base = smem + p.stage_off + slot * p.stage_bytes + phase + (size_t)wi * cb * BB;
        // four rows at a time: a row's chain (shared loads, dp4a chains, conversions, five dependent shuffles) is some
        // 500 cycles long, and independent rows are the only parallelism a warp has (a fill holds a multiple of four)
        for (uint32_t rr = 0; rr < nrows && !dead; rr += 4) {
            float tot[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                RawBlk<FMT> raw[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)  // rows past the fill's last read stale bytes of the stage; never used
                    load_blk<FMT>(base + (rr + u) * p.row_bytes + (have[j] ? (uint32_t)lane + 32 * j : 0u) * BB, raw[u]);
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (have[j] && rr + u < nrows) tot[u] += block_dot_i8<FMT>(raw[u], xr[j], xbs[j], xsc[j]);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int u = 0; u < 4; ++u) tot[u] += __shfl_xor_sync(0xFFFFFFFFu, tot[u], o);
            if (lane == 0) {
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (rr + u < nrows) part[(slot * FR + rr + u) * 4 + wi] = tot[u];
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + 8 * slot);
        // one warp of the group (they take turns) waits for its siblings, adds the quarter sums in K order, stores
        // the rows and refills the slot
        if (((f >> 2) & 3) == wi) {
            if (!dead && !mbar_wait(bar_empty + 8 * slot, par)) {
                dead = true;
                atomicOr(p.status, STATUS_TIMEOUT_EMPTY);
            }
            for (uint32_t rr = lane; rr < nrows && !dead; rr += 32) {
                const float4 q = *reinterpret_cast<const float4*>(part + (slot * FR + rr) * 4);
                const float tot = __fadd_rn(__fadd_rn(__fadd_rn(q.x, q.y), q.z), q.w);
                const size_t idx = r0 + rr;
                if (p.out_dtype == DT_F32) static_cast<float*>(p.out)[idx] = tot;
                else if (p.out_dtype == DT_BF16) static_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(tot);
                else static_cast<__half*>(p.out)[idx] = __float2half_rn(tot);
            }
            __syncwarp();
            if (!dead && f + p.nstages < nfill && lane == 0) issue_fill(f + p.nstages, slot);
        }
        slot += 4;
        if (slot >= p.nstages) {
            slot -= p.nstages;
            par ^= 1;
        }
    }
}

}  // namespace

bool gemv_m1_f32_supported(int fmt, size_t M, size_t K, size_t N) {
    return M == 1 && N >= 1 && (fmt == FMT_Q8_0 || fmt == FMT_Q4_0) && K % 32 == 0 && K >= 32 && K <= 8192;
}

cudaError_t launch_gemv_m1_f32(int fmt, const void* act, int act_dtype, const void* w, void* out, int out_dtype, size_t K,
                               size_t N, int sm_count, cudaStream_t st, unsigned int* status) {
    constexpr size_t SMEM_MAX = 232448 - 1024;
    GemvM1F32Params p{};
    p.w = static_cast<const uint8_t*>(w);
    p.act = act;
    p.out = out;
    p.K = (uint32_t)K;
    p.N = (uint32_t)N;
    p.nblk = (uint32_t)(K / 32);
    p.row_bytes = p.nblk * (fmt == FMT_Q8_0 ? 34u : 18u);
    p.rpw = 18432 / (4 * p.row_bytes);  // fills of about 18 KB
    if (p.rpw < 1) p.rpw = 1;
    if (p.rpw > 16) p.rpw = 16;
    p.stage_bytes = (4 * p.rpw * p.row_bytes + 32 + 127) & ~127u;  // + phase of an unaligned first row + round-up
    p.x_off = 256;
    const bool pieces = K % 256 == 0;  // int8 activation pieces per 256-run; ragged rows keep the f32 image
    p.part_off = (uint32_t)((p.x_off + ((K / 256 * 4 + 15) & ~(size_t)15) + p.nblk * XB_I8 + 15) & ~(size_t)15);
    p.stage_off = pieces ? (p.part_off + 16 * 4 * p.rpw * 16 + 127) & ~127u : (p.x_off + p.nblk * 36 * 4 + 127) & ~127u;
    p.nstages = (uint32_t)((SMEM_MAX - p.stage_off - 64) / p.stage_bytes);
    if (p.nstages > 16) p.nstages = 16;
    size_t grid = (N + 15) / 16;
    if (grid > (size_t)sm_count) grid = sm_count;
    p.rows_per_cta = (uint32_t)((N + grid - 1) / grid);
    grid = (N + p.rows_per_cta - 1) / p.rows_per_cta;
    p.act_dtype = act_dtype;
    p.out_dtype = out_dtype;
    p.status = status;
    const size_t smem = p.stage_off + (size_t)p.nstages * p.stage_bytes + 64;
    static PerDeviceOnce attrs;
    cudaError_t ae = attrs.run([] {
        cudaError_t e = cudaFuncSetAttribute(gemv_m1_f32_kernel<FMT_Q8_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_m1_f32_kernel<FMT_Q4_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_m1_i8_kernel<FMT_Q8_0, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_m1_i8_kernel<FMT_Q4_0, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_m1_i8_kernel<FMT_Q8_0, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_m1_i8_kernel<FMT_Q4_0, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_MAX);
        return e;
    });
    if (ae != cudaSuccess) return ae;
    cudaError_t le;
    if (pieces && p.nblk / 4 <= 32)
        le = fmt == FMT_Q8_0 ? launch_pdl(gemv_m1_i8_kernel<FMT_Q8_0, 1>, dim3((unsigned)grid), dim3(512), smem, st, p)
                             : launch_pdl(gemv_m1_i8_kernel<FMT_Q4_0, 1>, dim3((unsigned)grid), dim3(512), smem, st, p);
    else if (pieces)
        le = fmt == FMT_Q8_0 ? launch_pdl(gemv_m1_i8_kernel<FMT_Q8_0, 2>, dim3((unsigned)grid), dim3(512), smem, st, p)
                             : launch_pdl(gemv_m1_i8_kernel<FMT_Q4_0, 2>, dim3((unsigned)grid), dim3(512), smem, st, p);
    else
        le = fmt == FMT_Q8_0 ? launch_pdl(gemv_m1_f32_kernel<FMT_Q8_0>, dim3((unsigned)grid), dim3(512), smem, st, p)
                             : launch_pdl(gemv_m1_f32_kernel<FMT_Q4_0>, dim3((unsigned)grid), dim3(512), smem, st, p);
    note_launch();
    return le != cudaSuccess ? le : cudaGetLastError();
}

}  // namespace b200q
