// Memory-bound quantized small-M kernel (2 <= M <= 16 per pass, and every M = 1 shape the decode kernels do
// not take) for Q4_0, Q8_0, Q4_K, Q6_K.
//
// Stands in for boostr's quant_gemv_*_q8_1_mwr / quant_gemv_*_f32 / fused_swiglu_*_mwr kernels
// (src/quant/cuda/kernels/quant_gemv.cu:43-1215) and its separate activation-quantise launch
// (src/quant/cuda/kernels/quant_act.cu:17-69).
//
// Shape of the kernels
//   * act_prep_kernel: ONE small launch per call turns the activations into the "image" the main kernel
//     multiplies with: for every 256-wide run of K ("slice") and every tile of 8 activation rows, the
//     tensor-core B fragments of all 32 lanes, stored so that a warp fetches them with 16-byte loads.
//     Q4_K / Q6_K: the run quantised to Q8_K exactly as boostr's CPU path does (amax/127 scale,
//     round-half-even, src/quant/cpu/kernels/simd/quantize_act_q8k.rs:26-98) plus the 32-wide block
//     sums the Q4_K min term needs.  Q4_0 / Q8_0 (f32 activations on the CPU path,
//     src/quant/cpu/kernels/quant_matmul.rs:193-209): each value as a sum of int8 pieces
//     x = (amax/127) * (a1 + a2/254 + a3/254^2): three pieces for M <= 8 (relative error ~1e-7 of the
//     run's amax), two for M 9..16 per pass (~3e-5), so the weights' int8 codes go to the tensor cores
//     unconverted.
//   * gemv_kernel: persistent CTAs, one per SM, 16 warps.  A warp owns one slice of a K-chunk of up to 16
//     slices and keeps that slice's fragments for one or two 8-row tiles in registers for the whole
//     launch, so the only shared-memory traffic in the loop is the packed weights.  Slabs of 16 weight
//     rows per warp row-group stream through a ring of stages filled by bulk copies (cp.async.bulk +
//     mbarrier byte counts); the warps take turns requesting the refill of the stage they have just
//     released.  There is no block-wide barrier in the steady state: stages and per-slab partial sums
//     are handed over through mbarriers and warps drift apart freely.
//   * Dot products are mma.sync int8 (16 weight rows x 8 activation rows x 32 K per instruction).
//     Q4_K / Q6_K integer sums are exact and each block contributes (d*d8)*sumi - (dmin*d8)*sumi_mins
//     without FMA contraction (fused_q4k_q8k_dot.rs:111-172, fused_q6k_q8k_dot.rs:170-224); blocks are
//     added in K order, so for K <= 4096 the result is bit-identical to the CPU path.  Q4_0 / Q8_0: the
//     accumulator starts at the bit pattern of 1.5 * 2^23, so the finished integer sum is read as a float
//     without a conversion instruction, the pieces are combined in f32 and scaled by the block's d.
//   * When K is too long for one CTA's registers (K > 16 slices * chunks-per-CTA) the K-chunks are
//     spread over gridDim.y and a second small kernel adds the partials in K order.
#include "common.cuh"
#include "tmap.cuh"

namespace b200q {

struct GemvParams {
    const uint8_t* w[2];  // [1] = up-projection weight in SwiGLU mode
    const void* act;
    void* out;
    const uint4* img;     // activation image written by act_prep_kernel: [slice][tile][vector][lane]
    float* partial;       // [nmat][ksplit][M][N] f32 when ksplit > 1
    uint32_t M, K, N;
    uint32_t m0;          // first activation row of this launch
    uint32_t mcount;      // activation rows handled by this launch (<= 8*MT)
    uint32_t tiles_total; // 8-row tiles in the image (ceil(M / 8))
    uint32_t row_bytes;
    uint32_t nslices;     // ceil(K / 256)
    uint32_t spc;         // slices per chunk (<= 16) == compute warps per row group
    uint32_t nchunks;     // ceil(nslices / spc)
    uint32_t ksplit;      // gridDim.y
    uint32_t rgs;         // 16-row groups per slab
    uint32_t srow;        // shared-memory row stride (bytes, multiple of 16, odd multiple of 16)
    uint32_t stage_bytes;
    uint32_t nstages;
    uint32_t total_units; // slabs
    uint32_t red_off;     // byte offset of the reduction ring in dynamic smem
    uint32_t red_slot_bytes;
    uint32_t red_slots;   // slots in the reduction ring (3 or 4)
    uint32_t stage_off;   // byte offset of stage 0
    uint32_t rows_aligned;  // 1 when every row chunk starts and ends on a 16-byte boundary
    // Tiled fills: the packed weights are described to the copy engine as a 3-D tensor
    // [row_bytes / tma_w columns][N rows][tma_w bytes]; ONE copy brings the tma_cb columns of a K-chunk for all
    // rows of a slab and lays them out column by column, [tma_cb][rows per slab][tma_w].  tma_w is a whole number
    // of slices chosen so that consecutive rows (tma_w bytes apart) start in different shared-memory banks.
    uint32_t use_tma;
    uint32_t tma_w, tma_cb;
    int act_dtype, out_dtype;
    unsigned long long w_bytes;  // bytes of each weight tensor
    unsigned int* status;        // device status word (bounded-wait timeouts)
};

namespace {

constexpr int MAX_STAGES = 8;

// ---------------------------------------------------------------- activation access

__device__ __forceinline__ void load_act8(const void* act, int dt, size_t idx, float (&v)[8]) {
    if (dt == DT_F32) {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(act) + idx);
        float4 a = __ldg(p), b = __ldg(p + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        uint4 r = __ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(act) + idx));
        v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xFFFF0000u);
        v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xFFFF0000u);
        v[4] = __uint_as_float(r.z << 16); v[5] = __uint_as_float(r.z & 0xFFFF0000u);
        v[6] = __uint_as_float(r.w << 16); v[7] = __uint_as_float(r.w & 0xFFFF0000u);
    }
}
__device__ __forceinline__ void load_act4(const void* act, int dt, size_t idx, float (&v)[4]) {
    if (dt == DT_F32) {
        float4 a = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(act) + idx));
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    } else {
        uint2 r = __ldg(reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(act) + idx));
        v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xFFFF0000u);
        v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xFFFF0000u);
    }
}

// Q8_K code of one activation: rint(x * id) clamped to [-128, 127] (round half to even).
__device__ __forceinline__ int q8k_code(float x, float id) {
    int q = __float2int_rn(__fmul_rn(x, id));
    return max(-128, min(127, q));
}
__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
    return (uint32_t)(a & 0xFF) | ((uint32_t)(b & 0xFF) << 8) | ((uint32_t)(c & 0xFF) << 16) | ((uint32_t)(d & 0xFF) << 24);
}
__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, 2));
}
__device__ __forceinline__ int quad_sum(int v) {
    v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
    return v + __shfl_xor_sync(0xFFFFFFFFu, v, 2);
}

// ------------------------------------------------------------------ per-format state
//
// Lane naming follows the MMA fragment layout: g = lane / 4 (weight row within the 16-row
// group, and activation row within an 8-row tile), t = lane % 4 (position along K).

// Every format has two types:
//   TileB<FMT, P>      the fragments of ONE (slice, 8-row tile): built from the activations by the prep
//                      kernel (build), written to / read from the image (store / load);
//   SliceB<FMT, MT, P> what a warp of the main kernel keeps: MT tiles of its slice.
// P = number of int8 pieces per activation value (Q4_0 / Q8_0 only; 0 for the K-quants).
// Image layout of one (slice, tile): NV 16-byte vectors per lane, vector v of lane l at index v * 32 + l.

struct PrepParams {
    const void* act;
    uint4* img;
    uint32_t M, K;
    uint32_t nslices, tiles_total;
    int act_dtype;
};

template <int FMT, int P>
struct TileB;

// ---- Q4_K: int8 activations; sub-block j (32 wide) uses elements 8t..8t+7 of the lane ----
template <int P>
struct TileB<FMT_Q4_K, P> {
    static constexpr int NV = 5;
    uint32_t q[16];   // [2*j + half]: k32 B fragment of sub-block j
    uint32_t bs_lo;   // bytes: (bsum_j + 4096) & 127 for j = 4t..4t+3 (t < 2), else 0
    uint32_t bs_hi;   // bytes: (bsum_j + 4096) >> 7
    float d8[2];      // Q8_K scale of activation rows 2t, 2t+1 of the tile

    // rows = activation rows of this tile that exist (rows beyond it count as zero)
    __device__ __forceinline__ void build(const PrepParams& p, uint32_t slice, uint32_t m_first, uint32_t rows, int g, int t) {
        const bool on = (uint32_t)g < rows;
        const size_t base = (size_t)(m_first + g) * p.K + (size_t)slice * 256 + 8 * t;
        // one round of loads: the lane's 64 activations stay in registers for both passes
        float v[8][8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (on) load_act8(p.act, p.act_dtype, base + 32 * j, v[j]);
            else
#pragma unroll
                for (int i = 0; i < 8; ++i) v[j][i] = 0.f;
        }
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[j][i]));
        amax = quad_max(amax);
        float d = __fdiv_rn(amax, 127.0f);
        float id = amax != 0.f ? __fdiv_rn(127.0f, amax) : 0.f;
        uint32_t lo[2] = {0, 0}, hi[2] = {0, 0};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int c[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) c[i] = q8k_code(v[j][i], id);
            q[2 * j] = pack4(c[0], c[1], c[2], c[3]);
            q[2 * j + 1] = pack4(c[4], c[5], c[6], c[7]);
            int bsum = quad_sum(c[0] + c[1] + c[2] + c[3] + c[4] + c[5] + c[6] + c[7]) + 4096;
            lo[j >> 2] |= (uint32_t)(bsum & 127) << (8 * (j & 3));
            hi[j >> 2] |= (uint32_t)(bsum >> 7) << (8 * (j & 3));
        }
        bs_lo = !on ? 0u : t == 0 ? lo[0] : t == 1 ? lo[1] : 0u;
        bs_hi = !on ? 0u : t == 0 ? hi[0] : t == 1 ? hi[1] : 0u;
        float dd = on ? d : 0.f;
        d8[0] = __shfl_sync(0xFFFFFFFFu, dd, (2 * t) * 4);
        d8[1] = __shfl_sync(0xFFFFFFFFu, dd, (2 * t + 1) * 4);
    }
    __device__ __forceinline__ void store(uint4* dst, int lane) const {
#pragma unroll
        for (int v = 0; v < 4; ++v) dst[v * 32 + lane] = make_uint4(q[4 * v], q[4 * v + 1], q[4 * v + 2], q[4 * v + 3]);
        dst[4 * 32 + lane] = make_uint4(bs_lo, bs_hi, __float_as_uint(d8[0]), __float_as_uint(d8[1]));
    }
    __device__ __forceinline__ void load(const uint4* src, int lane) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            const uint4 x = __ldg(src + v * 32 + lane);
            q[4 * v] = x.x; q[4 * v + 1] = x.y; q[4 * v + 2] = x.z; q[4 * v + 3] = x.w;
        }
        const uint4 x = __ldg(src + 4 * 32 + lane);
        bs_lo = x.x; bs_hi = x.y; d8[0] = __uint_as_float(x.z); d8[1] = __uint_as_float(x.w);
    }
};

// Q5_K multiplies in the same order as Q4_K (see slice_q4k): the same fragments and block sums
template <int P>
struct TileB<FMT_Q5_K, P> : TileB<FMT_Q4_K, P> {};

// ---- Q6_K: int8 activations; sub-block sb (16 wide) uses elements 4t..4t+3 ----
template <int P>
struct TileB<FMT_Q6_K, P> {
    static constexpr int NV = 5;
    uint32_t q[16];  // [sb]: k16 B fragment of 16-wide sub-block sb
    float d8[2];

    __device__ __forceinline__ void build(const PrepParams& p, uint32_t slice, uint32_t m_first, uint32_t rows, int g, int t) {
        const bool on = (uint32_t)g < rows;
        const size_t base = (size_t)(m_first + g) * p.K + (size_t)slice * 256 + 4 * t;
        float v[16][4];
#pragma unroll
        for (int sb = 0; sb < 16; ++sb) {
            if (on) load_act4(p.act, p.act_dtype, base + 16 * sb, v[sb]);
            else
#pragma unroll
                for (int i = 0; i < 4; ++i) v[sb][i] = 0.f;
        }
        float amax = 0.f;
#pragma unroll
        for (int sb = 0; sb < 16; ++sb)
#pragma unroll
            for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fabsf(v[sb][i]));
        amax = quad_max(amax);
        float d = __fdiv_rn(amax, 127.0f);
        float id = amax != 0.f ? __fdiv_rn(127.0f, amax) : 0.f;
#pragma unroll
        for (int sb = 0; sb < 16; ++sb)
            q[sb] = pack4(q8k_code(v[sb][0], id), q8k_code(v[sb][1], id), q8k_code(v[sb][2], id), q8k_code(v[sb][3], id));
        float dd = on ? d : 0.f;
        d8[0] = __shfl_sync(0xFFFFFFFFu, dd, (2 * t) * 4);
        d8[1] = __shfl_sync(0xFFFFFFFFu, dd, (2 * t + 1) * 4);
    }
    __device__ __forceinline__ void store(uint4* dst, int lane) const {
#pragma unroll
        for (int v = 0; v < 4; ++v) dst[v * 32 + lane] = make_uint4(q[4 * v], q[4 * v + 1], q[4 * v + 2], q[4 * v + 3]);
        dst[4 * 32 + lane] = make_uint4(__float_as_uint(d8[0]), __float_as_uint(d8[1]), 0u, 0u);
    }
    __device__ __forceinline__ void load(const uint4* src, int lane) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            const uint4 x = __ldg(src + v * 32 + lane);
            q[4 * v] = x.x; q[4 * v + 1] = x.y; q[4 * v + 2] = x.z; q[4 * v + 3] = x.w;
        }
        const uint4 x = __ldg(src + 4 * 32 + lane);
        d8[0] = __uint_as_float(x.x); d8[1] = __uint_as_float(x.y);
    }
};

// ---- Q8_0 / Q4_0: every activation as P int8 pieces, x = (amax/127) * (a1 + a2/254 [+ a3/254^2]) ----
// K order inside a 32-block follows what the weight side reads without shuffling bytes:
//   Q8_0: the lane's two code words are bytes 4t..4t+3 and 16+4t..16+4t+3
//         -> k-slots 4t..4t+3 = elements 4t..4t+3, k-slots 16+4t.. = elements 16+4t..16+4t+3
//   Q4_0: byte i of the lane's word (bytes 4t..4t+3) holds elements 8t+2i (low nibble) and 8t+2i+1 (high nibble)
//         -> k-slots 4t..4t+3 = elements 8t+{0,2,4,6}, k-slots 16+4t.. = elements 8t+{1,3,5,7}
constexpr float PIECE_STEP = 254.0f;
template <int FMT, int P>
struct TileBI8 {
    static constexpr int NV = 4 * P + 1;
    uint32_t q[8][P][2];  // [block][piece][{b0, b1}]
    float scale[2];       // amax / 127 of activation rows 2t, 2t+1 of the tile (this slice)

    __device__ __forceinline__ void build(const PrepParams& p, uint32_t slice, uint32_t m_first, uint32_t rows, int g, int t) {
        const bool on = (uint32_t)g < rows;
        const uint32_t kleft = p.K - slice * 256;  // elements of this slice that exist (ragged last slice)
        const size_t base = (size_t)(m_first + g) * p.K + (size_t)slice * 256 + (FMT == FMT_Q8_0 ? 4 : 8) * t;
        float v[8][8];
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            if (on && 32u * b < kleft) {
                if constexpr (FMT == FMT_Q8_0) {
                    float lo4[4], hi4[4];
                    load_act4(p.act, p.act_dtype, base + 32 * b, lo4);
                    load_act4(p.act, p.act_dtype, base + 32 * b + 16, hi4);
#pragma unroll
                    for (int i = 0; i < 4; ++i) { v[b][i] = lo4[i]; v[b][4 + i] = hi4[i]; }
                } else {
                    load_act8(p.act, p.act_dtype, base + 32 * b, v[b]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[b][i] = 0.f;
            }
        }
        float amax = 0.f;
#pragma unroll
        for (int b = 0; b < 8; ++b)
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[b][i]));
        amax = quad_max(amax);
        const float id = amax != 0.f ? __fdiv_rn(127.0f, amax) : 0.f;
        constexpr int O8[8] = {0, 1, 2, 3, 4, 5, 6, 7};
        constexpr int O4[8] = {0, 2, 4, 6, 1, 3, 5, 7};
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            int c[P][8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float r = __fmul_rn(v[b][i], id);  // |r| <= 127 (+ one rounding)
#pragma unroll
                for (int pc = 0; pc < P; ++pc) {
                    const float a = rintf(r);
                    c[pc][i] = max(-127, min(127, (int)a));
                    r = __fmul_rn(__fsub_rn(r, (float)c[pc][i]), PIECE_STEP);  // remainder in [-0.5, 0.5] -> [-127, 127]
                }
            }
#pragma unroll
            for (int pc = 0; pc < P; ++pc) {
                if constexpr (FMT == FMT_Q8_0) {
                    q[b][pc][0] = pack4(c[pc][O8[0]], c[pc][O8[1]], c[pc][O8[2]], c[pc][O8[3]]);
                    q[b][pc][1] = pack4(c[pc][O8[4]], c[pc][O8[5]], c[pc][O8[6]], c[pc][O8[7]]);
                } else {
                    q[b][pc][0] = pack4(c[pc][O4[0]], c[pc][O4[1]], c[pc][O4[2]], c[pc][O4[3]]);
                    q[b][pc][1] = pack4(c[pc][O4[4]], c[pc][O4[5]], c[pc][O4[6]], c[pc][O4[7]]);
                }
            }
        }
        const float sc = on ? __fdiv_rn(amax, 127.0f) : 0.f;
        scale[0] = __shfl_sync(0xFFFFFFFFu, sc, (2 * t) * 4);
        scale[1] = __shfl_sync(0xFFFFFFFFu, sc, (2 * t + 1) * 4);
    }
    __device__ __forceinline__ void store(uint4* dst, int lane) const {
        const uint32_t* f = &q[0][0][0];
#pragma unroll
        for (int v = 0; v < 4 * P; ++v) dst[v * 32 + lane] = make_uint4(f[4 * v], f[4 * v + 1], f[4 * v + 2], f[4 * v + 3]);
        dst[4 * P * 32 + lane] = make_uint4(__float_as_uint(scale[0]), __float_as_uint(scale[1]), 0u, 0u);
    }
    __device__ __forceinline__ void load(const uint4* src, int lane) {
        uint32_t* f = &q[0][0][0];
#pragma unroll
        for (int v = 0; v < 4 * P; ++v) {
            const uint4 x = __ldg(src + v * 32 + lane);
            f[4 * v] = x.x; f[4 * v + 1] = x.y; f[4 * v + 2] = x.z; f[4 * v + 3] = x.w;
        }
        const uint4 x = __ldg(src + 4 * P * 32 + lane);
        scale[0] = __uint_as_float(x.x); scale[1] = __uint_as_float(x.y);
    }
};
template <int P>
struct TileB<FMT_Q8_0, P> : TileBI8<FMT_Q8_0, P> {};
template <int P>
struct TileB<FMT_Q4_0, P> : TileBI8<FMT_Q4_0, P> {};
template <int P>
struct TileB<FMT_Q5_0, P> : TileBI8<FMT_Q5_0, P> {};  // Q4_0's element order: even elements in the low nibbles

// pieces per activation value: K-quants none; Q4_0 / Q8_0 three while one 8-row tile is held, two beyond
__host__ __device__ constexpr int fmt_pieces(int fmt, int mt) { return (fmt == FMT_Q4_0 || fmt == FMT_Q5_0 || fmt == FMT_Q8_0) ? (mt == 1 ? 3 : 2) : 0; }
__host__ __device__ constexpr int fmt_image_vectors(int fmt, int mt) {
    return (fmt == FMT_Q4_0 || fmt == FMT_Q5_0 || fmt == FMT_Q8_0) ? 4 * fmt_pieces(fmt, mt) + 1 : 5;
}

template <int FMT, int MT, int P>
struct SliceB {
    TileB<FMT, P> tile[MT];
    // tiles [tile0, tile0 + MT) of `slice`; tiles past the image or an absent slice read as zero
    __device__ __forceinline__ void load(const GemvParams& p, uint32_t slice, bool valid, uint32_t tile0, int lane) {
        constexpr int NV = TileB<FMT, P>::NV;
#pragma unroll
        for (int tl = 0; tl < MT; ++tl) {
            if (valid && tile0 + tl < p.tiles_total) {
                tile[tl].load(p.img + ((size_t)slice * p.tiles_total + tile0 + tl) * (NV * 32), lane);
            } else {
                tile[tl] = TileB<FMT, P>{};
            }
        }
    }
};

// One warp per (slice, tile): builds the fragments and writes them to the image.
template <int FMT, int P>
__global__ void __launch_bounds__(128) act_prep_kernel(const PrepParams p) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint32_t unit = blockIdx.x * 4 + (threadIdx.x >> 5);
    grid_dep_launch();
    grid_dep_wait();  // the activations may be the previous kernel's output; the image may still be read by it
    if (unit >= p.nslices * p.tiles_total) return;
    const uint32_t slice = unit / p.tiles_total, tl = unit % p.tiles_total;
    const uint32_t m_first = tl * 8, rows = min(8u, p.M - m_first);
    TileB<FMT, P> b;
    b.build(p, slice, m_first, rows, g, t);
    b.store(p.img + (size_t)unit * (TileB<FMT, P>::NV * 32), lane);
}

// ------------------------------------------------------------------ slice x 16 rows

// Adds the contribution of one slice (K run of 256) of weight rows g and g+8 to acc.
// ra / rb: shared-memory byte address of the slice in row g / g+8.
// M1: only activation row 0 exists, so accumulator columns 1 and 3 (odd activation rows) are
// never stored and their scaling work is skipped.

// byte i of x, zero-extended / sign-extended, in one PRMT
template <int I>
__device__ __forceinline__ int byte_u(uint32_t x) { return (int)__byte_perm(x, 0u, 0x4440 | I); }
template <int I>
__device__ __forceinline__ int byte_s(uint32_t x) {
    // prmt selector nibble: bits 2..0 pick a byte, bit 3 replicates that byte's sign bit instead
    int r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(x), "r"(0u), "n"(((I | 8) << 12) | ((I | 8) << 8) | ((I | 8) << 4) | I));
    return r;
}

// Q4_K, and Q5_K (Q5 = true) in the element order of the reference's x86-64 dot product
// (src/quant/cpu/kernels/simd/fused_q5k_q8k_dot.rs:27-122): the same header, scales and nibble order as Q4_K, the
// nibbles 32 bytes further into the block, plus one high bit per element, bit (e % 8) of qh[e / 8] for element e.
template <int MT, bool M1, bool Q5>
__device__ __forceinline__ void slice_q4k(const SliceB<Q5 ? FMT_Q5_K : FMT_Q4_K, MT, 0>& B, const uint32_t ra, const uint32_t rb, int t,
                                          float (&acc)[MT][4]) {
    constexpr uint32_t QS = Q5 ? 48u : 16u;  // offset of the nibble bytes
    const int zero[4] = {0, 0, 0, 0};
    uint4 ha = sld128(ra), hb = sld128(rb);
    // 6-bit scales / mins as packed bytes (unpack_q4k_q5k_scales, q4k_q5k.rs:108-122)
    uint32_t sA[2], mA[2], sB[2], mB[2];
    sA[0] = ha.y & 0x3F3F3F3Fu;
    mA[0] = ha.z & 0x3F3F3F3Fu;
    sA[1] = (ha.w & 0x0F0F0F0Fu) | ((ha.y >> 2) & 0x30303030u);
    mA[1] = ((ha.w >> 4) & 0x0F0F0F0Fu) | ((ha.z >> 2) & 0x30303030u);
    sB[0] = hb.y & 0x3F3F3F3Fu;
    mB[0] = hb.z & 0x3F3F3F3Fu;
    sB[1] = (hb.w & 0x0F0F0F0Fu) | ((hb.y >> 2) & 0x30303030u);
    mB[1] = ((hb.w >> 4) & 0x0F0F0F0Fu) | ((hb.z >> 2) & 0x30303030u);

    // Q4_K: 16 * sumi (low-nibble sub-blocks enter with 16 * scale, high nibbles are used unshifted, 16 * q);
    // |16 * sumi| <= 16 * 8 * 63 * 32 * 15 * 127 < 2^31.  Q5_K: sumi itself (5-bit codes cannot stay in the high nibble).
    int isum[MT][4];
#pragma unroll
    for (int tl = 0; tl < MT; ++tl)
#pragma unroll
        for (int i = 0; i < 4; ++i) isum[tl][i] = 0;

#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {  // 32 bytes: low nibbles = sub-block 2jj, high = 2jj+1
        uint2 qa = sld64(ra + QS + 32 * jj + 8 * t), qb = sld64(rb + QS + 32 * jj + 8 * t);
        int scA0, scA1, scB0, scB1;
        if ((jj & 1) == 0) {
            scA0 = byte_u<0>(sA[jj >> 1]); scA1 = byte_u<1>(sA[jj >> 1]);
            scB0 = byte_u<0>(sB[jj >> 1]); scB1 = byte_u<1>(sB[jj >> 1]);
        } else {
            scA0 = byte_u<2>(sA[jj >> 1]); scA1 = byte_u<3>(sA[jj >> 1]);
            scB0 = byte_u<2>(sB[jj >> 1]); scB1 = byte_u<3>(sB[jj >> 1]);
        }
        uint32_t al0, al1, al2, al3, ah0, ah1, ah2, ah3;
        if constexpr (Q5) {
            // the lane's elements 8t .. 8t + 7 of sub-block 2jj take the eight bits of qh[8jj + t], those of sub-block
            // 2jj + 1 the bits of qh[8jj + 4 + t]; four bits are spread to bit 4 of four bytes by one multiplication
            const uint2 hqa = sld64(ra + 16 + 8 * jj), hqb = sld64(rb + 16 + 8 * jj);
            const uint32_t la = (hqa.x >> (8 * t)) & 0xFFu, ua = (hqa.y >> (8 * t)) & 0xFFu;
            const uint32_t lb = (hqb.x >> (8 * t)) & 0xFFu, ub = (hqb.y >> (8 * t)) & 0xFFu;
            auto spread = [](uint32_t n4) { return (n4 * 0x02040810u) & 0x10101010u; };  // n4 < 16
            al0 = (qa.x & 0x0F0F0F0Fu) | spread(la & 15u);
            al2 = (qa.y & 0x0F0F0F0Fu) | spread(la >> 4);
            al1 = (qb.x & 0x0F0F0F0Fu) | spread(lb & 15u);
            al3 = (qb.y & 0x0F0F0F0Fu) | spread(lb >> 4);
            ah0 = ((qa.x >> 4) & 0x0F0F0F0Fu) | spread(ua & 15u);
            ah2 = ((qa.y >> 4) & 0x0F0F0F0Fu) | spread(ua >> 4);
            ah1 = ((qb.x >> 4) & 0x0F0F0F0Fu) | spread(ub & 15u);
            ah3 = ((qb.y >> 4) & 0x0F0F0F0Fu) | spread(ub >> 4);
        } else {
            scA0 <<= 4;
            scB0 <<= 4;
            al0 = qa.x & 0x0F0F0F0Fu; al1 = qb.x & 0x0F0F0F0Fu; al2 = qa.y & 0x0F0F0F0Fu; al3 = qb.y & 0x0F0F0F0Fu;
            ah0 = qa.x & 0xF0F0F0F0u; ah1 = qb.x & 0xF0F0F0F0u; ah2 = qa.y & 0xF0F0F0F0u; ah3 = qb.y & 0xF0F0F0F0u;
        }
#pragma unroll
        for (int tl = 0; tl < MT; ++tl) {
            int d[4];
            mma_u8s8_k32(d, al0, al1, al2, al3, B.tile[tl].q[4 * jj], B.tile[tl].q[4 * jj + 1], zero);
            isum[tl][0] += scA0 * d[0];
            isum[tl][2] += scB0 * d[2];
            if (!M1) {
                isum[tl][1] += scA0 * d[1];
                isum[tl][3] += scB0 * d[3];
            }
            mma_u8s8_k32(d, ah0, ah1, ah2, ah3, B.tile[tl].q[4 * jj + 2], B.tile[tl].q[4 * jj + 3], zero);
            isum[tl][0] += scA1 * d[0];
            isum[tl][2] += scB1 * d[2];
            if (!M1) {
                isum[tl][1] += scA1 * d[1];
                isum[tl][3] += scB1 * d[3];
            }
        }
    }
    // sum_j mins_j * bsum_j as two tiny u8 MMAs over (bsum + 4096) = hi * 128 + lo
    const uint32_t am0 = t == 0 ? mA[0] : t == 1 ? mA[1] : 0u;
    const uint32_t am1 = t == 0 ? mB[0] : t == 1 ? mB[1] : 0u;
    const int sumA = __dp4a(mA[0], 0x01010101u, __dp4a(mA[1], 0x01010101u, 0u));
    const int sumB = __dp4a(mB[0], 0x01010101u, __dp4a(mB[1], 0x01010101u, 0u));
    const float dA = f16bits_to_f32(ha.x & 0xFFFF), dminA = f16bits_to_f32(ha.x >> 16);
    const float dB = f16bits_to_f32(hb.x & 0xFFFF), dminB = f16bits_to_f32(hb.x >> 16);
#pragma unroll
    for (int tl = 0; tl < MT; ++tl) {
        int ml[4], mh[4];
        mma_u8u8_k16(ml, am0, am1, B.tile[tl].bs_lo, zero);
        mma_u8u8_k16(mh, am0, am1, B.tile[tl].bs_hi, zero);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (M1 && (i & 1)) continue;
            const int sumi = Q5 ? isum[tl][i] : isum[tl][i] >> 4;
            const int summ = ml[i] + 128 * mh[i] - 4096 * (i < 2 ? sumA : sumB);
            const float d8 = B.tile[tl].d8[i & 1];
            const float dall = __fmul_rn(i < 2 ? dA : dB, d8);
            const float dmall = __fmul_rn(i < 2 ? dminA : dminB, d8);
            const float term = __fsub_rn(__fmul_rn(dall, (float)sumi), __fmul_rn(dmall, (float)summ));
            acc[tl][i] = __fadd_rn(acc[tl][i], term);
        }
    }
}

// Sign-extended byte `sb` (0..15) of four words; sb is a constant after unrolling.
__device__ __forceinline__ int byte_s_dyn(const uint32_t (&sc)[4], int sb) {
    const uint32_t w = sc[sb >> 2];
    switch (sb & 3) {
    case 0: return byte_s<0>(w);
    case 1: return byte_s<1>(w);
    case 2: return byte_s<2>(w);
    default: return byte_s<3>(w);
    }
}

// Signed scale sb (0..15) of a row from its four scale words.
template <int SB>
__device__ __forceinline__ int q6k_scale(const uint32_t (&sc)[4]) { return byte_s<SB & 3>(sc[SB >> 2]); }

// ALIGNED 1: both slices start on a 4-byte boundary (plain 32-bit loads); 2: both start exactly 2 bytes past one
// (a word = two aligned loads at constant offsets and one byte permute); 0: any 2-byte alignment.
template <int MT, bool M1, int ALIGNED>
__device__ __forceinline__ void slice_q6k(const SliceB<FMT_Q6_K, MT, 0>& B, const uint32_t ra, const uint32_t rb, int t,
                                          float (&acc)[MT][4]) {
    auto ld = [](uint32_t a) -> uint32_t {
        if (ALIGNED == 1) return sld32(a);
        if (ALIGNED == 2) return __byte_perm(sld32(a - 2), sld32(a + 2), 0x5432);  // every word exactly 2 bytes off
        return sld32_u(a);
    };
    const int zero[4] = {0, 0, 0, 0};
    int isum[MT][4];
#pragma unroll
    for (int tl = 0; tl < MT; ++tl)
#pragma unroll
        for (int i = 0; i < 4; ++i) isum[tl][i] = 0;
    uint32_t scA[4], scB[4];  // 16 signed 8-bit scales per row
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        scA[i] = ld(ra + 192 + 4 * i);
        scB[i] = ld(rb + 192 + 4 * i);
    }
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
        for (int is = 0; is < 2; ++is) {
            const uint32_t o = 64 * n + 16 * is + 4 * t;
            const uint32_t la0 = ld(ra + o), la1 = ld(ra + o + 32), hA = ld(ra + 128 + 32 * n + 16 * is + 4 * t);
            const uint32_t lb0 = ld(rb + o), lb1 = ld(rb + o + 32), hB = ld(rb + 128 + 32 * n + 16 * is + 4 * t);
#pragma unroll
            for (int gq = 0; gq < 4; ++gq) {
                // int8 value 4*(q-32): nibble -> bits 5..2, two high bits -> bits 7..6, flip bit 7
                const uint32_t qla = (gq & 1) ? la1 : la0, qlb = (gq & 1) ? lb1 : lb0;
                const uint32_t ua = ((hA << (6 - 2 * gq)) & 0xC0C0C0C0u) ^ 0x80808080u;
                const uint32_t ub = ((hB << (6 - 2 * gq)) & 0xC0C0C0C0u) ^ 0x80808080u;
                const uint32_t va = lop3_and_or(gq < 2 ? (qla << 2) : (qla >> 2), 0x3C3C3C3Cu, ua);
                const uint32_t vb = lop3_and_or(gq < 2 ? (qlb << 2) : (qlb >> 2), 0x3C3C3C3Cu, ub);
                const int sb = 8 * n + 2 * gq + is;
                const int sA_ = byte_s_dyn(scA, sb), sB_ = byte_s_dyn(scB, sb);
#pragma unroll
                for (int tl = 0; tl < MT; ++tl) {
                    int d[4];
                    mma_s8s8_k16(d, va, vb, B.tile[tl].q[sb], zero);
                    isum[tl][0] += sA_ * d[0];
                    isum[tl][2] += sB_ * d[2];
                    if (!M1) {
                        isum[tl][1] += sA_ * d[1];
                        isum[tl][3] += sB_ * d[3];
                    }
                }
            }
        }
    }
    const float dA = f16bits_to_f32(sld16(ra + 208)), dB = f16bits_to_f32(sld16(rb + 208));
#pragma unroll
    for (int tl = 0; tl < MT; ++tl)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (M1 && (i & 1)) continue;
            const float dall = __fmul_rn(i < 2 ? dA : dB, B.tile[tl].d8[i & 1]);
            acc[tl][i] = __fadd_rn(acc[tl][i], __fmul_rn(dall, (float)(isum[tl][i] >> 2)));
        }
}

// Q8_0 / Q4_0 slice: per 32-block one int8 MMA per activation piece.  The accumulator starts at the bit
// pattern of 1.5 * 2^23, so the finished integer sum S (|S| <= 32 * 128 * 127 < 2^22) reads back as the
// float 1.5 * 2^23 + S, and S itself costs one FADD instead of a conversion.
// ROWS4: both slices start on a 4-byte boundary (always so with tiled fills): every address is then the slice
// address plus a compile-time constant, blocks with an odd index hold their codes word-aligned, and those of
// even blocks sit exactly 2 bytes off, so a word is two aligned loads and one byte permute.
template <int FMT, int MT, int P, bool M1, bool ROWS4>
__device__ __forceinline__ void slice_i8(const SliceB<FMT, MT, P>& B, const uint32_t ra, const uint32_t rb, int t, uint32_t nblk,
                                         float (&acc)[MT][4]) {
    // word of a row at byte offset `off` (off = 2 mod 4 for even blocks, 0 mod 4 for odd ones when ROWS4)
    auto word = [](uint32_t row, uint32_t off, bool aligned) -> uint32_t {
        if (!ROWS4) return sld32_u(row + off);
        if (aligned) return sld32(row + off);
        return __byte_perm(sld32(row + off - 2), sld32(row + off + 2), 0x5432);
    };
    constexpr int BB = fmt_block_bytes(FMT);
    constexpr int MAGIC_I = 0x4B400000;
    constexpr float MAGIC_F = 12582912.0f;
    const int magic[4] = {MAGIC_I, MAGIC_I, MAGIC_I, MAGIC_I};
    constexpr float C1 = 1.0f / PIECE_STEP;
    // sacc: piece 1 (offset removed per block, exact); sacc2: pieces 2.. still carrying MAGIC * d per block — their
    // weight is 1/254 or less, so the cancellation error of removing sum(d) * MAGIC once per slice stays below 1e-6
    float sacc[MT][4], sacc2[MT][4], dsum[2] = {0.f, 0.f};
#pragma unroll
    for (int tl = 0; tl < MT; ++tl)
#pragma unroll
        for (int i = 0; i < 4; ++i) sacc[tl][i] = sacc2[tl][i] = 0.f;
#pragma unroll
    for (int b = 0; b < 8; ++b) {
        if ((uint32_t)b < nblk) {  // warp-uniform: ragged last slice when K % 256 != 0
            uint32_t a0, a1, a2, a3;  // row g k-slots 4t.. | row g+8 | row g k-slots 16+4t.. | row g+8
            float dA = f16bits_to_f32(sld16(ra + BB * b)), dB = f16bits_to_f32(sld16(rb + BB * b));
            if constexpr (FMT == FMT_Q8_0) {
                // block = f16 d | 32 x i8 (2-byte aligned); the lane's codes are bytes 4t..4t+3 and 16+4t..16+4t+3, so the
                // four lanes of a row read 16 contiguous bytes per load
                const bool al = (b & 1) != 0;  // 34 * b + 2 is a multiple of 4 for odd b
                a0 = word(ra, BB * b + 2 + 4 * t, al);
                a2 = word(ra, BB * b + 18 + 4 * t, al);
                a1 = word(rb, BB * b + 2 + 4 * t, al);
                a3 = word(rb, BB * b + 18 + 4 * t, al);
            } else if constexpr (FMT == FMT_Q5_0) {
                // Q5_0 block = f16 d | 32 high bits | 16 B nibbles, Q4_0's element order; element e takes bit e of the
                // high-bit word, so the lane's eight elements take byte t of it (even bits: low-nibble elements).  The
                // 5-bit code c goes to the top of a byte, (c << 3) ^ 0x80 = the int8 value 8 * (c - 16); the factor 8
                // leaves through the block scale.  (22 * b + 6 and 22 * b + 2 are multiples of 4 for odd b.)
                const bool al = (b & 1) != 0;
                const uint32_t wa = word(ra, BB * b + 6 + 4 * t, al), wb = word(rb, BB * b + 6 + 4 * t, al);
                const uint32_t ha = (word(ra, BB * b + 2, al) >> (8 * t)) & 0xFFu, hb = (word(rb, BB * b + 2, al) >> (8 * t)) & 0xFFu;
                // even bits of the byte -> bit 7 of bytes 0..3 (shifts 7, 13, 19, 25; stray products and their carries miss those bits)
                auto top = [](uint32_t bits) { return ((bits & 0x55u) * 0x02082080u) & 0x80808080u; };
                a0 = (((wa << 3) & 0x78787878u) | top(ha)) ^ 0x80808080u;
                a2 = (((wa >> 1) & 0x78787878u) | top(ha >> 1)) ^ 0x80808080u;
                a1 = (((wb << 3) & 0x78787878u) | top(hb)) ^ 0x80808080u;
                a3 = (((wb >> 1) & 0x78787878u) | top(hb >> 1)) ^ 0x80808080u;
                dA *= 0.125f;
                dB *= 0.125f;
            } else {
                // Q4_0 block = f16 d | 16 B; byte i = elements 2i (low nibble), 2i+1 (high); the lane's word = bytes 4t..4t+3.
                // (w ^ 0x88..) keeps each nibble as q - 8 in 4-bit two's complement; placed in the high nibble of a byte
                // it reads as the int8 value 16 * (q - 8): the factor 16 leaves through the block scale.
                const bool al = (b & 1) != 0;  // 18 * b + 2 is a multiple of 4 for odd b
                const uint32_t wa = word(ra, BB * b + 2 + 4 * t, al) ^ 0x88888888u, wb = word(rb, BB * b + 2 + 4 * t, al) ^ 0x88888888u;
                a0 = (wa << 4) & 0xF0F0F0F0u;
                a2 = wa & 0xF0F0F0F0u;
                a1 = (wb << 4) & 0xF0F0F0F0u;
                a3 = wb & 0xF0F0F0F0u;
                dA *= 0.0625f;
                dB *= 0.0625f;
            }
#pragma unroll
            for (int tl = 0; tl < MT; ++tl) {
                int d[P][4];
#pragma unroll
                for (int pc = 0; pc < P; ++pc) mma_s8s8_k32(d[pc], a0, a1, a2, a3, B.tile[tl].q[b][pc][0], B.tile[tl].q[b][pc][1], magic);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (M1 && (i & 1)) continue;
                    const float dr = i < 2 ? dA : dB;
                    sacc[tl][i] = fmaf(dr, __int_as_float(d[0][i]) - MAGIC_F, sacc[tl][i]);
                    float h2 = __int_as_float(d[1][i]);
                    if constexpr (P > 2) h2 = fmaf(__int_as_float(d[2][i]), C1, h2);  // (f2 + f3 / 254), offset MAGIC * (1 + 1/254)
                    sacc2[tl][i] = fmaf(dr, h2, sacc2[tl][i]);
                }
            }
            dsum[0] += dA;
            dsum[1] += dB;
        }
    }
    constexpr float OFF2 = MAGIC_F * (P > 2 ? 1.0f + C1 : 1.0f);
#pragma unroll
    for (int tl = 0; tl < MT; ++tl)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float s2 = sacc2[tl][i] - OFF2 * dsum[i >> 1];
            acc[tl][i] = fmaf(fmaf(s2, C1, sacc[tl][i]), B.tile[tl].scale[i & 1], acc[tl][i]);
        }
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

__device__ __forceinline__ void store_out(void* out, int dt, size_t idx, float v) {
    if (dt == DT_F32) static_cast<float*>(out)[idx] = v;
    else if (dt == DT_BF16) static_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
    else static_cast<__half*>(out)[idx] = __float2half_rn(v);
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
                 : "memory");
}

// ------------------------------------------------------------------------- the kernel
//
// FMT    block format
// MT     8-row activation tiles per launch (1 or 2)
// SL     K-chunks (of up to 16 slices) one CTA walks per slab; its activation fragments for all
//        of them stay in registers
// SWIGLU two weights (gate, up) and out = silu(gate) * up
// Cursor over the sequence of stage fills of one CTA: slab -> matrix -> K-chunk.
struct FillCursor {
    uint32_t unit;
    int mat, c;
    uint32_t it;     // running fill index
    uint32_t stage;  // it % nstages
    uint32_t par;    // (it / nstages) & 1
};

constexpr int RED_SLOTS = 4;  // upper bound; p.red_slots (3 or 4) are used
// dynamic shared memory header: full[8] | empty[8] | abort | red_full[4] | red_empty[4]
constexpr int OFF_EMPTY = 8 * MAX_STAGES, OFF_ABORT = 16 * MAX_STAGES, OFF_RFULL = OFF_ABORT + 8,
              OFF_REMPTY = OFF_RFULL + 8 * RED_SLOTS;

template <int FMT, int MT, int SL, bool M1, bool SWIGLU>
__global__ void __launch_bounds__(16 * 32, 1) gemv_kernel(const __grid_constant__ CUtensorMap tmap0, const __grid_constant__ CUtensorMap tmap1,
                                                          const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int P = fmt_pieces(FMT, MT);
    constexpr int NMAT = SWIGLU ? 2 : 1;
    constexpr int SLICE_B = fmt_slice_bytes(FMT);
    constexpr int PER_RG = MT * 4 * 32;  // floats one warp contributes per row group
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nwc = (int)(p.spc * p.rgs);  // warps in the CTA
    const uint32_t bar_full = smem_u32(smem), bar_empty = bar_full + OFF_EMPTY;
    const uint32_t bar_rfull = bar_full + OFF_RFULL, bar_rempty = bar_full + OFF_REMPTY;
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + OFF_ABORT);
    const uint32_t stage0 = smem_u32(smem + p.stage_off);
    const uint32_t rps = 16 * p.rgs;  // rows per slab
    const uint32_t ks = blockIdx.y;
    const int nch = (int)min((uint32_t)SL, p.nchunks - ks * SL);  // K-chunks this CTA walks (>= 1)

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.nstages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, nwc);
        }
        for (int s = 0; s < RED_SLOTS; ++s) {
            mbar_init(bar_rfull + 8 * s, nwc);
            mbar_init(bar_rempty + 8 * s, 1);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();

    // A warp that gives up on a wait marks the CTA dead; the others notice at their next slab.
    // Dead warps keep walking the loops (so every barrier still gets its arrivals) but skip
    // waits and arithmetic.
    bool dead = false;
    auto give_up = [&](unsigned code) {
        dead = true;
        *abort_flag = 1;
        atomicOr(p.status, code);
    };

    // Requests the fill at `cur`: the calling warp copies all rows of the stage, one row per
    // lane and pass.  The stage must have been released by every warp.
    auto issue_fill = [&](const FillCursor& cur) {
        const uint32_t stage = cur.stage;
        const uint32_t r0 = cur.unit * rps;
        const uint32_t nrows = min(rps, p.N - r0);
        const uint8_t* wbase = p.w[cur.mat];
        const uint32_t gc = ks * SL + cur.c;
        const uint32_t coff = gc * p.spc * SLICE_B;
        const uint32_t cbytes = min(p.spc * SLICE_B, p.row_bytes - coff);
        const uint32_t sdst = stage0 + stage * p.stage_bytes;
        const uint32_t bar = bar_full + 8 * stage;
        if (p.use_tma) {
            // one lane, one copy per box; rows past the end of the tensor are filled with zeros by the copy
            // engine and still count towards the byte total
            if (lane == 0) {
                mbar_expect_tx(bar, p.tma_cb * rps * p.tma_w);
                tma_load_3d(sdst, cur.mat ? &tmap1 : &tmap0, 0, (int)r0, (int)(coff / p.tma_w), bar);
            }
        } else if (p.rows_aligned) {
            if (lane == 0) mbar_expect_tx(bar, nrows * cbytes);
            __syncwarp();
            for (uint32_t r = lane; r < nrows; r += 32)
                bulk_g2s(sdst + r * p.srow, wbase + (size_t)(r0 + r) * p.row_bytes + coff, cbytes, bar);
        } else {
            // Each row's chunk is copied as the enclosing 16-byte-aligned range.  Only the last
            // row of the tensor can have a range that would end past the buffer: its final <16
            // bytes are moved with plain loads instead.
            const uint8_t* wend = wbase + p.w_bytes;
            uint32_t tx = 0;
            for (uint32_t r = lane; r < nrows; r += 32) {
                const uint8_t* gsrc = wbase + (size_t)(r0 + r) * p.row_bytes + coff;
                const uint8_t* gs = reinterpret_cast<const uint8_t*>(reinterpret_cast<uintptr_t>(gsrc) & ~(uintptr_t)15);
                const uint8_t* ge = gsrc + cbytes;
                const uint8_t* e16 = reinterpret_cast<const uint8_t*>((reinterpret_cast<uintptr_t>(ge) + 15) & ~(uintptr_t)15);
                if (e16 > wend) {
                    e16 = reinterpret_cast<const uint8_t*>(reinterpret_cast<uintptr_t>(ge) & ~(uintptr_t)15);
                    uint8_t* sd = smem + p.stage_off + stage * p.stage_bytes + r * p.srow;
                    for (const uint8_t* q = e16; q < ge; ++q) sd[q - gs] = __ldg(q);
                }
                tx += (uint32_t)(e16 - gs);
            }
            tx = __reduce_add_sync(0xFFFFFFFFu, tx);
            __syncwarp();
            if (lane == 0) mbar_expect_tx(bar, tx);
            __syncwarp();
            for (uint32_t r = lane; r < nrows; r += 32) {
                const uint8_t* gsrc = wbase + (size_t)(r0 + r) * p.row_bytes + coff;
                const uint8_t* gs = reinterpret_cast<const uint8_t*>(reinterpret_cast<uintptr_t>(gsrc) & ~(uintptr_t)15);
                const uint8_t* ge = gsrc + cbytes;
                const uint8_t* e16 = reinterpret_cast<const uint8_t*>((reinterpret_cast<uintptr_t>(ge) + 15) & ~(uintptr_t)15);
                if (e16 > wend) e16 = reinterpret_cast<const uint8_t*>(reinterpret_cast<uintptr_t>(ge) & ~(uintptr_t)15);
                const uint32_t n = (uint32_t)(e16 - gs);
                if (n) bulk_g2s(sdst + r * p.srow, gs, n, bar);
            }
        }
    };
    auto advance = [&](FillCursor& cur) {
        ++cur.it;
        if (++cur.stage == p.nstages) {
            cur.stage = 0;
            cur.par ^= 1;
        }
        if (++cur.c >= nch) {
            cur.c = 0;
            if (++cur.mat >= NMAT) {
                cur.mat = 0;
                cur.unit += gridDim.x;
            }
        }
    };

    // Fill f is requested by warp f % nwc: the first nstages fills right away, fill f >= nstages
    // when that warp has finished fill f - nstages (it then waits for the others to release the
    // stage).  Every warp walks the same cursor, so the role rotates without communication.
    FillCursor pc{blockIdx.x, 0, 0, 0, 0, 0};
    int pw = 0;  // warp that requests fill pc.it
    // Only two fills leave before the activations are fetched: responses return to an SM in request
    // order, so activation loads issued behind a full ring would wait for every stage to land.
    const uint32_t early = min(2u, p.nstages);
    for (uint32_t i = 0; i < early; ++i) {
        if (pc.unit < p.total_units && pw == warp) issue_fill(pc);
        advance(pc);
        if (++pw == nwc) pw = 0;
    }

    const int g = lane >> 2, t = lane & 3;
    const uint32_t s = warp % p.spc;   // slice within a chunk
    const uint32_t rg = warp / p.spc;  // row group within a slab
    // tiled fills: byte offset of row 0 of this warp's slice in a stage (column c of the chunk, then within the column)
    const uint32_t tma_off = p.use_tma ? ((s * SLICE_B) / p.tma_w) * (16u * p.rgs) * p.tma_w + (s * SLICE_B) % p.tma_w : 0u;

    grid_dep_launch();  // the next kernel may begin (its weight prefetch does not depend on us)
    grid_dep_wait();    // activations written by the previous kernel are complete from here on

    SliceB<FMT, MT, P> B[SL];  // written by act_prep_kernel, the previous launch in the stream
#pragma unroll
    for (int c = 0; c < SL; ++c) {
        const uint32_t gc = ks * SL + c;
        const uint32_t slice = gc * p.spc + s;
        B[c].load(p, slice, c < nch && slice < p.nslices, p.m0 >> 3, lane);
    }
    for (uint32_t i = early; i < p.nstages; ++i) {  // the rest of the ring
        if (pc.unit < p.total_units && pw == warp) issue_fill(pc);
        advance(pc);
        if (++pw == nwc) pw = 0;
    }

    // Adds up the partial sums of slab `unit_j` (ring slot `js`) and stores the results: one
    // output per lane and pass, the slices' terms added in K order.
    const uint32_t mcp = p.mcount <= 1 ? 1u : p.mcount <= 2 ? 2u : p.mcount <= 4 ? 4u : p.mcount <= 8 ? 8u : p.mcount <= 16 ? 16u : 32u;
    const uint32_t mcp_log = 31 - __clz(mcp);
    auto reduce_slab = [&](uint32_t unit_j, uint32_t js, uint32_t jpar) {
        if (!dead && !mbar_wait(bar_rfull + 8 * js, jpar)) give_up(STATUS_TIMEOUT_FULL);
        if (!dead) {
            const float* slot = reinterpret_cast<const float*>(smem + p.red_off + js * p.red_slot_bytes);
            const uint32_t r0 = unit_j * rps;
            for (uint32_t o = lane; o < rps * mcp; o += 32) {
                const uint32_t rr = o >> mcp_log, col = o & (mcp - 1);
                const uint32_t row = r0 + rr;
                if (row < p.N && col < p.mcount) {
                    const uint32_t rgi = rr >> 4, r16 = rr & 15;
                    const uint32_t i = (col >> 3) * 4 + (r16 >= 8 ? 2 : 0) + (col & 1);
                    const uint32_t ln = (r16 & 7) * 4 + ((col & 7) >> 1);
                    float v[NMAT];
#pragma unroll
                    for (int mat = 0; mat < NMAT; ++mat) {
                        const float* src = slot + ((size_t)mat * nwc + rgi * p.spc) * PER_RG + i * 32 + ln;
                        float sum = 0.f;
                        if (p.spc == 16) {  // all loads first, then the ordered adds
                            float x[16];
#pragma unroll
                            for (int ss = 0; ss < 16; ++ss) x[ss] = src[ss * PER_RG];
#pragma unroll
                            for (int ss = 0; ss < 16; ++ss) sum = __fadd_rn(sum, x[ss]);
                        } else {
                            for (uint32_t ss = 0; ss < p.spc; ++ss) sum = __fadd_rn(sum, src[(size_t)ss * PER_RG]);
                        }
                        v[mat] = sum;
                    }
                    if (p.ksplit == 1) {
                        float r = v[0];
                        if constexpr (SWIGLU) r = silu_f(v[0]) * v[1];
                        store_out(p.out, p.out_dtype, (size_t)(p.m0 + col) * p.N + row, r);
                    } else {
#pragma unroll
                        for (int mat = 0; mat < NMAT; ++mat)
                            p.partial[((size_t)(mat * p.ksplit + ks) * p.M + p.m0 + col) * p.N + row] = v[mat];
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_rempty + 8 * js);
    };
    uint32_t it = 0, stage = 0, par = 0;          // consumer position in the stage ring
    uint32_t rslot = 0, rpar = 0;                 // reduction ring: slot being written
    uint32_t jslot = 0, jpar = 0, junit = blockIdx.x;  // reduction ring: slab to be reduced next
    int jw = 0;                                   // warp that reduces slab junit
    const uint32_t lag = p.red_slots - 2;         // slabs between publishing partials and reducing them
    uint32_t published = 0;
    auto next_reduce = [&]() {
        if (jw == warp) reduce_slab(junit, jslot, jpar);
        junit += gridDim.x;
        if (++jslot == p.red_slots) {
            jslot = 0;
            jpar ^= 1;
        }
        if (++jw == nwc) jw = 0;
    };
    for (uint32_t unit = blockIdx.x; unit < p.total_units; unit += gridDim.x) {
        if (*abort_flag) dead = true;
        const uint32_t r0 = unit * rps;
        const uint32_t rowA = rg * 16 + g, rowB = rowA + 8;  // rows of the slab
        float accs[NMAT][MT][4];
#pragma unroll
        for (int mat = 0; mat < NMAT; ++mat) {
            float(&acc)[MT][4] = accs[mat];
#pragma unroll
            for (int tl = 0; tl < MT; ++tl)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[tl][i] = 0.f;
            // phase of a row inside its 16-byte-aligned copy (0 whenever row_bytes % 16 == 0)
            uint32_t phA = 0, phB = 0;
            if (!p.rows_aligned) {
                phA = (uint32_t)((reinterpret_cast<uintptr_t>(p.w[mat]) + (size_t)(r0 + rowA) * p.row_bytes) & 15);
                phB = (uint32_t)((reinterpret_cast<uintptr_t>(p.w[mat]) + (size_t)(r0 + rowB) * p.row_bytes) & 15);
            }
#pragma unroll
            for (int c = 0; c < SL; ++c) {
                if (c < nch) {
                    const uint32_t gc = ks * SL + c;
                    if (!dead && !mbar_wait(bar_full + 8 * stage, par)) give_up(STATUS_TIMEOUT_FULL);
                    const uint32_t slice = gc * p.spc + s;
                    if (!dead && slice < p.nslices) {
                        const uint32_t coff = gc * p.spc * SLICE_B;
                        uint32_t ra, rb;  // shared-window addresses of this warp's slice in rows g and g + 8
                        if (p.use_tma) {
                            const uint32_t sb = stage0 + stage * p.stage_bytes + tma_off;
                            ra = sb + rowA * p.tma_w;
                            rb = sb + rowB * p.tma_w;
                        } else {
                            const uint32_t sb = stage0 + stage * p.stage_bytes + s * SLICE_B;
                            ra = sb + rowA * p.srow + ((phA + coff) & 15);
                            rb = sb + rowB * p.srow + ((phB + coff) & 15);
                        }
                        if constexpr (FMT == FMT_Q4_K) slice_q4k<MT, M1, false>(B[c], ra, rb, t, acc);
                        else if constexpr (FMT == FMT_Q5_K) slice_q4k<MT, M1, true>(B[c], ra, rb, t, acc);
                        else if constexpr (FMT == FMT_Q6_K) {
                            const uint32_t al = (ra | rb) & 3u;
                            if (__all_sync(0xFFFFFFFFu, al == 0)) slice_q6k<MT, M1, 1>(B[c], ra, rb, t, acc);
                            else if (__all_sync(0xFFFFFFFFu, (ra & 3u) == 2 && (rb & 3u) == 2)) slice_q6k<MT, M1, 2>(B[c], ra, rb, t, acc);
                            else slice_q6k<MT, M1, 0>(B[c], ra, rb, t, acc);
                        } else {
                            const uint32_t kl = p.K - slice * 256;
                            const uint32_t nb8 = kl >= 256 ? 8u : kl / 32;
                            if (__all_sync(0xFFFFFFFFu, ((ra | rb) & 3u) == 0)) slice_i8<FMT, MT, P, M1, true>(B[c], ra, rb, t, nb8, acc);
                            else slice_i8<FMT, MT, P, M1, false>(B[c], ra, rb, t, nb8, acc);
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_empty + 8 * stage);
                    // whoever's turn it is refills the stage just released (fill it + nstages)
                    if (pc.unit < p.total_units && pw == warp) {
                        if (!dead && !mbar_wait(bar_empty + 8 * stage, par)) give_up(STATUS_TIMEOUT_EMPTY);
                        if (!dead) issue_fill(pc);
                    }
                    advance(pc);
                    if (++pw == nwc) pw = 0;
                    ++it;
                    if (++stage == p.nstages) {
                        stage = 0;
                        par ^= 1;
                    }
                }
            }
        }
        // publish the partial sums in the reduction ring ...
        float* slot = reinterpret_cast<float*>(smem + p.red_off + rslot * p.red_slot_bytes);
        if (!dead && !mbar_wait(bar_rempty + 8 * rslot, rpar ^ 1)) give_up(STATUS_TIMEOUT_EMPTY);
#pragma unroll
        for (int mat = 0; mat < NMAT; ++mat) {
            float* rdst = slot + ((size_t)mat * nwc + warp) * PER_RG;
#pragma unroll
            for (int tl = 0; tl < MT; ++tl)
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (!(M1 && (i & 1))) rdst[(tl * 4 + i) * 32 + lane] = accs[mat][tl][i];
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_rfull + 8 * rslot);
        if (++rslot == p.red_slots) {
            rslot = 0;
            rpar ^= 1;
        }
        ++published;
        // ... and one warp (taking turns) adds up an older slab, whose partials arrived long ago
        if (published > lag) next_reduce();
    }
    while (junit < p.total_units) next_reduce();  // drain the slabs still in the ring
}

// Adds split-K partials [nmat][ksplit][M][N] in K order and applies the SwiGLU gate.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partial, void* out, int out_dtype,
                                                            size_t mn, uint32_t ksplit, int swiglu) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < mn; i += (size_t)gridDim.x * blockDim.x) {
        float a = 0.f, b = 0.f;
        for (uint32_t k = 0; k < ksplit; ++k) a = __fadd_rn(a, partial[(size_t)k * mn + i]);
        if (swiglu) {
            for (uint32_t k = 0; k < ksplit; ++k) b = __fadd_rn(b, partial[(size_t)(ksplit + k) * mn + i]);
            a = silu_f(a) * b;
        }
        store_out(out, out_dtype, i, a);
    }
}

struct GemvMaps {
    CUtensorMap m[2];
};

template <int FMT, int MT, int SL, bool M1, bool SWIGLU>
cudaError_t launch_one(const GemvParams& p, const GemvMaps& maps, dim3 grid, int threads, size_t smem, cudaStream_t st) {
    auto k = gemv_kernel<FMT, MT, SL, M1, SWIGLU>;
    static PerDeviceOnce attrs;
    cudaError_t ae = attrs.run([&] { return cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448 - 1024); });
    if (ae != cudaSuccess) return ae;
    cudaError_t le = launch_pdl(k, grid, dim3(threads), smem, st, maps.m[0], maps.m[1], p);
    note_launch();
    return le != cudaSuccess ? le : cudaGetLastError();
}

template <int FMT, bool SWIGLU>
cudaError_t launch_gemv_fmt(const GemvParams& p, const GemvMaps& maps, int mt, int sl, dim3 grid, int threads, size_t smem, cudaStream_t st) {
    constexpr bool KQ = (FMT == FMT_Q4_K || FMT == FMT_Q5_K || FMT == FMT_Q6_K);
    const bool m1 = p.mcount == 1 && p.M == 1;
    if constexpr (KQ) {
        if (mt == 1 && sl == 1) return m1 ? launch_one<FMT, 1, 1, true, SWIGLU>(p, maps, grid, threads, smem, st)
                                          : launch_one<FMT, 1, 1, false, SWIGLU>(p, maps, grid, threads, smem, st);
        if (mt == 1 && sl == 2) return m1 ? launch_one<FMT, 1, 2, true, SWIGLU>(p, maps, grid, threads, smem, st)
                                          : launch_one<FMT, 1, 2, false, SWIGLU>(p, maps, grid, threads, smem, st);
        if (mt == 1 && sl == 4) return m1 ? launch_one<FMT, 1, 4, true, SWIGLU>(p, maps, grid, threads, smem, st)
                                          : launch_one<FMT, 1, 4, false, SWIGLU>(p, maps, grid, threads, smem, st);
        if (mt == 2 && sl == 1) return launch_one<FMT, 2, 1, false, SWIGLU>(p, maps, grid, threads, smem, st);
    } else {
        if (mt == 1 && sl == 1) return m1 ? launch_one<FMT, 1, 1, true, SWIGLU>(p, maps, grid, threads, smem, st)
                                          : launch_one<FMT, 1, 1, false, SWIGLU>(p, maps, grid, threads, smem, st);
        if (mt == 2 && sl == 1) return launch_one<FMT, 2, 1, false, SWIGLU>(p, maps, grid, threads, smem, st);
    }
    return cudaErrorInvalidValue;
}

template <int FMT>
cudaError_t launch_prep_fmt(const PrepParams& pp, int mt, cudaStream_t st) {
    const unsigned units = pp.nslices * pp.tiles_total;
    const dim3 grid((units + 3) / 4), block(128);
    constexpr bool KQ = (FMT == FMT_Q4_K || FMT == FMT_Q5_K || FMT == FMT_Q6_K);
    cudaError_t e;
    if constexpr (KQ) {
        e = launch_pdl(act_prep_kernel<FMT, 0>, grid, block, 0, st, pp);
    } else {
        e = mt == 1 ? launch_pdl(act_prep_kernel<FMT, 3>, grid, block, 0, st, pp) : launch_pdl(act_prep_kernel<FMT, 2>, grid, block, 0, st, pp);
    }
    note_launch();
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace

// K-chunks a CTA walks per slab (their activation fragments live in registers); the others are spread over
// gridDim.y.  Measured on 4096 x 14336 and the like: one chunk per CTA and a wider K split beats two or four chunks
// per CTA at every row count (Q6_K M = 16: 24.5 us against 33.7, where two chunks also spill; Q5_K M = 16: 23.3 / 29.3;
// Q4_K M = 3: 15.5 / 17.1); only single-tile launches over many rows (14336 x 8192, M = 1) are 5 % faster with more
// chunks per CTA, so those keep them.
int gemv_max_sl(int fmt, int mt, size_t N) {
    const bool kq = (fmt == FMT_Q4_K || fmt == FMT_Q5_K || fmt == FMT_Q6_K);
    return (kq && mt == 1 && N >= 8192) ? 4 : 1;
}

// 8-row tiles per pass: one for M <= 8, else two (16 activation rows per pass).  Four tiles per pass were
// measured (K-quants, K = 4096): the fragments of 32 rows leave the compiler no registers to overlap the
// tensor-core results with their scaling, and a pass took 2.1x the time of a 16-row pass; more than 16
// rows therefore run as consecutive 16-row passes (layer-sized weights are re-read from L2).
int gemv_tiles_per_pass(int fmt, size_t M, size_t K) {
    (void)fmt;
    (void)K;
    return M <= 8 ? 1 : 2;
}

struct GemvPlan {
    uint32_t spc, nslices, nchunks, sl, ksplit, rgs, srow, stage_bytes, nstages, total_units, red_off, stage_off;
    uint32_t red_slot_bytes, red_slots, rows_aligned;
    uint32_t use_tma, tma_w, tma_cb;
    size_t smem;
    int threads;
    dim3 grid;
};

// Shape-dependent launch geometry, shared by the launcher and the workspace query.
bool gemv_plan(int fmt, uint32_t K, uint32_t N, int mt, bool swiglu, int sm_count, GemvPlan& pl) {
    const uint32_t slice_b = fmt_slice_bytes(fmt);
    const uint32_t row_bytes = K / fmt_block_size(fmt) * fmt_block_bytes(fmt);
    pl.nslices = (K + 255) / 256;
    pl.spc = pl.nslices < 16 ? pl.nslices : 16;
    pl.nchunks = (pl.nslices + pl.spc - 1) / pl.spc;
    const uint32_t maxsl = gemv_max_sl(fmt, mt, N);
    uint32_t sl = pl.nchunks < maxsl ? pl.nchunks : maxsl;
    if (sl == 3) sl = 4;  // instantiated values: 1, 2, 4
    pl.sl = sl;
    pl.ksplit = (pl.nchunks + sl - 1) / sl;
    pl.rgs = 16 / pl.spc;
    if (pl.rgs < 1) pl.rgs = 1;
    // never stage more row groups than the tensor has
    const uint32_t need_rg = (N + 15) / 16;
    if (pl.rgs > need_rg) pl.rgs = need_rg;
    uint32_t cmax = pl.spc * slice_b < row_bytes ? pl.spc * slice_b : row_bytes;
    // Row stride in shared memory: room for the 16-byte phase of unaligned rows and for the
    // second word of a straddling load, then bumped so that the eight rows a warp touches at
    // once fall in distinct banks: Q4_K reads 8 bytes per lane (rows 32 bytes apart mod 128),
    // the other formats 4 bytes per lane (rows 16 bytes apart mod 32).
    uint32_t srow = (cmax + 19 + 15) & ~15u;
    if (fmt == FMT_Q4_K || fmt == FMT_Q5_K) {
        while ((srow & 63) != 32) srow += 16;
    } else {
        if ((srow & 31) == 0) srow += 16;
    }
    pl.rows_aligned = (row_bytes % 16 == 0 && (pl.spc * slice_b) % 16 == 0) ? 1u : 0u;
    pl.srow = srow;
    pl.stage_bytes = ((16 * pl.rgs * srow + 127) & ~127u) + 128;
    // Tiled fills (one copy per stage): column width = 2 slices of Q4_K / Q5_K (288 / 352 B: rows 32 / 96 B apart mod
    // 128 for the 8-byte reads), 1 slice of Q8_0 / Q4_0 (272 / 144 B: 16 B apart), 8 slices of Q6_K (1680 B, the smallest whole
    // number of 210-byte blocks that is a multiple of 16 bytes).  Rows must be a whole number of columns.
    const uint32_t tw = fmt == FMT_Q4_K ? 288u : fmt == FMT_Q5_K ? 352u : fmt == FMT_Q6_K ? 1680u : slice_b;
    pl.use_tma = 0;
    pl.tma_w = tw;
    pl.tma_cb = (cmax + tw - 1) / tw;
    if (tma_available() && K % 256 == 0 && row_bytes % tw == 0 && (pl.spc * slice_b) % tw == 0 && pl.tma_cb <= 256 && 16 * pl.rgs <= 256) {
        pl.use_tma = 1;
        pl.stage_bytes = ((pl.tma_cb * 16 * pl.rgs * tw + 127) & ~127u) + 128;
    }
    const int nwc = pl.spc * pl.rgs;
    pl.red_slot_bytes = (swiglu ? 2u : 1u) * nwc * mt * 4 * 32 * 4;
    const uint32_t budget = 232448 - 1024;
    pl.red_off = 256;
    // reduction ring: 4 slots when they are small, fewer when shared memory is short (with 2
    // slots a slab is reduced right after it is published, i.e. the warps meet once per slab)
    for (pl.red_slots = pl.red_slot_bytes * 4 <= 48 * 1024 ? 4u : 3u;; --pl.red_slots) {
        pl.stage_off = (pl.red_off + pl.red_slots * pl.red_slot_bytes + 127) & ~127u;
        if (pl.stage_off + 2 * pl.stage_bytes <= budget) break;
        if (pl.red_slots == 2) return false;
    }
    uint32_t ns = (budget - pl.stage_off) / pl.stage_bytes;
    if (ns > MAX_STAGES) ns = MAX_STAGES;
    pl.nstages = ns;
    pl.smem = pl.stage_off + (size_t)ns * pl.stage_bytes;
    pl.total_units = (N + 16 * pl.rgs - 1) / (16 * pl.rgs);
    pl.threads = nwc * 32;
    uint32_t gx = sm_count / pl.ksplit;
    if (gx < 1) gx = 1;
    if (gx > pl.total_units) gx = pl.total_units;
    pl.grid = dim3(gx, pl.ksplit, 1);
    return true;
}

// bytes of the activation image: [nslices][tiles_total][NV][32] 16-byte vectors, rounded up to 256
static size_t gemv_image_bytes(int fmt, size_t M, size_t K, int mt) {
    const size_t nslices = (K + 255) / 256, tiles = (M + 7) / 8;
    return (nslices * tiles * (size_t)fmt_image_vectors(fmt, mt) * 32 * 16 + 255) & ~(size_t)255;
}

size_t gemv_workspace_bytes(int fmt, size_t M, size_t K, size_t N, bool swiglu, int sm_count) {
    const int mt = gemv_tiles_per_pass(fmt, M, K);
    size_t need = gemv_image_bytes(fmt, M, K, mt);
    GemvPlan pl;
    if (gemv_plan(fmt, (uint32_t)K, (uint32_t)N, mt, swiglu, sm_count, pl) && pl.ksplit > 1)
        need += (size_t)(swiglu ? 2 : 1) * pl.ksplit * M * N * sizeof(float);
    return need;
}

// out[M,N] = act[M,K] x W^T for any M: one activation-image launch (none when the image is there already), then passes of up
// to 8 * MT activation rows.
cudaError_t launch_gemv(int fmt, const void* act, int act_dtype, const void* w0, const void* w1, void* out, int out_dtype,
                        size_t M, size_t K, size_t N, void* ws, size_t ws_bytes, bool swiglu, int sm_count, cudaStream_t st,
                        unsigned int* status, bool* ws_too_small, bool image_ready) {
    *ws_too_small = false;
    const int mt = gemv_tiles_per_pass(fmt, M, K);  // one geometry for every pass, so split-K partials line up
    GemvPlan pl;
    if (!gemv_plan(fmt, (uint32_t)K, (uint32_t)N, mt, swiglu, sm_count, pl)) return cudaErrorInvalidConfiguration;
    const size_t img_bytes = gemv_image_bytes(fmt, M, K, mt);
    const size_t part_bytes = pl.ksplit > 1 ? (size_t)(swiglu ? 2 : 1) * pl.ksplit * M * N * sizeof(float) : 0;
    if (!ws || ws_bytes < img_bytes + part_bytes || (reinterpret_cast<uintptr_t>(ws) & 15)) {
        *ws_too_small = true;
        return cudaSuccess;
    }
    PrepParams pp{};
    pp.act = act;
    pp.img = static_cast<uint4*>(ws);
    pp.M = (uint32_t)M;
    pp.K = (uint32_t)K;
    pp.nslices = pl.nslices;
    pp.tiles_total = (uint32_t)((M + 7) / 8);
    pp.act_dtype = act_dtype;
    // image_ready: the previous weight of a batch (same activations, same image format, same scratch) left the image there
    cudaError_t e = cudaSuccess;
    if (!image_ready)
    switch (fmt) {
    case FMT_Q4_0: e = launch_prep_fmt<FMT_Q4_0>(pp, mt, st); break;
    case FMT_Q5_0: e = launch_prep_fmt<FMT_Q5_0>(pp, mt, st); break;
    case FMT_Q8_0: e = launch_prep_fmt<FMT_Q8_0>(pp, mt, st); break;
    case FMT_Q4_K: e = launch_prep_fmt<FMT_Q4_K>(pp, mt, st); break;
    case FMT_Q5_K: e = launch_prep_fmt<FMT_Q5_K>(pp, mt, st); break;
    case FMT_Q6_K: e = launch_prep_fmt<FMT_Q6_K>(pp, mt, st); break;
    default: return cudaErrorInvalidValue;
    }
    if (e != cudaSuccess) return e;
    // tiled fills: one 3-D tensor map per weight, [row_bytes / tma_w][N][tma_w bytes as 8-byte elements]
    GemvMaps maps{};
    if (pl.use_tma) {
        const uint32_t row_bytes = (uint32_t)(K / fmt_block_size(fmt) * fmt_block_bytes(fmt));
        const cuuint64_t gdim[3] = {(cuuint64_t)(pl.tma_w / 8), (cuuint64_t)N, (cuuint64_t)(row_bytes / pl.tma_w)};
        const cuuint64_t gstride[2] = {(cuuint64_t)row_bytes, (cuuint64_t)pl.tma_w};
        const cuuint32_t box[3] = {pl.tma_w / 8, 16u * pl.rgs, pl.tma_cb};
        const cuuint32_t estr[3] = {1, 1, 1};
        const void* ws2[2] = {w0, w1 ? w1 : w0};
        for (int i = 0; i < 2 && pl.use_tma; ++i) {
            CUresult cr = encode_tiled()(&maps.m[i], CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, const_cast<void*>(ws2[i]), gdim, gstride, box, estr,
                                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (cr != CUDA_SUCCESS) pl.use_tma = 0;  // fall back to per-row copies
        }
        if (!pl.use_tma) {
            pl.stage_bytes = ((16 * pl.rgs * pl.srow + 127) & ~127u) + 128;
            uint32_t ns = (232448u - 1024u - pl.stage_off) / pl.stage_bytes;
            pl.nstages = ns > (uint32_t)MAX_STAGES ? (uint32_t)MAX_STAGES : ns;
            pl.smem = pl.stage_off + (size_t)pl.nstages * pl.stage_bytes;
        }
    }
    const uint32_t rows_per_pass = 8u * (uint32_t)mt;
    for (size_t m0 = 0; m0 < M; m0 += rows_per_pass) {
        const uint32_t mc = (uint32_t)(M - m0 < rows_per_pass ? M - m0 : rows_per_pass);
        GemvParams p{};
        p.w[0] = static_cast<const uint8_t*>(w0);
        p.w[1] = static_cast<const uint8_t*>(w1 ? w1 : w0);
        p.act = act;
        p.out = out;
        p.img = static_cast<const uint4*>(ws);
        p.tiles_total = pp.tiles_total;
        p.partial = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + img_bytes);
        p.M = (uint32_t)M; p.K = (uint32_t)K; p.N = (uint32_t)N;
        p.m0 = (uint32_t)m0; p.mcount = mc;
        p.row_bytes = (uint32_t)(K / fmt_block_size(fmt) * fmt_block_bytes(fmt));
        p.nslices = pl.nslices; p.spc = pl.spc; p.nchunks = pl.nchunks; p.ksplit = pl.ksplit; p.rgs = pl.rgs;
        p.srow = pl.srow; p.stage_bytes = pl.stage_bytes; p.nstages = pl.nstages; p.total_units = pl.total_units;
        p.red_off = pl.red_off; p.stage_off = pl.stage_off;
        p.red_slot_bytes = pl.red_slot_bytes; p.red_slots = pl.red_slots; p.rows_aligned = pl.rows_aligned;
        p.use_tma = pl.use_tma; p.tma_w = pl.tma_w; p.tma_cb = pl.tma_cb;
        p.act_dtype = act_dtype; p.out_dtype = out_dtype;
        p.w_bytes = (unsigned long long)N * p.row_bytes;
        p.status = status;
        switch (fmt) {
        case FMT_Q4_0: e = swiglu ? launch_gemv_fmt<FMT_Q4_0, true>(p, maps, mt, pl.sl, pl.grid, pl.threads, pl.smem, st)
                                  : launch_gemv_fmt<FMT_Q4_0, false>(p, maps, mt, pl.sl, pl.grid, pl.threads, pl.smem, st); break;
        case FMT_Q5_0: e = swiglu ? launch_gemv_fmt<FMT_Q5_0, true>(p, maps, mt, pl.sl, pl.grid, pl.threads, pl.smem, st)
                                  : launch_gemv_fmt<FMT_Q5_0, false>(p, maps, mt, pl.sl, pl.grid, pl.threads, pl.smem, st); break;
        case FMT_Q8_0: e = swiglu ? launch_gemv_fmt<FMT_Q8_0, true>(p, maps, mt, pl.sl, pl.grid, pl.threads, pl.smem, st)
                                  : launch_gemv_fmt<FMT_Q8_0, false>(p, maps, mt, pl.sl, pl.grid, pl.threads, pl.smem, st); break;
        case FMT_Q4_K: e = swiglu ? launch_gemv_fmt<FMT_Q4_K, true>(p, maps, mt, pl.sl, pl.grid, pl.threads, pl.smem, st)
                                  : launch_gemv_fmt<FMT_Q4_K, false>(p, maps, mt, pl.sl, pl.grid, pl.threads, pl.smem, st); break;
        case FMT_Q5_K: e = swiglu ? launch_gemv_fmt<FMT_Q5_K, true>(p, maps, mt, pl.sl, pl.grid, pl.threads, pl.smem, st)
                                  : launch_gemv_fmt<FMT_Q5_K, false>(p, maps, mt, pl.sl, pl.grid, pl.threads, pl.smem, st); break;
        case FMT_Q6_K: e = swiglu ? launch_gemv_fmt<FMT_Q6_K, true>(p, maps, mt, pl.sl, pl.grid, pl.threads, pl.smem, st)
                                  : launch_gemv_fmt<FMT_Q6_K, false>(p, maps, mt, pl.sl, pl.grid, pl.threads, pl.smem, st); break;
        default: return cudaErrorInvalidValue;
        }
        if (e != cudaSuccess) return e;
    }
    if (pl.ksplit > 1) {
        size_t mn = M * N;
        int grid = (int)((mn + 255) / 256);
        if (grid > sm_count * 8) grid = sm_count * 8;
        splitk_reduce_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const float*>(static_cast<uint8_t*>(ws) + img_bytes), out, out_dtype, mn,
                                                  pl.ksplit, swiglu ? 1 : 0);
        note_launch();
        return cudaGetLastError();
    }
    return cudaSuccess;
}

}  // namespace b200q
