// Decode GEMV (M = 1) for Q4_K: y[n] = sum_k x[k] * W[n,k], one activation row.
//
// Stands in for boostr's quant_gemv_q4_k_q8_1_mwr launch plus its activation-quantise launch
// (src/quant/cuda/kernels/quant_gemv.cu:285-379, quant_act.cu:17-69) when there is a single
// activation row, the shape every decode step of a quantised LLaMA produces.
//
// The kernel is bound by HBM: 144 bytes of packed weights per 256 multiply-adds.  Layout of work:
//   * persistent CTAs, one per SM, each owning a contiguous, evenly sized range of weight rows;
//   * the rows stream through a ring of up to 16 small fills (8 rows = 18 KB at K = 4096), each
//     fill one 1-D bulk copy (cp.async.bulk) signalled on an mbarrier and consumed by one group of
//     four warps (group g takes fills g, g + 4, ...), so about 220 KB of reads are in flight per
//     SM, no thread spends instructions on loads and the arithmetic starts when 18 KB have landed;
//   * the activation row is quantised to Q8_K once per CTA (exactly as boostr's CPU path does,
//     src/quant/cpu/kernels/simd/quantize_act_q8k.rs:26-98) and every lane keeps the int8 codes
//     of ONE 256-wide block in registers for the whole kernel;
//   * a warp takes two rows of a fill; lane (h, b) multiplies block b of row h against its
//     register-resident activation block with dp4a: 128-bit shared loads, nibbles unpacked with
//     one AND each (high nibbles stay in place and are divided out of the integer sum), 6-bit
//     scales and mins unpacked with a handful of byte-parallel logic ops, the min term through
//     byte-split block sums; then 16 lanes add their block terms with shuffles.
//   * a decode step is a chain of such launches, each short, so the time between one launch's last byte and
//     the next one's first byte counts: kernels start under programmatic dependent launch and send their
//     first fills before the grid dependency resolves, and a launch that has been told which weights follow
//     (NextHint) ends by pulling the head of those weights into L2.
// Integer sums are exact and each block contributes (d*d8)*sumi - (dmin*d8)*summ as in
// fused_dot_q4k_q8k (src/quant/cpu/kernels/simd/fused_q4k_q8k_dot.rs:111-172); only the order in
// which the K/256 block terms are added differs from the CPU loop (pairwise instead of serial).
#include "common.cuh"

namespace b200q {


// Where the launch AFTER this one starts to read, so that this launch can pull those bytes into L2 while its
// own ring drains.  A space is the virtual row range of up to three weights (or gate + up) that the next
// launch's CTAs cta0 .. cta0 + ncta - 1 divide into runs of rows_per_cta rows; CTA c of this launch
// prefetches the first `head` bytes of the run of CTA c of the next one.
struct NextSpace {
    const uint8_t* w[3];
    const uint8_t* w2;  // second weight with the same geometry (up-projection), or null
    uint32_t seg_end[3];
    uint32_t nseg, row_bytes, rows_per_cta, cta0, ncta;
};
struct NextHint {
    NextSpace sp[2];
    uint32_t nsp;   // 0: nothing to prefetch
    uint32_t head;  // bytes per CTA and weight
};

struct GemvM1Params {
    // Up to three weights that share the activation row (q/k/v-style batches) form one virtual row
    // space [0, N): segment s covers rows [seg_end[s-1], seg_end[s]) and writes its own output.
    const uint8_t* w[3];
    void* out[3];
    uint32_t seg_end[3];
    uint32_t nseg;
    const uint8_t* w2;   // up-projection weight (SwiGLU variant, single segment)
    const void* act;
    const float* norm_w; // RMSNorm prologue: the row is replaced by x * rsqrt(mean(x^2) + eps) * norm_w before it is quantised
    float norm_eps;
    uint32_t K, N;
    uint32_t nblk;       // K / 256 (<= 16)
    uint32_t row_bytes;  // nblk * 144
    uint32_t rows_per_cta;  // CTA c owns rows [c * rows_per_cta, min(N, (c + 1) * rows_per_cta)) of the virtual row space
    uint32_t lpr;           // lanes per row: nblk rounded up to a power of two
    uint32_t stage_bytes;   // one fill: 4 warps x (32 / lpr) rows, or 4 gate + 4 up rows in the SwiGLU variant
    uint32_t nstages;
    uint32_t act_off, stage_off;
    int act_dtype, out_dtype;
    unsigned int* status;
    PeerComm comm;  // row-parallel shard: push the partial row to every rank and add them up (single weight, f32 out)
    NextHint next;
};

namespace {

__device__ __forceinline__ int dp4a_u8s8(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t dp4a_u8u8(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
template <int I>
__device__ __forceinline__ int ubyte(uint32_t x) { return (int)__byte_perm(x, 0u, 0x4440 | I); }

// shared-memory image of the quantised activation row, per 256-block b (stride 400 B):
//   [0,256)   int8 codes   [256,264) (bsum_j + 4096) & 127, j = 0..7   [264,272) (bsum_j + 4096) >> 7
//   [272,276) f32 d8
// Every lane copies its block of the image into registers with 16-byte loads, 16 different blocks per warp.  The
// stride is 16 bytes past a multiple of 128, so the eight lanes of a quarter-warp hit all 32 banks once.
constexpr int ACT_STRIDE = 400;

// Loads 8 consecutive activation values of this lane (f32 or bf16 source).
__device__ __forceinline__ void load_act8(const void* act, int act_dtype, size_t base, float (&v)[8]) {
    if (act_dtype == DT_F32) {
        const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(act) + base);
        float4 a = __ldg(src), b = __ldg(src + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        uint4 r = __ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(act) + base));
        v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xFFFF0000u);
        v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xFFFF0000u);
        v[4] = __uint_as_float(r.z << 16); v[5] = __uint_as_float(r.z & 0xFFFF0000u);
        v[6] = __uint_as_float(r.w << 16); v[7] = __uint_as_float(r.w & 0xFFFF0000u);
    }
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ int dp4a_s8s8(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t f32_to_s8_rni_sat(float x) {
    int r;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(x));  // clamps to [-128, 127]; the code in the low byte
    return (uint32_t)r;
}

// Q8_K-quantises one 256-block held 8 values per lane: returns d8, the lane's 8 codes packed in `packed`
// and their sum in `s` (quantize_act_q8k.rs:26-98: d = amax / 127, id = 127 / amax, round half to even).
// This sits on every decode kernel's critical path, so the chain is kept short: one warp-wide integer
// max on the bit patterns (non-negative floats order like unsigned integers), saturating converts,
// byte permutes for the packing and dp4a for the sum.
__device__ __forceinline__ float quantize_block8(const float (&v)[8], uint2& packed, int& s) {
    const float m = fmaxf(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))),
                          fmaxf(fmaxf(fabsf(v[4]), fabsf(v[5])), fmaxf(fabsf(v[6]), fabsf(v[7]))));
    const float amax = __uint_as_float(__reduce_max_sync(0xFFFFFFFFu, __float_as_uint(m)));
    const float id = amax != 0.f ? __fdiv_rn(127.0f, amax) : 0.f;
    uint32_t c[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) c[i] = f32_to_s8_rni_sat(__fmul_rn(v[i], id));
    packed.x = prmt(prmt(c[0], c[1], 0x0040u), prmt(c[2], c[3], 0x0040u), 0x5410u);
    packed.y = prmt(prmt(c[4], c[5], 0x0040u), prmt(c[6], c[7], 0x0040u), 0x5410u);
    s = dp4a_s8s8(packed.x, 0x01010101u, dp4a_s8s8(packed.y, 0x01010101u, 0));
    return __fdiv_rn(amax, 127.0f);
}

// One lane: L2 prefetch of [ptr, ptr + len), shrunk to 16-byte boundaries (the bulk form wants both).
__device__ __forceinline__ void l2_prefetch(const uint8_t* ptr, uint32_t len) {
    const uint32_t skip = (uint32_t)(-(intptr_t)reinterpret_cast<uintptr_t>(ptr)) & 15u;
    if (len < skip + 16) return;
    const uint32_t n = (len - skip) & ~15u;
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(ptr + skip), "r"(n) : "memory");
}

// One lane of CTA `cta`: the head of the matching CTA's rows in the next launch goes to L2.  Called once the
// last fill of this CTA is on its way, so the prefetch queues behind every byte this launch still needs and
// fills the time in which this launch drains and the next one starts up.
__device__ __forceinline__ void prefetch_next(const NextHint& h, uint32_t cta) {
    for (uint32_t s = 0; s < h.nsp; ++s) {
        const NextSpace& sp = h.sp[s];
        const uint32_t c = cta - sp.cta0;
        if (c >= sp.ncta) continue;
        const uint32_t r0 = c * sp.rows_per_cta;
        uint32_t sg = 0, seg_begin = 0;
        while (sg + 1 < sp.nseg && r0 >= sp.seg_end[sg]) seg_begin = sp.seg_end[sg++];
        if (r0 >= sp.seg_end[sg]) continue;
        const uint32_t rows = min(sp.seg_end[sg] - r0, sp.rows_per_cta);
        const size_t off = (size_t)(r0 - seg_begin) * sp.row_bytes;
        const uint32_t len = (uint32_t)min((size_t)h.head, (size_t)rows * sp.row_bytes);
        l2_prefetch(sp.w[sg] + off, len);
        if (sp.w2) l2_prefetch(sp.w2 + off, len);
    }
}

// RMSNorm prologue.  Every warp adds the squares of the values it holds (0 for warps without a block), the 16 warp sums
// meet in shared memory (`red`, 16 floats) and every thread adds them in warp order, so all threads hold the same
// factor 1 / sqrt(mean(x^2) + eps).  Contains a block-wide barrier: all 512 threads call it.
__device__ __forceinline__ float rms_factor(float local_sq, float* red, int warp, int lane, uint32_t K, float eps) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local_sq += __shfl_xor_sync(0xFFFFFFFFu, local_sq, o);
    if (lane == 0) red[warp] = local_sq;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) tot += red[i];
    return 1.0f / sqrtf(tot / (float)K + eps);
}

// SWIGLU: two weights; a warp takes gate row r (lanes 0-15) and up row r (lanes 16-31) and stores
// silu(gate . x) * (up . x)  (quant_swiglu, src/quant/traits/quant_matmul.rs:122-127).
//
// The 16 warps form 4 groups; a fill is the 8 rows (SwiGLU: 4 gate + 4 up rows) that ONE group consumes,
// and group g takes fills g, g+4, g+8, ... of the CTA's row range.  Small fills let the arithmetic start
// as soon as the first 18 KB have landed, while the ring still keeps ~220 KB per SM in flight.
template <bool SWIGLU>
__device__ __forceinline__ void q4k_body(const GemvM1Params& p, const uint32_t cta, uint8_t* smem) {
    // A row takes `lpr` lanes (the block count rounded up to a power of two; 16 for SwiGLU), so a warp
    // takes 32 / lpr rows: short rows (K-split shards of a tensor-parallel group) keep all lanes busy.
    const uint32_t lpr = SWIGLU ? 16u : p.lpr, lpr_log = 31 - __clz(lpr), rpw = 32u >> lpr_log;
    const uint32_t FR = SWIGLU ? 4u : 4u * rpw;  // output rows per fill
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_full = smem_u32(smem), bar_empty = bar_full + 128;
    uint8_t* act_s = smem + p.act_off;
    const uint32_t stage0 = smem_u32(smem + p.stage_off);

    const uint32_t row_begin = cta * p.rows_per_cta;
    const uint32_t row_end = min(p.N, row_begin + p.rows_per_cta);
    const uint32_t nfill = row_end > row_begin ? (row_end - row_begin + FR - 1) / FR : 0;

    auto issue_fill = [&](uint32_t f, uint32_t slot) {  // one lane
        const uint32_t r0 = row_begin + f * FR;
        const uint32_t nrows = min(FR, row_end - r0);
        const uint32_t bytes = nrows * p.row_bytes;
        const uint32_t dst = stage0 + slot * p.stage_bytes, bar = bar_full + 8 * slot;
        if (SWIGLU) {
            mbar_expect_tx(bar, 2 * bytes);
            bulk_g2s(dst, p.w[0] + (size_t)r0 * p.row_bytes, bytes, bar);
            bulk_g2s(dst + FR * p.row_bytes, p.w2 + (size_t)r0 * p.row_bytes, bytes, bar);
        } else if (p.nseg == 1) {
            mbar_expect_tx(bar, bytes);
            bulk_g2s(dst, p.w[0] + (size_t)r0 * p.row_bytes, bytes, bar);
        } else {
            mbar_expect_tx(bar, bytes);
            uint32_t seg_begin = 0;
            for (uint32_t sg = 0; sg < p.nseg; ++sg) {  // the part of [r0, r0 + nrows) inside each segment
                const uint32_t lo = max(r0, seg_begin), hi = min(r0 + nrows, p.seg_end[sg]);
                if (lo < hi)
                    bulk_g2s(dst + (lo - r0) * p.row_bytes, p.w[sg] + (size_t)(lo - seg_begin) * p.row_bytes,
                             (hi - lo) * p.row_bytes, bar);
                seg_begin = p.seg_end[sg];
            }
        }
    };

    // Responses come back to an SM in request order, so an activation load issued behind a full ring
    // of weight fills would wait for all of them (several microseconds).  Hence: one fill per warp group
    // leaves before the grid dependency is resolved (the weights do not depend on the previous kernel),
    // then the activation loads, and only then the rest of the ring.
    if (warp == 15 && (uint32_t)lane < p.nstages) {
        mbar_init(bar_full + 8 * lane, 1);
        mbar_init(bar_empty + 8 * lane, 4);
        mbar_fence_init();
    }
    __syncthreads();
    if (warp == 15 && lane < 2 && (uint32_t)lane < nfill) issue_fill(lane, lane);
    grid_dep_launch();  // the next kernel may start its own weight prefetch as SMs free up
    grid_dep_wait();    // the previous kernel's output (our activations) is complete from here on
    const bool tp = !SWIGLU && p.comm.world > 1;
    const uint32_t tp_e = tp ? tp_epoch(p.comm) : 0u;

    // 1. quantise the activation row: warp w owns block w; each warp issues its load first and then
    // its share of the remaining first fills
    {
        float v[8];
        const bool on = (uint32_t)warp < p.nblk;
        if (on) load_act8(p.act, p.act_dtype, (size_t)warp * 256 + 8 * lane, v);
        const uint32_t f1 = 2 + (uint32_t)warp;  // the rest of the ring: one fill per warp
        if (lane == 0 && f1 < p.nstages && f1 < nfill) issue_fill(f1, f1);
        if (warp == 15 && lane == 0 && nfill <= p.nstages) prefetch_next(p.next, blockIdx.x);  // the whole range is on its way
        if (p.norm_w) {  // uniform over the launch
            float sq = 0.f;
            float g[8];
            if (on) {
                const float4 g0 = __ldg(reinterpret_cast<const float4*>(p.norm_w + (size_t)warp * 256 + 8 * lane));
                const float4 g1 = __ldg(reinterpret_cast<const float4*>(p.norm_w + (size_t)warp * 256 + 8 * lane) + 1);
                g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w; g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
#pragma unroll
                for (int i = 0; i < 8; ++i) sq = fmaf(v[i], v[i], sq);
            }
            const float rs = rms_factor(sq, reinterpret_cast<float*>(smem + 256), warp, lane, p.K, p.norm_eps);
            if (on)
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(__fmul_rn(v[i], rs), g[i]);
        }
        if (on) {  // warp-uniform
            uint2 packed;
            int s;
            const float d8 = quantize_block8(v, packed, s);
            uint8_t* blk = act_s + warp * ACT_STRIDE;
            *reinterpret_cast<uint2*>(blk + 8 * lane) = packed;
            // sum over the 4 lanes of a 32-element sub-block
            s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
            s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
            if ((lane & 3) == 0) {
                const int bs = s + 4096;
                blk[256 + (lane >> 2)] = (uint8_t)(bs & 127);
                blk[264 + (lane >> 2)] = (uint8_t)(bs >> 7);
            }
            if (lane == 0) *reinterpret_cast<float*>(blk + 272) = d8;
        }
    }
    __syncthreads();  // barriers initialised, activation image complete

    // 2. this lane's activation block goes to registers
    const int b = lane & (lpr - 1), h = lane >> lpr_log;
    const bool blk_on = (uint32_t)b < p.nblk;
    uint32_t a[64];
    uint32_t bs_lo[2], bs_hi[2];
    float d8 = 0.f;
    {
        const uint8_t* blk = act_s + (blk_on ? b : 0) * ACT_STRIDE;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            uint4 q = *reinterpret_cast<const uint4*>(blk + 16 * i);
            a[4 * i] = q.x; a[4 * i + 1] = q.y; a[4 * i + 2] = q.z; a[4 * i + 3] = q.w;
        }
        uint4 q = *reinterpret_cast<const uint4*>(blk + 256);
        bs_lo[0] = q.x; bs_lo[1] = q.y; bs_hi[0] = q.z; bs_hi[1] = q.w;
        d8 = blk_on ? *reinterpret_cast<const float*>(blk + 272) : 0.f;
    }
    const uint32_t grp = (uint32_t)warp >> 2, wi = (uint32_t)warp & 3;
    const uint32_t rr = SWIGLU ? wi : rpw * wi + h;  // output row of the fill handled by this lane group
    bool dead = false;
    uint32_t slot = grp, par = 0;  // fill f lives in ring slot f % nstages (nstages >= 4)
    for (uint32_t f = grp; f < nfill; f += 4) {
        if (!dead && !mbar_wait(bar_full + 8 * slot, par)) {
            dead = true;
            atomicOr(p.status, STATUS_TIMEOUT_FULL);
        }
        const uint32_t r0 = row_begin + f * FR;
        const uint32_t nrows = min(FR, row_end - r0);
        float term = 0.f;
        if (!dead && rr < nrows && blk_on) {
            const uint8_t* blk = smem + p.stage_off + slot * p.stage_bytes + (SWIGLU ? FR * h + wi : rr) * p.row_bytes + b * 144;
            const uint4 hd = *reinterpret_cast<const uint4*>(blk);
            // 6-bit scales / mins as packed bytes (unpack_q4k_q5k_scales, q4k_q5k.rs:108-122)
            uint32_t sc[2], mn[2];
            sc[0] = hd.y & 0x3F3F3F3Fu;
            mn[0] = hd.z & 0x3F3F3F3Fu;
            sc[1] = (hd.w & 0x0F0F0F0Fu) | ((hd.y >> 2) & 0x30303030u);
            mn[1] = ((hd.w >> 4) & 0x0F0F0F0Fu) | ((hd.z >> 2) & 0x30303030u);
            int sum_lo = 0, sum_hi = 0;  // sum_hi is 16x too large: high nibbles are used in place
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {  // 32 bytes: low nibbles = sub-block 2jj, high = 2jj+1
                const uint4 q0 = *reinterpret_cast<const uint4*>(blk + 16 + 32 * jj);
                const uint4 q1 = *reinterpret_cast<const uint4*>(blk + 32 + 32 * jj);
                const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                int dl = 0, dh = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    dl = dp4a_u8s8(w[i] & 0x0F0F0F0Fu, a[16 * jj + i], dl);
                    dh = dp4a_u8s8(w[i] & 0xF0F0F0F0u, a[16 * jj + 8 + i], dh);
                }
                const uint32_t sw = sc[jj >> 1];
                const int s0 = (jj & 1) ? ubyte<2>(sw) : ubyte<0>(sw);
                const int s1 = (jj & 1) ? ubyte<3>(sw) : ubyte<1>(sw);
                sum_lo += s0 * dl;
                sum_hi += s1 * dh;
            }
            const int sumi = sum_lo + (sum_hi >> 4);
            // sum_j mins_j * bsum_j with bsum_j + 4096 = hi * 128 + lo, all bytes
            const uint32_t mlo = dp4a_u8u8(mn[0], bs_lo[0], dp4a_u8u8(mn[1], bs_lo[1], 0u));
            const uint32_t mhi = dp4a_u8u8(mn[0], bs_hi[0], dp4a_u8u8(mn[1], bs_hi[1], 0u));
            const uint32_t msum = dp4a_u8u8(mn[0], 0x01010101u, dp4a_u8u8(mn[1], 0x01010101u, 0u));
            const int summ = (int)mlo + 128 * (int)mhi - 4096 * (int)msum;
            const float d = f16bits_to_f32(hd.x & 0xFFFF), dmin = f16bits_to_f32(hd.x >> 16);
            term = __fsub_rn(__fmul_rn(__fmul_rn(d, d8), (float)sumi), __fmul_rn(__fmul_rn(dmin, d8), (float)summ));
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + 8 * slot);
        // add the block terms of a row (lpr lanes)
#pragma unroll
        for (uint32_t o = 8; o > 0; o >>= 1)
            if (o < lpr) term += __shfl_xor_sync(0xFFFFFFFFu, term, o);
        if (SWIGLU) {
            const float up = __shfl_xor_sync(0xFFFFFFFFu, term, 16);
            term = term / (1.0f + expf(-term)) * up;  // meaningful in lane 0 (gate half)
        }
        if (b == 0 && (!SWIGLU || h == 0) && rr < nrows && !dead) {
            uint32_t v = r0 + rr, sg = 0, seg_begin = 0;
            while (sg + 1 < p.nseg && v >= p.seg_end[sg]) seg_begin = p.seg_end[sg++];
            const size_t idx = v - seg_begin;
            void* o = p.out[sg];
            if (tp && p.comm.gather) tp_push_gather(p.comm, tp_e, p.comm.rank * p.N + v, term);
            else if (tp) tp_push(p.comm, tp_e, v, term);
            else if (p.out_dtype == DT_F32) static_cast<float*>(o)[idx] = term;
            else if (p.out_dtype == DT_BF16) static_cast<__nv_bfloat16*>(o)[idx] = __float2bfloat16_rn(term);
            else static_cast<__half*>(o)[idx] = __float2half_rn(term);
        }
        // refill the slot just released: the four warps of the group take turns
        if (f + p.nstages < nfill && ((f >> 2) & 3) == wi) {
            if (!dead && !mbar_wait(bar_empty + 8 * slot, par)) {
                dead = true;
                atomicOr(p.status, STATUS_TIMEOUT_EMPTY);
            }
            if (!dead && lane == 0) {
                issue_fill(f + p.nstages, slot);
                if (f + p.nstages + 1 == nfill) prefetch_next(p.next, blockIdx.x);
            }
        }
        slot += 4;
        if (slot >= p.nstages) {
            slot -= p.nstages;
            par ^= 1;
        }
    }
    if (tp && p.comm.gather) tp_finish_gather(p.comm, tp_e, static_cast<float*>(p.out[0]), p.status);
    else if (tp) tp_finish(p.comm, tp_e, row_begin, row_end, static_cast<float*>(p.out[0]), p.status);
}

template <bool SWIGLU>
__global__ void __launch_bounds__(512, 1) gemv_m1_q4k_kernel(const __grid_constant__ GemvM1Params p) {
    extern __shared__ __align__(128) uint8_t smem[];
    q4k_body<SWIGLU>(p, blockIdx.x, smem);
}


// ------------------------------------------------------------------------------------ Q6_K, M = 1
//
// Same streaming structure as the Q4_K kernel (ring of small fills, one warp group per fill, activation
// loads ahead of the ring); the differences follow from the format:
//   * a 210-byte block is only 2-byte aligned inside its row, so a lane reads aligned 32-bit words and
//     re-assembles each needed word with one prmt whose selector depends on the block's parity;
//   * a block splits into two independent 128-element halves (64 B of low nibbles, 32 B of high bit
//     pairs, 8 signed scales each): lane (b, n) takes half n of block b of a 16-block chunk of K;
//   * NCHUNK = 1, 2 or 4 warps share a row (K up to 4096 * NCHUNK), so a fill of a 4-warp group is
//     4 / NCHUNK whole rows, which are contiguous in memory: one bulk copy per fill, rows of any
//     alignment; chunk sums of a row meet in a small table and the warp that refills the slot adds them;
//   * the 6-bit value is never assembled: nibbles and bit pairs are multiplied separately (dp4a) in
//     place and the place values (x16, x4, x16, x64) are shifted out of the integer sums;
//     sum (q-32)*a uses the activation's 16-wide block sums.  All integer arithmetic is exact, the block
//     term is (d*d8)*sumi as in fused_dot_q6k_q8k (src/quant/cpu/kernels/simd/fused_q6k_q8k_dot.rs:170-224).
struct GemvM1Q6Params {
    const uint8_t* w;
    const void* act;
    const float* norm_w;  // RMSNorm prologue (see GemvM1Params)
    float norm_eps;
    void* out;
    uint32_t K, N;
    uint32_t nblk;          // K / 256 (<= 64)
    uint32_t row_bytes;     // nblk * 210
    uint32_t rows_per_cta;  // CTA c owns rows [c * rows_per_cta, min(N, (c + 1) * rows_per_cta))
    uint32_t lpr;           // single chunk: lanes per row = 2 * (nblk rounded up to a power of two)
    uint32_t stage_bytes;   // rows of a fill + room for the phase of an unaligned first row
    uint32_t nstages;
    uint32_t act_off, stage_off;
    int act_dtype, out_dtype;
    unsigned int* status;
    PeerComm comm;  // row-parallel shard: push the partial row to every rank and add them up (f32 out)
    NextHint next;
};

// activation image per 256-block (stride 416 B), one 144-byte record per 128-element half n:
//   [144 n, 144 n + 128) int8 codes | [144 n + 128, 144 n + 144) 8 x int16 sums of 16;   [288,292) f32 d8
// Lane (b, n) copies record n of block b into registers with 16-byte loads; with the records 36 words apart and
// the blocks 8 words past a multiple of 32, the eight lanes of a quarter-warp hit all 32 banks once.
constexpr int ACT6_STRIDE = 416, ACT6_HALF = 144, ACT6_SUMS = 128, ACT6_SUMS_HALF = 144;
// half n: codes at ACT6_HALF * n, sums at ACT6_SUMS + ACT6_SUMS_HALF * n

template <int I>
__device__ __forceinline__ int sbyte(uint32_t x) {
    int r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(x), "r"(0u), "n"(((I | 8) << 12) | ((I | 8) << 8) | ((I | 8) << 4) | I));
    return r;
}


// Integer sum over half `n` (128 elements) of the Q6_K block at `blk` (2-byte aligned in shared memory)
// against the int8 codes `a` / 16-wide sums `bs` of the matching activation half; also returns d.
__device__ __forceinline__ int q6k_half_sum(const uint8_t* blk, int n, const uint32_t (&a)[32],
                                    const uint32_t (&bs)[4], float& d6) {
    int half_sum = 0;
    const uint32_t odd = (uint32_t)(reinterpret_cast<uintptr_t>(blk) & 2);     // the block starts 2 bytes past a word boundary
    const uint32_t sel = odd ? 0x5432u : 0x3210u;
    const uint32_t* W = reinterpret_cast<const uint32_t*>(blk - odd);          // aligned words covering the block
    auto word = [&](int i) { return __byte_perm(W[i], W[i + 1], sel); };   // bytes [4i, 4i+4) of the block
    const uint32_t sc0 = word(48 + 2 * n), sc1 = word(49 + 2 * n);          // 8 signed scales of this half
    d6 = f16bits_to_f32(*reinterpret_cast<const unsigned short*>(blk + 208));
#pragma unroll
    for (int is = 0; is < 2; ++is) {
        int dn[4] = {0, 0, 0, 0}, dh[4] = {0, 0, 0, 0};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = 4 * is + i;
            const uint32_t l0 = word(16 * n + idx), l1 = word(16 * n + 8 + idx), hw = word(32 + 8 * n + idx);
            dn[0] = dp4a_u8s8(l0 & 0x0F0F0F0Fu, a[4 * (0 + is) + i], dn[0]);
            dn[1] = dp4a_u8s8(l1 & 0x0F0F0F0Fu, a[4 * (2 + is) + i], dn[1]);
            dn[2] = dp4a_u8s8(l0 & 0xF0F0F0F0u, a[4 * (4 + is) + i], dn[2]);
            dn[3] = dp4a_u8s8(l1 & 0xF0F0F0F0u, a[4 * (6 + is) + i], dn[3]);
            dh[0] = dp4a_u8s8(hw & 0x03030303u, a[4 * (0 + is) + i], dh[0]);
            dh[1] = dp4a_u8s8(hw & 0x0C0C0C0Cu, a[4 * (2 + is) + i], dh[1]);
            dh[2] = dp4a_u8s8(hw & 0x30303030u, a[4 * (4 + is) + i], dh[2]);
            dh[3] = dp4a_u8s8(hw & 0xC0C0C0C0u, a[4 * (6 + is) + i], dh[3]);
        }
        // sub-block (gq, is): local index sb = 2 gq + is; q.a = nibble part + 16 * bit-pair part
        const int qa0 = dn[0] + (dh[0] << 4);
        const int qa1 = dn[1] + (dh[1] << 2);
        const int qa2 = (dn[2] >> 4) + dh[2];
        const int qa3 = (dn[3] >> 4) + (dh[3] >> 2);
        const int b0 = is ? (int)bs[0] >> 16 : (int)(short)(bs[0] & 0xFFFF);
        const int b1 = is ? (int)bs[1] >> 16 : (int)(short)(bs[1] & 0xFFFF);
        const int b2 = is ? (int)bs[2] >> 16 : (int)(short)(bs[2] & 0xFFFF);
        const int b3 = is ? (int)bs[3] >> 16 : (int)(short)(bs[3] & 0xFFFF);
        const int s0 = is ? sbyte<1>(sc0) : sbyte<0>(sc0);
        const int s1 = is ? sbyte<3>(sc0) : sbyte<2>(sc0);
        const int s2 = is ? sbyte<1>(sc1) : sbyte<0>(sc1);
        const int s3 = is ? sbyte<3>(sc1) : sbyte<2>(sc1);
        half_sum += s0 * (qa0 - 32 * b0) + s1 * (qa1 - 32 * b1) + s2 * (qa2 - 32 * b2) + s3 * (qa3 - 32 * b3);
    }
    return half_sum;
}

template <int NCHUNK>
__device__ __forceinline__ void q6k_body(const GemvM1Q6Params& p, const uint32_t cta, uint8_t* smem) {
    // One warp per row and chunk; with a single chunk a row takes only `lpr` lanes (twice the block count
    // rounded up to a power of two), so short rows (K-split shards) put 32 / lpr rows into a warp.
    const uint32_t lpr = NCHUNK == 1 ? p.lpr : 32u, lpr_log = 31 - __clz(lpr), rpw = 32u >> lpr_log;
    const uint32_t RPF = NCHUNK == 1 ? 4u * rpw : 4u / NCHUNK;  // rows per fill
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_full = smem_u32(smem), bar_empty = bar_full + 128;
    float* part = reinterpret_cast<float*>(smem + 256);  // [16 slots][4 warps of the group]
    uint8_t* act_s = smem + p.act_off;
    const uint32_t stage0 = smem_u32(smem + p.stage_off);

    const uint32_t row_begin = cta * p.rows_per_cta;
    const uint32_t row_end = min(p.N, row_begin + p.rows_per_cta);
    const uint32_t nfill = row_end > row_begin ? (row_end - row_begin + RPF - 1) / RPF : 0;

    auto issue_fill = [&](uint32_t f, uint32_t slot) {  // one lane
        const uint32_t r0 = row_begin + f * RPF;
        const uint32_t nrows = min(RPF, row_end - r0);
        fill_contiguous(stage0 + slot * p.stage_bytes, smem + p.stage_off + slot * p.stage_bytes, p.w + (size_t)r0 * p.row_bytes,
                        nrows * p.row_bytes, p.w + (size_t)p.N * p.row_bytes, bar_full + 8 * slot);
    };

    // Short rows: two fills leave before the grid dependency is resolved, the rest of the ring after the
    // activation loads (responses return in request order, so loads behind a full ring would wait for it).
    // Long rows (several warps per row, eight activation loads per lane): the whole ring leaves first.  This
    // kernel's end is set by when its weights arrive, and fills slip in between the many loads anyway.
    if (warp == 15 && (uint32_t)lane < p.nstages) {
        mbar_init(bar_full + 8 * lane, 1);
        mbar_init(bar_empty + 8 * lane, 4);
        mbar_fence_init();
    }
    __syncthreads();
    const uint32_t early = NCHUNK > 1 ? p.nstages : 2u;
    if (warp == 15 && (uint32_t)lane < early && (uint32_t)lane < nfill) issue_fill(lane, lane);
    grid_dep_launch();
    grid_dep_wait();
    const bool tp = p.comm.world > 1;
    const uint32_t tp_e = tp ? tp_epoch(p.comm) : 0u;

    // 1. quantise the activation row: warp w takes blocks w, w + 16, ... (8 values per lane)
    {
        float v[NCHUNK][8];
#pragma unroll
        for (int j = 0; j < NCHUNK; ++j) {
            const uint32_t qb = warp + 16 * j;
            if (qb < p.nblk) load_act8(p.act, p.act_dtype, (size_t)qb * 256 + 8 * lane, v[j]);
        }
        const uint32_t f1 = early + (uint32_t)warp;
        if (lane == 0 && f1 < p.nstages && f1 < nfill) issue_fill(f1, f1);
        if (warp == 15 && lane == 0 && nfill <= p.nstages) prefetch_next(p.next, blockIdx.x);
        if (p.norm_w) {  // uniform over the launch
            float sq = 0.f;
#pragma unroll
            for (int j = 0; j < NCHUNK; ++j)
                if (warp + 16 * j < p.nblk)
#pragma unroll
                    for (int i = 0; i < 8; ++i) sq = fmaf(v[j][i], v[j][i], sq);
            const float rs = rms_factor(sq, part, warp, lane, p.K, p.norm_eps);  // `part` is not in use yet
            __syncthreads();                                                     // ... and is free again before the loop
#pragma unroll
            for (int j = 0; j < NCHUNK; ++j) {
                const uint32_t qb = warp + 16 * j;
                if (qb < p.nblk) {
                    const float4 g0 = __ldg(reinterpret_cast<const float4*>(p.norm_w + (size_t)qb * 256 + 8 * lane));
                    const float4 g1 = __ldg(reinterpret_cast<const float4*>(p.norm_w + (size_t)qb * 256 + 8 * lane) + 1);
                    const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[j][i] = __fmul_rn(__fmul_rn(v[j][i], rs), g[i]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < NCHUNK; ++j) {
            const uint32_t qb = warp + 16 * j;
            if (qb < p.nblk) {  // warp-uniform
                uint2 packed;
                int s;
                const float d8 = quantize_block8(v[j], packed, s);
                uint8_t* blk = act_s + qb * ACT6_STRIDE;
                const int hn = lane >> 4;  // the half this lane's 8 values belong to
                *reinterpret_cast<uint2*>(blk + ACT6_HALF * hn + 8 * (lane & 15)) = packed;
                s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);  // 16 elements = 2 lanes
                if ((lane & 1) == 0) *reinterpret_cast<short*>(blk + ACT6_SUMS + ACT6_SUMS_HALF * hn + 2 * ((lane >> 1) & 7)) = (short)s;
                if (lane == 0) *reinterpret_cast<float*>(blk + 288) = d8;
            }
        }
    }
    __syncthreads();

    // 2. this lane's activation half-block goes to registers
    const uint32_t grp = (uint32_t)warp >> 2, wi = (uint32_t)warp & 3;
    const uint32_t r = NCHUNK == 1 ? wi * rpw + ((uint32_t)lane >> lpr_log) : wi / NCHUNK;  // row of the fill
    const uint32_t c = NCHUNK == 1 ? 0u : wi % NCHUNK;                                   // K-chunk
    const int b = (lane & (lpr - 1)) >> 1, n = lane & 1;
    const uint32_t gblk = c * 16 + b;
    const bool role = gblk < p.nblk;
    uint32_t a[32], bs[4];
    float d8 = 0.f;
    if (role) {
        const uint8_t* blk = act_s + gblk * ACT6_STRIDE;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            uint4 q = *reinterpret_cast<const uint4*>(blk + ACT6_HALF * n + 16 * i);
            a[4 * i] = q.x; a[4 * i + 1] = q.y; a[4 * i + 2] = q.z; a[4 * i + 3] = q.w;
        }
        uint4 q = *reinterpret_cast<const uint4*>(blk + ACT6_SUMS + ACT6_SUMS_HALF * n);
        bs[0] = q.x; bs[1] = q.y; bs[2] = q.z; bs[3] = q.w;
        d8 = *reinterpret_cast<const float*>(blk + 288);
    }

    auto store_row = [&](uint32_t row, float val) {
        if (tp && p.comm.gather) tp_push_gather(p.comm, tp_e, p.comm.rank * p.N + row, val);
        else if (tp) tp_push(p.comm, tp_e, row, val);
        else if (p.out_dtype == DT_F32) static_cast<float*>(p.out)[row] = val;
        else if (p.out_dtype == DT_BF16) static_cast<__nv_bfloat16*>(p.out)[row] = __float2bfloat16_rn(val);
        else static_cast<__half*>(p.out)[row] = __float2half_rn(val);
    };

    bool dead = false;
    uint32_t slot = grp, par = 0;  // fill f lives in ring slot f % nstages (nstages >= 4)
    for (uint32_t f = grp; f < nfill; f += 4) {
        if (!dead && !mbar_wait(bar_full + 8 * slot, par)) {
            dead = true;
            atomicOr(p.status, STATUS_TIMEOUT_FULL);
        }
        const uint32_t r0 = row_begin + f * RPF;
        const uint32_t nrows = min(RPF, row_end - r0);
        const uint32_t phase = (uint32_t)((reinterpret_cast<uintptr_t>(p.w) + (size_t)r0 * p.row_bytes) & 15);
        const bool on = !dead && role && r < nrows;
        int half_sum = 0;
        float d6 = 0.f;
        if (on) half_sum = q6k_half_sum(smem + p.stage_off + slot * p.stage_bytes + phase + r * p.row_bytes + gblk * 210, n, a, bs, d6);
        const int sumi = half_sum + __shfl_xor_sync(0xFFFFFFFFu, half_sum, 1);
        float term = on ? __fmul_rn(__fmul_rn(d6, d8), (float)sumi) : 0.f;
#pragma unroll
        for (uint32_t o = 16; o > 1; o >>= 1)
            if (o < lpr) term += __shfl_xor_sync(0xFFFFFFFFu, term, o);
        if (NCHUNK == 1) {
            if ((lane & (lpr - 1)) == 0 && on) store_row(r0 + r, term);
        } else {
            if (lane == 0) part[slot * 4 + wi] = term;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + 8 * slot);
        // one warp of the group (they take turns) waits for its siblings, adds the chunk sums of the
        // fill's rows and refills the slot
        const bool refill = f + p.nstages < nfill;
        if (((f >> 2) & 3) == wi && (NCHUNK > 1 || refill)) {
            if (!dead && !mbar_wait(bar_empty + 8 * slot, par)) {
                dead = true;
                atomicOr(p.status, STATUS_TIMEOUT_EMPTY);
            }
            if (NCHUNK > 1 && !dead && (uint32_t)lane < nrows) {
                float tot = 0.f;
#pragma unroll
                for (int k = 0; k < NCHUNK; ++k) tot = __fadd_rn(tot, part[slot * 4 + lane * NCHUNK + k]);
                store_row(r0 + lane, tot);
            }
            __syncwarp();
            if (!dead && refill && lane == 0) {
                issue_fill(f + p.nstages, slot);
                if (f + p.nstages + 1 == nfill) prefetch_next(p.next, blockIdx.x);
            }
        }
        slot += 4;
        if (slot >= p.nstages) {
            slot -= p.nstages;
            par ^= 1;
        }
    }
    if (tp && p.comm.gather) tp_finish_gather(p.comm, tp_e, static_cast<float*>(p.out), p.status);
    else if (tp) tp_finish(p.comm, tp_e, row_begin, row_end, static_cast<float*>(p.out), p.status);
}

template <int NCHUNK>
__global__ void __launch_bounds__(512, 1) gemv_m1_q6k_kernel(const __grid_constant__ GemvM1Q6Params p) {
    extern __shared__ __align__(128) uint8_t smem[];
    q6k_body<NCHUNK>(p, blockIdx.x, smem);
}

// Q4_K weights and one Q6_K weight that share the activation row (the q/k/v projections of a Q4_K_M
// model) in ONE launch: the first `split` CTAs stream the Q4_K rows, the others the Q6_K rows.
__global__ void __launch_bounds__(512, 1) gemv_m1_mixed_kernel(const __grid_constant__ GemvM1Params p4,
                                                               const __grid_constant__ GemvM1Q6Params p6, const uint32_t split) {
    extern __shared__ __align__(128) uint8_t smem[];
    if (blockIdx.x < split) q4k_body<false>(p4, blockIdx.x, smem);
    else q6k_body<1>(p6, blockIdx.x - split, smem);
}

}  // namespace

bool gemv_m1_supported(int fmt, size_t M, size_t K, size_t N, bool swiglu) {
    if (M != 1 || N < 1 || K % 256) return false;
    if (fmt == FMT_Q4_K) return K <= 4096;
    // Q6_K: the activation image must fit beside the stages
    if (fmt == FMT_Q6_K) return !swiglu && K <= 16384;
    return false;
}

constexpr size_t M1_SMEM_MAX = 232448 - 1024;

// Fills in the Q6_K parameters for a launch on at most `max_grid` CTAs; returns the grid, 0 if none.
static size_t setup_q6k(GemvM1Q6Params& p, uint32_t& nchunk, size_t& smem, const void* act, int act_dtype, const void* w, void* out,
                        int out_dtype, size_t K, size_t N, size_t max_grid, unsigned int* status) {
    p = GemvM1Q6Params{};
    p.w = static_cast<const uint8_t*>(w);
    p.act = act;
    p.out = out;
    p.K = (uint32_t)K;
    p.N = (uint32_t)N;
    p.nblk = (uint32_t)(K / 256);
    nchunk = p.nblk <= 16 ? 1 : p.nblk <= 32 ? 2 : 4;
    p.lpr = 2;
    while (p.lpr < 2 * p.nblk && p.lpr < 32) p.lpr *= 2;
    const uint32_t rpf = nchunk == 1 ? 4 * (32 / p.lpr) : 4 / nchunk;
    p.row_bytes = p.nblk * 210;
    p.stage_bytes = (rpf * p.row_bytes + 32 + 127) & ~127u;  // + phase of an unaligned first row + round-up
    p.act_off = 512;  // [0,256) barriers, [256,512) chunk-sum table
    p.stage_off = (p.act_off + p.nblk * ACT6_STRIDE + 127) & ~127u;
    p.nstages = (uint32_t)((M1_SMEM_MAX - p.stage_off - 64) / p.stage_bytes);
    if (p.nstages > 16) p.nstages = 16;
    // never fewer than ~16 rows per CTA
    size_t grid = (N + 15) / 16;
    if (grid > max_grid) grid = max_grid;
    p.rows_per_cta = (uint32_t)((N + grid - 1) / grid);
    grid = (N + p.rows_per_cta - 1) / p.rows_per_cta;
    p.act_dtype = act_dtype;
    p.out_dtype = out_dtype;
    p.status = status;
    smem = p.stage_off + (size_t)p.nstages * p.stage_bytes + 64;  // +64: the aligned word read past the last block
    return grid;
}

// Same for Q4_K: `nseg` weights (1..3) sharing one activation row, or gate/up for SwiGLU.
static size_t setup_q4k(GemvM1Params& p, size_t& smem, const void* act, int act_dtype, int nseg, const void* const* w,
                        const size_t* n, void* const* out, const void* w_up, int out_dtype, size_t K, size_t max_grid,
                        unsigned int* status) {
    p = GemvM1Params{};
    size_t N = 0;
    for (int i = 0; i < nseg && i < 3; ++i) {
        p.w[i] = static_cast<const uint8_t*>(w[i]);
        p.out[i] = out[i];
        N += n[i];
        p.seg_end[i] = (uint32_t)N;
    }
    p.nseg = (uint32_t)nseg;
    p.w2 = static_cast<const uint8_t*>(w_up);
    p.act = act;
    p.K = (uint32_t)K;
    p.N = (uint32_t)N;
    p.nblk = (uint32_t)(K / 256);
    p.row_bytes = p.nblk * 144;
    p.lpr = 1;
    while (p.lpr < p.nblk) p.lpr *= 2;
    if (p.lpr < 2) p.lpr = 2;
    p.stage_bytes = (w_up ? 8 : 4 * (32 / p.lpr)) * p.row_bytes;  // 4 warps x rows per warp (SwiGLU: 4 gate + 4 up); multiple of 128
    p.act_off = 320;  // [0,256) barriers, [256,320) the warp sums of the RMSNorm prologue
    p.stage_off = (p.act_off + 16 * ACT_STRIDE + 127) & ~127u;
    p.nstages = (uint32_t)((M1_SMEM_MAX - p.stage_off) / p.stage_bytes);
    if (p.nstages > 16) p.nstages = 16;
    size_t grid = (N + 15) / 16;
    if (grid > max_grid) grid = max_grid;
    p.rows_per_cta = (uint32_t)((N + grid - 1) / grid);
    grid = (N + p.rows_per_cta - 1) / p.rows_per_cta;
    p.act_dtype = act_dtype;
    p.out_dtype = out_dtype;
    p.status = status;
    smem = p.stage_off + (size_t)p.nstages * p.stage_bytes;
    return grid;
}

static cudaError_t m1_attrs() {
    static PerDeviceOnce attrs;
    return attrs.run([] {
    const int v = (int)M1_SMEM_MAX;
    cudaError_t e = cudaFuncSetAttribute(gemv_m1_q4k_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, v);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_m1_q4k_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, v);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_m1_q6k_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, v);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_m1_q6k_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, v);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_m1_q6k_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, v);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_m1_mixed_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, v);
    return e;
    });
}

// Number of CTAs that stream the Q6_K weight of a mixed launch: the SMs are divided in proportion to the
// packed bytes, Q6_K bytes counting 1.3x (more arithmetic per byte).
static size_t mixed_q6k_ctas(size_t n4, size_t n6, int sm_count) {
    const double b4 = (double)n4 * 144.0, b6 = (double)n6 * 210.0 * 1.3;
    size_t g6 = (size_t)((double)sm_count * b6 / (b4 + b6) + 0.5);
    if (g6 < 1) g6 = 1;
    if (g6 > (size_t)sm_count - 1) g6 = (size_t)sm_count - 1;
    return g6;
}

// ---- the hint about the launch after the next one (see NextHint) ----
namespace {
thread_local NextHint t_next = {};   // taken by the next M = 1 launch of this thread
thread_local NextHint t_stash = {};
thread_local int t_next_device = -1;  // the device that was current when the hint was given: its weights live there
NextHint take_next() {
    NextHint h = t_next;
    t_next.nsp = 0;
    int dev = -1;
    if (h.nsp && (cudaGetDevice(&dev) != cudaSuccess || dev != t_next_device)) h.nsp = 0;  // a launch on another device drops it
    return h;
}
void space_of(NextSpace& sp, const GemvM1Params& p, size_t grid, size_t cta0) {
    sp = NextSpace{};
    for (int i = 0; i < 3; ++i) {
        sp.w[i] = p.w[i];
        sp.seg_end[i] = p.seg_end[i];
    }
    sp.w2 = p.w2;
    sp.nseg = p.nseg;
    sp.row_bytes = p.row_bytes;
    sp.rows_per_cta = p.rows_per_cta;
    sp.cta0 = (uint32_t)cta0;
    sp.ncta = (uint32_t)grid;
}
void space_of(NextSpace& sp, const GemvM1Q6Params& p, size_t grid, size_t cta0) {
    sp = NextSpace{};
    sp.w[0] = p.w;
    sp.seg_end[0] = p.N;
    sp.nseg = 1;
    sp.row_bytes = p.row_bytes;
    sp.rows_per_cta = p.rows_per_cta;
    sp.cta0 = (uint32_t)cta0;
    sp.ncta = (uint32_t)grid;
}
}  // namespace

void m1_next_clear() { t_next.nsp = 0; }
void m1_next_stash() {
    t_stash = t_next;
    t_next.nsp = 0;
}
void m1_next_unstash() {
    t_next = t_stash;
    t_stash.nsp = 0;
}

// Describes the first launch of the coming single-row operation (the same choices as the dispatch makes):
// `n_weights` weights [N[i], K] sharing the activation row, or gate and up of a SwiGLU.  Returns false, and
// leaves no hint, when that operation would not run on the kernels of this file.
bool m1_next_set(bool swiglu, int n_weights, const int* formats, const void* const* w, const size_t* N, size_t K, int sm_count) {
    t_next.nsp = 0;
    if (n_weights < 1 || !formats || !w || !N || sm_count < 2) return false;
    for (int i = 0; i < n_weights && i < 4; ++i)
        if (!w[i] || N[i] == 0 || N[i] > 0x7FFFFFFFu) return false;
    // Bytes per CTA: what the memory system delivers to one SM while a launch drains and the next one starts up
    // (about 2 us at 1/148 of the HBM rate); measured flat between 80 and 104 KB, worse outside.
    constexpr uint32_t head_bytes = 96u * 1024u;
    NextHint h = {};
    h.head = head_bytes;
    void* const no_out[3] = {nullptr, nullptr, nullptr};
    size_t smem;
    if (swiglu) {
        if (n_weights != 2 || formats[0] != FMT_Q4_K || formats[1] != FMT_Q4_K || N[0] != N[1] || !gemv_m1_supported(FMT_Q4_K, 1, K, N[0], true))
            return false;
        GemvM1Params p;
        const size_t grid = setup_q4k(p, smem, nullptr, DT_F32, 1, w, N, no_out, w[1], DT_F32, K, (size_t)sm_count, nullptr);
        space_of(h.sp[0], p, grid, 0);
        h.nsp = 1;
        h.head = head_bytes / 2;
    } else if (formats[0] == FMT_Q4_K && gemv_m1_supported(FMT_Q4_K, 1, K, N[0], false)) {
        int run = 1;
        while (run < 3 && run < n_weights && formats[run] == FMT_Q4_K) ++run;
        const bool mixed = run < n_weights && formats[run] == FMT_Q6_K && gemv_m1_supported(FMT_Q6_K, 1, K, N[run], false);
        GemvM1Params p4;
        if (mixed) {
            size_t n4 = 0;
            for (int i = 0; i < run; ++i) n4 += N[i];
            const size_t g6 = mixed_q6k_ctas(n4, N[run], sm_count);
            GemvM1Q6Params p6;
            uint32_t nchunk;
            const size_t grid4 = setup_q4k(p4, smem, nullptr, DT_F32, run, w, N, no_out, nullptr, DT_F32, K, (size_t)sm_count - g6, nullptr);
            const size_t grid6 = setup_q6k(p6, nchunk, smem, nullptr, DT_F32, w[run], nullptr, DT_F32, K, N[run], g6, nullptr);
            space_of(h.sp[0], p4, grid4, 0);
            space_of(h.sp[1], p6, grid6, grid4);
            h.nsp = 2;
        } else {
            const size_t grid = setup_q4k(p4, smem, nullptr, DT_F32, run, w, N, no_out, nullptr, DT_F32, K, (size_t)sm_count, nullptr);
            space_of(h.sp[0], p4, grid, 0);
            h.nsp = 1;
        }
    } else if (formats[0] == FMT_Q6_K && gemv_m1_supported(FMT_Q6_K, 1, K, N[0], false)) {
        GemvM1Q6Params p6;
        uint32_t nchunk;
        const size_t grid = setup_q6k(p6, nchunk, smem, nullptr, DT_F32, w[0], nullptr, DT_F32, K, N[0], (size_t)sm_count, nullptr);
        space_of(h.sp[0], p6, grid, 0);
        h.nsp = 1;
    } else {
        return false;
    }
    if (cudaGetDevice(&t_next_device) != cudaSuccess) return false;
    t_next = h;
    return true;
}

static cudaError_t launch_gemv_m1_q6k(const void* act, int act_dtype, const void* w, void* out, int out_dtype, size_t K,
                                      size_t N, int sm_count, cudaStream_t st, unsigned int* status, const float* norm_w, float norm_eps) {
    GemvM1Q6Params p;
    uint32_t nchunk;
    size_t smem;
    const size_t grid = setup_q6k(p, nchunk, smem, act, act_dtype, w, out, out_dtype, K, N, (size_t)sm_count, status);
    p.norm_w = norm_w;
    p.norm_eps = norm_eps;
    p.next = take_next();
    cudaError_t e = m1_attrs();
    if (e != cudaSuccess) return e;
    cudaError_t le = nchunk == 1   ? launch_pdl(gemv_m1_q6k_kernel<1>, dim3((unsigned)grid), dim3(512), smem, st, p)
                     : nchunk == 2 ? launch_pdl(gemv_m1_q6k_kernel<2>, dim3((unsigned)grid), dim3(512), smem, st, p)
                                   : launch_pdl(gemv_m1_q6k_kernel<4>, dim3((unsigned)grid), dim3(512), smem, st, p);
    note_launch();
    return le != cudaSuccess ? le : cudaGetLastError();
}

// Q4_K, M = 1: `nseg` weights (1..3) sharing one activation row, each [n[i], K] with its own output.
cudaError_t launch_gemv_m1_batch(const void* act, int act_dtype, int nseg, const void* const* w, const size_t* n,
                                 void* const* out, const void* w_up, int out_dtype, size_t K, int sm_count, cudaStream_t st,
                                 unsigned int* status, const float* norm_w, float norm_eps) {
    GemvM1Params p;
    size_t smem;
    const size_t grid = setup_q4k(p, smem, act, act_dtype, nseg, w, n, out, w_up, out_dtype, K, (size_t)sm_count, status);
    p.norm_w = norm_w;
    p.norm_eps = norm_eps;
    p.next = take_next();
    cudaError_t e = m1_attrs();
    if (e != cudaSuccess) return e;
    cudaError_t le = w_up ? launch_pdl(gemv_m1_q4k_kernel<true>, dim3((unsigned)grid), dim3(512), smem, st, p)
                          : launch_pdl(gemv_m1_q4k_kernel<false>, dim3((unsigned)grid), dim3(512), smem, st, p);
    note_launch();
    return le != cudaSuccess ? le : cudaGetLastError();
}

// `nseg` Q4_K weights plus one Q6_K weight [n6, K] on the same activation row, one launch.
cudaError_t launch_gemv_m1_mixed(const void* act, int act_dtype, int nseg, const void* const* w, const size_t* n,
                                 void* const* out, const void* w6, size_t n6, void* out6, int out_dtype, size_t K, int sm_count,
                                 cudaStream_t st, unsigned int* status, const float* norm_w, float norm_eps) {
    size_t n4 = 0;
    for (int i = 0; i < nseg; ++i) n4 += n[i];
    const size_t g6 = mixed_q6k_ctas(n4, n6, sm_count);
    GemvM1Params p4;
    GemvM1Q6Params p6;
    uint32_t nchunk;
    size_t smem4, smem6;
    const size_t grid4 = setup_q4k(p4, smem4, act, act_dtype, nseg, w, n, out, nullptr, out_dtype, K, (size_t)sm_count - g6, status);
    const size_t grid6 = setup_q6k(p6, nchunk, smem6, act, act_dtype, w6, out6, out_dtype, K, n6, g6, status);
    p4.norm_w = p6.norm_w = norm_w;
    p4.norm_eps = p6.norm_eps = norm_eps;
    p4.next = p6.next = take_next();
    cudaError_t e = m1_attrs();
    if (e != cudaSuccess) return e;
    cudaError_t le = launch_pdl(gemv_m1_mixed_kernel, dim3((unsigned)(grid4 + grid6)), dim3(512), smem4 > smem6 ? smem4 : smem6, st,
                                p4, p6, (uint32_t)grid4);
    note_launch();
    return le != cudaSuccess ? le : cudaGetLastError();
}

// Row-parallel shard, M = 1: the local product's row is pushed to every rank and the rank-ordered sum
// lands in `out` (f32), all in this one launch.
cudaError_t launch_gemv_m1_rowpar(int fmt, const void* act, int act_dtype, const void* w, void* out, size_t K, size_t N,
                                  int sm_count, cudaStream_t st, unsigned int* status, const PeerComm& comm) {
    const NextHint next = take_next();
    cudaError_t e = m1_attrs();
    if (e != cudaSuccess) return e;
    cudaError_t le;
    size_t smem;
    if (fmt == FMT_Q6_K) {
        GemvM1Q6Params p;
        uint32_t nchunk;
        const size_t grid = setup_q6k(p, nchunk, smem, act, act_dtype, w, out, DT_F32, K, N, (size_t)sm_count, status);
        p.comm = comm;
        p.next = next;
            le = nchunk == 1   ? launch_pdl(gemv_m1_q6k_kernel<1>, dim3((unsigned)grid), dim3(512), smem, st, p)
             : nchunk == 2 ? launch_pdl(gemv_m1_q6k_kernel<2>, dim3((unsigned)grid), dim3(512), smem, st, p)
                           : launch_pdl(gemv_m1_q6k_kernel<4>, dim3((unsigned)grid), dim3(512), smem, st, p);
    } else {
        GemvM1Params p;
        const size_t grid = setup_q4k(p, smem, act, act_dtype, 1, &w, &N, &out, nullptr, DT_F32, K, (size_t)sm_count, status);
        p.comm = comm;
        p.next = next;
            le = launch_pdl(gemv_m1_q4k_kernel<false>, dim3((unsigned)grid), dim3(512), smem, st, p);
    }
    note_launch();
    return le != cudaSuccess ? le : cudaGetLastError();
}

cudaError_t launch_gemv_m1(int fmt, const void* act, int act_dtype, const void* w, const void* w_up, void* out,
                           int out_dtype, size_t K, size_t N, int sm_count, cudaStream_t st, unsigned int* status,
                           const float* norm_w, float norm_eps) {
    if (fmt == FMT_Q6_K) return launch_gemv_m1_q6k(act, act_dtype, w, out, out_dtype, K, N, sm_count, st, status, norm_w, norm_eps);
    return launch_gemv_m1_batch(act, act_dtype, 1, &w, &N, &out, w_up, out_dtype, K, sm_count, st, status, norm_w, norm_eps);
}

// Stand-alone RMSNorm (one CTA per row) for the shapes whose kernels have no fused prologue: the normalised row goes
// to scratch as f32 and the quantized product reads it from there.  Same expression as the fused form:
// x * (1 / sqrt(mean(x^2) + eps)) * w, squares added 8 per lane then across the warp, warp sums in warp order.
__global__ void __launch_bounds__(512) rmsnorm_kernel(const void* __restrict__ act, int act_dtype, const float* __restrict__ norm_w, float eps,
                                                      float* __restrict__ out, uint32_t K) {
    __shared__ float red[16];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t row = blockIdx.x;
    grid_dep_launch();
    grid_dep_wait();
    float sq = 0.f;
    for (uint32_t k0 = threadIdx.x * 8; k0 < K; k0 += 512 * 8) {
        float v[8];
        load_act8(act, act_dtype, row * K + k0, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) sq = fmaf(v[i], v[i], sq);
    }
    const float rs = rms_factor(sq, red, warp, lane, K, eps);
    for (uint32_t k0 = threadIdx.x * 8; k0 < K; k0 += 512 * 8) {
        float v[8];
        load_act8(act, act_dtype, row * K + k0, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) out[row * K + k0 + i] = __fmul_rn(__fmul_rn(v[i], rs), __ldg(norm_w + k0 + i));
    }
}

cudaError_t launch_rmsnorm(const void* act, int act_dtype, const float* norm_w, float eps, float* out, size_t M, size_t K, cudaStream_t st) {
    cudaError_t e = launch_pdl(rmsnorm_kernel, dim3((unsigned)M), dim3(512), 0, st, act, act_dtype, norm_w, eps, out, (uint32_t)K);
    note_launch();
    return e != cudaSuccess ? e : cudaGetLastError();
}

// All-reduce (sum) of `count` f32 values in place over the exchange buffers, for the small messages of row-parallel
// products that have no exchange inside their kernel (2 <= M <= 16 rows, or formats without a fused decode kernel):
// stands in for all_reduce_tensor + sync (src/distributed/comm_utils.rs:15-39).  Each CTA pushes its share of the
// values to every rank as tagged 8-byte stores and then adds, for the same elements, the ranks' values in rank order,
// so all ranks hold bit-identical sums.  Every poll is bounded (tp_finish).
__global__ void __launch_bounds__(256) tp_all_reduce_kernel(float* data, uint32_t count, const __grid_constant__ PeerComm comm,
                                                            unsigned int* status) {
    grid_dep_launch();
    grid_dep_wait();
    const uint32_t e = tp_epoch(comm);
    const uint32_t chunk = (count + gridDim.x - 1) / gridDim.x;
    const uint32_t begin = min(count, blockIdx.x * chunk), end = min(count, begin + chunk);
    for (uint32_t i = begin + threadIdx.x; i < end; i += blockDim.x) tp_push(comm, e, i, data[i]);
    tp_finish(comm, e, begin, end, data, status);
}

cudaError_t launch_tp_all_reduce(float* data, size_t count, const PeerComm& comm, int sm_count, cudaStream_t st, unsigned int* status) {
    unsigned grid = (unsigned)((count + 255) / 256);
    if (grid > (unsigned)sm_count) grid = (unsigned)sm_count;
    if (grid < 1) grid = 1;
    cudaError_t e = launch_pdl(tp_all_reduce_kernel, dim3(grid), dim3(256), 0, st, data, (uint32_t)count, comm, status);
    note_launch();
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace b200q
