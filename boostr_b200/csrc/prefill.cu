// Prefill GEMM (M >= 64) on the 5th-generation tensor cores:  out[M,N] = act[M,K] x dequant(W[N,K])^T.
//
// Stands in for boostr's quant_matmul_*_f32 "GEMM" kernels (src/quant/cuda/kernels/quant_matmul.cu:20-330:
// scalar decode + FFMA, no tensor cores).  Here the contraction runs on tcgen05.mma with the accumulator
// in tensor memory:
//   * orientation: the WEIGHT tile is the MMA's A operand (128 weight rows = the 128 TMEM lanes), the
//     ACTIVATION tile is the B operand (MT = 64/128/256 activation rows = TMEM columns).  The packed
//     weights are decoded once per (128 x MT) output tile, so a larger MT amortises the decode.
//   * persistent: one CTA per SM walks the output tiles; tensor memory holds TWO accumulators, so four
//     epilogue warps drain tile i (tcgen05.ld: lane = weight row, columns = activation rows; out[m, n]
//     stored with n contiguous across lanes) while the MMA warp already accumulates tile i + 1;
//   * activations are bf16 [M,K] (prepared once per call) and arrive by TMA (cp.async.bulk.tensor.2d,
//     128-byte swizzle, no multicast) into their own ring;
//   * four sets of four dequant warps take the K steps (64 wide) in turn; a thread owns a weight row and
//     decodes its 64 elements exactly in f32 (the dequant kernel's values: a byte permute and one FMA per
//     element), rounds once to bf16 and stores them into its lane of the step's tile in tensor memory,
//     from where the MMA reads its A operand;
//   * Q4_K: the packed blocks themselves arrive by TMA as tiles of 128 rows x one 144-byte block (four
//     K steps), double buffered, and are read from shared memory with conflict-free 16-byte loads
//     (per-thread 16-byte global loads touch 32 lines per warp instruction; they kept the L1 data pipe
//     73 % busy);
//   * one thread issues four 128 x MT x 16 tcgen05.mma per K step and commits the A and B slots back to
//     their producers through mbarriers; after the last step it commits the accumulator to the epilogue.
// Measured (M = 8192, N = 14336, K = 4096): 814 TFLOP/s; with the decode arithmetic and the tile stores
// switched off the same pipeline reaches 980 TFLOP/s, cuBLAS bf16 on the same shape 1455 TFLOP/s, so
// the single-CTA (cta_group::1) pipeline itself, not the decode, is the larger part of the gap.
// Output tiles are dealt round-robin, whole.  Cutting the tiles of the last, incomplete round along K (each SM an equal
// share of K steps, partial accumulators handed to the neighbouring CTA through global memory) was built and measured:
// it executed the same number of instructions but ran 5-8 % slower on every shape, so it was taken out again.
// Every mbarrier wait is bounded; on a timeout the CTA records a status code, skips the work that
// depended on the wait and still frees its tensor memory.
#include <cuda.h>

#include <cstdio>
#include <mutex>

#include "common.cuh"
#include "tmap.cuh"

namespace b200q {

struct PrefillParams {
    const uint8_t* w;
    void* out;
    uint32_t M, N, K;
    uint32_t row_bytes;
    uint32_t mt;      // activation rows per tile (MMA N): 64, 128 or 256
    uint32_t idesc;   // tcgen05 instruction descriptor
    uint32_t nkt;     // K / 64
    uint32_t ns;      // ring depth: stage s = ks decoded weight tiles in tensor memory + ks activation tiles in shared memory
    uint32_t ks;      // K steps (of 64) per stage, 1 or 2: at small mt the loop overhead of the MMA warp, not the MMAs, sets the pace
    uint32_t nr;      // ring depth of the packed-weight tiles (0: the rows are not staged)
    uint32_t ntn, ntiles;  // output tiles along N (128 weight rows each) and in total
    // Work distribution.  Tiles [0, nfull) are dealt whole, round-robin (nfull is a multiple of the grid).  The
    // remaining ntail tiles (fewer than one per CTA) are, when `split`, cut along K: their ntail * gpt granules of
    // `gran` K steps are shared evenly, CTA c taking granules [c Q / G, (c + 1) Q / G), which touches at most two
    // tiles; a piece that is not a whole tile is written as an f32 partial tile into `part` (pieces numbered in K order) and
    // prefill_reduce_kernel adds the pieces of each tile in K order.
    uint32_t nfull, ntail, split, gran, gpt;
    float* part;
    int out_dtype;
    unsigned int* status;
};

namespace {

constexpr int BK = 64;          // K elements per stage = one 128-byte swizzle row of bf16
// packed-weight tiles staged by TMA: 128 rows x the bytes of 256 elements (four K steps)
__host__ __device__ constexpr int raw_pitch(int fmt) { return fmt == FMT_Q8_0 ? 272 : fmt == FMT_Q6_K ? 212 : (fmt == FMT_Q5_K || fmt == FMT_Q5_0) ? 176 : 144; }
// tile bytes rounded up to 1 KB (the operand tiles behind them must stay 1 KB aligned).  Q6_K blocks (210 B) are not
// multiples of 16 bytes: where the ROWS are (K a multiple of 2048) TMA fetches the 240 bytes from the 16-byte boundary below
// the block (prefill_kernel's Q6BOX; measured 1.4-2.0x the speed of the copy below: M = 2048, 14336 x 4096: 371 -> 229 us);
// otherwise the dequant warps copy the blocks themselves with 4-byte asynchronous copies into rows of 212 bytes (4-byte
// aligned blocks, conflict-free row-per-thread reads).
__host__ __device__ constexpr int raw_tile_bytes(int fmt) { return (128 * raw_pitch(fmt) + 1023) & ~1023; }
constexpr int PF_THREADS = 23 * 32;  // warps 0-15 dequant | 16 activation TMA | 17 MMA issue, TMEM | 18 packed-weight TMA | 19-22 epilogue

// Bounded wait of the pipeline roles.  The fast path is one try_wait; only the slow path looks at the CTA's dead flag
// (set by whichever warp gave up first), so a healthy pipeline never pays for the check.
__device__ __noinline__ bool pf_wait_slow(uint32_t bar, uint32_t parity, volatile uint32_t* dead) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
#pragma unroll 1
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 8; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*dead || global_timer_ns() - t0 > 2000000000ull) return false;
        __nanosleep(40);
    }
}
__device__ __forceinline__ bool pf_wait(uint32_t bar, uint32_t parity, volatile uint32_t* dead) {
    if (mbar_try_wait(bar, parity)) return true;
    return pf_wait_slow(bar, parity, dead);
}
// Records why a role gave up (first failure only) and marks the CTA dead.
__device__ __noinline__ void pf_fail(volatile uint32_t* dead, unsigned int* status, unsigned int code) {
    if (!*dead) atomicOr(status, code);
    *dead = 1;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}
// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xFFFFFFFF;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The same with the A operand (128 rows x 16 bf16, row i in lane i, two elements per 32-bit column) in tensor memory.
__device__ __forceinline__ void tc_mma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 16 consecutive 32-bit columns of this thread's lane (the warp covers the 32 lanes of its quarter)
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
          "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
          "r"(r[30]), "r"(r[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// K-major operand tile, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;             // leading byte offset (unused for swizzled K-major): 1
    d |= (uint64_t)(1024 >> 4) << 32;   // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;             // descriptor version of this architecture
    d |= (uint64_t)2 << 61;             // layout type: 128-byte swizzle
    return d;
}
// The same descriptor from its low word ((addr >> 4) | 1 << 16; advancing K by 16 elements adds 2) and the constant
// high word, without 64-bit arithmetic in the issuing thread.
__device__ __forceinline__ uint64_t smem_desc_sw128_lo(uint32_t lo) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"((1024u >> 4) | (1u << 14) | (2u << 29)));
    return d;
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t g16(const uint8_t* p) { return __ldg(reinterpret_cast<const unsigned short*>(p)); }
__device__ __forceinline__ uint32_t g32(const uint8_t* p) {  // 4 bytes at a 2-byte-aligned address
    if ((reinterpret_cast<uintptr_t>(p) & 3u) == 0) return __ldg(reinterpret_cast<const uint32_t*>(p));
    return g16(p) | (g16(p + 2) << 16);
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
// float value of byte `I` of x (0..255) without an integer-to-float conversion instruction
template <int I>
__device__ __forceinline__ float byte_to_float(uint32_t x) {
    return __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7650 | I)) - 8388608.0f;
}

// Q4_0, Q8_0 and Q6_K weights, w = s * (c - z) with an integer code c and zero point z, cost a byte permute and ONE
// fused multiply-add each.  Byte I of x (a code c < 128) is placed in bits 16..23 of the float 2.0, which then reads
// 2 + c / 64, and w = fma(64 s, 2 + c / 64, -(128 + z) s): the product is exact and so is the constant (s has at most
// 18 significant bits), so the result is s * (c - z) exactly.  code_low() places codes up to 255 one byte lower
// (2 + c / 16384) for Q8_0.  Q4_K / Q5_K (w = s * c + t with unrelated s and t) cannot use it: t - 128 s is not exact
// in general, and a per-row test for exactness diverges within a warp and costs more than it saves (measured).
template <int I>
__device__ __forceinline__ float code_mid(uint32_t x) { return __uint_as_float(__byte_perm(x, 0x40000000u, 0x7044 | (I << 8))); }  // 2 + c / 64
template <int I>
__device__ __forceinline__ float code_low(uint32_t x) { return __uint_as_float(__byte_perm(x, 0x40000000u, 0x7404 | (I << 4))); }  // 2 + c / 16384
template <bool SM>
__device__ __forceinline__ uint32_t ld16(const uint8_t* p) { return SM ? (uint32_t)*reinterpret_cast<const unsigned short*>(p) : g16(p); }
template <bool SM>
__device__ __forceinline__ uint32_t ld32(const uint8_t* p) {  // 4 bytes at a 2-byte-aligned address
    if ((reinterpret_cast<uintptr_t>(p) & 3u) == 0) return SM ? *reinterpret_cast<const uint32_t*>(p) : __ldg(reinterpret_cast<const uint32_t*>(p));
    return ld16<SM>(p) | (ld16<SM>(p + 2) << 16);
}

// The 64 elements of K step jj (0..3) of a Q4_K / Q5_K block in shared memory: sub-blocks 2 jj (low nibbles) and
// 2 jj + 1 (high nibbles) of the same 32 bytes.  RNE bf16 of the exact f32 weight d * sc * q - dmin * m, the value
// the dequant kernel writes.  Q5_K in the element order of the reference's x86-64 dot product
// (src/quant/cpu/kernels/simd/fused_q5k_q8k_dot.rs:27-122): Q4_K's nibble order, the nibbles 32 bytes further into
// the block, plus bit (e % 8) of qh[e / 8] for element e, so sub-block j takes one 32-bit word of qh.
template <bool Q5>
__device__ __forceinline__ void decode64_q45k(const uint8_t* blk, uint32_t jj, uint32_t (&o)[32]) {
    const uint4 hd = *reinterpret_cast<const uint4*>(blk);
    const float d = f16bits_to_f32(hd.x & 0xFFFF), dmin = f16bits_to_f32(hd.x >> 16);
    uint32_t sc, mn;  // byte 0: sub-block 2 jj, byte 1: sub-block 2 jj + 1
    if (jj < 2) {
        sc = (hd.y >> (16 * jj)) & 0x3F3Fu;
        mn = (hd.z >> (16 * jj)) & 0x3F3Fu;
    } else {
        const uint32_t sh = 16 * (jj - 2);
        sc = ((hd.w >> sh) & 0x0F0Fu) | (((hd.y >> sh) >> 2) & 0x3030u);
        mn = (((hd.w >> sh) >> 4) & 0x0F0Fu) | (((hd.z >> sh) >> 2) & 0x3030u);
    }
    constexpr uint32_t QOFF = Q5 ? 48 : 16;
    const uint4 q0 = *reinterpret_cast<const uint4*>(blk + QOFF + 32 * jj), q1 = *reinterpret_cast<const uint4*>(blk + QOFF + 16 + 32 * jj);
    uint2 hb = make_uint2(0, 0);
    if constexpr (Q5) hb = *reinterpret_cast<const uint2*>(blk + 16 + 8 * jj);
    const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const float dl = d * byte_to_float<0>(sc >> (8 * h)), nml = -(dmin * byte_to_float<0>(mn >> (8 * h)));
        const uint32_t hbits = h ? hb.y : hb.x;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            uint32_t q = (w[i] >> (4 * h)) & 0x0F0F0F0Fu;
            // word i holds elements 4i .. 4i + 3; their fifth bits are bits 4i .. 4i + 3 of hbits
            if constexpr (Q5) q |= (((hbits >> (4 * i)) & 15u) * 0x02040810u) & 0x10101010u;
            // dl * q is exact (17 x 5 bits), so the fused form rounds once exactly like multiply-then-subtract
            o[16 * h + 2 * i] = pack_bf16(fmaf(dl, byte_to_float<0>(q), nml), fmaf(dl, byte_to_float<1>(q), nml));
            o[16 * h + 2 * i + 1] = pack_bf16(fmaf(dl, byte_to_float<2>(q), nml), fmaf(dl, byte_to_float<3>(q), nml));
        }
    }
}

// One 32-element Q8_0 / Q4_0 block (2-byte aligned) as 32 bf16.  SM: the block sits in shared memory.
// Q8_0: w = d * (u - 128) with u = q + 128 placed by code_low(): fma(16384 d, 2 + u / 16384, -32896 d);
// Q4_0: w = d * (q - 8): fma(64 d, 2 + q / 64, -136 d).  Both constants are exact (d has 11 significant bits).
template <int FMT, bool SM>
__device__ __forceinline__ void decode32_blk(const uint8_t* blk, uint32_t* o) {
    const float d = f16bits_to_f32(ld16<SM>(blk));
    if constexpr (FMT == FMT_Q8_0) {
        const float a = 16384.0f * d, c = -32896.0f * d;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t x = ld32<SM>(blk + 2 + 4 * i) ^ 0x80808080u;  // q + 128
            o[2 * i] = pack_bf16(fmaf(a, code_low<0>(x), c), fmaf(a, code_low<1>(x), c));
            o[2 * i + 1] = pack_bf16(fmaf(a, code_low<2>(x), c), fmaf(a, code_low<3>(x), c));
        }
    } else if constexpr (FMT == FMT_Q5_0) {
        // f16 d | 32 high bits | 16 B nibbles (Q4_0's element order; element e takes bit e of the high-bit word):
        // w = d * (c - 16) = fma(64 d, 2 + c / 64, -144 d)
        const float a = 64.0f * d, c = -144.0f * d;
        const uint32_t qh = ld32<SM>(blk + 2);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t x = ld32<SM>(blk + 6 + 4 * i), hb = (qh >> (8 * i)) & 0xFFu;
            // even bits of hb -> bit 4 of bytes 0..3 (shifts 4, 10, 16, 22; stray products and their carries miss those bits)
            const uint32_t lo = (x & 0x0F0F0F0Fu) | (((hb & 0x55u) * 0x00410410u) & 0x10101010u);
            const uint32_t hi = ((x >> 4) & 0x0F0F0F0Fu) | ((((hb >> 1) & 0x55u) * 0x00410410u) & 0x10101010u);
            o[4 * i] = pack_bf16(fmaf(a, code_mid<0>(lo), c), fmaf(a, code_mid<0>(hi), c));
            o[4 * i + 1] = pack_bf16(fmaf(a, code_mid<1>(lo), c), fmaf(a, code_mid<1>(hi), c));
            o[4 * i + 2] = pack_bf16(fmaf(a, code_mid<2>(lo), c), fmaf(a, code_mid<2>(hi), c));
            o[4 * i + 3] = pack_bf16(fmaf(a, code_mid<3>(lo), c), fmaf(a, code_mid<3>(hi), c));
        }
    } else {  // Q4_0: byte i = elements 2i (low nibble), 2i+1 (high)
        const float a = 64.0f * d, c = -136.0f * d;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t x = ld32<SM>(blk + 2 + 4 * i);
            const uint32_t lo = x & 0x0F0F0F0Fu, hi = (x >> 4) & 0x0F0F0F0Fu;
            o[4 * i] = pack_bf16(fmaf(a, code_mid<0>(lo), c), fmaf(a, code_mid<0>(hi), c));
            o[4 * i + 1] = pack_bf16(fmaf(a, code_mid<1>(lo), c), fmaf(a, code_mid<1>(hi), c));
            o[4 * i + 2] = pack_bf16(fmaf(a, code_mid<2>(lo), c), fmaf(a, code_mid<2>(hi), c));
            o[4 * i + 3] = pack_bf16(fmaf(a, code_mid<3>(lo), c), fmaf(a, code_mid<3>(hi), c));
        }
    }
}

// The 64 elements of K step jt (0..3) of the Q6_K block at `blk`: elements 128 n + 32 g + l, n = jt / 2,
// g = 2 (jt & 1) + {0, 1}.  w = (d * sc) * (q - 32) = fma(64 s, 2 + q / 64, -160 s) with s = d * sc (18 significant
// bits, so -160 s is exact).  SM: the block sits 4-byte aligned in shared memory; otherwise 2-byte aligned in global.
template <bool SM>
__device__ __forceinline__ void decode64_q6k(const uint8_t* blk, uint32_t jt, uint32_t (&o)[32]) {
    const uint32_t n = jt >> 1, g0 = (jt & 1) * 2;
    const float d = f16bits_to_f32(ld16<SM>(blk + 208));
    const uint8_t* qh = blk + 128 + 32 * n;
    const uint32_t scw = ld16<SM>(blk + 192 + 8 * n + 2 * g0) | (ld16<SM>(blk + 192 + 8 * n + 2 * g0 + 2) << 16);  // four int8 scales
    uint32_t hw[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) hw[i] = ld32<SM>(qh + 4 * i);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t gq = g0 + h;
        const uint8_t* ql = blk + 64 * n + 32 * h;  // gq & 1 == h
        const float s0 = d * (float)(int)(signed char)(scw >> (16 * h)), s1 = d * (float)(int)(signed char)(scw >> (16 * h + 8));
        const float a0 = 64.0f * s0, c0 = -160.0f * s0, a1 = 64.0f * s1, c1 = -160.0f * s1;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t lw = ld32<SM>(ql + 4 * i);
            const uint32_t nib = (g0 ? (lw >> 4) : lw) & 0x0F0F0F0Fu;
            const uint32_t q = nib | (((hw[i] >> (2 * gq)) & 0x03030303u) << 4);
            const float a = i < 4 ? a0 : a1, c = i < 4 ? c0 : c1;
            o[16 * h + 2 * i] = pack_bf16(fmaf(a, code_mid<0>(q), c), fmaf(a, code_mid<1>(q), c));
            o[16 * h + 2 * i + 1] = pack_bf16(fmaf(a, code_mid<2>(q), c), fmaf(a, code_mid<3>(q), c));
        }
    }
}

// The same for a block staged in shared memory at byte `sh` (0 or 2) of a 4-byte-aligned slot: aligned words are loaded
// and funnel-shifted, the same instructions for both alignments (rows of a warp differ in it).
__device__ __forceinline__ void decode64_q6k_staged(const uint8_t* slot, uint32_t sh, uint32_t jt, uint32_t (&o)[32]) {
    const uint32_t n = jt >> 1, g0 = (jt & 1) * 2, sb = 8 * sh;
    const uint8_t* blk = slot + sh;
    const float d = f16bits_to_f32(*reinterpret_cast<const unsigned short*>(blk + 208));
    const uint32_t scw = (uint32_t)*reinterpret_cast<const unsigned short*>(blk + 192 + 8 * n + 2 * g0) |
                         ((uint32_t)*reinterpret_cast<const unsigned short*>(blk + 192 + 8 * n + 2 * g0 + 2) << 16);  // four int8 scales
    uint32_t hw[9];
    const uint32_t* qh = reinterpret_cast<const uint32_t*>(slot + 128 + 32 * n);
#pragma unroll
    for (int i = 0; i < 9; ++i) hw[i] = qh[i];
#pragma unroll
    for (int i = 0; i < 8; ++i) hw[i] = __funnelshift_r(hw[i], hw[i + 1], sb);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t gq = g0 + h;
        const uint32_t* ql = reinterpret_cast<const uint32_t*>(slot + 64 * n + 32 * h);  // gq & 1 == h
        const float s0 = d * (float)(int)(signed char)(scw >> (16 * h)), s1 = d * (float)(int)(signed char)(scw >> (16 * h + 8));
        const float a0 = 64.0f * s0, c0 = -160.0f * s0, a1 = 64.0f * s1, c1 = -160.0f * s1;
        uint32_t lw[9];
#pragma unroll
        for (int i = 0; i < 9; ++i) lw[i] = ql[i];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t w = __funnelshift_r(lw[i], lw[i + 1], sb);
            const uint32_t nib = (g0 ? (w >> 4) : w) & 0x0F0F0F0Fu;
            const uint32_t q = nib | (((hw[i] >> (2 * gq)) & 0x03030303u) << 4);
            const float a = i < 4 ? a0 : a1, c = i < 4 ? c0 : c1;
            o[16 * h + 2 * i] = pack_bf16(fmaf(a, code_mid<0>(q), c), fmaf(a, code_mid<1>(q), c));
            o[16 * h + 2 * i + 1] = pack_bf16(fmaf(a, code_mid<2>(q), c), fmaf(a, code_mid<3>(q), c));
        }
    }
}

// Elements [64 kt, 64 kt + 64) of one weight row in global memory as 64 bf16 (rows whose packed tiles are not staged).
template <int FMT>
__device__ __forceinline__ void decode64_global(const uint8_t* row, uint32_t kt, uint32_t (&o)[32]) {
    if constexpr (FMT == FMT_Q6_K) {
        decode64_q6k<false>(row + (kt >> 2) * 210, kt & 3, o);
    } else if constexpr (FMT == FMT_Q5_K || FMT == FMT_Q4_K) {
        // never taken: K-quant rows are whole 256-element blocks, which are always staged in shared memory
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = 0;
    } else {
        constexpr uint32_t BB = fmt_block_bytes(FMT);
        decode32_blk<FMT, false>(row + (2 * kt) * BB, o);
        decode32_blk<FMT, false>(row + (2 * kt + 1) * BB, o + 16);
    }
}

// dynamic shared memory: [0,1024) barriers + TMEM base; then two packed-weight tiles and ns activation tiles of
// mt*128 B, all 1 KB aligned.  Stage s pairs activation tile s with decoded weight tile s in tensor memory.
constexpr int PF_OFF_FULL = 0, PF_OFF_EMPTY = 128, PF_OFF_ACC_FULL = 256,
              PF_OFF_ACC_EMPTY = 272, PF_OFF_TMEM = 288, PF_OFF_DEAD = 292, PF_OFF_FULL_RAW = 320, PF_OFF_EMPTY_RAW = 384;

// One piece of work of a CTA: K steps [k0, k0 + nk) of output tile `tile`; slot < 0: the whole tile, written to the
// output; otherwise a partial tile for the reduce kernel.
struct PfUnit {
    uint32_t tile, k0, nk;
    int slot;
};
// The it-th unit of this CTA (every role walks the same list).
__device__ __forceinline__ bool pf_unit(const PrefillParams& p, uint32_t it, PfUnit& u) {
    const uint32_t t = blockIdx.x + it * gridDim.x;
    if (t < p.nfull) {
        u.tile = t; u.k0 = 0; u.nk = p.nkt; u.slot = -1;
        return true;
    }
    const uint32_t j = it - p.nfull / gridDim.x;  // 0 or 1: piece of the tail
    if (!p.split) {
        if (j != 0 || blockIdx.x >= p.ntail) return false;
        u.tile = p.nfull + blockIdx.x; u.k0 = 0; u.nk = p.nkt; u.slot = -1;
        return true;
    }
    if (j > 1) return false;
    const uint32_t Q = p.ntail * p.gpt;
    const uint32_t a = (blockIdx.x * Q) / gridDim.x, b = ((blockIdx.x + 1) * Q) / gridDim.x;  // G * Q < 2^32 (checked by the launcher)
    if (a >= b) return false;
    const uint32_t t0 = a / p.gpt, e0 = min(b, (t0 + 1) * p.gpt);
    uint32_t lo, hi, tt;
    if (j == 0) { lo = a; hi = e0; tt = t0; }
    else {
        if (e0 >= b) return false;
        lo = e0; hi = b; tt = t0 + 1;
    }
    u.tile = p.nfull + tt;
    u.k0 = (lo - tt * p.gpt) * p.gran;
    u.nk = min((hi - lo) * p.gran, p.nkt - u.k0);
    // pieces in K order: one more at every CTA boundary and at every tile boundary (CTAs without work do not count)
    u.slot = (u.k0 == 0 && u.nk == p.nkt) ? -1 : (int)(min(blockIdx.x, a) + tt);
    return true;
}

// Persistent: one CTA per SM walks its work units (consecutive CTAs share an activation tile, which therefore stays
// in L2).  Tensor memory holds TWO accumulators while they fit, so the four epilogue warps drain unit i while the MMA
// warp is already accumulating unit i + 1 and the rings never run dry between units.
// RAW_TMA: packed weights staged in shared memory (by TMA where the rows are multiples of 16 bytes).  Q6BOX (Q6_K with rows
// that are multiples of 16 bytes, i.e. K a multiple of 2048): the 210-byte block comes by TMA as the 240 bytes from the
// 16-byte boundary below it, so it sits (210 b mod 16) bytes into every row of the tile; otherwise the dequant warps copy
// Q6_K tiles themselves with 4-byte asynchronous copies.
template <int FMT, bool RAW_TMA, bool Q6BOX = false>
__global__ void __launch_bounds__(PF_THREADS, 1) prefill_kernel(const __grid_constant__ CUtensorMap tmap_act,
                                                                const __grid_constant__ CUtensorMap tmap_w, const PrefillParams p) {
    constexpr uint32_t RAW_PITCH = Q6BOX ? 240u : (uint32_t)raw_pitch(FMT), RAW_TILE_BYTES = Q6BOX ? 128u * 240u : (uint32_t)raw_tile_bytes(FMT);
    constexpr bool COOP = RAW_TMA && FMT == FMT_Q6_K && !Q6BOX;  // packed tiles copied by the dequant warps instead of TMA
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // swizzled operand tiles need 1024-byte alignment; the launch reserves 1 KB of slack for this
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    // the warp index through a shuffle, so that the compiler treats the role branches (and what the roles compute
    // from kernel parameters) as warp-uniform
    const int warp = __shfl_sync(0xFFFFFFFFu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar_full = sbase + PF_OFF_FULL, bar_empty = sbase + PF_OFF_EMPTY;
    const uint32_t bar_acc_full = sbase + PF_OFF_ACC_FULL, bar_acc_empty = sbase + PF_OFF_ACC_EMPTY;
    const uint32_t bar_full_raw = sbase + PF_OFF_FULL_RAW, bar_empty_raw = sbase + PF_OFF_EMPTY_RAW;
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + PF_OFF_TMEM);
    volatile uint32_t* dead_flag = reinterpret_cast<volatile uint32_t*>(smem + PF_OFF_DEAD);
    const uint32_t b_tile_bytes = p.mt * 128;
    const uint32_t raw_bytes = RAW_TMA ? p.nr * RAW_TILE_BYTES : 0;
    const uint32_t raw_tiles = sbase + 1024, b_tiles = raw_tiles + raw_bytes;
    // Tensor memory (all 512 columns): nacc accumulators of mt columns (two while they fit beside the weight stages,
    // one at mt = 256), then the decoded weight tiles of 32 columns (128 rows x 64 bf16, two per column).
    const uint32_t tmem_cols = 512, nacc = p.mt <= 128 ? 2u : 1u, a_col0 = nacc * p.mt;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.ns; ++s) {
            // a stage is full when the four warps of a set have written the weight tile (to tensor memory) and the
            // activation tile's bytes have landed (one more arrival, with the byte count); one wait for the MMA warp
            mbar_init(bar_full + 8 * s, 4 * p.ks + 1);
            mbar_init(bar_empty + 8 * s, 1);  // released by the commit behind the stage's MMAs, for both producers
        }
        for (uint32_t s = 0; s < p.nr; ++s) {
            mbar_init(bar_full_raw + 8 * s, COOP ? 512 : 1);  // COOP: every dequant thread copies a share of the tile
            mbar_init(bar_empty_raw + 8 * s, 16);            // every dequant warp reads every packed tile
        }
        for (uint32_t s = 0; s < 2; ++s) {
            mbar_init(bar_acc_full + 8 * s, 1);
            mbar_init(bar_acc_empty + 8 * s, 4);   // the four epilogue warps
        }
        *dead_flag = 0;
        mbar_fence_init();
    }
    if (warp == 17) {  // tensor-memory columns for the accumulators, allocated by one whole warp
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sbase + PF_OFF_TMEM), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_acc = *tmem_holder;

    if (warp == 18) {
        // ------------------------------------------------------------ packed weight tiles by TMA
        if (RAW_TMA && !COOP && lane == 0) {
            uint32_t s = 0, par = 0;
            PfUnit u;
            for (uint32_t it = 0; pf_unit(p, it, u); ++it) {
                const uint32_t n0 = (u.tile % p.ntn) * 128, j0 = u.k0 / 4, nraw = (u.nk + 3) / 4;
                for (uint32_t j = 0; j < nraw; ++j) {
                    if (!pf_wait(bar_empty_raw + 8 * s, par ^ 1, dead_flag)) {
                        pf_fail(dead_flag, p.status, STATUS_TIMEOUT_EMPTY);
                        break;
                    }
                    mbar_expect_tx(bar_full_raw + 8 * s, RAW_TILE_BYTES);
                    // x in elements of the tensor map: bytes for the 144-byte formats, 16-bit units for Q8_0
                    const int x = Q6BOX ? (int)(((j0 + j) * 210u) & ~15u)
                                        : (int)((j0 + j) * (FMT == FMT_Q8_0 ? 136 : (FMT == FMT_Q5_K || FMT == FMT_Q5_0) ? 176 : 144));
                    tma_load_2d(raw_tiles + s * RAW_TILE_BYTES, &tmap_w, x, (int)n0, bar_full_raw + 8 * s);
                    if (++s == p.nr) { s = 0; par ^= 1; }
                }
                if (*dead_flag) break;
            }
        }
    } else if (warp == 16) {
        // ------------------------------------------------------------ activation tiles by TMA
        if (lane == 0) {
            uint32_t s = 0, par = 0;
            PfUnit u;
            for (uint32_t it = 0; pf_unit(p, it, u); ++it) {
                const uint32_t m0 = (u.tile / p.ntn) * p.mt;
                for (uint32_t kt = 0; kt < u.nk; kt += p.ks) {
                    if (!pf_wait(bar_empty + 8 * s, par ^ 1, dead_flag)) {
                        pf_fail(dead_flag, p.status, STATUS_TIMEOUT_EMPTY);
                        break;
                    }
                    mbar_expect_tx(bar_full + 8 * s, p.ks * b_tile_bytes);
                    for (uint32_t i = 0; i < p.ks; ++i)
                        tma_load_2d(b_tiles + (s * p.ks + i) * b_tile_bytes, &tmap_act, (int)((u.k0 + kt + i) * BK), (int)m0, bar_full + 8 * s);
                    if (++s == p.ns) { s = 0; par ^= 1; }
                }
                if (*dead_flag) break;
            }
        }
    } else if (warp == 17) {
        // ------------------------------------------------------------ MMA issue
        // The whole warp runs the loop and the waits, so that the stage counters and addresses are warp-uniform
        // values; one elected lane issues the MMAs and the commits.
        {
            uint32_t sa = 0, para = 0;
            const uint32_t a_tm0 = tmem_acc + a_col0, b_lo0 = ((b_tiles >> 4) & 0x3FFFu) | (1u << 16), b_lo_step = b_tile_bytes >> 4;
            bool ok = true;
            PfUnit un;
            for (uint32_t it = 0; ok && pf_unit(p, it, un); ++it) {
                const uint32_t acc = it % nacc, u = it / nacc;
                // the accumulator must have been drained by the epilogue of its previous use
                if (u > 0 && !pf_wait(bar_acc_empty + 8 * acc, (u - 1) & 1, dead_flag)) {
                    if (lane == 0) pf_fail(dead_flag, p.status, STATUS_TIMEOUT_EMPTY);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_acc + acc * p.mt;
                for (uint32_t kt = 0; kt < un.nk; kt += p.ks) {
                    if (!pf_wait(bar_full + 8 * sa, para, dead_flag)) {
                        if (lane == 0) pf_fail(dead_flag, p.status, STATUS_TIMEOUT_FULL);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_tm = a_tm0 + 32 * p.ks * sa, b_lo = b_lo0 + p.ks * sa * b_lo_step;
                    if (elect_one()) {
#pragma unroll
                        for (int k = 0; k < BK / 16; ++k)
                            tc_mma_bf16_ts(d_tmem, a_tm + 8 * k, smem_desc_sw128_lo(b_lo + 2 * k), p.idesc, (kt | k) != 0);
                        if (p.ks == 2) {
#pragma unroll
                            for (int k = 0; k < BK / 16; ++k)
                                tc_mma_bf16_ts(d_tmem, a_tm + 32 + 8 * k, smem_desc_sw128_lo(b_lo + b_lo_step + 2 * k), p.idesc, 1);
                        }
                        // the stage's tiles may be overwritten once these MMAs have read them
                        tc_commit(bar_empty + 8 * sa);
                    }
                    __syncwarp();
                    if (++sa == p.ns) { sa = 0; para ^= 1; }
                }
                if (ok && elect_one()) tc_commit(bar_acc_full + 8 * acc);  // arrives when every MMA of the unit has completed
                __syncwarp();
            }
        }
    } else if (warp >= 19) {
        // ------------------------------------------------------------ epilogue: accumulator -> out[m, n]
        // lane r of the accumulator = weight row n0 + r, column c = activation row m0 + c; a warp reaches the
        // 32 lanes of its quarter (warp & 3)
        const uint32_t quarter = (uint32_t)warp & 3, r = quarter * 32 + lane;
        bool ok = true;
        PfUnit un;
        for (uint32_t it = 0; ok && pf_unit(p, it, un); ++it) {
            const uint32_t acc = it % nacc, u = it / nacc;
            const uint32_t n0 = (un.tile % p.ntn) * 128, m0 = (un.tile / p.ntn) * p.mt;
            if (!pf_wait(bar_acc_full + 8 * acc, u & 1, dead_flag)) {
                pf_fail(dead_flag, p.status, STATUS_TIMEOUT_MMA);
                ok = false;
                break;
            }
            tc_fence_after();
            const bool row_ok = n0 + r < p.N;
            float* part = un.slot >= 0 ? p.part + (size_t)un.slot * p.mt * 128 : nullptr;
            for (uint32_t c0 = 0; c0 < p.mt; c0 += 16) {
                if (m0 + c0 >= p.M) break;  // warp-uniform
                uint32_t v[16];
                tmem_ld16(tmem_acc + ((quarter * 32) << 16) + acc * p.mt + c0, v);
                if (part) {
                    // partial tile [activation row][weight row]: lanes write consecutive floats
#pragma unroll
                    for (int i = 0; i < 16; ++i) part[(size_t)(c0 + i) * 128 + r] = __uint_as_float(v[i]);
                } else if (row_ok) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const uint32_t m = m0 + c0 + i;
                        if (m < p.M) {
                            const size_t idx = (size_t)m * p.N + n0 + r;
                            const float f = __uint_as_float(v[i]);
                            if (p.out_dtype == DT_F32) static_cast<float*>(p.out)[idx] = f;
                            else if (p.out_dtype == DT_BF16) static_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(f);
                            else static_cast<__half*>(p.out)[idx] = __float2half_rn(f);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty + 8 * acc);
        }
    } else {
        // ------------------------------------------------------------ dequant warps
        // thread (set, r): weight row r of the tile, all 64 elements of the K steps kt = set, set + 4, ... of every
        // unit: four sets of four warps, each taking one K step of every packed tile (one 256-element block per row)
        const uint32_t r = threadIdx.x & 127, set = threadIdx.x >> 7;
        bool ok = true;
        // COOP: packed tile c (counted over all units of this CTA) is copied by all 16 dequant warps, 8 rows each, one
        // tile ahead of its use; buffer c & 1 must have been released by every reader of tile c - 2
        uint32_t next_copy = 0, copy_it = 0, copy_base = 0;  // copy_base: first packed tile of unit copy_it
        uint32_t cs = 0, cpar = 0;                            // ring slot and phase of packed tile next_copy
        PfUnit cu;
        bool cu_ok = pf_unit(p, 0, cu);
        auto copy_upto = [&](uint32_t upto) {
            for (; next_copy <= upto; ++next_copy) {
                while (cu_ok && next_copy >= copy_base + (cu.nk + 3) / 4) {
                    copy_base += (cu.nk + 3) / 4;
                    cu_ok = pf_unit(p, ++copy_it, cu);
                }
                if (!cu_ok) return;  // no further packed tiles: next_copy stays, later calls return here again
                const uint32_t jc = cu.k0 / 4 + (next_copy - copy_base);
                if (ok && !pf_wait(bar_empty_raw + 8 * cs, cpar ^ 1, dead_flag)) {
                    pf_fail(dead_flag, p.status, STATUS_TIMEOUT_EMPTY);
                    ok = false;
                }
                if (ok) {
                    // Asynchronous 4-byte copies (no registers, nothing waits here).  A block starts 2-byte aligned:
                    // the copy starts at the 4-byte boundary at or below it, so the block lands at byte (start & 2) of
                    // its 212-byte row and the decoder shifts.  Rows past N are zero-filled; the last word is clipped
                    // where it would reach past the end of the tensor.
                    const uint32_t cn0 = (cu.tile % p.ntn) * 128;
                    const uint32_t dst = raw_tiles + cs * RAW_TILE_BYTES;
                    const uint8_t* wend = p.w + (size_t)p.N * p.row_bytes;
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        const uint32_t row = 8 * (uint32_t)warp + q;
                        const bool in = cn0 + row < p.N;
                        const uint8_t* blk = p.w + (size_t)(in ? cn0 + row : 0) * p.row_bytes + (size_t)jc * 210;
                        const uint8_t* src = blk - (reinterpret_cast<uintptr_t>(blk) & 2);
#pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            const uint32_t wd = lane + 32 * i;
                            if (wd < 53) {
                                const uint8_t* sp = src + 4 * wd;
                                const uint32_t nbytes = !in ? 0u : sp + 4 <= wend ? 4u : sp + 2 <= wend ? 2u : 0u;
                                asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst + row * RAW_PITCH + 4 * wd), "l"(in ? sp : p.w), "r"(nbytes) : "memory");
                            }
                        }
                    }
                    // arrives on the tile's barrier once this thread's copies have landed
                    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar_full_raw + 8 * cs) : "memory");
                } else {
                    mbar_arrive(bar_full_raw + 8 * cs);
                }
                if (++cs == p.nr) { cs = 0; cpar ^= 1; }
            }
        };
        uint32_t steps_done = 0, raws_done = 0;  // K steps and packed tiles of the units before this one
        uint32_t rs = 0, rpar = 0;                // ring slot and phase of the packed tile of this set's next K step
        PfUnit un;
        for (uint32_t it = 0; pf_unit(p, it, un); ++it) {
            const uint32_t n0 = (un.tile % p.ntn) * 128;
            const bool row_ok = n0 + r < p.N;
            const uint8_t* wrow = p.w + (size_t)(row_ok ? n0 + r : 0) * p.row_bytes;
            // stage and phase of this set's K steps: position steps_done + kt in the stream the MMA warp consumes
            // (with two K steps per stage, units are whole multiples of four steps and a set keeps its half of the stage)
            const uint32_t ksl = p.ks >> 1, sub = set & (p.ks - 1);
            uint32_t s = ((steps_done + set) >> ksl) % p.ns, par = (((steps_done + set) >> ksl) / p.ns) & 1;
            for (uint32_t kt = set; kt < un.nk; kt += 4) {
                uint32_t o[32];
                if constexpr (RAW_TMA) {
                    // packed tile raws_done + kt / 4 covers K steps 4j .. 4j+3; a set visits every packed tile once, in order
                    if constexpr (COOP) copy_upto(raws_done + (kt >> 2) + p.nr - 1);
                    if (ok && !pf_wait(bar_full_raw + 8 * rs, rpar, dead_flag)) {
                        pf_fail(dead_flag, p.status, STATUS_TIMEOUT_FULL);
                        ok = false;
                    }
                    const uint8_t* rrow = smem + 1024 + rs * RAW_TILE_BYTES + r * RAW_PITCH;
                    if (ok) {
                        if constexpr (FMT == FMT_Q4_K) decode64_q45k<false>(rrow, set, o);
                        else if constexpr (FMT == FMT_Q5_K) decode64_q45k<true>(rrow, set, o);
                        else if constexpr (FMT == FMT_Q6_K) {
                            if constexpr (Q6BOX) {
                                // the block sits `off` bytes into the row's 240: words from the 4-byte boundary below, the
                                // remaining 0 or 2 bytes through the decoder's shift
                                const uint32_t off = ((un.k0 / 4 + (kt >> 2)) * 210u) & 15u;
                                decode64_q6k_staged(rrow + (off & ~3u), off & 2u, set, o);
                            } else {
                                // where the row's block sits in its 212-byte slot: the low bits of its global address
                                const uint32_t sh = ((n0 + r) * p.row_bytes + (un.k0 / 4 + (kt >> 2)) * 210u) & 2u;
                                decode64_q6k_staged(rrow, sh, set, o);
                            }
                        }
                        else {
                            constexpr uint32_t BB = fmt_block_bytes(FMT);
                            decode32_blk<FMT, true>(rrow + (2 * set) * BB, o);
                            decode32_blk<FMT, true>(rrow + (2 * set + 1) * BB, o + 16);
                        }
                    }
                    // the warp's only K step in this packed tile (kt & 3 == set): release the tile
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_empty_raw + 8 * rs);
                    if (++rs == p.nr) { rs = 0; rpar ^= 1; }
                } else {
                    decode64_global<FMT>(wrow, un.k0 + kt, o);
                }
                if (!row_ok || !ok)
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = 0;
                if (ok && !pf_wait(bar_empty + 8 * s, par ^ 1, dead_flag)) {
                    pf_fail(dead_flag, p.status, STATUS_TIMEOUT_EMPTY);
                    ok = false;
                }
                // the thread's 64 bf16 go to its own lane (= weight row) of the stage's tensor-memory tile, 32 columns.
                // Executed by the whole warp (dead warps store what they hold: nobody reads it).
                tmem_st32(tmem_acc + ((((uint32_t)warp & 3u) * 32u) << 16) + a_col0 + 32 * (p.ks * s + sub), o);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_full + 8 * s);
                s += 4 >> ksl;
                while (s >= p.ns) { s -= p.ns; par ^= 1; }
            }
            steps_done += un.nk;
            raws_done += (un.nk + 3) / 4;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 17) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(tmem_cols) : "memory");
    }
}

// Adds the partial tiles of the K-split tail tiles in K order and writes the output.  Block = (eight activation rows of
// the tile, tail tile), thread = weight row of the tile; the pieces of tail tile t come from the CTAs whose granule range
// meets [t gpt, (t + 1) gpt), in CTA order, which is K order.
constexpr uint32_t PF_RED_ROWS = 8;
__global__ void __launch_bounds__(128) prefill_reduce_kernel(const PrefillParams p, uint32_t G) {
    __shared__ uint32_t slots[192];
    __shared__ uint32_t nslots;
    const uint32_t t = blockIdx.y, ml0 = blockIdx.x * PF_RED_ROWS, r = threadIdx.x;
    const uint32_t tile = p.nfull + t, n0 = (tile % p.ntn) * 128, m0 = (tile / p.ntn) * p.mt + ml0;
    if (m0 >= p.M) return;  // block-uniform
    if (threadIdx.x == 0) {
        const uint32_t Q = p.ntail * p.gpt, lo = t * p.gpt, hi = lo + p.gpt;
        uint32_t c = (lo * G) / Q, n = 0;
        while (c > 0 && (c * Q) / G > lo) --c;
        while (((c + 1) * Q) / G <= lo) ++c;  // first CTA whose range [a, b) ends beyond lo
        for (; c < G && n < 192; ++c) {
            const uint32_t a = (c * Q) / G, b = ((c + 1) * Q) / G;
            if (a >= hi) break;
            if (a >= b) continue;
            if (max(a, lo) == lo && min(b, hi) == hi) { n = 0; break; }  // computed whole and written by its CTA
            slots[n++] = min(c, a) + t;  // the numbering of pf_unit()
        }
        nslots = n;
    }
    __syncthreads();
    const uint32_t ns = nslots;
    if (ns == 0 || n0 + r >= p.N) return;
    // four pieces x eight rows of loads are in flight together (a tile of a small matrix is cut into up to ~20 pieces: one
    // load at a time was 20 L2 round trips); the additions stay in K order
    float sum[PF_RED_ROWS];
    for (uint32_t i0 = 0; i0 < ns; i0 += 4) {
        float v[4][PF_RED_ROWS];
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
            if (i0 + i < ns) {
                const float* src = p.part + ((size_t)slots[i0 + i] * p.mt + ml0) * 128 + r;
#pragma unroll
                for (uint32_t j = 0; j < PF_RED_ROWS; ++j) v[i][j] = __ldcg(src + j * 128);  // rows up to mt exist in every piece
            }
        }
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
            if (i0 + i < ns) {
#pragma unroll
                for (uint32_t j = 0; j < PF_RED_ROWS; ++j) sum[j] = i0 + i == 0 ? v[i][j] : sum[j] + v[i][j];
            }
        }
    }
#pragma unroll
    for (uint32_t j = 0; j < PF_RED_ROWS; ++j) {
        const uint32_t m = m0 + j;
        if (m >= p.M) break;
        const size_t idx = (size_t)m * p.N + n0 + r;
        if (p.out_dtype == DT_F32) static_cast<float*>(p.out)[idx] = sum[j];
        else if (p.out_dtype == DT_BF16) static_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(sum[j]);
        else static_cast<__half*>(p.out)[idx] = __float2half_rn(sum[j]);
    }
}

__global__ void __launch_bounds__(256) f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, size_t n) {
    const size_t n4 = n / 4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(in) + i);
        uint2 r;
        r.x = pack_bf16(v.x, v.y);
        r.y = pack_bf16(v.z, v.w);
        reinterpret_cast<uint2*>(out)[i] = r;
    }
}

// K-quants: boostr's CPU path multiplies Q8_K-quantised activations (one f32 scale per 256, int8
// codes; src/quant/cpu/kernels/simd/quantize_act_q8k.rs:26-98).  The tensor-core path follows it:
// each 256-run is quantised exactly that way and d8 * code is then rounded to bf16, so what
// separates the two results is bf16 rounding only, not a second, different activation quantiser.
// One warp per 256-run, 8 values per lane.
template <typename InT>
__global__ void __launch_bounds__(256) act_q8k_to_bf16_kernel(const InT* __restrict__ in, __nv_bfloat16* __restrict__ out, size_t nruns) {
    const int lane = threadIdx.x & 31;
    for (size_t run = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5); run < nruns; run += (size_t)gridDim.x * 8) {
        float v[8];
        const size_t base = run * 256 + 8 * lane;
        if constexpr (sizeof(InT) == 4) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(in + base)), b = __ldg(reinterpret_cast<const float4*>(in + base) + 1);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
            const uint4 r = __ldg(reinterpret_cast<const uint4*>(in + base));
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
        const float d8 = __fdiv_rn(amax, 127.0f);
        const float id = amax != 0.f ? __fdiv_rn(127.0f, amax) : 0.f;
        float q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = __fmul_rn(d8, (float)max(-128, min(127, __float2int_rn(__fmul_rn(v[i], id)))));
        uint4 r;
        r.x = pack_bf16(q[0], q[1]); r.y = pack_bf16(q[2], q[3]); r.z = pack_bf16(q[4], q[5]); r.w = pack_bf16(q[6], q[7]);
        *reinterpret_cast<uint4*>(out + base) = r;
    }
}

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

uint32_t pick_mt(size_t M) { return M >= 256 ? 256u : M > 64 ? 128u : 64u; }

template <int FMT, bool RAW, bool Q6BOX = false>
cudaError_t launch_fmt(const CUtensorMap& map, const CUtensorMap& wmap, const PrefillParams& p, dim3 grid, size_t smem, cudaStream_t st) {
    static PerDeviceOnce attrs;
    cudaError_t ae = attrs.run([] { return cudaFuncSetAttribute(prefill_kernel<FMT, RAW, Q6BOX>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448 - 1024); });
    if (ae != cudaSuccess) return ae;
    prefill_kernel<FMT, RAW, Q6BOX><<<grid, PF_THREADS, smem, st>>>(map, wmap, p);
    note_launch();
    return cudaGetLastError();
}

}  // namespace

// Smallest M that takes the tensor-core path; below it the memory-bound small-M kernel runs (in passes of
// up to 32 activation rows).
#ifndef B200Q_PREFILL_MIN_M
#define B200Q_PREFILL_MIN_M 64
#endif
bool prefill_supported(int fmt, size_t M, size_t K, size_t N) {
    (void)fmt;
    return M >= B200Q_PREFILL_MIN_M && K % 64 == 0 && K % 8 == 0 && N >= 1;
}

namespace {
// How the output tiles are dealt to the CTAs (the fields of PrefillParams with the same names).
struct PfPlan {
    uint32_t mt, ntn, ntiles, grid, nfull, ntail, split, gran, gpt;
    size_t part_bytes;
};
PfPlan pf_plan(size_t M, size_t K, size_t N, int sm_count) {
    PfPlan pl{};
    pl.mt = pick_mt(M);
    pl.ntn = (uint32_t)((N + 127) / 128);
    pl.ntiles = pl.ntn * (uint32_t)((M + pl.mt - 1) / pl.mt);
    const uint32_t G = (uint32_t)sm_count, nkt = (uint32_t)(K / BK);
    pl.gran = nkt % 4 == 0 ? 4u : 1u;  // whole packed tiles (256 elements) where rows consist of them
    pl.gpt = nkt / pl.gran;
    pl.nfull = pl.ntiles / G * G;
    pl.ntail = pl.ntiles - pl.nfull;
    // cut the tail along K when it fills less than two thirds of the SMs (the partial tiles and the reduce launch cost a
    // few microseconds: measured, a tail of 86 tiles on 148 SMs gains 14 % cut, one of 112 tiles loses 3-20 %) and the
    // 32-bit granule arithmetic holds
    pl.split = pl.ntail > 0 && pl.ntail * 3 <= G * 2 && pl.gpt >= 2 && (uint64_t)(G + 1) * pl.ntail * pl.gpt < 0xFFFFFFFFull && G <= 190;
    pl.grid = (pl.split || pl.ntiles >= G) ? G : pl.ntiles;
    const size_t Q = (size_t)pl.ntail * pl.gpt;
    pl.part_bytes = pl.split ? ((Q < G ? Q : G) + pl.ntail) * pl.mt * 128 * sizeof(float) : 0;
    return pl;
}
}  // namespace

size_t prefill_workspace_bytes(int fmt, int act_dtype, size_t M, size_t K, size_t N, int sm_count) {
    const bool kq = (fmt == FMT_Q4_K || fmt == FMT_Q5_K || fmt == FMT_Q6_K);  // always re-quantised (see act_q8k_to_bf16_kernel)
    const size_t acts = (act_dtype == DT_BF16 && !kq) ? 0 : ((M * K * 2 + 255) & ~(size_t)255);
    return acts + pf_plan(M, K, N, sm_count).part_bytes;
}

cudaError_t launch_prefill(int fmt, const void* act, int act_dtype, const void* w, void* out, int out_dtype, size_t M,
                           size_t K, size_t N, void* ws, size_t ws_bytes, int sm_count, cudaStream_t st,
                           unsigned int* status, bool* ws_too_small, char* err, size_t err_len, bool acts_prepared) {
    *ws_too_small = false;
    const void* act_bf16 = act;
    const bool kq = (fmt == FMT_Q4_K || fmt == FMT_Q5_K || fmt == FMT_Q6_K);
    const PfPlan pl = pf_plan(M, K, N, sm_count);
    const size_t need = prefill_workspace_bytes(fmt, act_dtype, M, K, N, sm_count), act_bytes = need - pl.part_bytes;
    if (need && (!ws || ws_bytes < need || (reinterpret_cast<uintptr_t>(ws) & 15))) { *ws_too_small = true; return cudaSuccess; }
    if ((act_dtype != DT_BF16 || kq) && acts_prepared) {
        act_bf16 = ws;  // a previous call with the same activations and scratch left them there (gate, then up)
    } else if (act_dtype != DT_BF16 || kq) {
        const size_t n = M * K;
        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(ws);
        if (kq) {
            const size_t nruns = n / 256;
            int grid = (int)((nruns + 7) / 8);
            if (grid > sm_count * 16) grid = sm_count * 16;
            if (grid < 1) grid = 1;
            if (act_dtype == DT_F32) act_q8k_to_bf16_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(act), dst, nruns);
            else act_q8k_to_bf16_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(act), dst, nruns);
        } else {
            int grid = (int)((n / 4 + 255) / 256);
            if (grid > sm_count * 16) grid = sm_count * 16;
            if (grid < 1) grid = 1;
            f32_to_bf16_kernel<<<grid, 256, 0, st>>>(static_cast<const float*>(act), dst, n);
        }
        note_launch();
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
        act_bf16 = ws;
    }
    EncodeTiledFn enc = encode_tiled();
    if (!enc) {
        snprintf(err, err_len, "cuTensorMapEncodeTiled is not available from this driver");
        return cudaErrorNotSupported;
    }
    PrefillParams p{};
    p.w = static_cast<const uint8_t*>(w);
    p.out = out;
    p.M = (uint32_t)M; p.N = (uint32_t)N; p.K = (uint32_t)K;
    p.row_bytes = (uint32_t)(K / fmt_block_size(fmt) * fmt_block_bytes(fmt));
    p.mt = pl.mt;
    p.idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((p.mt >> 3) << 17) | ((128u >> 4) << 24);  // f32 acc, bf16 x bf16, K-major, N = mt, M = 128
    p.nkt = (uint32_t)(K / BK);
    // packed tiles by TMA need rows that are a multiple of 16 bytes and whole 256-element tiles
    // (Q6_K's tiles are copied by the dequant warps and only need whole blocks, which the format guarantees)
    const bool raw = K % 256 == 0 && (fmt == FMT_Q6_K || p.row_bytes % 16 == 0);
    const bool q6box = raw && fmt == FMT_Q6_K && p.row_bytes % 16 == 0;  // K a multiple of 2048
    const uint32_t raw_tile = !raw ? 0u : q6box ? 128u * 240u : (uint32_t)raw_tile_bytes(fmt);
    // the paths that still fetch packed bytes with loads keep ~30 KB of the SM's 256 KB as L1
    const uint32_t budget = (raw ? 232448u - 1024u : 200704u) - 2048u, b_tile = p.mt * 128;
    // activation tiles first (at least two packed tiles stay), then as many packed tiles as fit: at small M the packed
    // weights stream from HBM and the ring has to cover that latency
    uint32_t nsb = (budget - 2 * raw_tile) / b_tile;  // activation tiles = decoded weight tiles
    const uint32_t tmem_tiles = (512u - (p.mt <= 128 ? 2u : 1u) * p.mt) / 32u;  // 32 columns each beside the accumulators
    if (nsb > tmem_tiles) nsb = tmem_tiles;
    if (nsb > 12) nsb = 12;
    if (nsb > p.nkt) nsb = p.nkt;
    // two K steps per stage where the MMAs are short (mt <= 128) and every unit is a whole number of stages
    p.ks = (p.mt <= 128 && p.nkt % 4 == 0 && nsb >= 4) ? 2u : 1u;
    p.ns = nsb / p.ks;
    nsb = p.ns * p.ks;
    uint32_t nr = raw ? (budget - nsb * b_tile) / raw_tile : 0u;
    if (nr > 8) nr = 8;
    p.nr = nr;
    const uint32_t raw_bytes = nr * raw_tile;
    p.ntn = pl.ntn;
    p.ntiles = pl.ntiles;
    p.nfull = pl.nfull; p.ntail = pl.ntail; p.split = pl.split; p.gran = pl.gran; p.gpt = pl.gpt;
    p.part = pl.split ? reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + act_bytes) : nullptr;
    p.out_dtype = out_dtype;
    p.status = status;
    const size_t smem = 2048 + raw_bytes + (size_t)nsb * b_tile;

    CUtensorMap map;
    const cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t gstride[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, p.mt};
    const cuuint32_t estr[2] = {1, 1};
    CUresult cr = enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(act_bf16), gdim, gstride, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) {
        snprintf(err, err_len, "cuTensorMapEncodeTiled failed with code %d (activation pointer %p, K=%zu, M=%zu)", (int)cr, act_bf16, K, M);
        return cudaErrorInvalidValue;
    }
    // packed weights as a matrix [N, row_bytes]: tiles of 128 rows x the bytes of 256 elements (bytes for the
    // 144-byte formats, 16-bit units for Q8_0's 272 bytes: a box dimension holds at most 256 elements)
    CUtensorMap wmap = map;
    if (raw && (fmt != FMT_Q6_K || q6box)) {
        const bool q8 = fmt == FMT_Q8_0;
        const cuuint64_t wdim[2] = {(cuuint64_t)(q8 ? p.row_bytes / 2 : p.row_bytes), (cuuint64_t)N};
        const cuuint64_t wstride[1] = {(cuuint64_t)p.row_bytes};
        const cuuint32_t wbox[2] = {q6box ? 240u : q8 ? 136u : (fmt == FMT_Q5_K || fmt == FMT_Q5_0) ? 176u : 144u, 128u};
        cr = enc(&wmap, q8 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(w), wdim, wstride, wbox,
                 estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) {
            snprintf(err, err_len, "cuTensorMapEncodeTiled failed with code %d (weight pointer %p, row bytes %u, N=%zu)", (int)cr, w, p.row_bytes, N);
            return cudaErrorInvalidValue;
        }
    }
    dim3 grid(pl.grid, 1, 1);
    cudaError_t le;
    switch (fmt) {
    case FMT_Q4_0: le = raw ? launch_fmt<FMT_Q4_0, true>(map, wmap, p, grid, smem, st) : launch_fmt<FMT_Q4_0, false>(map, wmap, p, grid, smem, st); break;
    case FMT_Q5_0: le = raw ? launch_fmt<FMT_Q5_0, true>(map, wmap, p, grid, smem, st) : launch_fmt<FMT_Q5_0, false>(map, wmap, p, grid, smem, st); break;
    case FMT_Q8_0: le = raw ? launch_fmt<FMT_Q8_0, true>(map, wmap, p, grid, smem, st) : launch_fmt<FMT_Q8_0, false>(map, wmap, p, grid, smem, st); break;
    case FMT_Q4_K: le = launch_fmt<FMT_Q4_K, true>(map, wmap, p, grid, smem, st); break;
    case FMT_Q5_K: le = launch_fmt<FMT_Q5_K, true>(map, wmap, p, grid, smem, st); break;
    case FMT_Q6_K: le = q6box ? launch_fmt<FMT_Q6_K, true, true>(map, wmap, p, grid, smem, st) : launch_fmt<FMT_Q6_K, true>(map, wmap, p, grid, smem, st); break;
    default: return cudaErrorInvalidValue;
    }
    if (le != cudaSuccess || !pl.split) return le;
    // the K-split tail tiles: add their pieces in K order
    const uint32_t rows = (uint32_t)(M < p.mt ? M : p.mt);
    prefill_reduce_kernel<<<dim3((rows + PF_RED_ROWS - 1) / PF_RED_ROWS, pl.ntail, 1), 128, 0, st>>>(p, pl.grid);
    note_launch();
    return cudaGetLastError();
}

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
