// Dequantise packed GGUF blocks (Q4_0, Q5_0, Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K) straight to f32 / bf16 / f16 / f64.
//
// Stands in for boostr's dequant_*_f32 kernels (src/quant/cuda/kernels/dequant.cu:18-206, one
// thread per block, scalar stores) plus the separate cast pass of CudaClient::dequantize
// (src/quant/cuda/dequant.rs:141-145): the output is produced in a single pass in its final type.
//
// Persistent CTAs, two per SM.  The packed blocks stream through a shared-memory ring of stages of 64
// runs of 256 elements (9-17 KB), each stage ONE bulk copy (cp.async.bulk) signalled on an mbarrier, so
// no thread waits on a global load; a stage is released for refilling as soon as its bytes are in
// registers, before the arithmetic.  A warp decodes two runs per pass: Q4_K lanes take the 8 bytes that
// hold 8 elements of a sub-block in their low nibbles and 8 elements of the next sub-block in their high
// nibbles (the scale/min unpacking is shared by the 16 elements); the other formats take 8 consecutive
// elements per lane and run.  Results leave with 16-byte stores, 64-512 bytes contiguous per warp instruction.
// The kernel is bound by HBM writes: 2 or 4 bytes written per element against 0.56-1.06 bytes read.
//
// Every dequantised value is exactly representable in f32 (block scales are fp16, codes have at
// most 8 bits), so the f32 result is independent of evaluation order; Q4_K's final
// d*sc*q - dmin*m is one rounding of an exact product, written without FMA contraction.
#include "common.cuh"

namespace b200q {

namespace {

// the packed bytes are read from shared memory (plain loads)
__device__ __forceinline__ uint32_t ldg_u16(const uint8_t* p) { return *reinterpret_cast<const unsigned short*>(p); }

// 4 bytes at a 2-byte-aligned address
__device__ __forceinline__ uint32_t ldg_w(const uint8_t* p) { return lds32_u(p); }

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
    } else if constexpr (FMT == FMT_Q5_0) {
        // block = f16 d | 32 high bits | 16 B nibbles; byte i -> elements 2i (low), 2i+1 (high); element e takes bit e of
        // the high-bit word (src/quant/cpu/kernels/dequant_simple.rs:66-95)
        const uint8_t* blk = u + (lane >> 2) * 22;
        float d = f16bits_to_f32(ldg_u16(blk));
        const uint32_t hb = (ldg_w(blk + 2) >> (8 * (lane & 3))) & 0xFFu;  // the high bits of this lane's 8 elements
        const uint32_t w = ldg_w(blk + 6 + 4 * (lane & 3));
        // even bits -> bit 4 of bytes 0..3 (shifts 4, 10, 16, 22; the stray products and their carries miss bits 4, 12, 20, 28)
        const uint32_t lo = (w & 0x0F0F0F0Fu) | (((hb & 0x55u) * 0x00410410u) & 0x10101010u);
        const uint32_t hi = ((w >> 4) & 0x0F0F0F0Fu) | ((((hb >> 1) & 0x55u) * 0x00410410u) & 0x10101010u);
        v[0] = (byte_to_float<0>(lo) - 16.0f) * d; v[1] = (byte_to_float<0>(hi) - 16.0f) * d;
        v[2] = (byte_to_float<1>(lo) - 16.0f) * d; v[3] = (byte_to_float<1>(hi) - 16.0f) * d;
        v[4] = (byte_to_float<2>(lo) - 16.0f) * d; v[5] = (byte_to_float<2>(hi) - 16.0f) * d;
        v[6] = (byte_to_float<3>(lo) - 16.0f) * d; v[7] = (byte_to_float<3>(hi) - 16.0f) * d;
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
    } else if constexpr (FMT == FMT_Q2_K) {
        // block = 16 scale bytes (low nibble scale, high nibble min) | 64 B of 2-bit codes | f16 d | f16 dmin; element
        // e = 128 n + 32 g + 16 h + l takes bits 2g..2g+1 of byte 32 n + 16 h + l and scale byte e / 16
        // (src/quant/cpu/kernels/dequant_k_quants/q2k_q3k.rs:13-58).  d * sc * q is exact, so the fused form rounds once
        // exactly like the reference's multiply-then-subtract.
        const int n = lane >> 4, g = (lane >> 2) & 3, h = (lane >> 1) & 1;
        const uint32_t dm = *reinterpret_cast<const uint32_t*>(u + 80);
        const float d = f16bits_to_f32(dm & 0xFFFF), dmin = f16bits_to_f32(dm >> 16);
        const uint32_t sc = u[lane >> 1];
        const float dl = d * (float)(sc & 15u), nml = -(dmin * (float)(sc >> 4));
        const uint32_t* w = reinterpret_cast<const uint32_t*>(u + 16 + 32 * n + 16 * h + 8 * (lane & 1));  // blocks are 4-byte aligned
        const uint32_t q0 = (w[0] >> (2 * g)) & 0x03030303u, q1 = (w[1] >> (2 * g)) & 0x03030303u;
        v[0] = fmaf(dl, byte_to_float<0>(q0), nml); v[1] = fmaf(dl, byte_to_float<1>(q0), nml);
        v[2] = fmaf(dl, byte_to_float<2>(q0), nml); v[3] = fmaf(dl, byte_to_float<3>(q0), nml);
        v[4] = fmaf(dl, byte_to_float<0>(q1), nml); v[5] = fmaf(dl, byte_to_float<1>(q1), nml);
        v[6] = fmaf(dl, byte_to_float<2>(q1), nml); v[7] = fmaf(dl, byte_to_float<3>(q1), nml);
    } else if constexpr (FMT == FMT_Q3_K) {
        // block = 32 B high-bit masks | 64 B of 2-bit codes | 12 B packed 6-bit scales | f16 d (2-byte aligned); element
        // e = 128 n + 32 g + 16 h + l: low bits 2g..2g+1 of qs[32 n + 16 h + l], high bit 4 n + g of hmask[16 h + l], a
        // clear high bit subtracts 4; scale e / 16 (src/quant/cpu/kernels/dequant_k_quants/q2k_q3k.rs:64-144).
        // (d * scale) * (code - 4) is exact in f32.
        const int n = lane >> 4, g = (lane >> 2) & 3, h = (lane >> 1) & 1, j = lane >> 1;
        const float d = f16bits_to_f32(ldg_u16(u + 108));
        const uint32_t low4 = ((uint32_t)u[96 + (j & 7)] >> (4 * (j >> 3))) & 15u, high2 = ((uint32_t)u[104 + (j & 3)] >> (2 * (j >> 2))) & 3u;
        const float dl = d * (float)((int)(low4 | (high2 << 4)) - 32);
        const uint8_t* qp = u + 32 + 32 * n + 16 * h + 8 * (lane & 1);
        const uint8_t* hp = u + 16 * h + 8 * (lane & 1);
        const uint32_t q0 = (ldg_w(qp) >> (2 * g)) & 0x03030303u, q1 = (ldg_w(qp + 4) >> (2 * g)) & 0x03030303u;
        const uint32_t h0 = (ldg_w(hp) >> (4 * n + g)) & 0x01010101u, h1 = (ldg_w(hp + 4) >> (4 * n + g)) & 0x01010101u;
        const uint32_t c0 = q0 | (h0 << 2), c1 = q1 | (h1 << 2);  // codes 0..7
        v[0] = dl * (byte_to_float<0>(c0) - 4.0f); v[1] = dl * (byte_to_float<1>(c0) - 4.0f);
        v[2] = dl * (byte_to_float<2>(c0) - 4.0f); v[3] = dl * (byte_to_float<3>(c0) - 4.0f);
        v[4] = dl * (byte_to_float<0>(c1) - 4.0f); v[5] = dl * (byte_to_float<1>(c1) - 4.0f);
        v[6] = dl * (byte_to_float<2>(c1) - 4.0f); v[7] = dl * (byte_to_float<3>(c1) - 4.0f);
    } else if constexpr (FMT == FMT_Q4_K) {
        // block = f16 d | f16 dmin | 12 B packed 6-bit scales/mins | 128 B nibbles
        // (src/quant/cpu/kernels/dequant_k_quants/q4k_q5k.rs:10-47, :108-122)
        const int j = lane >> 2;  // 32-element sub-block
        const uint32_t* hd = reinterpret_cast<const uint32_t*>(u);
        const uint4 hq = *reinterpret_cast<const uint4*>(hd);
        const uint32_t dm = hq.x, h1 = hq.y, h2 = hq.z, h3 = hq.w;
        const float d = f16bits_to_f32(dm & 0xFFFF), dmin = f16bits_to_f32(dm >> 16);
        // the four 6-bit scales / mins of sub-blocks 0-3 or 4-7 as packed bytes
        const uint32_t scw = j < 4 ? (h1 & 0x3F3F3F3Fu) : ((h3 & 0x0F0F0F0Fu) | ((h1 >> 2) & 0x30303030u));
        const uint32_t mnw = j < 4 ? (h2 & 0x3F3F3F3Fu) : (((h3 >> 4) & 0x0F0F0F0Fu) | ((h2 >> 2) & 0x30303030u));
        const int sh8 = 8 * (j & 3);
        // d * sc and dmin * m are exact (11 x 6 bits), and so is (d * sc) * q: the fused multiply-add below
        // rounds once, exactly like the multiply-then-subtract of the reference
        const float dl = d * (float)((scw >> sh8) & 0xFF), nml = -(dmin * (float)((mnw >> sh8) & 0xFF));
        const uint2 w = *reinterpret_cast<const uint2*>(u + 16 + (j >> 1) * 32 + 8 * (lane & 3));
        const int sh = (j & 1) * 4;
        const uint32_t q0 = (w.x >> sh) & 0x0F0F0F0Fu, q1 = (w.y >> sh) & 0x0F0F0F0Fu;
        v[0] = fmaf(dl, byte_to_float<0>(q0), nml); v[1] = fmaf(dl, byte_to_float<1>(q0), nml);
        v[2] = fmaf(dl, byte_to_float<2>(q0), nml); v[3] = fmaf(dl, byte_to_float<3>(q0), nml);
        v[4] = fmaf(dl, byte_to_float<0>(q1), nml); v[5] = fmaf(dl, byte_to_float<1>(q1), nml);
        v[6] = fmaf(dl, byte_to_float<2>(q1), nml); v[7] = fmaf(dl, byte_to_float<3>(q1), nml);
    } else if constexpr (FMT == FMT_Q5_K) {
        // block = f16 d | f16 dmin | 12 B packed scales/mins (as Q4_K) | 32 B qh | 128 B qs
        // (src/quant/cpu/kernels/dequant_k_quants/q4k_q5k.rs:56-106).  Element 32 j + l takes nibble (l % 2) of
        // qs[16 j + l / 2] and bit ((32 j + l) % 8) of qh[(32 j + l) / 8]: the lane's elements 8 lane .. 8 lane + 7 are the
        // four bytes qs[4 lane .. 4 lane + 3] (low nibble first) and the eight bits of qh[lane].
        const int j = lane >> 2;
        const uint4 hq = *reinterpret_cast<const uint4*>(u);
        const uint32_t dm = hq.x, h1 = hq.y, h2 = hq.z, h3 = hq.w;
        const float d = f16bits_to_f32(dm & 0xFFFF), dmin = f16bits_to_f32(dm >> 16);
        const uint32_t scw = j < 4 ? (h1 & 0x3F3F3F3Fu) : ((h3 & 0x0F0F0F0Fu) | ((h1 >> 2) & 0x30303030u));
        const uint32_t mnw = j < 4 ? (h2 & 0x3F3F3F3Fu) : (((h3 >> 4) & 0x0F0F0F0Fu) | ((h2 >> 2) & 0x30303030u));
        const int sh8 = 8 * (j & 3);
        const float dl = d * (float)((scw >> sh8) & 0xFF), nml = -(dmin * (float)((mnw >> sh8) & 0xFF));
        const uint32_t w = *reinterpret_cast<const uint32_t*>(u + 48 + 4 * lane);
        const uint32_t hb = u[16 + lane];
        // even elements: low nibbles + bits 0, 2, 4, 6 of hb; odd elements: high nibbles + bits 1, 3, 5, 7
        const uint32_t be = ((hb & 1u) | ((hb & 4u) << 6) | ((hb & 16u) << 12) | ((hb & 64u) << 18)) << 4;
        const uint32_t bo = (((hb >> 1) & 1u) | (((hb >> 1) & 4u) << 6) | (((hb >> 1) & 16u) << 12) | (((hb >> 1) & 64u) << 18)) << 4;
        const uint32_t qe = (w & 0x0F0F0F0Fu) | be, qo = ((w >> 4) & 0x0F0F0F0Fu) | bo;
        v[0] = fmaf(dl, byte_to_float<0>(qe), nml); v[1] = fmaf(dl, byte_to_float<0>(qo), nml);
        v[2] = fmaf(dl, byte_to_float<1>(qe), nml); v[3] = fmaf(dl, byte_to_float<1>(qo), nml);
        v[4] = fmaf(dl, byte_to_float<2>(qe), nml); v[5] = fmaf(dl, byte_to_float<2>(qo), nml);
        v[6] = fmaf(dl, byte_to_float<3>(qe), nml); v[7] = fmaf(dl, byte_to_float<3>(qo), nml);
    } else {
        // Q6_K block = 128 B ql | 64 B qh | 16 x i8 scales | f16 d
        // (src/quant/cpu/kernels/dequant_k_quants/q6k_q8k.rs:10-56)
        int n = lane >> 4, gq = (lane >> 2) & 3, l0 = 8 * (lane & 3);
        float d = f16bits_to_f32(ldg_u16(u + 208));
        int sc = (int)(signed char)u[192 + 8 * n + 2 * gq + (l0 >> 4)];
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

// Q4_K, 16 elements per lane: lane (jj, t) of a 16-lane group takes bytes [32 jj + 8 t, +8) of the block's 128 nibble
// bytes: low nibbles = elements 64 jj + 8 t .. of sub-block 2 jj, high nibbles = the same positions of sub-block 2 jj + 1.
__device__ __forceinline__ void decode16_q4k(const uint8_t* blk, int jj, int t, float (&lo)[8], float (&hi)[8]) {
    const uint4 hq = *reinterpret_cast<const uint4*>(blk);
    const float d = f16bits_to_f32(hq.x & 0xFFFF), dmin = f16bits_to_f32(hq.x >> 16);
    // 6-bit scales / mins of sub-blocks 0-3 and 4-7 as packed bytes (unpack_q4k_q5k_scales, q4k_q5k.rs:108-122)
    const uint32_t sc03 = hq.y & 0x3F3F3F3Fu, mn03 = hq.z & 0x3F3F3F3Fu;
    const uint32_t sc47 = (hq.w & 0x0F0F0F0Fu) | ((hq.y >> 2) & 0x30303030u);
    const uint32_t mn47 = ((hq.w >> 4) & 0x0F0F0F0Fu) | ((hq.z >> 2) & 0x30303030u);
    // sub-blocks 2 jj and 2 jj + 1 are two neighbouring bytes of one of those words
    const uint32_t scw = (jj < 2 ? sc03 : sc47) >> (16 * (jj & 1)), mnw = (jj < 2 ? mn03 : mn47) >> (16 * (jj & 1));
    const float dl0 = d * byte_to_float<0>(scw), dl1 = d * byte_to_float<1>(scw);
    const float nm0 = -(dmin * byte_to_float<0>(mnw)), nm1 = -(dmin * byte_to_float<1>(mnw));
    const uint2 w = *reinterpret_cast<const uint2*>(blk + 16 + 32 * jj + 8 * t);
    const uint32_t l0 = w.x & 0x0F0F0F0Fu, l1 = w.y & 0x0F0F0F0Fu, h0 = (w.x >> 4) & 0x0F0F0F0Fu, h1 = (w.y >> 4) & 0x0F0F0F0Fu;
    // d * sc and (d * sc) * q are exact, so the fused form rounds once exactly like multiply-then-subtract
    lo[0] = fmaf(dl0, byte_to_float<0>(l0), nm0); lo[1] = fmaf(dl0, byte_to_float<1>(l0), nm0);
    lo[2] = fmaf(dl0, byte_to_float<2>(l0), nm0); lo[3] = fmaf(dl0, byte_to_float<3>(l0), nm0);
    lo[4] = fmaf(dl0, byte_to_float<0>(l1), nm0); lo[5] = fmaf(dl0, byte_to_float<1>(l1), nm0);
    lo[6] = fmaf(dl0, byte_to_float<2>(l1), nm0); lo[7] = fmaf(dl0, byte_to_float<3>(l1), nm0);
    hi[0] = fmaf(dl1, byte_to_float<0>(h0), nm1); hi[1] = fmaf(dl1, byte_to_float<1>(h0), nm1);
    hi[2] = fmaf(dl1, byte_to_float<2>(h0), nm1); hi[3] = fmaf(dl1, byte_to_float<3>(h0), nm1);
    hi[4] = fmaf(dl1, byte_to_float<0>(h1), nm1); hi[5] = fmaf(dl1, byte_to_float<1>(h1), nm1);
    hi[6] = fmaf(dl1, byte_to_float<2>(h1), nm1); hi[7] = fmaf(dl1, byte_to_float<3>(h1), nm1);
}

constexpr int DQ_STAGE_UNITS = 64, DQ_WARPS = 8;
constexpr int DQ_OFF_EMPTY = 64, DQ_OFF_STAGE0 = 256;  // full[8] | empty[8] | stages

// unit = 256 elements (one K-quant block, eight Q4_0 / Q8_0 blocks); the last unit of a Q4_0 / Q8_0 tensor may be
// partial (tail_elems of 256).  Stage g of the tensor = units [64 g, 64 g + 64); CTA c takes stages c, c + grid, ...
template <int FMT, typename OutT>
__global__ void __launch_bounds__(DQ_WARPS * 32, 2) dequant_kernel(const uint8_t* __restrict__ w, OutT* __restrict__ out, size_t nunits,
                                                                   int tail_elems, size_t w_bytes, uint32_t nstages,
                                                                   unsigned int* status) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int UB = fmt_slice_bytes(FMT);
    constexpr uint32_t STAGE_BYTES = DQ_STAGE_UNITS * UB + 128;  // + room for the 16-byte rounding of the last copy
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar_full = smem_u32(smem), bar_empty = bar_full + DQ_OFF_EMPTY;
    const uint32_t stage0 = smem_u32(smem + DQ_OFF_STAGE0);
    const size_t total_stages = (nunits + DQ_STAGE_UNITS - 1) / DQ_STAGE_UNITS;
    const size_t my_stages = total_stages > blockIdx.x ? (total_stages - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    auto issue_fill = [&](size_t i, uint32_t slot) {  // one lane: my i-th stage into ring slot `slot`
        const size_t g = blockIdx.x + i * gridDim.x;
        const size_t begin = g * DQ_STAGE_UNITS * (size_t)UB;
        size_t bytes = (size_t)DQ_STAGE_UNITS * UB;
        if (begin + bytes > w_bytes) bytes = w_bytes - begin;
        fill_contiguous(stage0 + slot * STAGE_BYTES, smem + DQ_OFF_STAGE0 + slot * STAGE_BYTES, w + begin, (uint32_t)bytes, w + w_bytes,
                        bar_full + 8 * slot);
    };

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < nstages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, DQ_WARPS);
        }
        mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 0)
        for (uint32_t s = 0; s < nstages && s < my_stages; ++s) issue_fill(s, s);

    bool dead = false;
    uint32_t slot = 0, par = 0;
    for (size_t i = 0; i < my_stages; ++i) {
        if (!dead && !mbar_wait(bar_full + 8 * slot, par)) {
            dead = true;
            atomicOr(status, STATUS_TIMEOUT_FULL);
        }
        const size_t g = blockIdx.x + i * gridDim.x;
        const size_t unit0 = g * DQ_STAGE_UNITS + (size_t)warp * (DQ_STAGE_UNITS / DQ_WARPS);  // this warp's 8 units of the stage
        const uint8_t* src = smem + DQ_OFF_STAGE0 + slot * STAGE_BYTES + (size_t)warp * (DQ_STAGE_UNITS / DQ_WARPS) * UB;
        if constexpr (FMT == FMT_Q4_K) {
            // 4 passes of two blocks; a 16-lane group per block
            const int bsel = lane >> 4, jj = (lane >> 2) & 3, t = lane & 3;
            float lo[4][8], hi[4][8];
#pragma unroll
            for (int ps = 0; ps < 4; ++ps)
                if (!dead && unit0 + 2 * ps + bsel < nunits) decode16_q4k(src + (2 * ps + bsel) * UB, jj, t, lo[ps], hi[ps]);
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * slot);  // the stage's bytes are in registers
#pragma unroll
            for (int ps = 0; ps < 4; ++ps)
                if (!dead && unit0 + 2 * ps + bsel < nunits) {
                    OutT* o = out + (unit0 + 2 * ps + bsel) * 256 + 64 * jj + 8 * t;
                    store8<OutT>(o, lo[ps]);
                    store8<OutT>(o + 32, hi[ps]);
                }
        } else {
            // 8 consecutive elements per lane and unit; four units are decoded before any is stored
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                float v[4][8];
                int ok[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const size_t unit = unit0 + 4 * half + q;
                    const int valid = unit >= nunits ? 0 : (unit + 1 == nunits && tail_elems) ? tail_elems : 256;
                    ok[q] = !dead && 8 * lane < valid;  // elements come in whole 32-blocks: 8-lane groups are all-or-nothing
                    if (ok[q]) decode8<FMT>(src + (4 * half + q) * UB, lane, v[q]);
                }
                if (half == 1) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_empty + 8 * slot);
                }
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (ok[q]) store8<OutT>(out + (unit0 + 4 * half + q) * 256 + 8 * lane, v[q]);
            }
        }
        // refill the slot with my stage i + nstages once every warp has released it
        if (warp == 0 && i + nstages < my_stages) {
            if (!dead && !mbar_wait(bar_empty + 8 * slot, par)) {
                dead = true;
                atomicOr(status, STATUS_TIMEOUT_EMPTY);
            }
            if (!dead && lane == 0) issue_fill(i + nstages, slot);
        }
        if (++slot == nstages) {
            slot = 0;
            par ^= 1;
        }
    }
}

template <int FMT, typename OutT>
cudaError_t launch_dequant_t(const uint8_t* w, OutT* out, size_t nunits, int tail, size_t w_bytes, int grid, cudaStream_t st,
                             unsigned int* status) {
    constexpr uint32_t STAGE_BYTES = DQ_STAGE_UNITS * fmt_slice_bytes(FMT) + 128;
    constexpr uint32_t NST = 6;  // 56-105 KB per CTA: two CTAs share an SM for every format
    constexpr size_t SMEM = DQ_OFF_STAGE0 + (size_t)NST * STAGE_BYTES;
    static PerDeviceOnce attrs;
    cudaError_t ae = attrs.run([] { return cudaFuncSetAttribute(dequant_kernel<FMT, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM); });
    if (ae != cudaSuccess) return ae;
    dequant_kernel<FMT, OutT><<<grid, DQ_WARPS * 32, SMEM, st>>>(w, out, nunits, tail, w_bytes, NST, status);
    note_launch();
    return cudaGetLastError();
}

template <int FMT>
cudaError_t launch_dequant_fmt(const void* w, size_t nblocks, void* out, int out_dtype, cudaStream_t st, int sm_count, unsigned int* status) {
    constexpr int per_unit = 256 / fmt_block_size(FMT);
    const size_t nunits = (nblocks + per_unit - 1) / per_unit;
    const int tail = (int)(nblocks % per_unit) * fmt_block_size(FMT);
    const size_t w_bytes = nblocks * (size_t)fmt_block_bytes(FMT);
    const size_t nstage = (nunits + DQ_STAGE_UNITS - 1) / DQ_STAGE_UNITS;
    int grid = (int)(nstage < (size_t)sm_count * 2 ? nstage : (size_t)sm_count * 2);
    if (grid < 1) grid = 1;
    const uint8_t* wp = static_cast<const uint8_t*>(w);
    switch (out_dtype) {
    case DT_F32: return launch_dequant_t<FMT, float>(wp, static_cast<float*>(out), nunits, tail, w_bytes, grid, st, status);
    case DT_BF16: return launch_dequant_t<FMT, __nv_bfloat16>(wp, static_cast<__nv_bfloat16*>(out), nunits, tail, w_bytes, grid, st, status);
    case DT_F16: return launch_dequant_t<FMT, __half>(wp, static_cast<__half*>(out), nunits, tail, w_bytes, grid, st, status);
    case DT_F64: return launch_dequant_t<FMT, double>(wp, static_cast<double*>(out), nunits, tail, w_bytes, grid, st, status);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace

cudaError_t launch_dequant(int fmt, const void* w, size_t nblocks, void* out, int out_dtype, cudaStream_t st, int sm_count,
                           unsigned int* status) {
    switch (fmt) {
    case FMT_Q4_0: return launch_dequant_fmt<FMT_Q4_0>(w, nblocks, out, out_dtype, st, sm_count, status);
    case FMT_Q8_0: return launch_dequant_fmt<FMT_Q8_0>(w, nblocks, out, out_dtype, st, sm_count, status);
    case FMT_Q4_K: return launch_dequant_fmt<FMT_Q4_K>(w, nblocks, out, out_dtype, st, sm_count, status);
    case FMT_Q2_K: return launch_dequant_fmt<FMT_Q2_K>(w, nblocks, out, out_dtype, st, sm_count, status);
    case FMT_Q3_K: return launch_dequant_fmt<FMT_Q3_K>(w, nblocks, out, out_dtype, st, sm_count, status);
    case FMT_Q5_0: return launch_dequant_fmt<FMT_Q5_0>(w, nblocks, out, out_dtype, st, sm_count, status);
    case FMT_Q5_K: return launch_dequant_fmt<FMT_Q5_K>(w, nblocks, out, out_dtype, st, sm_count, status);
    case FMT_Q6_K: return launch_dequant_fmt<FMT_Q6_K>(w, nblocks, out, out_dtype, st, sm_count, status);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace b200q
