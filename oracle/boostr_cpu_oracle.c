/*
 * CPU oracle for the quantized-linear hot path of ml-rust/boostr (v0.2.0).
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of boostr's own
 * CPU algorithms for QuantTensor dequantisation and quantized matmul (formats
 * Q4_0, Q8_0, Q4_K, Q6_K).  It is the checker for the CUDA kernels and the timed
 * CPU baseline of the benchmark.  Nothing in the product path links, imports or
 * calls it.
 *
 * Parity status.  boostr is Rust and cannot be compiled where this was written
 * (no rustc/cargo; its tensor crate numr 0.6.1 is not vendored), so the
 * restatement is pinned against
 *   (a) every known-answer test the reference holds for this path
 *       (src/quant/cpu/kernels/dequant_simple.rs:185-289,
 *        src/quant/cpu/kernels/dequant_k_quants/q4k_q5k.rs:129-190,
 *        src/quant/cpu/kernels/dequant_k_quants/q6k_q8k.rs:89-98,
 *        src/quant/cpu/kernels/quant_matmul.rs:415-510,
 *        src/quant/cpu/quant_matmul/tests.rs:19-88,
 *        src/quant/cpu/kernels/simd/quantize_act_q8k.rs:145-171,
 *        src/quant/cpu/kernels/simd/fused_q4k_q8k_dot.rs:181-245,
 *        src/quant/cpu/kernels/simd/fused_q6k_q8k_dot.rs:233-297), and
 *   (b) the gguf-py 0.19.0 dequantisers as an independent witness for Q8_0, Q4_K
 *       and Q6_K (bit-equal; NOT for Q4_0, whose element order in boostr differs
 *       from ggml's).
 * One piece is "parity unpinned": the f32 -> bf16/f16 cast of `dequantize` lives in
 * numr (`cast`, called at src/quant/cpu/dequant.rs:124) whose source is absent and
 * which no boostr test pins by value; round-to-nearest-even is assumed here.
 * `quant_swiglu`'s silu_mul is numr's as well (src/quant/cpu/quant_matmul/impl_ops.rs:347-358);
 * x/(1+exp(-x)) in f32 is assumed and compared with a tolerance, never bit-wise.
 *
 * Build: gcc -O2 -mavx2 -mfma -mf16c -ffp-contract=off -fPIC -shared -pthread
 * (-ffp-contract=off because rustc never contracts a*b+c; the one place the
 * reference fuses, dot_f32_avx2_fma, is written with explicit fmaf below).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#if defined(__AVX2__)
#include <immintrin.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* Format ids follow QuantFormat::format_id (src/quant/format.rs:204-230). */
enum { FMT_Q4_0 = 0, FMT_Q5_0 = 2, FMT_Q8_0 = 4, FMT_Q2_K = 6, FMT_Q3_K = 7, FMT_Q4_K = 8, FMT_Q5_K = 9, FMT_Q6_K = 10 };

/* block_size / block_bytes: src/quant/format.rs:81-140 */
ORACLE_API int oracle_block_size(int fmt) {
    switch (fmt) {
    case FMT_Q4_0: case FMT_Q5_0: case FMT_Q8_0: return 32;
    case FMT_Q2_K: case FMT_Q3_K: case FMT_Q4_K: case FMT_Q5_K: case FMT_Q6_K: return 256;
    default: return 0;
    }
}
ORACLE_API int oracle_block_bytes(int fmt) {
    switch (fmt) {
    case FMT_Q4_0: return 18;
    case FMT_Q5_0: return 22;
    case FMT_Q8_0: return 34;
    case FMT_Q2_K: return 84;
    case FMT_Q3_K: return 110;
    case FMT_Q4_K: return 144;
    case FMT_Q5_K: return 176;
    case FMT_Q6_K: return 210;
    default: return 0;
    }
}

/* IEEE binary16 -> binary32, exact (what half 2.7.1 f16::to_f32 computes). */
static float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}
static inline uint16_t rd16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

ORACLE_API float oracle_f16_to_f32(uint16_t h) { return f16_to_f32(h); }

/* ------------------------------------------------------------------ dequant */

/* dequant_q4_0: src/quant/cpu/kernels/dequant_simple.rs:11-32.
 * NOTE the interleaved order: byte i gives out[2i] (low nibble), out[2i+1] (high). */
static void dequant_q4_0(const uint8_t *blocks, size_t nblocks, float *out) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = blocks + b * 18;
        float d = f16_to_f32(rd16(blk));
        const uint8_t *qs = blk + 2;
        float *o = out + b * 32;
        for (int i = 0; i < 16; i++) {
            int lo = (int)(qs[i] & 0x0F) - 8;
            int hi = (int)((qs[i] >> 4) & 0x0F) - 8;
            o[2 * i] = (float)lo * d;
            o[2 * i + 1] = (float)hi * d;
        }
    }
}

/* dequant_q5_0: src/quant/cpu/kernels/dequant_simple.rs:66-95.  Block = f16 d | 32 high bits | 16 bytes of nibbles;
 * element 2 i = low nibble of byte i, element 2 i + 1 = its high nibble (boostr's interleaved order, as for Q4_0),
 * and element e takes bit e of the high-bit word; value = (5-bit code - 16) * d. */
static void dequant_q5_0(const uint8_t *blocks, size_t nblocks, float *out) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = blocks + b * 22;
        float d = f16_to_f32(rd16(blk));
        uint32_t qh = (uint32_t)blk[2] | ((uint32_t)blk[3] << 8) | ((uint32_t)blk[4] << 16) | ((uint32_t)blk[5] << 24);
        const uint8_t *qs = blk + 6;
        float *o = out + b * 32;
        for (int i = 0; i < 16; i++) {
            int lo = (int)((qs[i] & 0x0F) | (((qh >> (2 * i)) & 1u) << 4)) - 16;
            int hi = (int)(((qs[i] >> 4) & 0x0F) | (((qh >> (2 * i + 1)) & 1u) << 4)) - 16;
            o[2 * i] = (float)lo * d;
            o[2 * i + 1] = (float)hi * d;
        }
    }
}

/* dequant_q8_0: src/quant/cpu/kernels/dequant_simple.rs:137-155 */
static void dequant_q8_0(const uint8_t *blocks, size_t nblocks, float *out) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = blocks + b * 34;
        float d = f16_to_f32(rd16(blk));
        const int8_t *qs = (const int8_t *)(blk + 2);
        float *o = out + b * 32;
        for (int i = 0; i < 32; i++) o[i] = (float)qs[i] * d;
    }
}

/* unpack_q4k_q5k_scales: src/quant/cpu/kernels/dequant_k_quants/q4k_q5k.rs:108-122 */
static void unpack_q4k_scales(const uint8_t *sc, uint8_t scales[8], uint8_t mins[8]) {
    for (int i = 0; i < 4; i++) {
        scales[i] = sc[i] & 0x3F;
        mins[i] = sc[i + 4] & 0x3F;
    }
    for (int i = 4; i < 8; i++) {
        scales[i] = (uint8_t)((sc[i + 4] & 0x0F) | ((sc[i - 4] >> 6) << 4));
        mins[i] = (uint8_t)((sc[i + 4] >> 4) | ((sc[i] >> 6) << 4));
    }
}

/* dequant_q4k: src/quant/cpu/kernels/dequant_k_quants/q4k_q5k.rs:10-47 */
static void dequant_q4k(const uint8_t *blocks, size_t nblocks, float *out) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = blocks + b * 144;
        float d = f16_to_f32(rd16(blk));
        float dmin = f16_to_f32(rd16(blk + 2));
        const uint8_t *qs = blk + 16;
        uint8_t scales[8], mins[8];
        unpack_q4k_scales(blk + 4, scales, mins);
        float *o = out + b * 256;
        for (int j = 0; j < 8; j++) {
            float dl = d * (float)scales[j];
            float ml = dmin * (float)mins[j];
            int base = (j / 2) * 32;
            int high = j & 1;
            for (int l = 0; l < 32; l++) {
                float q = high ? (float)((qs[base + l] >> 4) & 0x0F) : (float)(qs[base + l] & 0x0F);
                o[j * 32 + l] = dl * q - ml;
            }
        }
    }
}

/* dequant_q5k: src/quant/cpu/kernels/dequant_k_quants/q4k_q5k.rs:56-106.
 * Block = f16 d | f16 dmin | 12 B scales (as Q4_K) | 32 B qh | 128 B qs.  NOTE the element order: element l of
 * sub-block j takes nibble (l % 2) of qs[16 j + l / 2] (interleaved, 16 bytes per sub-block) and bit (idx % 8) of
 * qh[idx / 8] with idx = 32 j + l.  This is neither ggml's Q5_K order nor the order the reference's own Q8_K dot
 * product uses on x86 (dot_q5k_q8k_avx2order below); the restatement follows each function as it is written. */
static void dequant_q5k(const uint8_t *blocks, size_t nblocks, float *out) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = blocks + b * 176;
        float d = f16_to_f32(rd16(blk));
        float dmin = f16_to_f32(rd16(blk + 2));
        const uint8_t *qh = blk + 16, *qs = blk + 48;
        uint8_t scales[8], mins[8];
        unpack_q4k_scales(blk + 4, scales, mins);
        float *o = out + b * 256;
        for (int j = 0; j < 8; j++) {
            float dl = d * (float)scales[j];
            float ml = dmin * (float)mins[j];
            for (int l = 0; l < 32; l++) {
                int idx = j * 32 + l;
                int byte = qs[j * 16 + l / 2];
                int low4 = (l % 2 == 0) ? (byte & 0x0F) : ((byte >> 4) & 0x0F);
                int high1 = (qh[idx / 8] >> (idx % 8)) & 1;
                float q = (float)(low4 | (high1 << 4));
                o[idx] = dl * q - ml;
            }
        }
    }
}

/* dequant_q6k: src/quant/cpu/kernels/dequant_k_quants/q6k_q8k.rs:10-56 */
static void dequant_q6k(const uint8_t *blocks, size_t nblocks, float *out) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = blocks + b * 210;
        const uint8_t *ql = blk;
        const uint8_t *qh = blk + 128;
        const int8_t *sc = (const int8_t *)(blk + 192);
        float d = f16_to_f32(rd16(blk + 208));
        float *o = out + b * 256;
        for (int n = 0; n < 2; n++) {
            int yb = n * 128, qlb = n * 64, qhb = n * 32, scb = n * 8;
            for (int l = 0; l < 32; l++) {
                int is = l / 16;
                int8_t q1 = (int8_t)((ql[qlb + l] & 0x0F) | ((qh[qhb + l] & 0x03) << 4)) - 32;
                int8_t q2 = (int8_t)((ql[qlb + l + 32] & 0x0F) | (((qh[qhb + l] >> 2) & 0x03) << 4)) - 32;
                int8_t q3 = (int8_t)((ql[qlb + l] >> 4) | (((qh[qhb + l] >> 4) & 0x03) << 4)) - 32;
                int8_t q4 = (int8_t)((ql[qlb + l + 32] >> 4) | (((qh[qhb + l] >> 6) & 0x03) << 4)) - 32;
                /* d * sc * q, evaluated left to right as the Rust expression is */
                o[yb + l] = d * (float)sc[scb + is] * (float)q1;
                o[yb + l + 32] = d * (float)sc[scb + is + 2] * (float)q2;
                o[yb + l + 64] = d * (float)sc[scb + is + 4] * (float)q3;
                o[yb + l + 96] = d * (float)sc[scb + is + 6] * (float)q4;
            }
        }
    }
}

/* dequant_q2k: src/quant/cpu/kernels/dequant_k_quants/q2k_q3k.rs:13-58.  Block = 16 scale bytes (low nibble: sub-block
 * scale, high nibble: sub-block min) | 64 bytes of 2-bit codes | f16 d | f16 dmin.  Element e = 128 n + 32 g + 16 h + l
 * takes bits 2 g .. 2 g + 1 of byte 32 n + 16 h + l and the scale byte e / 16; value = d * sc * q - dmin * m (the
 * product and the subtraction each rounded, as the reference writes them). */
static void dequant_q2k(const uint8_t *blocks, size_t nblocks, float *out) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = blocks + b * 84;
        const uint8_t *sc = blk, *qs = blk + 16;
        float d = f16_to_f32(rd16(blk + 80)), dmin = f16_to_f32(rd16(blk + 82));
        float *o = out + b * 256;
        int y = 0, is = 0;
        for (int n = 0; n < 2; n++) {
            const uint8_t *q = qs + 32 * n;
            for (int shift = 0; shift < 8; shift += 2) {
                for (int h = 0; h < 2; h++) {
                    float dl = d * (float)(sc[is] & 0x0F);
                    float ml = dmin * (float)(sc[is] >> 4);
                    is++;
                    for (int l = 0; l < 16; l++) {
                        volatile float p = dl * (float)((q[16 * h + l] >> shift) & 3);  /* no contraction into an FMA */
                        o[y++] = p - ml;
                    }
                }
            }
        }
    }
}

/* unpack_q3k_scales: src/quant/cpu/kernels/dequant_k_quants/q2k_q3k.rs:115-144.  Sixteen 6-bit scales from 12 bytes:
 * low four bits from the nibbles of bytes 0..7, high two bits from the bit pairs of bytes 8..11; value - 32. */
static void unpack_q3k_scales(const uint8_t *sc, int8_t *out) {
    for (int j = 0; j < 16; j++) {
        int low4 = (sc[j & 7] >> (4 * (j >> 3))) & 15;
        int high2 = (sc[8 + (j & 3)] >> (2 * (j >> 2))) & 3;
        out[j] = (int8_t)((low4 | (high2 << 4)) - 32);
    }
}

/* The 3-bit code minus 4 of element e = 128 n + 32 g + 16 h + l of a Q3_K block: two low bits from qs[32 n + 16 h + l]
 * (bits 2g..2g+1), the high bit from hmask[16 h + l] (bit 4 n + g); a clear high bit subtracts 4
 * (q2k_q3k.rs:64-110). */
static inline int q3k_code(const uint8_t *blk, int e) {
    int n = e >> 7, g = (e >> 5) & 3, hl = e & 31;
    int low2 = (blk[32 + 32 * n + hl] >> (2 * g)) & 3;
    int hbit = (blk[hl] >> (4 * n + g)) & 1;
    return low2 - (hbit ? 0 : 4);
}

/* dequant_q3k: src/quant/cpu/kernels/dequant_k_quants/q2k_q3k.rs:64-110.  Block = 32 B high-bit masks | 64 B of 2-bit
 * codes | 12 B packed scales | f16 d; value = (d * scale[e / 16]) * (code - 4). */
static void dequant_q3k(const uint8_t *blocks, size_t nblocks, float *out) {
    for (size_t b = 0; b < nblocks; b++) {
        const uint8_t *blk = blocks + b * 110;
        int8_t scales[16];
        unpack_q3k_scales(blk + 96, scales);
        float d = f16_to_f32(rd16(blk + 108));
        for (int e = 0; e < 256; e++) {
            float dl = d * (float)scales[e >> 4];
            out[b * 256 + e] = dl * (float)q3k_code(blk, e);
        }
    }
}

/* dequant_row_f32 (src/quant/cpu/kernels/quant_matmul.rs:378-407) restricted to the
 * four formats on the path; also the body of CpuClient::dequantize
 * (src/quant/cpu/dequant.rs:91-115). Returns 0, or -1 for an unknown format. */
ORACLE_API int oracle_dequant_f32(int fmt, const uint8_t *blocks, size_t nblocks, float *out) {
    switch (fmt) {
    case FMT_Q4_0: dequant_q4_0(blocks, nblocks, out); return 0;
    case FMT_Q5_0: dequant_q5_0(blocks, nblocks, out); return 0;
    case FMT_Q8_0: dequant_q8_0(blocks, nblocks, out); return 0;
    case FMT_Q2_K: dequant_q2k(blocks, nblocks, out); return 0;
    case FMT_Q3_K: dequant_q3k(blocks, nblocks, out); return 0;
    case FMT_Q4_K: dequant_q4k(blocks, nblocks, out); return 0;
    case FMT_Q5_K: dequant_q5k(blocks, nblocks, out); return 0;
    case FMT_Q6_K: dequant_q6k(blocks, nblocks, out); return 0;
    default: return -1;
    }
}

/* f32 -> bf16, round to nearest even, NaN kept quiet.  Stands in for numr's cast
 * (parity unpinned, see the header). */
ORACLE_API uint16_t oracle_f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u);
    uint32_t r = 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)((u + r) >> 16);
}

/* f32 -> f16, round to nearest even (parity unpinned, as above). */
ORACLE_API uint16_t oracle_f32_to_f16(float f) {
#if defined(__F16C__)
    return (uint16_t)_cvtss_sh(f, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC);
#else
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax > 0x7F800000u) return (uint16_t)(sign | 0x7E00u);
    if (ax >= 0x47800000u) return (uint16_t)(sign | 0x7C00u);
    if (ax < 0x38800000u) { /* subnormal or zero in f16 */
        if (ax < 0x33000000u) return (uint16_t)sign;
        int e = (int)(ax >> 23);
        uint32_t m = (ax & 0x7FFFFFu) | 0x800000u;
        int shift = 126 - e; /* 14..24 */
        uint32_t half = m >> shift;
        uint32_t rem = m & ((1u << shift) - 1u);
        uint32_t mid = 1u << (shift - 1);
        if (rem > mid || (rem == mid && (half & 1u))) half++;
        return (uint16_t)(sign | half);
    }
    uint32_t v = ax - 0x38000000u;
    uint32_t half = v >> 13;
    uint32_t rem = v & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++;
    return (uint16_t)(sign | half);
#endif
}

/* dequantize to a 16-bit target: f32 kernel, then the cast (src/quant/cpu/dequant.rs:118-125).
 * out_kind: 1 = bf16, 2 = f16. */
ORACLE_API int oracle_dequant_16(int fmt, const uint8_t *blocks, size_t nblocks, uint16_t *out, int out_kind) {
    int bs = oracle_block_size(fmt);
    if (!bs) return -1;
    float tmp[256];
    int bb = oracle_block_bytes(fmt);
    for (size_t b = 0; b < nblocks; b++) {
        oracle_dequant_f32(fmt, blocks + b * (size_t)bb, 1, tmp);
        for (int i = 0; i < bs; i++)
            out[b * (size_t)bs + i] = out_kind == 1 ? oracle_f32_to_bf16(tmp[i]) : oracle_f32_to_f16(tmp[i]);
    }
    return 0;
}

/* ------------------------------------------------------- Q8_K activations */

#define Q8K_BLOCK_BYTES 292

/* quantize_f32_to_q8k, AVX2 semantics: src/quant/cpu/kernels/simd/quantize_act_q8k.rs:26-98.
 * The x86 reference rounds half-to-even (_mm256_round_ps NEAREST, then cvtps_epi32);
 * its scalar fallback (:114-138) rounds half away and is NOT what an x86 host runs.
 * rintf() under the default rounding mode is round-half-even.
 * Block layout (292 B): f32 d | 256 x i8 | 16 x i16 sums of 16. */
ORACLE_API void oracle_quantize_q8k(const float *x, size_t n, uint8_t *out) {
    size_t nb = n / 256;
    for (size_t b = 0; b < nb; b++) {
        const float *src = x + b * 256;
        uint8_t *dst = out + b * Q8K_BLOCK_BYTES;
        float amax = 0.0f;
        for (int i = 0; i < 256; i++) {
            float a = fabsf(src[i]);
            if (a > amax) amax = a; /* max_ps(amax, |v|): keeps amax when v is NaN-free */
        }
        float d = amax / 127.0f;
        float id = amax != 0.0f ? 127.0f / amax : 0.0f;
        memcpy(dst, &d, 4);
        for (int sub = 0; sub < 16; sub++) {
            int16_t bsum = 0;
            for (int j = 0; j < 16; j++) {
                int idx = sub * 16 + j;
                float r = rintf(src[idx] * id);
                if (r > 127.0f) r = 127.0f;
                if (r < -128.0f) r = -128.0f;
                int8_t q = (int8_t)(int32_t)r;
                dst[4 + idx] = (uint8_t)q;
                bsum = (int16_t)(bsum + q);
            }
            dst[260 + sub * 2] = (uint8_t)(bsum & 0xFF);
            dst[260 + sub * 2 + 1] = (uint8_t)((bsum >> 8) & 0xFF);
        }
    }
}

/* fused_dot_q4k_q8k: scalar form src/quant/cpu/kernels/simd/fused_q4k_q8k_dot.rs:111-172
 * (the AVX2 form :27-96 produces the same integers and the same f32 expression). */
static float dot_q4k_q8k_scalar(const uint8_t *act_q8k, const uint8_t *w, size_t k) {
    size_t nb = k / 256;
    float sumf = 0.0f;
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *q4 = w + b * 144;
        float d = f16_to_f32(rd16(q4));
        float dmin = f16_to_f32(rd16(q4 + 2));
        const uint8_t *qs = q4 + 16;
        uint8_t scales[8], mins[8];
        unpack_q4k_scales(q4 + 4, scales, mins);
        const uint8_t *a = act_q8k + b * Q8K_BLOCK_BYTES;
        float d8;
        memcpy(&d8, a, 4);
        const int8_t *q8 = (const int8_t *)(a + 4);
        const uint8_t *bs = a + 260;
        float dall = d * d8;
        float dmin_all = dmin * d8;
        int32_t sumi = 0, sumi_mins = 0;
        for (int j = 0; j < 8; j++) {
            int base = (j / 2) * 32;
            int high = j & 1;
            int32_t dot = 0;
            for (int l = 0; l < 32; l++) {
                int nib = high ? (qs[base + l] >> 4) & 0x0F : qs[base + l] & 0x0F;
                dot += nib * (int32_t)q8[j * 32 + l];
            }
            sumi += dot * (int32_t)scales[j];
            int32_t bsum = (int32_t)(int16_t)rd16(bs + j * 4) + (int32_t)(int16_t)rd16(bs + j * 4 + 2);
            sumi_mins += (int32_t)mins[j] * bsum;
        }
        float t = dall * (float)sumi - dmin_all * (float)sumi_mins;
        sumf += t;
    }
    return sumf;
}

/* fused_dot_q6k_q8k: scalar form src/quant/cpu/kernels/simd/fused_q6k_q8k_dot.rs:170-224 */
static float dot_q6k_q8k_scalar(const uint8_t *act_q8k, const uint8_t *w, size_t k) {
    size_t nb = k / 256;
    float sumf = 0.0f;
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = w + b * 210;
        const uint8_t *ql = blk, *qh = blk + 128;
        const int8_t *sc = (const int8_t *)(blk + 192);
        float d6 = f16_to_f32(rd16(blk + 208));
        const uint8_t *a = act_q8k + b * Q8K_BLOCK_BYTES;
        float d8;
        memcpy(&d8, a, 4);
        const int8_t *q8 = (const int8_t *)(a + 4);
        float dall = d6 * d8;
        int32_t sumi = 0;
        for (int half = 0; half < 2; half++) {
            int qlb = half * 64, qhb = half * 32, scb = half * 8, q8b = half * 128;
            for (int l = 0; l < 32; l++) {
                uint8_t lo = ql[qlb + l], hi = ql[qlb + 32 + l], h = qh[qhb + l];
                int is = l / 16;
                int32_t q1 = (int32_t)((lo & 0x0F) | ((h & 0x03) << 4)) - 32;
                int32_t q2 = (int32_t)((hi & 0x0F) | (((h >> 2) & 0x03) << 4)) - 32;
                int32_t q3 = (int32_t)((lo >> 4) | (((h >> 4) & 0x03) << 4)) - 32;
                int32_t q4 = (int32_t)((hi >> 4) | (((h >> 6) & 0x03) << 4)) - 32;
                sumi += (int32_t)sc[scb + is] * q1 * (int32_t)q8[q8b + l];
                sumi += (int32_t)sc[scb + is + 2] * q2 * (int32_t)q8[q8b + 32 + l];
                sumi += (int32_t)sc[scb + is + 4] * q3 * (int32_t)q8[q8b + 64 + l];
                sumi += (int32_t)sc[scb + is + 6] * q4 * (int32_t)q8[q8b + 96 + l];
            }
        }
        sumf += dall * (float)sumi;
    }
    return sumf;
}

#if defined(__AVX2__)
static inline int32_t hsum_epi32(__m256i v) {
    __m128i s = _mm_add_epi32(_mm256_castsi256_si128(v), _mm256_extracti128_si256(v, 1));
    s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0x4E));
    s = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0xB1));
    return _mm_cvtsi128_si32(s);
}

/* AVX2 maddubs form of the Q4_K x Q8_K dot (same SIMD class the reference times with,
 * fused_q4k_q8k_dot.rs:27-96).  Integer-exact, so bit-identical to the scalar form. */
static float dot_q4k_q8k_avx2(const uint8_t *act_q8k, const uint8_t *w, size_t k) {
    size_t nb = k / 256;
    float sumf = 0.0f;
    const __m256i m4 = _mm256_set1_epi8(0x0F);
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *q4 = w + b * 144;
        float d = f16_to_f32(rd16(q4));
        float dmin = f16_to_f32(rd16(q4 + 2));
        const uint8_t *qs = q4 + 16;
        uint8_t scales[8], mins[8];
        unpack_q4k_scales(q4 + 4, scales, mins);
        const uint8_t *a = act_q8k + b * Q8K_BLOCK_BYTES;
        float d8;
        memcpy(&d8, a, 4);
        const uint8_t *q8 = a + 4;
        const uint8_t *bs = a + 260;
        __m256i acc = _mm256_setzero_si256();
        int32_t sumi_mins = 0;
        for (int j = 0; j < 4; j++) {
            __m256i raw = _mm256_loadu_si256((const __m256i *)(qs + j * 32));
            __m256i lo = _mm256_and_si256(raw, m4);
            __m256i hi = _mm256_and_si256(_mm256_srli_epi16(raw, 4), m4);
            __m256i a_lo = _mm256_loadu_si256((const __m256i *)(q8 + j * 64));
            __m256i a_hi = _mm256_loadu_si256((const __m256i *)(q8 + j * 64 + 32));
            __m256i p_lo = _mm256_madd_epi16(_mm256_maddubs_epi16(lo, a_lo), _mm256_set1_epi16(scales[2 * j]));
            __m256i p_hi = _mm256_madd_epi16(_mm256_maddubs_epi16(hi, a_hi), _mm256_set1_epi16(scales[2 * j + 1]));
            acc = _mm256_add_epi32(acc, _mm256_add_epi32(p_lo, p_hi));
            int32_t b_lo = (int32_t)(int16_t)rd16(bs + j * 8) + (int32_t)(int16_t)rd16(bs + j * 8 + 2);
            int32_t b_hi = (int32_t)(int16_t)rd16(bs + j * 8 + 4) + (int32_t)(int16_t)rd16(bs + j * 8 + 6);
            sumi_mins += (int32_t)mins[2 * j] * b_lo + (int32_t)mins[2 * j + 1] * b_hi;
        }
        int32_t sumi = hsum_epi32(acc);
        float t = (d * d8) * (float)sumi - (dmin * d8) * (float)sumi_mins;
        sumf += t;
    }
    return sumf;
}

/* AVX2 form of the Q6_K x Q8_K dot (fused_q6k_q8k_dot.rs:27-154): unsigned 6-bit
 * values through maddubs, minus 32 * (sum of activations), per 16-element scale. */
static float dot_q6k_q8k_avx2(const uint8_t *act_q8k, const uint8_t *w, size_t k) {
    size_t nb = k / 256;
    float sumf = 0.0f;
    const __m256i m4 = _mm256_set1_epi8(0x0F), m2 = _mm256_set1_epi8(0x03), m30 = _mm256_set1_epi8(0x30);
    const __m256i ones = _mm256_set1_epi8(1);
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = w + b * 210;
        const int8_t *sc = (const int8_t *)(blk + 192);
        float d6 = f16_to_f32(rd16(blk + 208));
        const uint8_t *a = act_q8k + b * Q8K_BLOCK_BYTES;
        float d8;
        memcpy(&d8, a, 4);
        const uint8_t *q8 = a + 4;
        __m256i acc = _mm256_setzero_si256();
        for (int half = 0; half < 2; half++) {
            __m256i ql0 = _mm256_loadu_si256((const __m256i *)(blk + half * 64));
            __m256i ql1 = _mm256_loadu_si256((const __m256i *)(blk + half * 64 + 32));
            __m256i qh = _mm256_loadu_si256((const __m256i *)(blk + 128 + half * 32));
            for (int g = 0; g < 4; g++) {
                __m256i q6;
                switch (g) {
                case 0: q6 = _mm256_or_si256(_mm256_and_si256(ql0, m4), _mm256_slli_epi16(_mm256_and_si256(qh, m2), 4)); break;
                case 1: q6 = _mm256_or_si256(_mm256_and_si256(ql1, m4), _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(qh, 2), m2), 4)); break;
                case 2: q6 = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(ql0, 4), m4), _mm256_and_si256(qh, m30)); break;
                default: q6 = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(ql1, 4), m4), _mm256_and_si256(_mm256_srli_epi16(qh, 2), m30)); break;
                }
                __m256i a8 = _mm256_loadu_si256((const __m256i *)(q8 + half * 128 + g * 32));
                __m256i dot = _mm256_maddubs_epi16(q6, a8);
                __m256i asum = _mm256_maddubs_epi16(ones, a8);
                __m256i cor = _mm256_sub_epi16(dot, _mm256_slli_epi16(asum, 5));
                int so = half * 8 + g * 2;
                __m256i sv = _mm256_set_m128i(_mm_set1_epi16(sc[so + 1]), _mm_set1_epi16(sc[so]));
                acc = _mm256_add_epi32(acc, _mm256_madd_epi16(cor, sv));
            }
        }
        sumf += (d6 * d8) * (float)hsum_epi32(acc);
    }
    return sumf;
}
#endif

/* fused_dot_q5k_q8k.  The reference dispatches to its AVX2 form on x86-64 (src/quant/cpu/kernels/simd/fused_q5k_q8k_dot.rs:
 * 27-122, dispatch :139-148); that form is what the CPU matmul computes there and what this function restates
 * (`scalar_order` = 0).  Per chunk j of 64 elements it takes the LOW nibbles of qs[32 j .. 32 j + 32) as elements
 * 64 j .. 64 j + 32 and the HIGH nibbles as elements 64 j + 32 .. 64 j + 64 (the Q4_K order), with high bit
 * (qh[e / 8] >> (e % 8)) & 1 for element e, scales[2 j] / scales[2 j + 1], and the min term from the Q8_K block sums.
 * Its scalar fallback (:151-212, `scalar_order` = 1) uses the interleaved order of dequant_q5k instead, so the two
 * forms of the reference disagree with each other on the same bytes; integer arithmetic is exact in both. */
static float dot_q5k_q8k(const uint8_t *act_q8k, const uint8_t *w, size_t k, int scalar_order) {
    size_t nb = k / 256;
    float sumf = 0.0f;
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *q5 = w + b * 176;
        float d = f16_to_f32(rd16(q5));
        float dmin = f16_to_f32(rd16(q5 + 2));
        const uint8_t *qh = q5 + 16, *qs = q5 + 48;
        uint8_t scales[8], mins[8];
        unpack_q4k_scales(q5 + 4, scales, mins);
        const uint8_t *a = act_q8k + b * Q8K_BLOCK_BYTES;
        float d8;
        memcpy(&d8, a, 4);
        const int8_t *q8 = (const int8_t *)(a + 4);
        const uint8_t *bs = a + 260;
        float dall = d * d8;
        float dmin_all = dmin * d8;
        int32_t sumi = 0, sumi_mins = 0;
        for (int j = 0; j < 8; j++) {
            int32_t dot = 0;
            for (int l = 0; l < 32; l++) {
                int idx = j * 32 + l;
                int low4;
                if (scalar_order) {
                    int byte = qs[j * 16 + l / 2];
                    low4 = (l % 2 == 0) ? (byte & 0x0F) : ((byte >> 4) & 0x0F);
                } else {
                    int byte = qs[(j / 2) * 32 + l];
                    low4 = (j & 1) ? ((byte >> 4) & 0x0F) : (byte & 0x0F);
                }
                int high1 = (qh[idx / 8] >> (idx % 8)) & 1;
                dot += (low4 | (high1 << 4)) * (int32_t)q8[idx];
            }
            sumi += dot * (int32_t)scales[j];
            int32_t bsum = (int32_t)(int16_t)rd16(bs + j * 4) + (int32_t)(int16_t)rd16(bs + j * 4 + 2);
            sumi_mins += (int32_t)mins[j] * bsum;
        }
        float t = dall * (float)sumi - dmin_all * (float)sumi_mins;
        sumf += t;
    }
    return sumf;
}

/* fused_dot_q2k_q8k: src/quant/cpu/kernels/simd/fused_q2k_q8k_dot.rs:152-214 (scalar) and :28-137 (AVX2: the same
 * integers through maddubs / madd).  Per block: summs = sum_j bsums[j] * (sc[j] >> 4) over the sixteen 16-wide sums of
 * the activation block, isum = sum_j (sc[j] & 15) * sum_l q * a, sumf += (d * d8) * isum - (dmin * d8) * summs. */
static float dot_q2k_q8k(const uint8_t *act_q8k, const uint8_t *w, size_t k) {
    size_t nb = k / 256;
    float sumf = 0.0f;
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = w + b * 84;
        const uint8_t *sc = blk, *qs = blk + 16;
        float d = f16_to_f32(rd16(blk + 80)), dmin = f16_to_f32(rd16(blk + 82));
        const uint8_t *a = act_q8k + b * Q8K_BLOCK_BYTES;
        float d8;
        memcpy(&d8, a, 4);
        const int8_t *q8 = (const int8_t *)(a + 4);
        const uint8_t *bs = a + 260;
        float dall = d * d8, dmin_all = dmin * d8;
        int32_t summs = 0;
        for (int j = 0; j < 16; j++) {
            int16_t v;
            memcpy(&v, bs + 2 * j, 2);
            summs += (int32_t)v * (int32_t)(sc[j] >> 4);
        }
        int32_t isum = 0;
        int is = 0, off = 0;
        for (int n = 0; n < 2; n++) {
            const uint8_t *q = qs + 32 * n;
            for (int shift = 0; shift < 8; shift += 2) {
                for (int h = 0; h < 2; h++) {
                    int32_t isuml = 0;
                    for (int l = 0; l < 16; l++) isuml += (int32_t)q8[off + 16 * h + l] * (int32_t)((q[16 * h + l] >> shift) & 3);
                    isum += (int32_t)(sc[is++] & 0x0F) * isuml;
                }
                off += 32;
            }
        }
        volatile float t1 = dall * (float)isum, t2 = dmin_all * (float)summs;  /* no contraction */
        sumf += t1 - t2;
    }
    return sumf;
}

/* fused_dot_q3k_q8k.  scalar_form = 0: the AVX2 form x86-64 runs (src/quant/cpu/kernels/simd/fused_q3k_q8k_dot.rs:33-205):
 * one integer sum per block, sumf += (d * d8) * isum.  scalar_form = 1: the scalar fallback (:225-292), which keeps eight
 * float accumulators (element index mod 8) across blocks and adds them at the end.  Same integers, different f32 sums. */
static float dot_q3k_q8k(const uint8_t *act_q8k, const uint8_t *w, size_t k, int scalar_form) {
    size_t nb = k / 256;
    float sumf = 0.0f, sums[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (size_t b = 0; b < nb; b++) {
        const uint8_t *blk = w + b * 110;
        int8_t scales[16];
        unpack_q3k_scales(blk + 96, scales);
        float d_all = f16_to_f32(rd16(blk + 108));
        const uint8_t *a = act_q8k + b * Q8K_BLOCK_BYTES;
        float d8;
        memcpy(&d8, a, 4);
        const int8_t *q8 = (const int8_t *)(a + 4);
        float d = d_all * d8;
        int32_t aux32[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int e = 0; e < 256; e++) aux32[e & 7] += (int32_t)scales[e >> 4] * ((int32_t)q8[e] * q3k_code(blk, e));
        if (scalar_form) {
            for (int l = 0; l < 8; l++) sums[l] += d * (float)aux32[l];
        } else {
            int32_t isum = 0;
            for (int l = 0; l < 8; l++) isum += aux32[l];
            sumf += d * (float)isum;
        }
    }
    if (scalar_form)
        for (int l = 0; l < 8; l++) sumf += sums[l];
    return sumf;
}

/* simd: 1 = the forms the reference runs on x86-64 (AVX2), 0 = its scalar fallbacks.  For Q4_K and Q6_K the two give
 * identical bits; for Q5_K they are different functions of the weight bytes (see dot_q5k_q8k). */
ORACLE_API float oracle_dot_q8k(int fmt, const uint8_t *act_q8k, const uint8_t *w, size_t k, int simd) {
    if (fmt == FMT_Q5_K) return dot_q5k_q8k(act_q8k, w, k, simd ? 0 : 1);
    if (fmt == FMT_Q3_K) return dot_q3k_q8k(act_q8k, w, k, simd ? 0 : 1);
    if (fmt == FMT_Q2_K) return dot_q2k_q8k(act_q8k, w, k);  /* the AVX2 form computes the same integers */
#if defined(__AVX2__)
    if (simd) return fmt == FMT_Q4_K ? dot_q4k_q8k_avx2(act_q8k, w, k) : dot_q6k_q8k_avx2(act_q8k, w, k);
#endif
    (void)simd;
    return fmt == FMT_Q4_K ? dot_q4k_q8k_scalar(act_q8k, w, k) : dot_q6k_q8k_scalar(act_q8k, w, k);
}

/* dot_f32_avx2_fma + hsum_f32_avx2: src/quant/cpu/kernels/simd/dot_f32.rs:13-61.
 * Eight independent FMA lanes, then (lo+hi), (+movehl), (+lane 1), then a scalar tail
 * of separately rounded multiply and add.  The fmaf form is bit-identical to the
 * intrinsic form; the intrinsic form is used when available (it is what gets timed). */
ORACLE_API float oracle_dot_f32(const float *a, const float *b, size_t len) {
    size_t chunks = len / 8;
    float result;
#if defined(__AVX2__) && defined(__FMA__)
    __m256 acc = _mm256_setzero_ps();
    for (size_t i = 0; i < chunks; i++)
        acc = _mm256_fmadd_ps(_mm256_loadu_ps(a + 8 * i), _mm256_loadu_ps(b + 8 * i), acc);
    __m128 s = _mm_add_ps(_mm256_castps256_ps128(acc), _mm256_extractf128_ps(acc, 1));
    s = _mm_add_ps(s, _mm_movehl_ps(s, s));
    s = _mm_add_ss(s, _mm_shuffle_ps(s, s, 1));
    result = _mm_cvtss_f32(s);
#else
    float lane[8] = {0};
    for (size_t i = 0; i < chunks; i++)
        for (int l = 0; l < 8; l++) lane[l] = fmaf(a[8 * i + l], b[8 * i + l], lane[l]);
    float s0 = lane[0] + lane[4], s1 = lane[1] + lane[5], s2 = lane[2] + lane[6], s3 = lane[3] + lane[7];
    s0 = s0 + s2;
    s1 = s1 + s3;
    result = s0 + s1;
#endif
    for (size_t i = chunks * 8; i < len; i++) {
        float p = a[i] * b[i];
        result = result + p;
    }
    return result;
}

/* ------------------------------------------------------------ quant_matmul */

typedef struct {
    const float *act;
    const uint8_t *act_q8k;
    const uint8_t *w;
    float *out;
    size_t m, k, n, row_bytes, q8k_row;
    int fmt, simd;
    size_t j0, j1;
} mm_job;

/* Body of the per-chunk closure of quant_matmul_f32
 * (src/quant/cpu/kernels/quant_matmul.rs:138-211). */
static void mm_chunk(const mm_job *J) {
    if (J->act_q8k) {
        for (size_t i = 0; i < J->m; i++) {
            const uint8_t *arow = J->act_q8k + i * J->q8k_row;
            for (size_t j = J->j0; j < J->j1; j++)
                J->out[i * J->n + j] = oracle_dot_q8k(J->fmt, arow, J->w + j * J->row_bytes, J->k, J->simd);
        }
    } else {
        float *row = (float *)malloc(J->k * sizeof(float));
        size_t nblk = J->k / (size_t)oracle_block_size(J->fmt);
        for (size_t j = J->j0; j < J->j1; j++) {
            oracle_dequant_f32(J->fmt, J->w + j * J->row_bytes, nblk, row);
            for (size_t i = 0; i < J->m; i++) J->out[i * J->n + j] = oracle_dot_f32(J->act + i * J->k, row, J->k);
        }
        free(row);
    }
}

/* Persistent worker pool (rayon keeps one too: src/quant/cpu/kernels/quant_matmul.rs:138 runs on the
 * global rayon pool).  Workers sleep on a condition variable between calls; a call publishes its job
 * array under a new generation number, workers and the caller claim chunks with an atomic counter, and
 * the caller waits until every claimed chunk has finished.  One call at a time (calls serialise on
 * run_mu); the pool only grows. */
#define MM_MAX_WORKERS 256
typedef struct {
    pthread_mutex_t mu, run_mu;
    pthread_cond_t wake, done;
    pthread_t th[MM_MAX_WORKERS];
    size_t nworkers;
    unsigned long generation;
    mm_job *jobs;
    size_t njobs, active_limit; /* workers with index >= active_limit sit a call out */
    size_t next;                /* atomic: next chunk to claim */
    size_t finished;            /* guarded by mu: workers that have drained the queue of this generation */
    size_t participants;
} mm_pool;
static mm_pool g_pool = {PTHREAD_MUTEX_INITIALIZER, PTHREAD_MUTEX_INITIALIZER, PTHREAD_COND_INITIALIZER,
                         PTHREAD_COND_INITIALIZER, {0}, 0, 0, NULL, 0, 0, 0, 0, 0};

static void mm_drain(mm_pool *P) {
    for (;;) {
        size_t i = __atomic_fetch_add(&P->next, 1, __ATOMIC_RELAXED);
        if (i >= P->njobs) break;
        mm_chunk(&P->jobs[i]);
    }
}

static void *mm_worker(void *arg) {
    mm_pool *P = &g_pool;
    size_t me = (size_t)(uintptr_t)arg;
    unsigned long seen = 0;
    pthread_mutex_lock(&P->mu);
    for (;;) {
        while (P->generation == seen) pthread_cond_wait(&P->wake, &P->mu);
        seen = P->generation;
        if (me >= P->active_limit) continue;
        pthread_mutex_unlock(&P->mu);
        mm_drain(P);
        pthread_mutex_lock(&P->mu);
        if (++P->finished == P->participants) pthread_cond_signal(&P->done);
    }
    return NULL;
}

/* Runs jobs[0..njobs) on `threads` threads (the caller is one of them). */
static void mm_run(mm_job *jobs, size_t njobs, size_t threads) {
    mm_pool *P = &g_pool;
    if (threads > MM_MAX_WORKERS + 1) threads = MM_MAX_WORKERS + 1;
    pthread_mutex_lock(&P->run_mu);
    pthread_mutex_lock(&P->mu);
    while (P->nworkers + 1 < threads) {
        if (pthread_create(&P->th[P->nworkers], NULL, mm_worker, (void *)(uintptr_t)P->nworkers) != 0) break;
        pthread_detach(P->th[P->nworkers]);
        P->nworkers++;
    }
    size_t helpers = threads - 1 < P->nworkers ? threads - 1 : P->nworkers;
    P->jobs = jobs;
    P->njobs = njobs;
    P->active_limit = helpers;
    P->participants = helpers;
    P->finished = 0;
    __atomic_store_n(&P->next, 0, __ATOMIC_RELAXED);
    P->generation++;
    pthread_cond_broadcast(&P->wake);
    pthread_mutex_unlock(&P->mu);
    mm_drain(P);
    pthread_mutex_lock(&P->mu);
    while (P->finished < P->participants) pthread_cond_wait(&P->done, &P->mu);
    pthread_mutex_unlock(&P->mu);
    pthread_mutex_unlock(&P->run_mu);
}

/* quant_matmul_f32: src/quant/cpu/kernels/quant_matmul.rs:55-212.
 *   act [M,K] f32 row-major, w packed [N,K] (blocks along K), out [M,N] f32.
 *   K-quants with K % 256 == 0 quantise each activation row to Q8_K first (:119-135)
 *   and use integer dots; Q4_0/Q8_0 dequantise a weight row and use dot_f32 (:193-209).
 *   Columns are split into chunks of max(16, ceil(N / (T or 4T))) (:84-87).
 * K-quants with K % 256 != 0 cannot occur (block size is 256), so the f32 fused-dot
 * branch (:159-192) is not restated.
 * threads <= 0 means 1.  simd != 0 selects the AVX2 integer dots (same results).
 * Returns 0, -1 unknown format, -2 K not a multiple of the block size. */
ORACLE_API int oracle_quant_matmul(int fmt, const float *act, const uint8_t *w, float *out, size_t m, size_t k,
                                   size_t n, int threads, int simd) {
    int bs = oracle_block_size(fmt);
    if (!bs) return -1;
    if (k % (size_t)bs) return -2;
    if (threads <= 0) threads = 1;
    size_t row_bytes = (k / (size_t)bs) * (size_t)oracle_block_bytes(fmt);
    int kq = (fmt == FMT_Q2_K || fmt == FMT_Q3_K || fmt == FMT_Q4_K || fmt == FMT_Q5_K || fmt == FMT_Q6_K);
    size_t q8k_row = (k / 256) * Q8K_BLOCK_BYTES;
    uint8_t *aq = NULL;
    if (kq) {
        aq = (uint8_t *)malloc(m * q8k_row + 1);
        for (size_t i = 0; i < m; i++) oracle_quantize_q8k(act + i * k, k, aq + i * q8k_row);
    }
    size_t target = (m == 1) ? (size_t)threads : (size_t)threads * 4;
    size_t chunk = (n + target - 1) / target;
    if (chunk < 16) chunk = 16;
    size_t njobs = (n + chunk - 1) / chunk;
    mm_job *jobs = (mm_job *)malloc(sizeof(mm_job) * (njobs ? njobs : 1));
    for (size_t c = 0; c < njobs; c++) {
        mm_job J = {act, aq, w, out, m, k, n, row_bytes, q8k_row, fmt, simd, c * chunk, 0};
        J.j1 = J.j0 + chunk < n ? J.j0 + chunk : n;
        jobs[c] = J;
    }
    if (threads == 1 || njobs <= 1) {
        for (size_t c = 0; c < njobs; c++) mm_chunk(&jobs[c]);
    } else {
        mm_run(jobs, njobs, (size_t)threads < njobs ? (size_t)threads : njobs);
    }
    free(jobs);
    free(aq);
    return 0;
}

/* quant_swiglu on CPU: two quant_matmuls then silu(gate) * up
 * (src/quant/cpu/quant_matmul/impl_ops.rs:347-358).  silu_mul itself is numr's
 * (parity unpinned); x / (1 + exp(-x)) in f32 is what boostr's own CUDA kernel
 * uses (src/quant/cuda/kernels/quant_gemv.cu:791-793). */
ORACLE_API int oracle_quant_swiglu(int fmt, const float *act, const uint8_t *wg, const uint8_t *wu, float *out,
                                   size_t m, size_t k, size_t n, int threads, int simd) {
    float *g = (float *)malloc(sizeof(float) * m * n + 4);
    int rc = oracle_quant_matmul(fmt, act, wg, g, m, k, n, threads, simd);
    if (rc == 0) rc = oracle_quant_matmul(fmt, act, wu, out, m, k, n, threads, simd);
    if (rc == 0)
        for (size_t i = 0; i < m * n; i++) {
            float x = g[i];
            float s = x / (1.0f + expf(-x));
            out[i] = s * out[i];
        }
    free(g);
    return rc;
}

/* Diagnostic only (not the parity reference): exact-weight x f32-activation dot in f64. */
ORACLE_API int oracle_matmul_exact_f64(int fmt, const float *act, const uint8_t *w, double *out, size_t m, size_t k,
                                       size_t n) {
    int bs = oracle_block_size(fmt);
    if (!bs || k % (size_t)bs) return -1;
    size_t row_bytes = (k / (size_t)bs) * (size_t)oracle_block_bytes(fmt);
    float *row = (float *)malloc(k * sizeof(float));
    for (size_t j = 0; j < n; j++) {
        oracle_dequant_f32(fmt, w + j * row_bytes, k / (size_t)bs, row);
        for (size_t i = 0; i < m; i++) {
            double s = 0.0;
            for (size_t t = 0; t < k; t++) s += (double)act[i * k + t] * (double)row[t];
            out[i * n + j] = s;
        }
    }
    free(row);
    return 0;
}
