// Small-M quantized matmul (2 <= M <= 32) for Q4_K on the 5th-generation tensor cores' INTEGER path:
//   out[M,N] = act[M,K] x W[N,K]^T  with boostr's CPU arithmetic (activations quantised to Q8_K,
//   src/quant/cpu/kernels/simd/quantize_act_q8k.rs:26-98; per 256-block (d*d8)*sumi - (dmin*d8)*sumi_mins with exact
//   integer sums, src/quant/cpu/kernels/simd/fused_q4k_q8k_dot.rs:111-172).
//
// The mma.sync kernel (gemv.cu) spends ~540 warp instructions per (16 weight rows x 256 K x 16 activation rows), is bound
// by instruction issue, and takes more than 16 activation rows in several passes over the weights.  Here ONE
// tcgen05.mma.kind::i8 (128 weight rows x MP activation rows x 32 K) computes the integer dot products of a whole
// 32-wide sub-block for 128 rows, and the per-sub-block scales are applied by the warps that drain the accumulator:
//   * tile = 128 weight rows (the MMA's M = the 128 lanes of tensor memory); the activations are the B operand,
//     MP = 16 or 32 rows (MMA N); every 32-wide sub-block j of a 256-block gets its OWN accumulator columns
//     [MP j, MP j + MP), so no scale has to enter the tensor core; tensor memory holds two such accumulators;
//   * packed weight blocks arrive by TMA as tiles of 128 rows x 144 bytes (conflict-free 16-byte reads, one thread
//     per row); two sets of four decode warps, taking the blocks in turn, split the nibbles into bytes and write them
//     as the K-major, 128-byte-swizzled A operand in shared memory (two tiles of 128 rows x 128 codes per block), and
//     leave the row's 6-bit scales, mins, d and dmin in a small ring of records for the drain;
//   * the activations are quantised once per call (i8_act_prep_kernel) into an int8 image [M][K] that TMA brings in
//     as the B operand; the Q8_K scales and the 32-wide block sums the min term needs travel beside the records;
//   * one thread issues the 8 MMAs of a block; two teams of eight drain warps, one per accumulator (a thread owns a
//     weight row and half of the activation rows), read the 8 x MP integer sums from tensor memory, form
//     sumi = sum_j sc_j dot_j and sumi_mins = sum_j m_j bsum_j in integers and the block's f32 term; the running f32
//     sums pass from team to team through shared memory, so the blocks are still added in K order;
//   * work = (tile, block) pairs dealt to the CTAs as equal contiguous ranges.  Where the matrix has enough tiles the
//     ranges are whole tiles and the result has the CPU's bits.  Otherwise a range may cut a tile along K: such pieces
//     go to scratch as f32 partial tiles and the CTA that writes a tile's last piece (a counter per tile) adds them in
//     K order; a cut tile differs from the CPU's bits by f32 rounding only (the grouping of the sum).
// What bounds it: the drain is ~200 instructions per (weight row, 8 activation rows, block), about 2600 warp
// instructions per (128 rows x 256 K x 16 activation rows) for the whole CTA against ~4300 in the mma.sync kernel.
// Every mbarrier wait is bounded; on a timeout the CTA records a status code and still frees its tensor memory.
#include <cuda.h>

#include <cstdio>

#include "common.cuh"
#include "tmap.cuh"

namespace b200q {

struct I8Params {
    const uint8_t* w;
    void* out;
    float* part;          // [slot][MP][128] f32 pieces of cut tiles
    unsigned int* cnt;    // [ntiles] pieces of a cut tile that have been written; 0 between calls
    const uint8_t* aux;   // [nblk][aux_bytes(MP)]: per block the eight int16 sums of 32 codes of every activation row, then the rows' Q8_K scales
    uint32_t M, N, K;
    uint32_t MP;          // activation rows of the MMA (16 or 32)
    uint32_t nblk;        // K / 256
    uint32_t ntiles;      // ceil(N / 128)
    uint32_t Q;           // ntiles * nblk (tile, block) pairs
    uint32_t unit;        // pairs are dealt in items of `unit` pairs: 1, or nblk (whole tiles: nothing is cut)
    uint32_t qbase, qrem; // items / grid and items % grid: CTA c takes items [c qbase + min(c, qrem), ...)
    uint32_t ns;          // ring depth of operand stages (one 256-block each)
    uint32_t nr;          // ring depth of packed-weight tiles
    uint32_t nsc;         // ring depth of the scale records
    uint32_t idesc;
    int out_dtype;
    unsigned int* status;
};

namespace {


constexpr int DEC_WARPS = 8, DRAIN_WARPS = 16;  // decode: two sets of four warps; drain: two teams of eight warps
constexpr int I8_THREADS = (DEC_WARPS + DRAIN_WARPS + 3) * 32;  // decode | drain | packed-weight TMA | activation TMA | MMA issue, TMEM
constexpr int W_RAW = DEC_WARPS + DRAIN_WARPS, W_ACT = W_RAW + 1, W_MMA = W_RAW + 2;
constexpr uint32_t RAW_PITCH = 144, RAW_TILE = 128 * RAW_PITCH;  // 18432 = 18 x 1024
constexpr uint32_t A_ATOM = 128 * 128;                            // 128 rows x 128 codes
constexpr uint32_t SC_WORDS = 5;                                  // d|dmin, 8 scales, 8 mins
constexpr uint32_t SC_REC = 128 * SC_WORDS * 4;                  // the 128 row records of a block
constexpr uint32_t SC_SLOT = SC_REC + 32 * 20;                    // + the activation side of the block (aux_bytes(32))
__host__ __device__ constexpr uint32_t aux_bytes(uint32_t MP) { return MP * 20; }  // per block: MP x 8 int16 block sums | MP x f32 d8
// barriers (8 bytes each) at the start of dynamic shared memory
constexpr int OFF_FULL = 0, OFF_EMPTY = 64, OFF_RAW_FULL = 128, OFF_RAW_EMPTY = 192, OFF_ACC_FULL = 256, OFF_ACC_EMPTY = 272,
              OFF_SC_FULL = 320, OFF_TMEM = 448, OFF_DEAD = 452, OFF_RED = 456, OFF_LAST = 464, OFF_NSLOT = 472, OFF_XFER = 480, OFF_SLOTS = 512,
              OFF_SC = 1024;  // OFF_SLOTS: two lists of 64 slots

__device__ __noinline__ bool i8_wait_slow(uint32_t bar, uint32_t parity, volatile uint32_t* dead) {
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
__device__ __forceinline__ bool i8_wait(uint32_t bar, uint32_t parity, volatile uint32_t* dead) {
    if (mbar_try_wait(bar, parity)) return true;
    return i8_wait_slow(bar, parity, dead);
}
__device__ __noinline__ void i8_fail(volatile uint32_t* dead, unsigned int* status, unsigned int code) {
    if (!*dead) atomicOr(status, code);
    *dead = 1;
}
__device__ __forceinline__ void tma2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ bool elect_one_lane() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xFFFFFFFF;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit_to(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[128 x N] (int32, tensor memory) = A[128 x 32] (int8, shared) x B[N x 32]^T (int8, shared); never accumulates:
// every sub-block has its own columns
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc)
        : "memory");
}
// K-major operand tile with 128-byte swizzle (rows of 128 bytes, 8-row groups 1024 bytes apart), from the low word
// ((addr >> 4) | 1 << 16; 32 bytes further along K adds 2)
__device__ __forceinline__ uint64_t desc_sw128(uint32_t lo) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"((1024u >> 4) | (1u << 14) | (2u << 29)));
    return d;
}
__device__ __forceinline__ uint32_t desc_lo(uint32_t addr) { return ((addr >> 4) & 0x3FFFu) | (1u << 16); }
// 16 consecutive 32-bit columns of this thread's lane; the caller waits (tmem_ld_wait) before using them
__device__ __forceinline__ void tmem_ld16_async(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld8_async(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// One piece of work of a CTA: blocks [b0, b0 + nb) of tile `tile`; slot < 0: the whole tile, written to the output.
struct I8Unit {
    uint32_t tile, b0, nb;
    int slot;
};
// First (tile, block) pair of CTA c: the first qrem CTAs take one item more than the others
__device__ __forceinline__ uint32_t i8_range_begin(const I8Params& p, uint32_t c) { return (c * p.qbase + min(c, p.qrem)) * p.unit; }
// The CTA whose range holds pair x
__device__ __forceinline__ uint32_t i8_cta_of(const I8Params& p, uint32_t x) {
    const uint32_t y = x / p.unit, big = p.qrem * (p.qbase + 1);
    return y < big ? y / (p.qbase + 1) : p.qrem + (y - big) / p.qbase;
}
// The it-th unit of this CTA (every role walks the same list): the CTA's range cut at the tile boundaries
__device__ __forceinline__ bool i8_unit(const I8Params& p, uint32_t it, I8Unit& u) {
    const uint32_t a = i8_range_begin(p, blockIdx.x), b = i8_range_begin(p, blockIdx.x + 1);
    const uint32_t t = a / p.nblk + it;
    const uint32_t lo = max(a, t * p.nblk), hi = min(b, (t + 1) * p.nblk);
    if (t >= p.ntiles || lo >= hi) return false;
    u.tile = t;
    u.b0 = lo - t * p.nblk;
    u.nb = hi - lo;
    u.slot = u.nb == p.nblk ? -1 : (int)(2 * blockIdx.x + (it == 0 ? 0u : 1u));
    return true;
}

template <int I>
__device__ __forceinline__ int ubyte(uint32_t x) { return (int)__byte_perm(x, 0u, 0x4440 | I); }

template <int MP>
__global__ void __launch_bounds__(I8_THREADS, 1) smallm_i8_q4k_kernel(const __grid_constant__ CUtensorMap tmap_act,
                                                                      const __grid_constant__ CUtensorMap tmap_w, const I8Params p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);  // the launch reserves 1 KB of slack
    const int warp = __shfl_sync(0xFFFFFFFFu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar_full = sbase + OFF_FULL, bar_empty = sbase + OFF_EMPTY, bar_raw_full = sbase + OFF_RAW_FULL,
                   bar_raw_empty = sbase + OFF_RAW_EMPTY, bar_acc_full = sbase + OFF_ACC_FULL, bar_acc_empty = sbase + OFF_ACC_EMPTY,
                   bar_sc_full = sbase + OFF_SC_FULL;
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + OFF_TMEM);
    volatile uint32_t* dead = reinterpret_cast<volatile uint32_t*>(smem + OFF_DEAD);
    constexpr uint32_t NACC = 2, ACC_COLS = 8 * MP, TMEM_COLS = NACC * ACC_COLS < 32 ? 32 : NACC * ACC_COLS;  // 256 or 512
    constexpr uint32_t B_ATOM = MP * 128, STAGE = 2 * A_ATOM + 2 * B_ATOM;
    // shared memory: barriers | scale records | exchange buffer of the drain teams | packed tiles | operand stages (A atom
    // 0, A atom 1, B atom 0, B atom 1)
    const uint32_t sc_off = OFF_SC, x_off = sc_off + p.nsc * SC_SLOT, raw_off = (x_off + 128 * MP * 4 + 1023u) & ~1023u,
                   st_off = raw_off + p.nr * RAW_TILE;

    constexpr int MH = MP / 2;  // activation rows of a drain warp: a team is 2 groups of 4 warps
    const uint32_t team_warps = 4 * min(2u, (p.M + MH - 1) / MH);  // warps of a team whose activation rows exist
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.ns; ++s) {
            mbar_init(bar_full + 8 * s, 5);   // the four decode warps of a set + the activation copy (with its byte count)
            mbar_init(bar_empty + 8 * s, 1);  // the commit behind the block's MMAs
        }
        for (uint32_t s = 0; s < p.nr; ++s) {
            mbar_init(bar_raw_full + 8 * s, 1);
            mbar_init(bar_raw_empty + 8 * s, 4);
        }
        for (uint32_t s = 0; s < NACC; ++s) {
            mbar_init(bar_acc_full + 8 * s, 1);
            mbar_init(bar_acc_empty + 8 * s, team_warps);  // the team that drains this accumulator
            mbar_init(sbase + OFF_XFER + 8 * s, team_warps);  // the team's running sums are in the exchange buffer
        }
        for (uint32_t s = 0; s < p.nsc; ++s) mbar_init(bar_sc_full + 8 * s, 5);  // four decode warps write the records, one copy brings the activation side
        mbar_init(sbase + OFF_RED, 2 * team_warps);  // both teams meet here around the hand-over of a cut tile
        *dead = 0;
        mbar_fence_init();
    }
    if (warp == W_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sbase + OFF_TMEM), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_before();
    __syncthreads();
    tc_after();
    const uint32_t tmem = *tmem_holder;
    grid_dep_launch();

    if (warp == W_RAW) {
        // ------------------------------------------------------------ packed weight tiles (do not depend on the previous kernel)
        if (lane == 0) {
            uint32_t s = 0, par = 0;
            I8Unit u;
            for (uint32_t it = 0; i8_unit(p, it, u) && !*dead; ++it) {
                for (uint32_t j = 0; j < u.nb; ++j) {
                    if (!i8_wait(bar_raw_empty + 8 * s, par ^ 1, dead)) {
                        i8_fail(dead, p.status, STATUS_TIMEOUT_EMPTY);
                        break;
                    }
                    mbar_expect_tx(bar_raw_full + 8 * s, RAW_TILE);
                    tma2d(sbase + raw_off + s * RAW_TILE, &tmap_w, (int)((u.b0 + j) * RAW_PITCH), (int)(u.tile * 128), bar_raw_full + 8 * s);
                    if (++s == p.nr) { s = 0; par ^= 1; }
                }
            }
        }
    } else if (warp == W_ACT) {
        // ------------------------------------------------------------ activation codes (written by the previous kernel)
        if (lane == 0) {
            grid_dep_wait();
            uint32_t s = 0, par = 0, i = 0;
            I8Unit u;
            for (uint32_t it = 0; i8_unit(p, it, u) && !*dead; ++it) {
                for (uint32_t j = 0; j < u.nb; ++j, ++i) {
                    if (!i8_wait(bar_empty + 8 * s, par ^ 1, dead)) {
                        i8_fail(dead, p.status, STATUS_TIMEOUT_EMPTY);
                        break;
                    }
                    const uint32_t b0 = sbase + st_off + s * STAGE + 2 * A_ATOM;
                    mbar_expect_tx(bar_full + 8 * s, 2 * B_ATOM);
                    tma2d(b0, &tmap_act, (int)((u.b0 + j) * 256), 0, bar_full + 8 * s);
                    tma2d(b0 + B_ATOM, &tmap_act, (int)((u.b0 + j) * 256 + 128), 0, bar_full + 8 * s);
                    // block sums and scales of the activation rows, next to the row records (same life time)
                    const uint32_t q = i % p.nsc;
                    mbar_expect_tx(bar_sc_full + 8 * q, aux_bytes(MP));
                    bulk_g2s(sbase + sc_off + q * SC_SLOT + SC_REC, p.aux + (size_t)(u.b0 + j) * aux_bytes(MP), aux_bytes(MP), bar_sc_full + 8 * q);
                    if (++s == p.ns) { s = 0; par ^= 1; }
                }
            }
        }
    } else if (warp == W_MMA) {
        // ------------------------------------------------------------ MMA issue: 8 sub-blocks, 8 column groups
        uint32_t s = 0, par = 0, i = 0;
        bool ok = true;
        I8Unit u;
        for (uint32_t it = 0; ok && i8_unit(p, it, u); ++it) {
            for (uint32_t j = 0; j < u.nb; ++j, ++i) {
                const uint32_t buf = i % NACC, use = i / NACC;
                if (!i8_wait(bar_full + 8 * s, par, dead)) {
                    if (lane == 0) i8_fail(dead, p.status, STATUS_TIMEOUT_FULL);
                    ok = false;
                    break;
                }
                if (use > 0 && !i8_wait(bar_acc_empty + 8 * buf, (use - 1) & 1, dead)) {
                    if (lane == 0) i8_fail(dead, p.status, STATUS_TIMEOUT_EMPTY);
                    ok = false;
                    break;
                }
                tc_after();
                if (elect_one_lane()) {
                    const uint32_t a_lo = desc_lo(sbase + st_off + s * STAGE), b_lo = desc_lo(sbase + st_off + s * STAGE + 2 * A_ATOM);
                    const uint32_t d0 = tmem + buf * ACC_COLS;
#pragma unroll
                    for (uint32_t sb = 0; sb < 8; ++sb)
                        tc_mma_i8(d0 + MP * sb, desc_sw128(a_lo + (sb >> 2) * (A_ATOM >> 4) + 2 * (sb & 3)),
                                  desc_sw128(b_lo + (sb >> 2) * (B_ATOM >> 4) + 2 * (sb & 3)), p.idesc);
                    tc_commit_to(bar_empty + 8 * s);         // the stage may be overwritten once these MMAs have read it
                    tc_commit_to(bar_acc_full + 8 * buf);    // and the sums are complete
                }
                __syncwarp();
                if (++s == p.ns) { s = 0; par ^= 1; }
            }
        }
    } else if (warp < DEC_WARPS) {
        // ------------------------------------------------------------ decode: nibbles -> int8 A operand, one thread per row
        // the sets of four warps take the CTA's blocks in turn, so DEC_WARPS / 4 blocks are in work at a time
        const uint32_t r = threadIdx.x & 127, set = threadIdx.x >> 7;
        const uint32_t row_sw = (r >> 3) * 1024 + (r & 7) * 128, x7 = r & 7;
        bool ok = true;
        I8Unit u;
        uint32_t i = 0;
        for (uint32_t it = 0; i8_unit(p, it, u); ++it) {
            const bool row_ok = u.tile * 128 + r < p.N;
            for (uint32_t j = 0; j < u.nb; ++j, ++i) {
                if (i % (DEC_WARPS / 4) != set) continue;
                const uint32_t rs = i % p.nr, rpar = (i / p.nr) & 1, s = i % p.ns, par = (i / p.ns) & 1;
                if (ok && !i8_wait(bar_raw_full + 8 * rs, rpar, dead)) {
                    i8_fail(dead, p.status, STATUS_TIMEOUT_FULL);
                    ok = false;
                }
                const uint4* src = reinterpret_cast<const uint4*>(smem + raw_off + rs * RAW_TILE + r * RAW_PITCH);
                uint4 h = make_uint4(0, 0, 0, 0), q[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) q[k] = make_uint4(0, 0, 0, 0);
                if (ok && row_ok) {
                    h = src[0];
#pragma unroll
                    for (int k = 0; k < 8; ++k) q[k] = src[1 + k];
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_raw_empty + 8 * rs);
                if (ok && !i8_wait(bar_empty + 8 * s, par ^ 1, dead)) {
                    i8_fail(dead, p.status, STATUS_TIMEOUT_EMPTY);
                    ok = false;
                }
                // 16 nibble bytes q[k] = bytes 16k .. 16k+15 of qs: low nibbles -> sub-block 2 (k / 2), codes 16 (k & 1) ..;
                // high nibbles -> sub-block 2 (k / 2) + 1.  Sub-block sb sits at bytes 32 sb .. of the 256-byte operand
                // row: 16-byte chunk c = 2 sb + (k & 1) -> tile (c / 8), chunk (c % 8) ^ (row % 8) of the swizzled row.
                uint8_t* a0 = smem + st_off + s * STAGE + row_sw;
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint32_t c_lo = 4 * (k >> 1) + (k & 1), c_hi = c_lo + 2;
                    const uint4 lo = make_uint4(q[k].x & 0x0F0F0F0Fu, q[k].y & 0x0F0F0F0Fu, q[k].z & 0x0F0F0F0Fu, q[k].w & 0x0F0F0F0Fu);
                    const uint4 hi = make_uint4((q[k].x >> 4) & 0x0F0F0F0Fu, (q[k].y >> 4) & 0x0F0F0F0Fu, (q[k].z >> 4) & 0x0F0F0F0Fu,
                                                (q[k].w >> 4) & 0x0F0F0F0Fu);
                    *reinterpret_cast<uint4*>(a0 + (c_lo >> 3) * A_ATOM + (((c_lo & 7) ^ x7) << 4)) = lo;
                    *reinterpret_cast<uint4*>(a0 + (c_hi >> 3) * A_ATOM + (((c_hi & 7) ^ x7) << 4)) = hi;
                }
                // the row's record for the drain: d | dmin, the 6-bit scales and mins as bytes (unpack_q4k_q5k_scales,
                // src/quant/cpu/kernels/dequant_k_quants/q4k_q5k.rs:108-122)
                uint32_t* rec = reinterpret_cast<uint32_t*>(smem + sc_off + (i % p.nsc) * SC_SLOT) + r * SC_WORDS;
                rec[0] = h.x;
                rec[1] = h.y & 0x3F3F3F3Fu;
                rec[2] = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u);
                rec[3] = h.z & 0x3F3F3F3Fu;
                rec[4] = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
                proxy_fence();  // the operand bytes are read by the tensor core (async proxy)
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(bar_full + 8 * s);
                    mbar_arrive(bar_sc_full + 8 * (i % p.nsc));
                }
            }
        }
    } else {
        // ------------------------------------------------------------ drain: integer sums -> scaled f32 terms
        // Two teams of eight warps take the CTA's blocks in turn (team = block index & 1 = accumulator), so the latencies
        // of two blocks overlap.  In a team, a thread owns one weight row (two warps per quarter of the rows) and MH of
        // the activation rows; warps whose rows do not exist have nothing to do.  The f32 sums still grow block by block,
        // in K order: the running sums of a tile pass from team to team through a buffer in shared memory.
        // The CTA's pairs are the contiguous range [xa, xb): pair x = block x % nblk of tile x / nblk.
        const uint32_t dw = (uint32_t)warp - DEC_WARPS, team = dw >> 3, quarter = dw & 3, r = quarter * 32 + lane, m_lo = ((dw >> 2) & 1) * MH;
        const bool rows_exist = m_lo < p.M;
        const uint32_t lane_addr = (quarter * 32) << 16;
        const uint32_t xa = i8_range_begin(p, blockIdx.x), xb = i8_range_begin(p, blockIdx.x + 1);
        const uint32_t bar_red = sbase + OFF_RED, bar_x = sbase + OFF_XFER;
        volatile uint32_t* last_flag = reinterpret_cast<volatile uint32_t*>(smem + OFF_LAST);   // [2]
        volatile uint32_t* nslot = reinterpret_cast<volatile uint32_t*>(smem + OFF_NSLOT);      // [2]
        volatile uint32_t* slot_list = reinterpret_cast<volatile uint32_t*>(smem + OFF_SLOTS);  // [2][64]
        float* xch = reinterpret_cast<float*>(smem + x_off) + m_lo * 128 + r;                   // [activation row][weight row]
        grid_dep_wait();  // the output and the scratch may still be in use by the previous kernel
        uint32_t red_phase = 0;
        bool ok = true;
        auto store_out = [&](uint32_t n, uint32_t m, float v) {
            const size_t idx = (size_t)m * p.N + n;
            if (p.out_dtype == DT_F32) static_cast<float*>(p.out)[idx] = v;
            else if (p.out_dtype == DT_BF16) static_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(v);
            else static_cast<__half*>(p.out)[idx] = __float2half_rn(v);
        };
        // the drain warps meet (bounded: a warp that gave up marks the CTA dead and the others leave too)
        auto meet = [&]() {
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_red);
            if (!i8_wait(bar_red, red_phase & 1, dead)) {
                i8_fail(dead, p.status, STATUS_TIMEOUT_EMPTY);
                ok = false;
            }
            ++red_phase;
        };
        // pieces of cut tiles this CTA writes: of its first tile (0) and / or of its last one (1)
        const uint32_t t_first = xa / p.nblk, t_last = xb > xa ? (xb - 1) / p.nblk : t_first;
        const bool have[2] = {xb > xa && (xa != t_first * p.nblk || xb < (t_first + 1) * p.nblk), t_last != t_first && xb != (t_last + 1) * p.nblk};
        const uint32_t cut_tile[2] = {t_first, t_last};
        for (uint32_t x = xa + team; x < xb && ok && rows_exist; x += 2) {
            const uint32_t i = x - xa, buf = team, use = i >> 1, q = i % p.nsc;
            const uint32_t tile = x / p.nblk, blk = x - tile * p.nblk;
            if (!i8_wait(bar_sc_full + 8 * q, (i / p.nsc) & 1, dead)) {
                i8_fail(dead, p.status, STATUS_TIMEOUT_FULL);
                ok = false;
                break;
            }
            const uint8_t* slot = smem + sc_off + q * SC_SLOT;
            const uint32_t* rec = reinterpret_cast<const uint32_t*>(slot) + r * SC_WORDS;
            const uint32_t hd = rec[0], s0 = rec[1], s1 = rec[2], m0 = rec[3], m1 = rec[4];
            const uint4* bsum = reinterpret_cast<const uint4*>(slot + SC_REC) + m_lo;
            const float* d8s = reinterpret_cast<const float*>(slot + SC_REC + MP * 16) + m_lo;
            const int sc[8] = {ubyte<0>(s0), ubyte<1>(s0), ubyte<2>(s0), ubyte<3>(s0), ubyte<0>(s1), ubyte<1>(s1), ubyte<2>(s1), ubyte<3>(s1)};
            if (!i8_wait(bar_acc_full + 8 * buf, use & 1, dead)) {
                i8_fail(dead, p.status, STATUS_TIMEOUT_MMA);
                ok = false;
                break;
            }
            tc_after();
            const uint32_t t0 = tmem + lane_addr + buf * ACC_COLS + m_lo;
            constexpr int GB = 2;  // sub-blocks whose loads are in flight together
            int sumi[MH];
#pragma unroll
            for (int m = 0; m < MH; ++m) sumi[m] = 0;
#pragma unroll
            for (int g = 0; g < 8 / GB; ++g) {
                uint32_t v[GB][MH];
#pragma unroll
                for (int k = 0; k < GB; ++k) {
                    if constexpr (MH == 16) tmem_ld16_async(t0 + MP * (GB * g + k), v[k]);
                    else tmem_ld8_async(t0 + MP * (GB * g + k), v[k]);
                }
                tmem_ld_wait();
#pragma unroll
                for (int k = 0; k < GB; ++k)
#pragma unroll
                    for (int m = 0; m < MH; ++m) sumi[m] += sc[GB * g + k] * (int)v[k][m];
            }
            tc_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);  // the MMA warp may reuse the columns
            // the block's terms: (d d8) sumi - (dmin d8) sum_j m_j bsum_j
            const float d = f16bits_to_f32(hd & 0xFFFF), dmin = f16bits_to_f32(hd >> 16);
            float term[MH];
#pragma unroll
            for (int m = 0; m < MH; ++m) {
                const uint4 bs = bsum[m];
                const float d8 = d8s[m];
                const int summ = __dp2a_lo((int)bs.x, (int)m0, __dp2a_hi((int)bs.y, (int)m0, __dp2a_lo((int)bs.z, (int)m1, __dp2a_hi((int)bs.w, (int)m1, 0))));
                term[m] = __fsub_rn(__fmul_rn(__fmul_rn(d, d8), (float)sumi[m]), __fmul_rn(__fmul_rn(dmin, d8), (float)summ));
            }
            // the running sums after the previous block (the other team's); every block waits for its predecessor, so the
            // teams never drift apart by more than one block
            const bool first_of_tile = blk == 0 || x == xa;
            if (i > 0 && !i8_wait(bar_x + 8 * (team ^ 1), ((i - 1) >> 1) & 1, dead)) {
                i8_fail(dead, p.status, STATUS_TIMEOUT_EMPTY);
                ok = false;
                break;
            }
            if (!first_of_tile)
#pragma unroll
                for (int m = 0; m < MH; ++m) term[m] = __fadd_rn(xch[m * 128], term[m]);
            const bool last_of_tile = blk + 1 == p.nblk || x + 1 == xb;
            if (!last_of_tile)
#pragma unroll
                for (int m = 0; m < MH; ++m) xch[m * 128] = term[m];
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_x + 8 * team);
            if (!last_of_tile) continue;
            // ---- the CTA's last block of this tile
            const uint32_t n = tile * 128 + r;
            const bool whole = (tile * p.nblk >= xa) && ((tile + 1) * p.nblk <= xb);
            if (whole) {
                if (n < p.N)
#pragma unroll
                    for (int m = 0; m < MH; ++m)
                        if (m_lo + m < p.M) store_out(n, m_lo + m, term[m]);
            } else {
                // a piece of a cut tile goes to scratch; the hand-over follows when all blocks are done
                const uint32_t which = tile == t_first ? 0u : 1u;
                float* part = p.part + ((size_t)(2 * blockIdx.x + which) * MP + m_lo) * 128;
#pragma unroll
                for (int m = 0; m < MH; ++m) part[m * 128 + r] = term[m];
            }
        }
        // ---- cut tiles: whoever writes a tile's last piece adds all of them, in K order, and stores the rows
        if (ok && rows_exist && (have[0] || have[1])) {
            meet();  // every drain thread's pieces are written
            if (ok && warp == DEC_WARPS && lane == 0) {
                uint32_t old[2] = {0, 0}, np[2] = {0, 0};
#pragma unroll
                for (uint32_t which = 0; which < 2; ++which) {
                    if (!have[which]) continue;
                    // the CTAs whose ranges meet the tile's pairs [x0, x1), in order
                    const uint32_t tile = cut_tile[which], x0 = tile * p.nblk, x1 = x0 + p.nblk, G = gridDim.x;
                    uint32_t k = 0;
                    for (uint32_t cc = i8_cta_of(p, x0); cc < G && k < 64; ++cc) {
                        const uint32_t a = i8_range_begin(p, cc);
                        if (a >= x1) break;
                        slot_list[64 * which + k++] = 2 * cc + (tile == a / p.nblk ? 0u : 1u);
                    }
                    nslot[which] = np[which] = k;
                    // release: the pieces (seen through the meeting) are visible to whoever reads the count; acquire: the
                    // pieces counted before are visible here.  The two counts are on their way together.
                    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(old[which]) : "l"(p.cnt + tile) : "memory");
                }
#pragma unroll
                for (uint32_t which = 0; which < 2; ++which) {
                    const bool last = have[which] && old[which] + 1 == np[which];
                    if (last) p.cnt[cut_tile[which]] = 0;  // ready for the next call
                    last_flag[which] = last ? 1u : 0u;
                }
            }
            meet();
            // the rows of a tile are shared out over both teams: team t adds the activation rows of its parity
            for (uint32_t which = 0; ok && which < 2; ++which) {
                if (!have[which] || !last_flag[which]) continue;
                const uint32_t ns = nslot[which], n = cut_tile[which] * 128 + r;
                for (uint32_t m = m_lo + team; m < m_lo + MH && m < p.M; m += 2) {
                    float tot = 0.f;
                    for (uint32_t k0 = 0; k0 < ns; k0 += 8) {
                        float v[8];
#pragma unroll
                        for (uint32_t k = 0; k < 8; ++k)
                            if (k0 + k < ns) v[k] = __ldcg(p.part + ((size_t)slot_list[64 * which + k0 + k] * MP + m) * 128 + r);
#pragma unroll
                        for (uint32_t k = 0; k < 8; ++k)
                            if (k0 + k < ns) tot = k0 + k == 0 ? v[k] : __fadd_rn(tot, v[k]);
                    }
                    if (n < p.N) store_out(n, m, tot);
                }
            }
        }
    }
    tc_before();
    __syncthreads();
    if (warp == W_MMA) {
        tc_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// One warp per (activation row, 256-block): Q8_K codes (quantize_act_q8k.rs:26-98: d = amax / 127, id = 127 / amax,
// round half to even) into the int8 image [M][K]; the eight sums of 32 codes and the scale go to the block's record in
// `aux` (aux_bytes).  Also clears the piece counters of the main kernel.
template <typename InT>
__global__ void __launch_bounds__(256) i8_act_prep_kernel(const InT* __restrict__ act, uint8_t* __restrict__ codes, uint8_t* __restrict__ aux,
                                                          unsigned int* __restrict__ cnt, uint32_t ntiles, uint32_t M, uint32_t nblk,
                                                          uint32_t MP) {
    const int lane = threadIdx.x & 31;
    grid_dep_launch();
    grid_dep_wait();  // the activations may be the previous kernel's output; the image may still be read by it
    for (uint32_t t = blockIdx.x * 256 + threadIdx.x; t < ntiles; t += gridDim.x * 256) cnt[t] = 0;  // piece counters of the cut tiles
    const uint32_t run = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (run >= M * nblk) return;
    const uint32_t m = run / nblk, b = run % nblk;
    float v[8];
    const size_t base = (size_t)run * 256 + 8 * lane;  // row m, block b of [M][K]
    if constexpr (sizeof(InT) == 4) {
        const float4 x = __ldg(reinterpret_cast<const float4*>(act + base)), y = __ldg(reinterpret_cast<const float4*>(act + base) + 1);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; v[4] = y.x; v[5] = y.y; v[6] = y.z; v[7] = y.w;
    } else {
        const uint4 rr = __ldg(reinterpret_cast<const uint4*>(act + base));
        v[0] = __uint_as_float(rr.x << 16); v[1] = __uint_as_float(rr.x & 0xFFFF0000u);
        v[2] = __uint_as_float(rr.y << 16); v[3] = __uint_as_float(rr.y & 0xFFFF0000u);
        v[4] = __uint_as_float(rr.z << 16); v[5] = __uint_as_float(rr.z & 0xFFFF0000u);
        v[6] = __uint_as_float(rr.w << 16); v[7] = __uint_as_float(rr.w & 0xFFFF0000u);
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
        c[i] = max(-128, min(127, __float2int_rn(__fmul_rn(v[i], id))));
        s += c[i];
    }
    uint32_t w0 = 0, w1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        w0 |= (uint32_t)(c[i] & 0xFF) << (8 * i);
        w1 |= (uint32_t)(c[4 + i] & 0xFF) << (8 * i);
    }
    *reinterpret_cast<uint2*>(codes + base) = make_uint2(w0, w1);
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);  // 32 codes = four lanes
    s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
    uint8_t* ab = aux + (size_t)b * aux_bytes(MP);
    if ((lane & 3) == 0) reinterpret_cast<short*>(ab)[m * 8 + (lane >> 2)] = (short)s;
    if (lane == 0) reinterpret_cast<float*>(ab + MP * 16)[m] = __fdiv_rn(amax, 127.0f);
}

// ---------------------------------------------------------------------------------------------------------------------
// Q8_0, 17..32 activation rows (f32 activations on boostr's CPU path: dequantised row . f32 dot,
// src/quant/cpu/kernels/quant_matmul.rs:193-209).  The weight codes are int8 already; every activation is two int8
// PIECES, x = amax/127 (a1 + a2/254) with amax over its 256-run (~3e-5 of the run's amax), stacked as 2 x 32 rows of the
// B operand.  One MMA per 32-block (128 weight rows x 64 x 32) leaves the block's integer sums of both pieces in its own
// columns; the drain converts them, weighs the pieces, multiplies by the block's d and adds in f32.  Same pipeline as
// above with these differences: an accumulator holds the four blocks of half a 256-run (one 128-byte operand tile, 256
// columns), so a stage feeds both accumulators and each is reused every block; all sixteen drain warps work on every
// accumulator (four groups of four warps, 8 activation rows each) and keep their sums in registers for the whole tile;
// only whole tiles are dealt (no hand-over).
struct Q8Params {
    const uint8_t* w;
    void* out;
    const float* scale;   // [nblk256][32] amax / 127 of (256-run, activation row)
    uint32_t M, N, K;
    uint32_t nblk;        // K / 256
    uint32_t ntiles;      // ceil(N / 128)
    uint32_t ns, nr, nsc;
    uint32_t idesc;
    int out_dtype;
    unsigned int* status;
};
constexpr uint32_t Q8_RAW_PITCH = 272, Q8_RAW_TILE = 128 * Q8_RAW_PITCH;  // 34816 = 34 x 1024
constexpr uint32_t Q8_REC_WORDS = 4;                                       // the eight f16 d of a row's 256-run
constexpr uint32_t Q8_REC = 128 * Q8_REC_WORDS * 4;
constexpr uint32_t Q8_SLOT = Q8_REC + 32 * 4;                              // + the activation rows' scales of the run
constexpr float Q8_STEP = 254.0f;

__global__ void __launch_bounds__(I8_THREADS, 1) smallm_i8_q8_0_kernel(const __grid_constant__ CUtensorMap tmap_act,
                                                                       const __grid_constant__ CUtensorMap tmap_w, const Q8Params p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int warp = __shfl_sync(0xFFFFFFFFu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar_full = sbase + OFF_FULL, bar_empty = sbase + OFF_EMPTY, bar_raw_full = sbase + OFF_RAW_FULL,
                   bar_raw_empty = sbase + OFF_RAW_EMPTY, bar_acc_full = sbase + OFF_ACC_FULL, bar_acc_empty = sbase + OFF_ACC_EMPTY,
                   bar_sc_full = sbase + OFF_SC_FULL;
    volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + OFF_TMEM);
    volatile uint32_t* dead = reinterpret_cast<volatile uint32_t*>(smem + OFF_DEAD);
    constexpr uint32_t MP = 32, P = 2;                   // activation rows of the MMA, pieces per activation
    constexpr uint32_t NB = P * MP;                      // MMA N: the pieces' rows
    constexpr uint32_t ACC_COLS = 4 * NB;                // four 32-blocks
    constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;         // 512
    constexpr uint32_t B_ATOM = NB * 128, STAGE = 2 * A_ATOM + 2 * B_ATOM;
    constexpr int MH = 8;                                // activation rows of a drain thread
    const uint32_t sc_off = OFF_SC, raw_off = (sc_off + p.nsc * Q8_SLOT + 1023u) & ~1023u, st_off = raw_off + p.nr * Q8_RAW_TILE;
    // drain warps whose activation rows exist, per accumulator
    const uint32_t groups = min((uint32_t)MP / MH, (p.M + MH - 1) / MH), acc_warps = 4 * groups;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.ns; ++s) {
            mbar_init(bar_full + 8 * s, 5);   // the four decode warps of a set + the activation copy
            mbar_init(bar_empty + 8 * s, 1);  // the commit behind the stage's second group of MMAs
        }
        for (uint32_t s = 0; s < p.nr; ++s) {
            mbar_init(bar_raw_full + 8 * s, 1);
            mbar_init(bar_raw_empty + 8 * s, 4);
        }
        for (uint32_t s = 0; s < 2; ++s) {
            mbar_init(bar_acc_full + 8 * s, 1);
            mbar_init(bar_acc_empty + 8 * s, acc_warps);
        }
        for (uint32_t s = 0; s < p.nsc; ++s) mbar_init(bar_sc_full + 8 * s, 5);
        *dead = 0;
        mbar_fence_init();
    }
    if (warp == W_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sbase + OFF_TMEM), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_before();
    __syncthreads();
    tc_after();
    const uint32_t tmem = *tmem_holder;
    grid_dep_launch();
    // the CTA's tiles: blockIdx.x, blockIdx.x + gridDim.x, ...; block i of the CTA = block i % nblk of its (i / nblk)-th tile
    const uint32_t my_tiles = p.ntiles > blockIdx.x ? (p.ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;
    const uint32_t nblocks = my_tiles * p.nblk;

    if (warp == W_RAW) {
        if (lane == 0) {
            for (uint32_t i = 0; i < nblocks && !*dead; ++i) {
                const uint32_t s = i % p.nr, par = (i / p.nr) & 1, tile = blockIdx.x + (i / p.nblk) * gridDim.x, blk = i % p.nblk;
                if (!i8_wait(bar_raw_empty + 8 * s, par ^ 1, dead)) {
                    i8_fail(dead, p.status, STATUS_TIMEOUT_EMPTY);
                    break;
                }
                mbar_expect_tx(bar_raw_full + 8 * s, Q8_RAW_TILE);
                tma2d(sbase + raw_off + s * Q8_RAW_TILE, &tmap_w, (int)(blk * 136), (int)(tile * 128), bar_raw_full + 8 * s);  // x in 16-bit units
            }
        }
    } else if (warp == W_ACT) {
        if (lane == 0) {
            grid_dep_wait();
            for (uint32_t i = 0; i < nblocks && !*dead; ++i) {
                const uint32_t s = i % p.ns, par = (i / p.ns) & 1, blk = i % p.nblk, q = i % p.nsc;
                if (!i8_wait(bar_empty + 8 * s, par ^ 1, dead)) {
                    i8_fail(dead, p.status, STATUS_TIMEOUT_EMPTY);
                    break;
                }
                const uint32_t b0 = sbase + st_off + s * STAGE + 2 * A_ATOM;
                mbar_expect_tx(bar_full + 8 * s, 2 * B_ATOM);
                tma2d(b0, &tmap_act, (int)(blk * 256), 0, bar_full + 8 * s);
                tma2d(b0 + B_ATOM, &tmap_act, (int)(blk * 256 + 128), 0, bar_full + 8 * s);
                mbar_expect_tx(bar_sc_full + 8 * q, MP * 4);
                bulk_g2s(sbase + sc_off + q * Q8_SLOT + Q8_REC, p.scale + (size_t)blk * MP, MP * 4, bar_sc_full + 8 * q);
            }
        }
    } else if (warp == W_MMA) {
        // ------------------------------------------------------------ MMA issue: per stage two accumulators of four blocks
        bool ok = true;
        for (uint32_t i = 0; ok && i < nblocks; ++i) {
            const uint32_t s = i % p.ns, par = (i / p.ns) & 1;
            if (!i8_wait(bar_full + 8 * s, par, dead)) {
                if (lane == 0) i8_fail(dead, p.status, STATUS_TIMEOUT_FULL);
                break;
            }
            for (uint32_t h = 0; h < 2; ++h) {  // accumulator h = half-run h of the block: use number i of this accumulator
                if (i > 0 && !i8_wait(bar_acc_empty + 8 * h, (i - 1) & 1, dead)) {
                    if (lane == 0) i8_fail(dead, p.status, STATUS_TIMEOUT_EMPTY);
                    ok = false;
                    break;
                }
                tc_after();
                if (elect_one_lane()) {
                    const uint32_t a_lo = desc_lo(sbase + st_off + s * STAGE + h * A_ATOM), b_lo = desc_lo(sbase + st_off + s * STAGE + 2 * A_ATOM + h * B_ATOM);
#pragma unroll
                    for (uint32_t b = 0; b < 4; ++b) tc_mma_i8(tmem + h * ACC_COLS + NB * b, desc_sw128(a_lo + 2 * b), desc_sw128(b_lo + 2 * b), p.idesc);
                    if (h == 1) tc_commit_to(bar_empty + 8 * s);
                    tc_commit_to(bar_acc_full + 8 * h);
                }
                __syncwarp();
            }
        }
    } else if (warp < DEC_WARPS) {
        // ------------------------------------------------------------ decode: copy the codes into the A operand, one thread per row
        // Raw row of a 256-run: eight blocks of 34 bytes (f16 d | 32 x i8) = 68 words.  The codes of block b start at byte
        // 34 b + 2: on a word boundary for odd b, two bytes past one for even b (a word = two neighbours and a byte permute).
        const uint32_t r = threadIdx.x & 127, set = threadIdx.x >> 7;
        const uint32_t row_sw = (r >> 3) * 1024 + (r & 7) * 128, x7 = r & 7;
        bool ok = true;
        for (uint32_t i = set; i < nblocks; i += DEC_WARPS / 4) {
            const uint32_t rs = i % p.nr, rpar = (i / p.nr) & 1, s = i % p.ns, par = (i / p.ns) & 1;
            const bool row_ok = (blockIdx.x + (i / p.nblk) * gridDim.x) * 128 + r < p.N;
            if (ok && !i8_wait(bar_raw_full + 8 * rs, rpar, dead)) {
                i8_fail(dead, p.status, STATUS_TIMEOUT_FULL);
                ok = false;
            }
            if (ok && !i8_wait(bar_empty + 8 * s, par ^ 1, dead)) {
                i8_fail(dead, p.status, STATUS_TIMEOUT_EMPTY);
                ok = false;
            }
            const uint4* src = reinterpret_cast<const uint4*>(smem + raw_off + rs * Q8_RAW_TILE + r * Q8_RAW_PITCH);
            uint8_t* a0 = smem + st_off + s * STAGE + row_sw;
            uint32_t dd[8];
#pragma unroll
            for (int b = 0; b < 8; ++b) {
                constexpr int K0[8] = {0, 9, 17, 26, 34, 43, 51, 60};  // first word that holds codes of block b
                const int q0 = (K0[b] - (b & 1)) / 4, off = K0[b] - 4 * q0;  // three 16-byte loads from word 4 q0 cover d and the codes
                uint32_t a[12];
                if (ok && row_ok) {
                    const uint4 u0 = src[q0], u1 = src[q0 + 1], u2 = src[q0 + 2];
                    a[0] = u0.x; a[1] = u0.y; a[2] = u0.z; a[3] = u0.w; a[4] = u1.x; a[5] = u1.y; a[6] = u1.z; a[7] = u1.w;
                    a[8] = u2.x; a[9] = u2.y; a[10] = u2.z; a[11] = u2.w;
                } else {
#pragma unroll
                    for (int k = 0; k < 12; ++k) a[k] = 0;
                }
                uint32_t o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = (b & 1) ? a[off + j] : __byte_perm(a[off + j], a[off + j + 1], 0x5432);
                dd[b] = (b & 1) ? a[off - 1] >> 16 : a[off] & 0xFFFFu;
                // block b = bytes 32 b .. of the 256-byte operand row: 16-byte chunks 2 b, 2 b + 1 -> tile b / 4
                uint8_t* at = a0 + (b >> 2) * A_ATOM;
                *reinterpret_cast<uint4*>(at + ((((2 * b) & 7) ^ x7) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                *reinterpret_cast<uint4*>(at + ((((2 * b + 1) & 7) ^ x7) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_raw_empty + 8 * rs);
            uint32_t* rec = reinterpret_cast<uint32_t*>(smem + sc_off + (i % p.nsc) * Q8_SLOT) + r * Q8_REC_WORDS;
#pragma unroll
            for (int k = 0; k < 4; ++k) rec[k] = dd[2 * k] | (dd[2 * k + 1] << 16);
            proxy_fence();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(bar_full + 8 * s);
                mbar_arrive(bar_sc_full + 8 * (i % p.nsc));
            }
        }
    } else {
        // ------------------------------------------------------------ drain: four groups of four warps, 8 activation rows each
        const uint32_t dw = (uint32_t)warp - DEC_WARPS, quarter = dw & 3, r = quarter * 32 + lane, m_lo = (dw >> 2) * MH;
        const bool rows_exist = m_lo < p.M;
        const uint32_t lane_addr = (quarter * 32) << 16;
        grid_dep_wait();
        bool ok = true;
        float acc[MH];
#pragma unroll
        for (int m = 0; m < MH; ++m) acc[m] = 0.f;
        constexpr float C1 = 1.0f / Q8_STEP;
        for (uint32_t i = 0; i < nblocks && ok && rows_exist; ++i) {
            const uint32_t q = i % p.nsc, blk = i % p.nblk, tl = i / p.nblk;
            if (!i8_wait(bar_sc_full + 8 * q, (i / p.nsc) & 1, dead)) {
                i8_fail(dead, p.status, STATUS_TIMEOUT_FULL);
                ok = false;
                break;
            }
            const uint8_t* slot = smem + sc_off + q * Q8_SLOT;
            const uint32_t* rec = reinterpret_cast<const uint32_t*>(slot) + r * Q8_REC_WORDS;
            const float* scl = reinterpret_cast<const float*>(slot + Q8_REC) + m_lo;
#pragma unroll
            for (uint32_t h = 0; h < 2; ++h) {  // the two half-runs of the block
                const uint32_t d01 = rec[2 * h], d23 = rec[2 * h + 1];
                const float db[4] = {f16bits_to_f32(d01 & 0xFFFF), f16bits_to_f32(d01 >> 16), f16bits_to_f32(d23 & 0xFFFF), f16bits_to_f32(d23 >> 16)};
                if (!i8_wait(bar_acc_full + 8 * h, i & 1, dead)) {
                    i8_fail(dead, p.status, STATUS_TIMEOUT_MMA);
                    ok = false;
                    break;
                }
                tc_after();
                float sacc[MH];
#pragma unroll
                for (int m = 0; m < MH; ++m) sacc[m] = 0.f;
                const uint32_t t0 = tmem + lane_addr + h * ACC_COLS + m_lo;
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    uint32_t v[P][MH];
#pragma unroll
                    for (int pc = 0; pc < (int)P; ++pc) tmem_ld8_async(t0 + NB * b + MP * pc, v[pc]);
                    tmem_ld_wait();
                    // the two pieces meet as integers, 254 a1 + a2 (|.| < 2^28), so a block costs one conversion and one FMA
#pragma unroll
                    for (int m = 0; m < MH; ++m) sacc[m] = fmaf(db[b], (float)(254 * (int)v[0][m] + (int)v[1][m]), sacc[m]);
                }
                tc_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_empty + 8 * h);
#pragma unroll
                for (int m = 0; m < MH; ++m) acc[m] = fmaf(sacc[m], scl[m] * C1, acc[m]);
            }
            if (!ok || blk + 1 != p.nblk) continue;
            // ---- the tile is complete
            const uint32_t n = (blockIdx.x + tl * gridDim.x) * 128 + r;
            if (n < p.N)
#pragma unroll
                for (int m = 0; m < MH; ++m) {
                    if (m_lo + m < p.M) {
                        const size_t idx = (size_t)(m_lo + m) * p.N + n;
                        if (p.out_dtype == DT_F32) static_cast<float*>(p.out)[idx] = acc[m];
                        else if (p.out_dtype == DT_BF16) static_cast<__nv_bfloat16*>(p.out)[idx] = __float2bfloat16_rn(acc[m]);
                        else static_cast<__half*>(p.out)[idx] = __float2half_rn(acc[m]);
                    }
                }
#pragma unroll
            for (int m = 0; m < MH; ++m) acc[m] = 0.f;
        }
    }
    tc_before();
    __syncthreads();
    if (warp == W_MMA) {
        tc_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// One warp per (activation row, 256-run): the run's amax / 127 into scale[run][row] and every value as P int8 pieces,
// x = amax/127 (a1 + a2/254 + a3/254^2), piece pc of row m into row pc MP + m of the image [P MP][K]; rows that do not
// exist are written as zeros (the B operand reads all MP rows of a piece).
template <typename InT, int P>
__global__ void __launch_bounds__(256) q8_act_prep_kernel(const InT* __restrict__ act, uint8_t* __restrict__ img, float* __restrict__ scale,
                                                          uint32_t M, uint32_t K, uint32_t MP) {
    const int lane = threadIdx.x & 31;
    grid_dep_launch();
    grid_dep_wait();
    const uint32_t nblk = K / 256, run = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (run >= MP * nblk) return;
    const uint32_t m = run / nblk, b = run % nblk;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = 0.f;
    if (m < M) {
        const size_t base = (size_t)m * K + (size_t)b * 256 + 8 * lane;
        if constexpr (sizeof(InT) == 4) {
            const float4 x = __ldg(reinterpret_cast<const float4*>(act + base)), y = __ldg(reinterpret_cast<const float4*>(act + base) + 1);
            v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w; v[4] = y.x; v[5] = y.y; v[6] = y.z; v[7] = y.w;
        } else {
            const uint4 rr = __ldg(reinterpret_cast<const uint4*>(act + base));
            v[0] = __uint_as_float(rr.x << 16); v[1] = __uint_as_float(rr.x & 0xFFFF0000u);
            v[2] = __uint_as_float(rr.y << 16); v[3] = __uint_as_float(rr.y & 0xFFFF0000u);
            v[4] = __uint_as_float(rr.z << 16); v[5] = __uint_as_float(rr.z & 0xFFFF0000u);
            v[6] = __uint_as_float(rr.w << 16); v[7] = __uint_as_float(rr.w & 0xFFFF0000u);
        }
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    const float id = amax != 0.f ? __fdiv_rn(127.0f, amax) : 0.f;
    uint32_t w[P][2];
#pragma unroll
    for (int pc = 0; pc < P; ++pc) w[pc][0] = w[pc][1] = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float rr = __fmul_rn(v[i], id);  // |rr| <= 127 (+ one rounding)
#pragma unroll
        for (int pc = 0; pc < P; ++pc) {
            const int c = max(-127, min(127, (int)rintf(rr)));
            w[pc][i >> 2] |= (uint32_t)(c & 0xFF) << (8 * (i & 3));
            rr = __fmul_rn(__fsub_rn(rr, (float)c), Q8_STEP);  // remainder in [-0.5, 0.5] -> [-127, 127]
        }
    }
#pragma unroll
    for (int pc = 0; pc < P; ++pc)
        *reinterpret_cast<uint2*>(img + ((size_t)(pc * MP + m) * K + (size_t)b * 256 + 8 * lane)) = make_uint2(w[pc][0], w[pc][1]);
    if (lane == 0) scale[(size_t)b * MP + m] = m < M ? __fdiv_rn(amax, 127.0f) : 0.f;
}

struct I8Layout {
    uint32_t MP, nblk, ntiles, Q, grid, unit;
    size_t codes_bytes, aux_off, part_off, cnt_off, total;
};
I8Layout i8_layout(size_t M, size_t K, size_t N, int sm_count) {
    I8Layout l{};
    l.MP = M <= 16 ? 16u : 32u;
    l.nblk = (uint32_t)(K / 256);
    l.ntiles = (uint32_t)((N + 127) / 128);
    l.Q = l.ntiles * l.nblk;
    // Whole tiles per CTA (nothing to hand over) unless cutting the tiles along K shortens the longest CTA by more than
    // the hand-over costs (about eight blocks' worth of time).
    const uint32_t G = (uint32_t)sm_count;
    const uint32_t whole_cost = (l.ntiles + G - 1) / G * l.nblk, cut_cost = (l.Q + G - 1) / G + 8;
    l.unit = whole_cost <= cut_cost ? l.nblk : 1u;
    const uint32_t items = l.Q / l.unit;
    l.grid = items < G ? items : G;
    l.codes_bytes = (M * K + 255) & ~(size_t)255;
    l.aux_off = l.codes_bytes;
    l.part_off = l.aux_off + (((size_t)l.nblk * aux_bytes(l.MP) + 255) & ~(size_t)255);
    l.cnt_off = l.part_off + (size_t)2 * l.grid * l.MP * 128 * 4;
    l.total = l.cnt_off + (((size_t)l.ntiles * 4 + 255) & ~(size_t)255);
    return l;
}

struct Q8Layout {
    uint32_t MP, P, nblk, ntiles, grid;
    size_t img_bytes, scale_off, total;
};
Q8Layout q8_layout(size_t M, size_t K, size_t N, int sm_count) {
    Q8Layout l{};
    (void)M;
    l.MP = 32u;  // 17..32 rows
    l.P = 2u;
    l.nblk = (uint32_t)(K / 256);
    l.ntiles = (uint32_t)((N + 127) / 128);
    l.grid = l.ntiles < (uint32_t)sm_count ? l.ntiles : (uint32_t)sm_count;
    l.img_bytes = ((size_t)l.P * l.MP * K + 255) & ~(size_t)255;
    l.scale_off = l.img_bytes;
    l.total = l.scale_off + (((size_t)l.nblk * l.MP * 4 + 255) & ~(size_t)255);
    return l;
}

cudaError_t launch_q8_kernel(const CUtensorMap& amap, const CUtensorMap& wmap, const Q8Params& p, uint32_t grid, size_t smem, cudaStream_t st) {
    static PerDeviceOnce attrs;
    cudaError_t e = attrs.run([] { return cudaFuncSetAttribute(smallm_i8_q8_0_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448); });
    if (e != cudaSuccess) return e;
    return launch_pdl(smallm_i8_q8_0_kernel, dim3(grid), dim3(I8_THREADS), smem, st, amap, wmap, p);
}

cudaError_t launch_smallm_q8_0(const void* act, int act_dtype, const void* w, void* out, int out_dtype, size_t M, size_t K, size_t N, void* ws,
                               size_t ws_bytes, int sm_count, cudaStream_t st, unsigned int* status, bool* ws_too_small, char* err,
                               size_t err_len, bool acts_prepared) {
    *ws_too_small = false;
    const Q8Layout l = q8_layout(M, K, N, sm_count);
    if (!ws || ws_bytes < l.total || (reinterpret_cast<uintptr_t>(ws) & 15)) { *ws_too_small = true; return cudaSuccess; }
    uint8_t* base = static_cast<uint8_t*>(ws);
    float* scale = reinterpret_cast<float*>(base + l.scale_off);
    if (!acts_prepared) {
        const dim3 pg((l.MP * l.nblk + 7) / 8);
        cudaError_t e;
        if (act_dtype == DT_F32)
            e = launch_pdl(q8_act_prep_kernel<float, 2>, pg, dim3(256), 0, st, static_cast<const float*>(act), base, scale, (uint32_t)M, (uint32_t)K, l.MP);
        else
            e = launch_pdl(q8_act_prep_kernel<__nv_bfloat16, 2>, pg, dim3(256), 0, st, static_cast<const __nv_bfloat16*>(act), base, scale, (uint32_t)M,
                           (uint32_t)K, l.MP);
        note_launch();
        if (e != cudaSuccess) return e;
    }
    EncodeTiledFn enc = encode_tiled();
    if (!enc) {
        snprintf(err, err_len, "cuTensorMapEncodeTiled is not available from this driver");
        return cudaErrorNotSupported;
    }
    Q8Params p{};
    p.w = static_cast<const uint8_t*>(w);
    p.out = out;
    p.scale = scale;
    p.M = (uint32_t)M; p.N = (uint32_t)N; p.K = (uint32_t)K;
    p.nblk = l.nblk; p.ntiles = l.ntiles;
    const uint32_t NB = l.P * l.MP;
    p.idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((NB >> 3) << 17) | ((128u >> 4) << 24);  // int32 <- s8 x s8, K-major, N = P MP, M = 128
    p.out_dtype = out_dtype;
    p.status = status;
    const uint32_t stage = 2 * A_ATOM + 2 * NB * 128;
    p.ns = 2;
    p.nsc = p.ns + 2 + 2;
    const uint32_t fixed = 1024 + ((p.nsc * Q8_SLOT + 1023u) & ~1023u) + p.ns * stage;
    p.nr = ((232448u - 1024u - 1024u - fixed) / Q8_RAW_TILE) & ~1u;  // even: see launch_smallm_i8
    if (p.nr > 4) p.nr = 4;
    const size_t smem = 1024 + fixed + (size_t)p.nr * Q8_RAW_TILE;

    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap amap, wmap;
    {
        const cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)NB};
        const cuuint64_t gstride[1] = {(cuuint64_t)K};
        const cuuint32_t box[2] = {128u, NB};
        CUresult cr = enc(&amap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) {
            snprintf(err, err_len, "cuTensorMapEncodeTiled failed with code %d (activation image %p, K=%zu, rows %u)", (int)cr, (void*)base, K, NB);
            return cudaErrorInvalidValue;
        }
    }
    {
        // packed rows as 16-bit units (a box dimension holds at most 256 elements): 136 units = the 272 bytes of a 256-run
        const uint32_t row_bytes = l.nblk * 272;
        const cuuint64_t gdim[2] = {(cuuint64_t)(row_bytes / 2), (cuuint64_t)N};
        const cuuint64_t gstride[1] = {(cuuint64_t)row_bytes};
        const cuuint32_t box[2] = {136u, 128u};
        CUresult cr = enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(w), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) {
            snprintf(err, err_len, "cuTensorMapEncodeTiled failed with code %d (weight pointer %p, row bytes %u, N=%zu)", (int)cr, w, row_bytes, N);
            return cudaErrorInvalidValue;
        }
    }
    cudaError_t e = launch_q8_kernel(amap, wmap, p, l.grid, smem, st);
    note_launch();
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace

// Shapes the integer tensor-core kernels take.  Q4_K: 2 <= M <= 32, whole 256-blocks (rows are multiples of 16 bytes:
// 144-byte blocks), pair counts within 32 bits.  Q8_0: 17 <= M <= 32 (up to 16 rows the mma.sync kernel is as fast), K a multiple
// of 256 (rows of whole 272-byte runs), whole tiles only.
bool smallm_i8_supported(int fmt, size_t M, size_t K, size_t N) {
    if (M < 2 || M > 32 || K % 256 != 0 || K < 256 || N < 1 || (N + 127) / 128 * (K / 256) >= (1u << 30)) return false;
    return (fmt == FMT_Q8_0 && M > 16) || (fmt == FMT_Q4_K && K / 256 <= 64);
}
size_t smallm_i8_workspace_bytes(int fmt, size_t M, size_t K, size_t N, int sm_count) {
    return fmt == FMT_Q8_0 ? q8_layout(M, K, N, sm_count).total : i8_layout(M, K, N, sm_count).total;
}
// Where they beat the mma.sync kernel (measured).  Q4_K: matrices with enough 128-row tiles to give every SM whole tiles
// (nothing to hand over), from 8 activation rows on; and every shape above 16 rows, which the mma.sync kernel takes in
// two passes over the weights.  Q8_0: above 16 rows (one pass over the weights instead of two), matrices with enough
// tiles to occupy half of the SMs (only whole tiles are dealt).
bool smallm_i8_preferred(int fmt, size_t M, size_t K, size_t N, int sm_count) {
    if (!smallm_i8_supported(fmt, M, K, N)) return false;
    if (fmt == FMT_Q8_0) return M > 16 && (N + 127) / 128 >= (size_t)sm_count / 2;
    if (M > 16) return true;
    const I8Layout l = i8_layout(M, K, N, sm_count);
    return M >= 8 && l.unit == l.nblk && l.ntiles >= (uint32_t)sm_count * 3 / 4;
}

// acts_prepared: a previous call with the same activations and scratch left the image there (gate, then up).
cudaError_t launch_smallm_i8(int fmt, const void* act, int act_dtype, const void* w, void* out, int out_dtype, size_t M, size_t K,
                             size_t N, void* ws, size_t ws_bytes, int sm_count, cudaStream_t st, unsigned int* status,
                             bool* ws_too_small, char* err, size_t err_len, bool acts_prepared) {
    if (fmt == FMT_Q8_0)
        return launch_smallm_q8_0(act, act_dtype, w, out, out_dtype, M, K, N, ws, ws_bytes, sm_count, st, status, ws_too_small, err, err_len, acts_prepared);
    *ws_too_small = false;
    const I8Layout l = i8_layout(M, K, N, sm_count);
    if (!ws || ws_bytes < l.total || (reinterpret_cast<uintptr_t>(ws) & 15)) { *ws_too_small = true; return cudaSuccess; }
    uint8_t* base = static_cast<uint8_t*>(ws);
    uint8_t* codes = base;
    uint8_t* aux = base + l.aux_off;
    unsigned int* cnt = reinterpret_cast<unsigned int*>(base + l.cnt_off);
    if (!acts_prepared) {
        const uint32_t runs = (uint32_t)M * l.nblk;
        const dim3 pg((runs + 7) / 8);
        cudaError_t e = act_dtype == DT_F32
                            ? launch_pdl(i8_act_prep_kernel<float>, pg, dim3(256), 0, st, static_cast<const float*>(act), codes, aux, cnt, l.ntiles, (uint32_t)M, l.nblk, l.MP)
                            : launch_pdl(i8_act_prep_kernel<__nv_bfloat16>, pg, dim3(256), 0, st, static_cast<const __nv_bfloat16*>(act), codes, aux, cnt,
                                         l.ntiles, (uint32_t)M, l.nblk, l.MP);
        note_launch();
        if (e != cudaSuccess) return e;
    }
    EncodeTiledFn enc = encode_tiled();
    if (!enc) {
        snprintf(err, err_len, "cuTensorMapEncodeTiled is not available from this driver");
        return cudaErrorNotSupported;
    }
    I8Params p{};
    p.w = static_cast<const uint8_t*>(w);
    p.out = out;
    p.part = reinterpret_cast<float*>(base + l.part_off);
    p.cnt = cnt;
    p.aux = aux;
    p.M = (uint32_t)M; p.N = (uint32_t)N; p.K = (uint32_t)K;
    p.MP = l.MP; p.nblk = l.nblk; p.ntiles = l.ntiles; p.Q = l.Q;
    p.unit = l.unit;
    p.qbase = (l.Q / l.unit) / l.grid; p.qrem = (l.Q / l.unit) % l.grid;
    // int32 accumulator, signed 8-bit x signed 8-bit, both K-major, N = MP, M = 128
    p.idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((p.MP >> 3) << 17) | ((128u >> 4) << 24);
    p.out_dtype = out_dtype;
    p.status = status;
    const uint32_t stage = 2 * A_ATOM + 2 * p.MP * 128;
    p.ns = 3;
    p.nsc = p.ns + 2 + 2;
    const uint32_t fixed = 1024 + ((p.nsc * SC_SLOT + 128 * p.MP * 4 + 1023u) & ~1023u) + p.ns * stage;
    // The ring of packed tiles must have an EVEN depth: block i lives in slot i % nr and is read by decode set i & 1, so with
    // an even depth a slot always belongs to one set and that set sees every phase of the slot's barrier.  With an odd depth
    // the sets would alternate on a slot, a set would wait for phase k having last seen phase k - 2, and a parity wait cannot
    // tell those apart when the fill in between is late (fills may complete out of order).
    p.nr = ((232448u - 1024u - 1024u - fixed) / RAW_TILE) & ~1u;
    if (p.nr > 6) p.nr = 6;
    const size_t smem = 1024 + fixed + (size_t)p.nr * RAW_TILE;

    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap amap, wmap;
    {
        const cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)M};
        const cuuint64_t gstride[1] = {(cuuint64_t)K};
        const cuuint32_t box[2] = {128u, p.MP};
        CUresult cr = enc(&amap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, codes, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) {
            snprintf(err, err_len, "cuTensorMapEncodeTiled failed with code %d (activation image %p, K=%zu, M=%zu)", (int)cr, (void*)codes, K, M);
            return cudaErrorInvalidValue;
        }
    }
    {
        const uint32_t row_bytes = l.nblk * 144;
        const cuuint64_t gdim[2] = {(cuuint64_t)row_bytes, (cuuint64_t)N};
        const cuuint64_t gstride[1] = {(cuuint64_t)row_bytes};
        const cuuint32_t box[2] = {RAW_PITCH, 128u};
        CUresult cr = enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(w), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS) {
            snprintf(err, err_len, "cuTensorMapEncodeTiled failed with code %d (weight pointer %p, row bytes %u, N=%zu)", (int)cr, w, row_bytes, N);
            return cudaErrorInvalidValue;
        }
    }
    static PerDeviceOnce attrs;
    cudaError_t e = attrs.run([] {
        cudaError_t a = cudaFuncSetAttribute(smallm_i8_q4k_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
        if (a == cudaSuccess) a = cudaFuncSetAttribute(smallm_i8_q4k_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448);
        return a;
    });
    if (e != cudaSuccess) return e;
    e = p.MP == 16 ? launch_pdl(smallm_i8_q4k_kernel<16>, dim3(l.grid), dim3(I8_THREADS), smem, st, amap, wmap, p)
                   : launch_pdl(smallm_i8_q4k_kernel<32>, dim3(l.grid), dim3(I8_THREADS), smem, st, amap, wmap, p);
    note_launch();
    if (e != cudaSuccess) return e;
    return cudaGetLastError();
}

}  // namespace b200q
