// Shared device helpers for the sm_100a quantized-linear kernels: mbarrier and bulk-copy
// (TMA) wrappers with bounded waits, legacy-tensor-core MMA wrappers for the memory-bound
// small-M kernels, unaligned shared-memory loads for the 2-byte-aligned GGUF blocks.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

namespace b200q {

// Block formats (QuantFormat::format_id of the reference).
enum : int { FMT_Q4_0 = 0, FMT_Q5_0 = 2, FMT_Q8_0 = 4, FMT_Q2_K = 6, FMT_Q3_K = 7, FMT_Q4_K = 8, FMT_Q5_K = 9, FMT_Q6_K = 10 };
enum : int { DT_F32 = 0, DT_BF16 = 1, DT_F16 = 2, DT_F64 = 3 };

// Device status word (one per device, owned by the C-ABI translation unit and handed to
// kernels as a pointer): a kernel that gives up on a bounded wait ORs a code in here and
// finishes without touching the data it waited for.
enum : unsigned { STATUS_TIMEOUT_FULL = 1u, STATUS_TIMEOUT_EMPTY = 2u, STATUS_TIMEOUT_MMA = 4u, STATUS_TIMEOUT_TMEM = 8u, STATUS_TIMEOUT_PEER = 16u };

__host__ __device__ constexpr int fmt_block_size(int f) { return (f == FMT_Q4_0 || f == FMT_Q5_0 || f == FMT_Q8_0) ? 32 : 256; }
__host__ __device__ constexpr int fmt_block_bytes(int f) {
    return f == FMT_Q4_0 ? 18 : f == FMT_Q5_0 ? 22 : f == FMT_Q8_0 ? 34 : f == FMT_Q2_K ? 84 : f == FMT_Q3_K ? 110 : f == FMT_Q4_K ? 144 : f == FMT_Q5_K ? 176 : f == FMT_Q6_K ? 210 : 0;
}
// Bytes of one 256-element run of a row ("slice"): the unit one warp of the small-M kernel owns.
__host__ __device__ constexpr int fmt_slice_bytes(int f) { return fmt_block_bytes(f) * (256 / fmt_block_size(f)); }

// Host-side count of kernel launches issued by the library (see b200q_launch_count).
void note_launch(unsigned n = 1);

// Per-device "done once" flags for host-side set-up (kernel attributes): the action runs until it has
// succeeded once on the current device; concurrent first calls may both run it, which is harmless for
// idempotent CUDA attribute calls, and the flag itself is an atomic.
struct PerDeviceOnce {
    std::atomic<bool> done[64];
    template <typename F>
    cudaError_t run(F&& action) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        if (dev < 0 || dev >= 64) return action();
        if (done[dev].load(std::memory_order_acquire)) return cudaSuccess;
        e = action();
        if (e == cudaSuccess) done[dev].store(true, std::memory_order_release);
        return e;
    }
};

// ---------------------------------------------------------------- shared memory / mbarrier

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking test of a phase (try_wait may suspend the thread for a while when it fails).
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: gives up after two seconds of wall time, in which case the caller records a
// status code and stops using the data it waited for.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
#pragma unroll 1
    for (int i = 0; i < 128; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
#pragma unroll 1
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 8; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_timer_ns() - t0 > 2000000000ull) return false;
        __nanosleep(40);
    }
}

// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier.
// dst, src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Copies the 2-byte-aligned global range [src, src + bytes) into shared memory as the enclosing 16-byte
// aligned range (bulk copies need 16-byte alignment): the data lands at dst + (src & 15).  If that range
// would end past the tensor (`wend`), the last <16 bytes are moved with plain loads.  One lane calls this.
__device__ __forceinline__ void fill_contiguous(uint32_t dst_s, uint8_t* dst_g, const uint8_t* src, uint32_t bytes,
                                                const uint8_t* wend, uint32_t bar) {
    const uint8_t* gs = reinterpret_cast<const uint8_t*>(reinterpret_cast<uintptr_t>(src) & ~(uintptr_t)15);
    const uint8_t* ge = src + bytes;
    const uint8_t* e16 = reinterpret_cast<const uint8_t*>((reinterpret_cast<uintptr_t>(ge) + 15) & ~(uintptr_t)15);
    if (e16 > wend) {
        e16 = reinterpret_cast<const uint8_t*>(reinterpret_cast<uintptr_t>(ge) & ~(uintptr_t)15);
        for (const uint8_t* q = e16; q < ge; ++q) dst_g[q - gs] = __ldg(q);
    }
    const uint32_t n = (uint32_t)(e16 - gs);
    mbar_expect_tx(bar, n);  // release: the plain stores above are visible to whoever sees the phase complete
    if (n) bulk_g2s(dst_s, gs, n, bar);
}

// ------------------------------------------------------------- programmatic dependent launch
// Kernels of this library are launched so that a grid may begin while its predecessor in the
// stream is still draining (launch_pdl below).  grid_dep_launch() lets the NEXT grid start early;
// grid_dep_wait() blocks until the PREVIOUS grid has completed and its writes are visible — it
// must precede the first read of activations and the first write of any output or scratch.
// Weights never change, so their prefetch may be issued before the wait.
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ------------------------------------------------------------------- peer exchange (tensor parallel)
// Row-parallel decode products end in an all-reduce of one f32 row.  Instead of a separate collective
// the GEMV kernel pushes every element of its partial row into EVERY rank's exchange buffer over NVLink
// as one 64-bit scalar store {epoch : value bits}: the epoch travels with the value, so a reader that sees the
// expected epoch has the value (an aligned 64-bit scalar access is single-copy atomic) and no fence, flag or
// barrier is needed.
// Each CTA then collects, for ITS OWN rows, the P partial values (all ranks split the rows alike) and
// adds them in rank order, so every rank stores the same bits.  Waits are bounded.
//
// Exchange buffer of a rank (TP_BUF_BYTES, zeroed at allocation):
//   [0]   u32 epoch: number of exchanges completed by this rank (advanced by the CTA that finishes last)
//   [4]   u32 count of local CTAs that finished (reset by the same CTA)
//   [1024 + (((e & 1) * 8 + r) * 16384 + row) * 8]  {bits, e}: element `row` of rank r's partial row, epoch e
// Two parities suffice: a rank can push epoch e + 2 only after it has collected e + 1 from every peer,
// which a peer pushes after it finished collecting epoch e.
constexpr uint32_t TP_MAX_WORLD = 8, TP_MAX_N = 65536;
constexpr size_t TP_BUF_BYTES = 1024 + 2 * (size_t)TP_MAX_WORLD * TP_MAX_N * 8;
struct PeerComm {
    uint32_t world, rank;  // world <= 1: no exchange
    uint32_t gather;       // 0: add the ranks' partial rows (row-parallel); 1: place the ranks' row slices side by side (column-parallel)
    uint32_t n_total;      // gather: length of the assembled row (world * local rows, <= TP_MAX_WORLD * TP_MAX_N)
    uint8_t* buf[TP_MAX_WORLD];
};
__device__ __forceinline__ size_t tp_slot(uint32_t e, uint32_t src, uint32_t row) {
    return 1024 + (((size_t)(e & 1u) * TP_MAX_WORLD + src) * TP_MAX_N + row) * 8;
}
// epoch this launch takes part in (call after grid_dep_wait)
__device__ __forceinline__ uint32_t tp_epoch(const PeerComm& c) {
    return *reinterpret_cast<volatile const uint32_t*>(c.buf[c.rank]) + 1u;
}
__device__ __forceinline__ void tp_push(const PeerComm& c, uint32_t e, uint32_t row, float v) {
    const size_t off = tp_slot(e, c.rank, row);
    // one 64-bit scalar {epoch : value bits}: a single-copy-atomic access, so the tag and the value arrive together
    const unsigned long long word = ((unsigned long long)e << 32) | (unsigned long long)__float_as_uint(v);
    for (uint32_t r = 0; r < c.world; ++r)
        asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(c.buf[r] + off), "l"(word) : "memory");
}
// Column-parallel gather: element `col` of the assembled row [0, n_total) lives at slot `col` of the epoch's
// parity half (the same memory the row-parallel exchange uses as [rank][row]; the two kinds of exchange may
// alternate freely because consecutive epochs never share a half).
__device__ __forceinline__ size_t tp_gather_slot(uint32_t e, uint32_t col) {
    return 1024 + ((size_t)(e & 1u) * TP_MAX_WORLD * TP_MAX_N + col) * 8;
}
__device__ __forceinline__ void tp_push_gather(const PeerComm& c, uint32_t e, uint32_t col, float v) {
    const size_t off = tp_gather_slot(e, col);
    const unsigned long long word = ((unsigned long long)e << 32) | (unsigned long long)__float_as_uint(v);
    for (uint32_t r = 0; r < c.world; ++r)
        asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(c.buf[r] + off), "l"(word) : "memory");
}
// Called by ALL threads of every CTA after its last tp_push_gather: CTA b copies columns
// [b * chunk, (b + 1) * chunk) of the assembled row from this rank's buffer to `out` once their tags have arrived.
__device__ __forceinline__ void tp_finish_gather(const PeerComm& c, uint32_t e, float* out, unsigned int* status) {
    bool lost = (*reinterpret_cast<volatile unsigned int*>(status) & STATUS_TIMEOUT_PEER) != 0;
    const uint32_t chunk = (c.n_total + gridDim.x - 1) / gridDim.x;
    const uint32_t begin = min(c.n_total, blockIdx.x * chunk), end = min(c.n_total, begin + chunk);
    for (uint32_t col = begin + threadIdx.x; col < end; col += blockDim.x) {
        const uint8_t* slot = c.buf[c.rank] + tp_gather_slot(e, col);
        unsigned long long word = 0;
        uint64_t t0 = 0;
        for (uint32_t spin = 0;; ++spin) {
            asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(word) : "l"(slot) : "memory");
            if ((uint32_t)(word >> 32) == e || lost) break;
            if ((spin & 63u) == 63u) {
                const uint64_t now = global_timer_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > 1000000000ull) {
                    atomicOr(status, STATUS_TIMEOUT_PEER);
                    lost = true;
                }
            }
        }
        out[col] = __uint_as_float((uint32_t)word);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t* ctl = reinterpret_cast<uint32_t*>(c.buf[c.rank]);
        if (atomicAdd(ctl + 1, 1u) == gridDim.x - 1) {  // the CTA that finishes last closes the epoch
            ctl[1] = 0;
            ctl[0] = e;
        }
    }
}
// Called by ALL threads of every CTA after its last tp_push: adds up rows [row_begin, row_end).
__device__ __forceinline__ void tp_finish(const PeerComm& c, uint32_t e, uint32_t row_begin, uint32_t row_end, float* out,
                                          unsigned int* status) {
    bool lost = (*reinterpret_cast<volatile unsigned int*>(status) & STATUS_TIMEOUT_PEER) != 0;  // a peer was lost before
    for (uint32_t row = row_begin + threadIdx.x; row < row_end; row += blockDim.x) {
        // all ranks' slots are read at once (independent loads: one round trip, not one per rank); only
        // the slots whose epoch has not arrived yet are read again
        uint32_t bits[TP_MAX_WORLD], tag[TP_MAX_WORLD];
        uint32_t pending = (1u << c.world) - 1u;
        uint64_t t0 = 0;
        for (uint32_t spin = 0; pending; ++spin) {
#pragma unroll
            for (uint32_t r = 0; r < TP_MAX_WORLD; ++r)
                if (pending >> r & 1u) {
                    const uint8_t* slot = c.buf[c.rank] + tp_slot(e, r, row);
                    unsigned long long word;
                    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(word) : "l"(slot) : "memory");
                    bits[r] = (uint32_t)word;
                    tag[r] = (uint32_t)(word >> 32);
                }
#pragma unroll
            for (uint32_t r = 0; r < TP_MAX_WORLD; ++r)
                if ((pending >> r & 1u) && (tag[r] == e || lost)) pending &= ~(1u << r);
            if (pending && (spin & 63u) == 63u) {
                const uint64_t now = global_timer_ns();
                if (t0 == 0) t0 = now;
                else if (now - t0 > 1000000000ull) {
                    atomicOr(status, STATUS_TIMEOUT_PEER);
                    lost = true;
                }
            }
        }
        float sum = 0.f;
#pragma unroll
        for (uint32_t r = 0; r < TP_MAX_WORLD; ++r)
            if (r < c.world) sum = __fadd_rn(sum, __uint_as_float(bits[r]));
        out[row] = sum;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t* ctl = reinterpret_cast<uint32_t*>(c.buf[c.rank]);
        if (atomicAdd(ctl + 1, 1u) == gridDim.x - 1) {  // the CTA that finishes last closes the epoch
            ctl[1] = 0;
            ctl[0] = e;
        }
    }
}

// ------------------------------------------------------------------- shared-memory loads
// Plain C++ loads (not asm) so the compiler can schedule them freely between the barrier
// operations, whose asm statements carry memory clobbers.

__device__ __forceinline__ uint32_t lds32(const uint8_t* a) { return *reinterpret_cast<const uint32_t*>(a); }
__device__ __forceinline__ uint2 lds64(const uint8_t* a) { return *reinterpret_cast<const uint2*>(a); }
__device__ __forceinline__ uint4 lds128(const uint8_t* a) { return *reinterpret_cast<const uint4*>(a); }
__device__ __forceinline__ uint32_t lds16(const uint8_t* a) { return *reinterpret_cast<const unsigned short*>(a); }
// 32-bit word at a 2-byte-aligned shared address.
__device__ __forceinline__ uint32_t lds32_u(const uint8_t* a) {
    const uintptr_t v = reinterpret_cast<uintptr_t>(a);
    const uint32_t* base = reinterpret_cast<const uint32_t*>(v & ~(uintptr_t)3);
    return __funnelshift_r(base[0], base[1], (uint32_t)(v & 3u) * 8u);
}

// The same loads through 32-bit shared-window addresses (ld.shared): no 64-bit generic address arithmetic.
// volatile keeps them in program order relative to the barrier waits (also volatile); it does not
// stop the assembler from overlapping them.
__device__ __forceinline__ uint32_t sld32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t sld16(uint32_t a) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 sld64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 sld128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
// 32-bit word at a 2-byte-aligned shared address
__device__ __forceinline__ uint32_t sld32_u(uint32_t a) {
    const uint32_t base = a & ~3u;
    return __funnelshift_r(sld32(base), sld32(base + 4), (a & 3u) * 8u);
}

// ------------------------------------------------------------------------------- MMA

// D(16x8,s32) = A(16x32,u8,row) * B(32x8,s8,col) + C
__device__ __forceinline__ void mma_u8s8_k32(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1, const int (&c)[4]) {
    asm(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}
// D(16x8,s32) = A(16x32,s8,row) * B(32x8,s8,col) + C
__device__ __forceinline__ void mma_s8s8_k32(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1, const int (&c)[4]) {
    asm(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}
// D(16x8,s32) = A(16x16,s8,row) * B(16x8,s8,col) + C
__device__ __forceinline__ void mma_s8s8_k16(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0, const int (&c)[4]) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}
// D(16x8,s32) = A(16x16,u8,row) * B(16x8,u8,col) + C
__device__ __forceinline__ void mma_u8u8_k16(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0, const int (&c)[4]) {
    asm("mma.sync.aligned.m16n8k16.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}
// D(16x8,f32) = A(16x16,f16,row) * B(16x8,f16,col) + C
__device__ __forceinline__ void mma_f16_k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                            uint32_t b1, const float (&c)[4]) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

// ---------------------------------------------------------------------------- numerics

__device__ __forceinline__ float f16bits_to_f32(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a & mask) | orv
    return r;
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

}  // namespace b200q
