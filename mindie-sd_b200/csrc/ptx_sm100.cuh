// Thin inline-PTX wrappers for the sm_100a features the attention kernels use:
// mbarriers, TMA tiled loads, tensor memory (TMEM) management, tcgen05 MMA / load / store.
// Every wait is bounded in time: a wait that gives up returns false and the caller unwinds.
#pragma once
#include <cuda_runtime.h>
#include <cuda.h>
#include <cstdint>

namespace sdb {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ----------------------------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Time limit of a bounded wait.  The longest legitimate wait inside these kernels is that of the
// warps of an idle query tile, which sit on one barrier for the whole life of their thread block:
// tens of milliseconds at the largest sizes and the lowest clocks.  One second is far beyond that
// and short enough that a grid of stuck thread blocks drains at once (the blocks that are resident
// give up together; the ones that start afterwards see the status word and leave).
constexpr uint32_t kWaitLimitUs = 1000000u;

// Waits for the phase with the given parity, for at most limit_us microseconds of wall-clock time
// (the nanosecond timer of the device, which does not depend on the SM clock).  Returns false if
// the wait gave up (limit reached, or another role of the thread block raised the abort flag); the
// first to give up raises the flag and leaves `site` (a small number naming the wait) next to it.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int site = 0,
                                          uint32_t limit_us = kWaitLimitUs) {
    // Kept small on purpose: this is inlined in front of every barrier wait of the kernels, and their hot
    // loops measured 5 % slower with one more polling loop here.  (Each attempt suspends the thread for a
    // hardware-chosen while by itself; the timer and the flag are looked at every 64 attempts.)
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    for (uint32_t i = 1;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 0u) {
            if (*abort_flag) return false;
            if (global_timer_ns() - t0 > static_cast<uint64_t>(limit_us) * 1000u) break;
        }
    }
    if (*abort_flag == 0) abort_flag[1] = site;
    *abort_flag = 1;
    return false;
}

// The wait of a thread that must see its own asynchronous copies land before the thread block may
// exit: it does not look at the abort flag (the copies are in flight whatever the other roles
// decided) and is bounded by time alone.
__device__ __forceinline__ bool mbar_wait_drain(uint32_t bar, uint32_t parity, uint32_t limit_us = kWaitLimitUs) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    for (uint32_t i = 1;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 0u && global_timer_ns() - t0 > static_cast<uint64_t>(limit_us) * 1000u) return false;
    }
}

// ----------------------------------------------------------------------------------------------
// TMA (tiled bulk tensor loads, each CTA fetching its own tiles)
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int c0, int c1,
                                            int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
// ----------------------------------------------------------------------------------------------
// Tensor memory
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane (base+i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
          "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
          "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
        : "memory");
}

// ----------------------------------------------------------------------------------------------
// tcgen05.mma (one CTA, issued by a single thread) and its completion signal
// ----------------------------------------------------------------------------------------------
// D[tmem] (+)= A * B with A from shared memory (ss) or tensor memory (ts) and B from shared memory.
// Descriptors are given as (low word, high word) pairs.  The thread that
// issues the MMAs runs alone, so every scalar instruction between two MMAs is exposed latency:
// callers keep the high word constant and derive the low word (start address field) with one add.
template <bool kFp8>
__device__ __forceinline__ void umma_ss_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi,
                                             uint32_t idesc, uint32_t accumulate) {
    if constexpr (kFp8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
            "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\tsetp.ne.b32 p, %5, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %4, p;\n\t}"
            ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
            "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\tsetp.ne.b32 p, %5, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
            ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}
template <bool kFp8>
__device__ __forceinline__ void umma_ts_lohi(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t hi,
                                             uint32_t idesc, uint32_t accumulate) {
    if constexpr (kFp8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
            "mov.b64 db, {%2, %3};\n\tsetp.ne.b32 p, %5, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], db, %4, p;\n\t}"
            ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
            "mov.b64 db, {%2, %3};\n\tsetp.ne.b32 p, %5, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
            ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}
// Shared-memory matrix descriptor of a 128-byte-swizzled operand tile, as low and high word.
//   bits  0..13  start address >> 4        bits 16..29  leading byte offset >> 4
//   bits 32..45  stride byte offset >> 4   bit 46 descriptor version   bits 61..63  2 = 128-byte swizzle
//   K-major  (rows of 128 B along the contraction dim): lbo unused (16), sbo = bytes between 8-row groups.
//   MN-major (rows of 128 B along the M/N dim): lbo = bytes between 128-B column groups,
//                                               sbo = bytes between 8-row (K) groups.
// sbo is 1024 for every operand tile of these kernels, so one high word serves them all.
__device__ __forceinline__ uint32_t desc_lo(uint32_t addr, uint32_t lbo_bytes) {
    return ((addr & 0x3FFFFu) >> 4) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
constexpr uint32_t kDescHiSbo1024 = (1024u >> 4) | (1u << 14) | (2u << 29);

// The mbarrier receives one arrival once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// Instruction descriptor: fp32 accumulate, A and B of one operand format, M x N tile.
//   fmt: kind::f16 -> 0 fp16, 1 bf16; kind::f8f6f4 -> 0 e4m3, 1 e5m2.
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t fmt, uint32_t m, uint32_t n, bool a_mn_major,
                                                  bool b_mn_major) {
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(a_mn_major) << 15) |
           (static_cast<uint32_t>(b_mn_major) << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Packed pairs of fp32 values in one 64-bit register: the f32x2 arithmetic of this architecture
// issues one instruction for two lanes' worth of work.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// 2^x for a packed pair on the FMA and integer pipes, leaving the exponent unit (16 results per clock
// per SM) to other values: x = n + f with n = round(x) taken from the low mantissa bits of x + 1.5 * 2^23,
// a cubic for 2^f on [-0.5, 0.5] (relative error 7.5e-5, well inside the rounding of a two-byte or
// e4m3 probability), and n added to the exponent field.  x is clamped to [lo, hi] inside [-125, 126]
// so that the exponent arithmetic cannot wrap; -inf (a masked score) gives 2^lo, i.e. nothing.
template <bool kClampHigh>
__device__ __forceinline__ void ex2_poly2(uint64_t x2, float& e0, float& e1) {
    float x0, x1;
    unpack2(x2, x0, x1);
    x0 = fmaxf(x0, -125.0f);
    x1 = fmaxf(x1, -125.0f);
    if constexpr (kClampHigh) {
        x0 = fminf(x0, 126.0f);
        x1 = fminf(x1, 126.0f);
    }
    const uint64_t x = pack2(x0, x1);
    const uint64_t magic = pack2(12582912.0f, 12582912.0f);
    const uint64_t t = add2(x, magic);
    const uint64_t f = sub2(x, sub2(t, magic));
    uint64_t p = fma2(pack2(0.055171650f, 0.055171650f), f, pack2(0.24261113f, 0.24261113f));
    p = fma2(p, f, pack2(0.69326097f, 0.69326097f));
    p = fma2(p, f, pack2(0.99992806f, 0.99992806f));
    uint32_t plo, phi, tlo, thi;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(plo), "=r"(phi) : "l"(p));
    asm("mov.b64 {%0, %1}, %2;" : "=r"(tlo), "=r"(thi) : "l"(t));
    e0 = __uint_as_float(plo + (tlo << 23));
    e1 = __uint_as_float(phi + (thi << 23));
}

// Three-input maximum (one instruction on this architecture).
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace sdb
