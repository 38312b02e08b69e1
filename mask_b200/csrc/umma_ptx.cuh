// Inline-PTX helpers shared by the tcgen05 / tensor-memory kernels: mbarriers with bounded waits,
// shared-memory matrix descriptors, the TF32 MMA, its commit, tensor-memory loads and cp.async.
#pragma once

#include "spmm_common.cuh"

namespace mask {

constexpr long long kUmmaWaitCycles = 2000000000LL;   // bound of every wait: about a second of SM clock
constexpr uint32_t kUmmaSuspendHintNs = 20000;   // upper bound of one try_wait's sleep; completion of the phase wakes the thread at once

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// try_wait parks the thread in hardware until the phase completes or a short, implementation-defined
// time slice ends, so a waiting warp costs almost no issue slots (a test_wait spin loop here made the
// idle epilogue warps execute as many instructions as the whole kernel needs).
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(kUmmaSuspendHintNs)
        : "memory");
    return ok != 0;
}
// Non-suspending probe of a phase (one instruction, returns at once).
__device__ __forceinline__ bool mbar_probe(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: false if the block is aborting (this wait or somebody else's ran out of time).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_test(bar, parity)) return true;
    const long long start = clock64();
    while (true) {
        if (mbar_test(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - start > kUmmaWaitCycles) {
            *abort_flag = 1;
            return false;
        }
    }
}
// Bounded wait that spins on the probe instead of letting the hardware park the thread: the lowest
// wake-up latency, at the price of issue slots; for the one thread that paces a block.
__device__ __forceinline__ bool mbar_wait_spin(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    const long long start = clock64();
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 64; i++)
            if (mbar_probe(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - start > kUmmaWaitCycles) {
            *abort_flag = 1;
            return false;
        }
    }
}

__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t saddr, uint32_t lbo16, uint32_t sbo16, uint32_t layout) {
    // bits [0,14) start address >> 4, [16,30) leading byte offset >> 4, [32,46) stride byte offset >> 4,
    // [46,48) descriptor version (1 on sm_100), [61,64) swizzle mode
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)(lbo16 & 0x3FFF) << 16) | ((uint64_t)(sbo16 & 0x3FFF) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)layout << 61);
}
constexpr uint32_t kSwizzle128B32B = 1, kSwizzle32B = 6;   // 128-byte swizzle with 32-byte base; 32-byte swizzle
// instruction descriptor: D = F32, A = B = TF32, A MN-major, B K-major, N = 16, M = 128
constexpr uint32_t kUmmaIdesc = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | (0u << 16) | ((16u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(kUmmaIdesc), "r"(accumulate)
        : "memory");
}
// The same MMA with each descriptor given as its two 32-bit halves: the low half carries the start
// address (>> 4), so stepping through operands that lie at fixed distances is one 32-bit add.
__device__ __forceinline__ void umma_tf32_split(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                                uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %5, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(kUmmaIdesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void cp16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}


}  // namespace mask
