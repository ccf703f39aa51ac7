// tc5.cuh - the pieces of a tcgen05 (5th-generation tensor core) kernel that its users share: mbarriers with time-bounded
// waits, K-major 128-byte-swizzled shared-memory operand descriptors, the kind::f16 MMA and its commit, tensor-memory loads.
#pragma once
#include <cstdint>

#include "common.cuh"

namespace bsx {

constexpr unsigned long long kWaitNs = 200ull * 1000 * 1000;   // every mbarrier wait gives up after 200 ms; the caller reports it

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("{\n.reg .b64 st;\nmbarrier.arrive.shared::cta.b64 st, [%0];\n}\n" ::"r"(smem_u32(bar)) : "memory");
}
// Waits for the phase with the given parity, at most kWaitNs of wall time; false when it gave up.  A few non-blocking polls
// first (the common case: the phase completes within a microsecond), then try_wait with a suspend-time hint: the hardware parks
// the thread and wakes it when the phase completes - no sleep granularity between the completion and the waiter - or after the
// hint at the latest, and the clock is read between two such waits, so the bound is the clock's and every single wait is short.
constexpr uint32_t kWaitHintNs = 4000;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t a = smem_u32(bar);
    uint32_t ok;
#pragma unroll 1
    for (int i = 0; i < 16; ++i) {
        asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok)
                     : "r"(a), "r"(parity)
                     : "memory");
        if (ok) return true;
    }
    unsigned long long t0;
    asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t0));
    for (;;) {
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok)
                     : "r"(a), "r"(parity), "r"(kWaitHintNs)
                     : "memory");
        if (ok) return true;
        unsigned long long now;
        asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(now));
        if (now - t0 > kWaitNs) return false;
    }
}

// K-major, 128-byte swizzle: 8-row atoms of 1024 bytes stacked along M/N (stride byte offset 1024), descriptor version 1
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    return (uint64_t) ((addr & 0x3FFFFu) >> 4) | ((uint64_t) 1 << 16) | ((uint64_t) (1024 >> 4) << 32) | ((uint64_t) 1 << 46) |
           ((uint64_t) 2 << 61);
}
// kind::f16 instruction descriptor: D fp32, A and B fp16, both K-major, M x N
__host__ __device__ constexpr uint32_t instr_desc_f16(int m, int n) { return (1u << 4) | ((uint32_t) (n >> 3) << 17) | ((uint32_t) (m >> 4) << 24); }

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d), "l"(adesc),
                 "l"(bdesc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    __syncwarp();   // the load is warp-wide: all 32 lanes must arrive together
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
        "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]),
          "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    __syncwarp();
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

// position of column c inside its 16-column group in the permuted k order (0,8,1,9,...,7,15) both operands are stored in
__host__ __device__ constexpr int perm16(int j) { return 2 * (j & 7) + (j >> 3); }

}  // namespace bsx
