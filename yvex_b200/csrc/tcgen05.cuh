// Thin inline-PTX wrappers for the sm_100a features the grouped GEMM uses: mbarriers with
// bounded waits, TMA tiled loads, tcgen05 (TMEM allocation, UMMA issue/commit, TMEM loads) and
// the shared-memory matrix descriptors of the K-major 128-byte-swizzle canonical layout.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace yb {
namespace sm100 {

// Bounded waits: a wait gives up once this much time has passed on the device's nanosecond clock
// (%globaltimer), whatever a single poll costs; the poll count is only a backstop.
constexpr uint64_t kWaitLimitNs = 2000000000ull;
constexpr uint32_t kSpinLimit = 1u << 30;
// Optional suspend-time hint of a try_wait (how long one poll may keep the thread suspended before it
// reports "not yet"). A streaming kernel whose consumers wait on copies for microseconds gives it so that
// its waiting warps leave the issue slots alone; the grouped GEMM, whose two-stage rings turn every
// cycle of wake-up latency into pipeline time, polls without it (measured: 3 % faster).
constexpr uint32_t kTryWaitHintNs = 2000u;

__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}"
                 ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
template <uint32_t kHintNs = 0>
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    if constexpr (kHintNs != 0) {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(kHintNs) : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    }
    return ok != 0;
}
// Waits for the phase with the given parity to complete. Gives up after `limit_ns` (or as soon as
// another thread of the CTA gave up), raising `abort` so every role unwinds.
template <uint32_t kHintNs = 0>
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort,
                                          uint64_t limit_ns = kWaitLimitNs) {
    if (mbar_try_wait<kHintNs>(bar, parity)) return true;
    const uint64_t t0 = global_ns();
    for (uint32_t i = 1; i < kSpinLimit; ++i) {
        if (mbar_try_wait<kHintNs>(bar, parity)) return true;
        if ((i & 63u) == 0u) {
            if (*abort) return false;
            if (global_ns() - t0 > limit_ns) break;
        }
    }
    *abort = 1;
    return false;
}

// The same wait for a whole warp: every lane waits, and all 32 lanes get the same answer, so a warp
// never splits between lanes that saw the phase complete and lanes that gave up (the code after
// such waits uses warp-wide synchronising instructions). (Every lane polls: a wait by one elected
// lane with the answer broadcast measured 60 % slower in the grouped GEMM.)
template <uint32_t kHintNs = 0>
__device__ __forceinline__ bool mbar_wait_warp(uint64_t *bar, uint32_t parity, volatile int *abort,
                                               uint64_t limit_ns = kWaitLimitNs) {
    return __all_sync(0xffffffffu, mbar_wait<kHintNs>(bar, parity, abort, limit_ns)) != 0;
}

// generic-proxy writes (st.shared) -> visible to the async proxy (UMMA / TMA reads)
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// Untiled bulk copy global -> shared: both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- tensor memory ---------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t columns) {      // one full warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(columns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {        // same warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// mbarrier arrives once every previously issued UMMA of this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem], fp16 inputs, f32 accumulate, M=128, N from the instruction
// descriptor, K=16 per instruction. One thread issues.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns: thread i of the warp gets lane (32*(warp%4) + i).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Instruction descriptor: kind::f16, A = B = fp16, D = f32, both operands K-major, M = 128.
__host__ __device__ constexpr uint32_t idesc_f16(uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

// Shared-memory matrix descriptor, K-major, 128-byte swizzle: rows of 128 bytes, 8-row atoms 1024
// bytes apart (stride byte offset), descriptor version 1 (Blackwell). `byte_offset` advances
// along K inside the swizzled row (32 bytes per K=16 step).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
    return static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}

// Byte offset of 16-byte chunk `c` (0..7) of row `r` inside a K-major SW128 tile (64 fp16 per row).
__device__ __forceinline__ uint32_t sw128_offset(uint32_t r, uint32_t c) { return r * 128u + ((c ^ (r & 7u)) << 4); }

}  // namespace sm100
}  // namespace yb
