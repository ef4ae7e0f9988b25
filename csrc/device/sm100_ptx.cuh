// sm100_ptx.cuh - thin inline-PTX wrappers for the Blackwell (sm_100a) tensor path:
// mbarrier, TMA tiled loads/stores (cp.async.bulk.tensor), tensor memory management and the
// tcgen05 MMA / load / commit instructions, plus the shared-memory and instruction descriptors.
//
// Conventions used by every kernel built on this header
//   * one elected thread issues TMA and tcgen05.mma; completion is tracked with mbarriers;
//   * every wait is bounded: MbarWait returns false after kSpinLimit polls, the caller then raises
//     the kernel's error flag, stops issuing work, still frees its tensor memory and returns;
//   * TMA loads never carry a cluster-multicast qualifier and only ever read this GPU's memory.
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace sm100 {

constexpr uint32_t kSpinLimit = 1u << 26;   // polls before a wait is declared dead (seconds, not minutes)

__device__ __forceinline__ uint32_t SmemAddr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool ElectOne()
{
    uint32_t pred = 0;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// ---------------------------------------------------------------------------------- mbarrier

__device__ __forceinline__ void MbarInit(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void MbarFenceInit() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void MbarExpectTx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SmemAddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void MbarArrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(SmemAddr(bar)) : "memory");
}
__device__ __forceinline__ bool MbarTryWait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(SmemAddr(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  `abortFlag` (shared memory) lets one failed role stop the others quickly.
__device__ __forceinline__ bool MbarWait(uint64_t *bar, uint32_t parity, volatile uint32_t *abortFlag)
{
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (MbarTryWait(bar, parity)) return true;
        if ((i & 1023) == 1023 && *abortFlag) return false;
    }
    *abortFlag = 1;
    return false;
}

// --------------------------------------------------------------------------------------- TMA

__device__ __forceinline__ void TmaPrefetchDescriptor(const CUtensorMap *m)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
// 2-D tiled load global -> shared; x is the innermost (contiguous) coordinate and must be a multiple of
// 16 bytes worth of elements.
__device__ __forceinline__ void TmaLoad2d(void *smemDst, const CUtensorMap *m, uint64_t *bar, int32_t x, int32_t y)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(SmemAddr(smemDst)), "l"(m), "r"(SmemAddr(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void TmaStore2d(const CUtensorMap *m, const void *smemSrc, int32_t x, int32_t y)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(m), "r"(SmemAddr(smemSrc)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void TmaStoreCommit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void TmaStoreWaitRead() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N> __device__ __forceinline__ void TmaStoreWait() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void FenceProxyAsyncShared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ------------------------------------------------------------------------------ tensor memory

// Allocates nCols (power of two, 32..512) columns; the base address lands in *smemResult.  Warp-wide.
__device__ __forceinline__ void TmemAlloc(uint32_t *smemResult, uint32_t nCols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(smemResult)), "r"(nCols) : "memory");
}
__device__ __forceinline__ void TmemRelinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void TmemDealloc(uint32_t taddr, uint32_t nCols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(nCols) : "memory");
}
__device__ __forceinline__ void TcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void TcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ------------------------------------------------------------------------------- descriptors

// Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128 bytes with the
// 128-byte swizzle TMA applies (8-row groups are 1024 bytes apart).
__device__ __forceinline__ uint64_t SmemDescKMajorSw128(const void *smemTile)
{
    uint64_t d = 0;
    d |= (uint64_t)((SmemAddr(smemTile) & 0x3FFFF) >> 4);        // start address, 16-byte units
    d |= (uint64_t)1 << 16;                                      // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                            // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                                      // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                                      // layout: 128-byte swizzle
    return d;
}
// Instruction descriptor, kind::f16: bf16 x bf16 -> fp32, both operands K-major, tile M x N.
__host__ __device__ constexpr uint32_t InstrDescBf16(uint32_t M, uint32_t N)
{
    return (1u << 4) /* D fp32 */ | (1u << 7) /* A bf16 */ | (1u << 10) /* B bf16 */ | ((N >> 3) << 17) | ((M >> 4) << 24);
}
// kind::f8f6f4 with e4m3 operands (format code 0) and fp32 accumulation.
__host__ __device__ constexpr uint32_t InstrDescE4m3(uint32_t M, uint32_t N)
{
    return (1u << 4) | (0u << 7) | (0u << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
__device__ __forceinline__ void MmaBf16(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, bool accumulate)
{
    uint32_t acc = accumulate ? 1u : 0u;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void MmaF8(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, bool accumulate)
{
    uint32_t acc = accumulate ? 1u : 0u;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(acc) : "memory");
}
// Makes the mbarrier complete once all MMAs issued so far by this thread have finished.
__device__ __forceinline__ void MmaCommit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(SmemAddr(bar)) : "memory");
}

// Reads 32 consecutive fp32 columns of this warp's 32 lanes: thread l gets row (laneBase + l).
__device__ __forceinline__ void TmemLoad32x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void TmemLoadWait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace sm100
