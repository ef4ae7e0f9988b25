// gemm_sm100_2sm.cuh - the persistent bf16 GEMM main loop on CTA pairs (tcgen05 cta_group::2).
//
// Two CTAs on neighbouring SMs form a cluster and compute one 256 x 256 tile together:
//   * CTA r of the pair loads rows [r*128, r*128+128) of the A tile and rows [r*128, r*128+128) of the B tile
//     (half of the 256 output columns) - 32 KB per CTA and k-block instead of the 48 KB a lone CTA needs for a
//     128 x 256 tile, so the operand traffic L2 -> shared memory per FLOP drops by a third and the ring holds six
//     stages instead of four;
//   * one thread of the leader CTA (cluster rank 0) issues tcgen05.mma.cta_group::2 with M = 256: each SM's tensor
//     core produces its own 128 accumulator rows in its own tensor memory and reads the other half of B from the
//     peer's shared memory;
//   * all four TMA loads of a stage complete on the LEADER's "full" mbarrier (loads carry .cta_group::2, which
//     allows the barrier to live in the peer CTA; no load carries a multicast qualifier);
//   * tcgen05.commit with a two-CTA mask releases the stage ("empty") and publishes the accumulator
//     ("tmemFull") in both CTAs at once; the epilogue warps of both CTAs hand the accumulator back on the
//     leader's "tmemEmpty" barrier (remote mbarrier arrive for the peer).
// Policies (TileOrder, Epilogue) are the ones of gemm_sm100.cuh; tile row blocks here are 256 rows tall.
// Every wait is bounded; the CTAs of a pair always meet at the final cluster barrier before either exits.
#pragma once
#include "gemm_sm100.cuh"

namespace hcgemm {

constexpr int kPairM = 256;

constexpr int kStagingBytesPerWarp = 32 * 128 * 2;      // 32 rows x 128 bf16 columns
constexpr int kStagingBytes = 4 * kStagingBytesPerWarp;  // one slab per epilogue warp

// BN: width of the pair's tile, a multiple of 32 between 128 and 256 (each CTA holds BN / 2 rows of B, whole 8-row
// swizzle groups, and the epilogue reads 32 columns at a time).  Widths below 256 exist for the tail: a problem whose
// tile count at 256 columns leaves most of the last wave idle runs faster on narrower tiles.
template <int BN, int STAGES = 6, bool STAGING = false, int EXTRA = 0> struct Config2 {
    static_assert(BN % 32 == 0 && BN >= 128 && BN <= 256, "tile widths: 128, 160, 192, 224, 256");
    static_assert(STAGES >= 2 && STAGES <= 8, "the ring must fit 227 KB of shared memory and the 8-entry barrier arrays");
    static_assert(!STAGING || BN % 128 == 0, "the staged epilogue sends 128-column slabs");
    static constexpr int kStages = STAGES;
    static constexpr int kStaging = STAGING ? kStagingBytes : 0;
    static constexpr int kABytes = kBlockM * kBlockK * 2;          // 128 rows of A per CTA
    static constexpr int kBBytes = (BN / 2) * kBlockK * 2;         // 128 of the 256 B rows per CTA
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemCols = 2 * BN <= 256 ? 256 : 512;    // two accumulators; allocations are powers of two
    static constexpr int kExtra = EXTRA;                           // shared memory of the Extra policy
    static constexpr int kSmemBytes = kStages * kStageBytes + kStaging + kExtra + 1024 + 256;
    static_assert(kSmemBytes <= 227 * 1024, "shared memory per CTA");
};

// Epilogue policies without a staged path.
struct NoStaging { static constexpr bool kStaged = false; };

namespace pair {

__device__ __forceinline__ uint32_t ClusterCtaRank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t ClusterId()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t NumClusters()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void ClusterSync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `p` (a shared-memory object of this CTA) as seen in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t MapToCta(const void *p, uint32_t rank)
{
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(SmemAddr(p)), "r"(rank));
    return out;
}
__device__ __forceinline__ void RemoteArrive(uint32_t clusterAddr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(clusterAddr) : "memory");
}
// 2-D tiled load into this CTA's shared memory; completion is signalled on `barClusterAddr`, which may be the
// leader CTA's barrier.
__device__ __forceinline__ void TmaLoad2dPair(void *smemDst, const CUtensorMap *m, uint32_t barClusterAddr, int32_t x, int32_t y)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(SmemAddr(smemDst)), "l"(m), "r"(barClusterAddr), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void TmemAlloc2(uint32_t *smemResult, uint32_t nCols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(smemResult)), "r"(nCols) : "memory");
}
__device__ __forceinline__ void TmemRelinquish2() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void TmemDealloc2(uint32_t taddr, uint32_t nCols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(nCols) : "memory");
}
__device__ __forceinline__ void MmaBf16Pair(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, bool accumulate)
{
    uint32_t acc = accumulate ? 1u : 0u;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmemD), "l"(descA), "l"(descB), "r"(idesc), "r"(acc) : "memory");
}
// Arrives on the barrier at this shared-memory offset in BOTH CTAs once all MMAs issued so far have finished.
__device__ __forceinline__ void MmaCommitPair(uint64_t *bar)
{
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(SmemAddr(bar)), "h"(mask) : "memory");
}

// Epilogue staging: a warp parks 32 rows x 128 bf16 columns (256 bytes per row) in shared memory so that the rows
// can leave as whole 256-byte segments - two rows per warp store - instead of 16-byte pieces at a row stride.
// 16-byte chunks are XOR-swizzled with the row so that neither the row-wise writes nor the segment-wise reads pile
// up on the same banks.
__device__ __forceinline__ void StagePut(uint8_t *slab, int row, int chunk, uint4 v)
{
    *(uint4 *)(slab + row * 256 + ((chunk ^ (row & 15)) << 4)) = v;
}
__device__ __forceinline__ uint4 StageGet(const uint8_t *slab, int row, int chunk)
{
    return *(const uint4 *)(slab + row * 256 + ((chunk ^ (row & 15)) << 4));
}
// Writes the slab to dst[row * pitchBytes + 0..255] for rows 0..31 (dst may be peer memory).
__device__ __forceinline__ void StageFlushRows(const uint8_t *slab, char *dst, size_t pitchBytes, int lane)
{
    const int chunk = lane & 15, half = lane >> 4;
#pragma unroll 4
    for (int it = 0; it < 16; ++it) {
        const int row = it * 2 + half;
        *(uint4 *)(dst + (size_t)row * pitchBytes + (chunk << 4)) = StageGet(slab, row, chunk);
    }
}

}  // namespace pair

// Writes bf16 rows of C through the per-warp slab: every warp store covers two 256-byte row segments.
// For shapes whose tiles are complete (M a multiple of 256, N a multiple of 256).
struct StoreBf16Staged {
    static constexpr bool kStaged = true;
    static constexpr bool kReportsTiles = false;
    __nv_bfloat16 *C;
    int ldc;
    __device__ __forceinline__ bool StagedTile(int) const { return true; }
    __device__ __forceinline__ void BeginTile(int, int, int) const {}
    __device__ __forceinline__ void EndTile(int, int, int) const {}
    __device__ __forceinline__ void Fragment(int, int, int, int, const uint32_t (&)[32]) const {}
    __device__ __forceinline__ void StoreStaged(int, int, int rowBase, int colBase, const uint8_t *slab, int lane) const
    {
        pair::StageFlushRows(slab, (char *)(C + (size_t)rowBase * ldc + colBase), (size_t)ldc * sizeof(__nv_bfloat16), lane);
    }
};

// g.tilesM counts 256-row blocks here.  Launch with a cluster of two CTAs along x and an even grid.
// The Gate policy is asked per CTA with the index of the 128-row block that CTA loads (2 * mb + cluster rank).
template <int BN, int STAGES, typename TileOrder, typename Epilogue, typename Gate = NoGate, typename Extra = NoExtra>
__device__ __forceinline__ void GemmMainLoopPair(const CUtensorMap *tmA, const CUtensorMap *tmB, const GemmShape &g, TileOrder order, Epilogue epi,
                                                 Gate gate = Gate(), const CUtensorMap *tmA2 = nullptr, Extra extra = Extra())
{
    using Cfg = Config2<BN, STAGES, Epilogue::kStaged, Extra::kSmemBytes>;
    using namespace pair;
    extern __shared__ uint8_t smemRaw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smemRaw + 1023) & ~(uintptr_t)1023);
    uint8_t *staging = smem + Cfg::kStages * Cfg::kStageBytes;
    uint8_t *extraSmem = staging + Cfg::kStaging;
    SharedState *st = (SharedState *)(extraSmem + Cfg::kExtra);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t ctaRank = ClusterCtaRank();
    const bool leader = ctaRank == 0;
    const int numTiles = g.tilesM * g.tilesN;
    const int kBlocks = (g.K + kBlockK - 1) / kBlockK;
    const int firstTile = (int)ClusterId(), tileStep = g.clusters > 0 ? g.clusters : (int)NumClusters();

    if (threadIdx.x == 0) {
        if (g.phase) g.phase[(size_t)blockIdx.x * kPhaseSlots + kPhaseStart] = GlobalTimer();
        for (int s = 0; s < Cfg::kStages; ++s) { MbarInit(&st->full[s], 1); MbarInit(&st->empty[s], 1); }
        for (int a = 0; a < 2; ++a) { MbarInit(&st->tmemFull[a], 1); MbarInit(&st->tmemEmpty[a], 8); }   // 4 epilogue warps x 2 CTAs
        st->abort = 0;
        for (int i = 0; i < Cfg::kExtra / 4; ++i) ((volatile uint32_t *)extraSmem)[i] = 0;
        MbarFenceInit();
        TmaPrefetchDescriptor(tmA);
        TmaPrefetchDescriptor(tmB);
    }
    if (warp == 1) {
        TmemAlloc2(&st->tmemBase, Cfg::kTmemCols);
        TmemRelinquish2();
    }
    TcFenceBefore();
    __syncthreads();
    ClusterSync();          // the peer's barriers are initialised before anything signals them
    TcFenceAfter();
    const uint32_t tmemBase = st->tmemBase;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (ElectOne()) {
            uint32_t it = 0;
            bool alive = true;
            for (int t = firstTile; t < numTiles && alive; t += tileStep) {
                int mb, nb;
                order(t, g, &mb, &nb);
                const int mb128 = mb * 2 + (int)ctaRank;
                int aRow = mb128 * kBlockM;
                const CUtensorMap *mapA = tmA;
                if (!gate(mb128, nb, &st->abort, &aRow, tmA, tmA2, &mapA)) { alive = false; break; }
                const int bRow = nb * BN + (int)ctaRank * (BN / 2);
                for (int kb = 0; kb < kBlocks; ++kb, ++it) {
                    const int s = it % Cfg::kStages;
                    const uint32_t ph = (it / Cfg::kStages) & 1;
                    if (!MbarWait(&st->empty[s], ph ^ 1, &st->abort)) { alive = false; break; }
                    uint8_t *sa = smem + s * Cfg::kStageBytes, *sb = sa + Cfg::kABytes;
                    if (leader) MbarExpectTx(&st->full[s], 2 * Cfg::kStageBytes);      // both CTAs' loads land on this barrier
                    const uint32_t bar = MapToCta(&st->full[s], 0);
                    TmaLoad2dPair(sa, mapA, bar, kb * kBlockK, aRow);
                    TmaLoad2dPair(sb, tmB, bar, kb * kBlockK, bRow);
                }
            }
            // After a wait that ran out, copies already issued still write into this CTA's shared memory.  They take
            // microseconds; the CTA stays for a fixed, much longer time before it goes on to the exit barrier.
            if (!alive) __nanosleep(500000);
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------------- MMA issuer (leader CTA only)
        if (leader && ElectOne()) {
            constexpr uint32_t idesc = InstrDescBf16(kPairM, BN);
            uint32_t it = 0, tileIter = 0;
            bool alive = true;
            for (int t = firstTile; t < numTiles && alive; t += tileStep, ++tileIter) {
                const uint32_t acc = tileIter & 1, accPh = (tileIter >> 1) & 1;
                if (!MbarWait(&st->tmemEmpty[acc], accPh ^ 1, &st->abort)) { alive = false; break; }
                TcFenceAfter();
                const uint32_t tmemD = tmemBase + acc * BN;
                for (int kb = 0; kb < kBlocks; ++kb, ++it) {
                    const int s = it % Cfg::kStages;
                    const uint32_t ph = (it / Cfg::kStages) & 1;
                    if (!MbarWait(&st->full[s], ph, &st->abort)) { alive = false; break; }
                    TcFenceAfter();
                    uint8_t *sa = smem + s * Cfg::kStageBytes, *sb = sa + Cfg::kABytes;
                    const uint64_t da = SmemDescKMajorSw128(sa), db = SmemDescKMajorSw128(sb);
#pragma unroll
                    for (int k = 0; k < kBlockK / kUmmaK; ++k) MmaBf16Pair(tmemD, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0);
                    MmaCommitPair(&st->empty[s]);
                }
                if (alive) MmaCommitPair(&st->tmemFull[acc]);
            }
        }
    } else if (warp >= 6) {
        // -------------------------------------------------- extra warps (communication roles of fused kernels)
        extra(warp - 6, lane, &st->abort, extraSmem);
    } else {
        // ---------------------------------------------------------------------- epilogue (both CTAs)
        const int q = warp & 3;
        uint32_t tileIter = 0;
        bool alive = true;
        for (int t = firstTile; t < numTiles && alive; t += tileStep, ++tileIter) {
            int mb, nb;
            order(t, g, &mb, &nb);
            const uint32_t acc = tileIter & 1, accPh = (tileIter >> 1) & 1;
            if (g.phase && q == 0 && lane == 0) {
                // phase clock: time this CTA's epilogue spent waiting for an accumulator (main loop or its inputs late)
                const uint64_t t0 = GlobalTimer();
                const bool ok = MbarWait(&st->tmemFull[acc], accPh, &st->abort);
                g.phase[(size_t)blockIdx.x * kPhaseSlots + kPhaseAccWait] += GlobalTimer() - t0;
                if (!ok) st->abort = 1;
            }
            if (!MbarWait(&st->tmemFull[acc], accPh, &st->abort)) { alive = false; break; }
            TcFenceAfter();
            const int row = mb * kPairM + (int)ctaRank * kBlockM + q * 32 + lane;
            epi.BeginTile(mb, nb, row);
            bool staged = false;
            if constexpr (Epilogue::kStaged) staged = epi.StagedTile(mb);
            if (staged) {
                if constexpr (Epilogue::kStaged) {
                    uint8_t *slab = staging + q * kStagingBytesPerWarp;
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 128) {
#pragma unroll 1
                        for (int c = 0; c < 128; c += 32) {
                            uint32_t frag[32];
                            TmemLoad32x32(tmemBase + ((uint32_t)(q * 32) << 16) + acc * BN + c0 + c, frag);
                            TmemLoadWait();
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                uint4 pk;
                                uint32_t *pw = (uint32_t *)&pk;
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(frag[v * 8 + 2 * j]), __uint_as_float(frag[v * 8 + 2 * j + 1]));
                                    pw[j] = *(uint32_t *)&h;
                                }
                                StagePut(slab, lane, (c >> 3) + v, pk);
                            }
                        }
                        __syncwarp();
                        epi.StoreStaged(mb, nb, row - lane, nb * BN + c0, slab, lane);
                        __syncwarp();
                    }
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t frag[32];
                    TmemLoad32x32(tmemBase + ((uint32_t)(q * 32) << 16) + acc * BN + c, frag);
                    TmemLoadWait();
                    epi.Fragment(mb, nb, row, nb * BN + c, frag);
                }
            }
            TcFenceBefore();
            __syncwarp();
            if (lane == 0) {
                if (leader) MbarArrive(&st->tmemEmpty[acc]);
                else RemoteArrive(MapToCta(&st->tmemEmpty[acc], 0));
            }
            epi.EndTile(mb, nb, row);
            // epilogues that leave the publication of their tiles to another warp count them here
            if constexpr (Epilogue::kReportsTiles) epi.TileDone(q, tileIter + 1, extraSmem, lane);
        }
    }
    // Nobody leaves while the peer may still read this CTA's shared memory, signal its barriers or use its
    // tensor memory: both CTAs meet here, also after a wait that ran out.
    TcFenceBefore();
    __syncthreads();
    ClusterSync();
    if (warp == 1) TmemDealloc2(tmemBase, Cfg::kTmemCols);
    if (threadIdx.x == 0 && st->abort && g.errFlag) atomicExch(g.errFlag, 1u);
    if (threadIdx.x == 0 && g.phase) g.phase[(size_t)blockIdx.x * kPhaseSlots + kPhaseEnd] = GlobalTimer();
}

}  // namespace hcgemm
