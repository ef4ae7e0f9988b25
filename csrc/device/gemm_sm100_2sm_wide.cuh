// gemm_sm100_2sm_wide.cuh - the CTA-pair bf16 GEMM main loop with 256 x 512 tiles.
//
// Same machinery as gemm_sm100_2sm.cuh (tcgen05 cta_group::2, loads of both CTAs completing on the leader's barrier,
// two-CTA commits), with a tile twice as wide: every CTA keeps ONE 128 x 512 fp32 accumulator, which is all 512 columns
// of its tensor memory, and holds two 128-row blocks of B per stage (48 KB per stage, four stages).  A k-step is two
// MMAs of N = 256, one per half of the tile's columns.
//
// Why: operand traffic.  A 256 x 256 tile fetches (256 + 256) rows of K per 65536 outputs, a 256 x 512 tile
// (256 + 512) rows per 131072: a quarter less L2 -> shared-memory traffic and fewer panels per wave from DRAM.  On a
// GPU that runs dense bf16 at its power cap that traffic is what sets the clock (ncu on 8192 x 28672 x 8192: the
// 256-wide kernel needs 3.33 M cycles, 99.5 % tensor-pipe activity, 30 GB from L2 and 4.2 - 4.9 GB from DRAM, and ran
// at 1.27 GHz; cuBLAS' kernel of this tile shape 3.40 M cycles, 96 %, 22.5 GB and 2.9 GB, at 1.43 GHz).
// The price: with one accumulator the tensor core waits while the epilogue empties it; the producer keeps loading the
// next tile's first stages meanwhile.  To keep that wait short the accumulator is handed back as soon as its last
// column has been READ: every warp converts 64 columns at a time into a 4 KB shared-memory slab (128-byte rows with
// the 128-byte swizzle, so the row-per-lane writes spread over all banks) and one TMA store per slab carries it to C.
// Stores issued by the lanes themselves (16 bytes per lane at a row stride) kept the load/store unit busy for about a
// tenth of the time of an 8192-deep tile, all of it on the tensor core's critical path.
#pragma once
#include "gemm_sm100_2sm.cuh"

namespace hcgemm {

constexpr int kWideN = 512;
constexpr int kWideThreads = 320;       // producer, MMA issuer and eight epilogue warps: two per 32-lane quarter, one per half of the columns

template <int STAGES = 4> struct ConfigWide {
    static constexpr int kStages = STAGES;
    static constexpr int kABytes = kBlockM * kBlockK * 2;           // 128 rows of A per CTA
    static constexpr int kBBlock = 128 * kBlockK * 2;               // 128 rows of B: this CTA's share of one half of the tile's columns
    static constexpr int kStageBytes = kABytes + 2 * kBBlock;
    static constexpr int kTmemCols = 512;
    static constexpr int kSlabBytes = 32 * 64 * 2;                  // epilogue staging per warp: 32 rows x 64 bf16 columns (128-byte rows)
    static constexpr int kStaging = 8 * kSlabBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + kStaging + 1024 + 256;
    static_assert(kSmemBytes <= 227 * 1024, "shared memory per CTA");
};

// g.tilesM counts 256-row blocks, g.tilesN 512-column blocks; N a multiple of 512.  The B tensor map has 128-row boxes,
// the C tensor map boxes of 32 rows x 64 columns with the 128-byte swizzle.
template <int STAGES, typename TileOrder>
__device__ __forceinline__ void GemmMainLoopPairWide(const CUtensorMap *tmA, const CUtensorMap *tmB, const CUtensorMap *tmC, const GemmShape &g, TileOrder order)
{
    using Cfg = ConfigWide<STAGES>;
    using namespace pair;
    extern __shared__ uint8_t smemRaw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smemRaw + 1023) & ~(uintptr_t)1023);
    uint8_t *staging = smem + Cfg::kStages * Cfg::kStageBytes;                  // 1024-byte aligned: stages are multiples of 1 KB
    SharedState *st = (SharedState *)(staging + Cfg::kStaging);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t ctaRank = ClusterCtaRank();
    const bool leader = ctaRank == 0;
    const int numTiles = g.tilesM * g.tilesN;
    const int kBlocks = (g.K + kBlockK - 1) / kBlockK;
    const int firstTile = (int)ClusterId(), tileStep = (int)NumClusters();

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::kStages; ++s) { MbarInit(&st->full[s], 1); MbarInit(&st->empty[s], 1); }
        TmaPrefetchDescriptor(tmC);
        MbarInit(&st->tmemFull[0], 1);
        MbarInit(&st->tmemEmpty[0], 16);                    // 8 epilogue warps x 2 CTAs
        st->abort = 0;
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
    ClusterSync();
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
                const int aRow = (mb * 2 + (int)ctaRank) * kBlockM;
                const int bRow = nb * kWideN + (int)ctaRank * 128;              // block j adds j * 256
                for (int kb = 0; kb < kBlocks; ++kb, ++it) {
                    const int s = it % Cfg::kStages;
                    const uint32_t ph = (it / Cfg::kStages) & 1;
                    if (!MbarWait(&st->empty[s], ph ^ 1, &st->abort)) { alive = false; break; }
                    uint8_t *sa = smem + s * Cfg::kStageBytes, *sb = sa + Cfg::kABytes;
                    if (leader) MbarExpectTx(&st->full[s], 2 * Cfg::kStageBytes);
                    const uint32_t bar = MapToCta(&st->full[s], 0);
                    TmaLoad2dPair(sa, tmA, bar, kb * kBlockK, aRow);
                    TmaLoad2dPair(sb, tmB, bar, kb * kBlockK, bRow);
                    TmaLoad2dPair(sb + Cfg::kBBlock, tmB, bar, kb * kBlockK, bRow + 256);
                }
            }
            if (!alive) __nanosleep(500000);                // copies already issued land long before this ends
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------------- MMA issuer (leader CTA only)
        if (leader && ElectOne()) {
            constexpr uint32_t idesc = InstrDescBf16(kPairM, 256);
            uint32_t it = 0, tileIter = 0;
            bool alive = true;
            for (int t = firstTile; t < numTiles && alive; t += tileStep, ++tileIter) {
                if (!MbarWait(&st->tmemEmpty[0], (tileIter & 1) ^ 1, &st->abort)) { alive = false; break; }
                TcFenceAfter();
                for (int kb = 0; kb < kBlocks; ++kb, ++it) {
                    const int s = it % Cfg::kStages;
                    const uint32_t ph = (it / Cfg::kStages) & 1;
                    if (!MbarWait(&st->full[s], ph, &st->abort)) { alive = false; break; }
                    TcFenceAfter();
                    uint8_t *sa = smem + s * Cfg::kStageBytes, *sb = sa + Cfg::kABytes;
                    const uint64_t da = SmemDescKMajorSw128(sa), db0 = SmemDescKMajorSw128(sb), db1 = SmemDescKMajorSw128(sb + Cfg::kBBlock);
#pragma unroll
                    for (int k = 0; k < kBlockK / kUmmaK; ++k) {
                        MmaBf16Pair(tmemBase, da + (uint64_t)(k * 2), db0 + (uint64_t)(k * 2), idesc, (kb | k) != 0);
                        MmaBf16Pair(tmemBase + 256, da + (uint64_t)(k * 2), db1 + (uint64_t)(k * 2), idesc, (kb | k) != 0);
                    }
                    MmaCommitPair(&st->empty[s]);
                }
                if (alive) MmaCommitPair(&st->tmemFull[0]);
            }
        }
    } else if (warp < 10) {
        // ---------------------------------------------------------------------- epilogue (both CTAs)
        // The tensor core waits while the accumulator is emptied, so eight warps do it: warp w reads lane quarter w % 4
        // (the lanes a warp may touch) and the column half (w - 2) / 4, two 32-column loads in flight at a time.
        const int q = warp & 3, half = (warp - 2) >> 2;
        uint8_t *slab = staging + (warp - 2) * Cfg::kSlabBytes;
        uint8_t *mine = slab + lane * 128;                      // this lane's row of the slab
        uint32_t tileIter = 0;
        bool alive = true;
        for (int t = firstTile; t < numTiles && alive; t += tileStep, ++tileIter) {
            int mb, nb;
            order(t, g, &mb, &nb);
            if (!MbarWait(&st->tmemFull[0], tileIter & 1, &st->abort)) { alive = false; break; }
            TcFenceAfter();
            const int row0 = mb * kPairM + (int)ctaRank * kBlockM + q * 32;
#pragma unroll 1
            for (int c = half * 256; c < half * 256 + 256; c += 64) {
                uint32_t f0[32], f1[32];
                TmemLoad32x32(tmemBase + ((uint32_t)(q * 32) << 16) + c, f0);
                TmemLoad32x32(tmemBase + ((uint32_t)(q * 32) << 16) + c + 32, f1);
                TmemLoadWait();
                if (c + 64 == half * 256 + 256) {
                    // the accumulator has been read: hand it back before the rows are on their way
                    TcFenceBefore();
                    __syncwarp();
                    if (lane == 0) {
                        if (leader) MbarArrive(&st->tmemEmpty[0]);
                        else RemoteArrive(MapToCta(&st->tmemEmpty[0], 0));
                    }
                }
                if (lane == 0) TmaStoreWaitRead<0>();           // the previous store has read the slab
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t *f = j < 4 ? f0 : f1;
                    const int o = (j & 3) * 8;
                    uint4 pk;
                    uint32_t *pw = (uint32_t *)&pk;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(f[o + 2 * e]), __uint_as_float(f[o + 2 * e + 1]));
                        pw[e] = *(uint32_t *)&h;
                    }
                    *(uint4 *)(mine + ((j ^ (lane & 7)) << 4)) = pk;
                }
                FenceProxyAsyncShared();                        // my writes, before the copy engine reads them
                __syncwarp();
                if (lane == 0) {
                    TmaStore2d(tmC, slab, nb * kWideN + c, row0);
                    TmaStoreCommit();
                }
            }
        }
        if (lane == 0) TmaStoreWait<0>();                       // nobody leaves with a store still reading shared memory
    }
    TcFenceBefore();
    __syncthreads();
    ClusterSync();
    if (warp == 1) TmemDealloc2(tmemBase, Cfg::kTmemCols);
    if (threadIdx.x == 0 && st->abort && g.errFlag) atomicExch(g.errFlag, 1u);
}

}  // namespace hcgemm
