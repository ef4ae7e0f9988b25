// gemm_sm100.cuh - persistent warp-specialised bf16 GEMM main loop for sm_100a, shared by the plain
// GEMM and the fused GEMM + collective kernels.
//
//   C[M,N] = A[M,K] * B[N,K]^T        A, B bf16 row-major with K contiguous ("TN"), fp32 accumulation
//
// One CTA per SM, 192 threads:
//   warp 0      TMA producer: streams 128 x 64 tiles of A and BN x 64 tiles of B into a ring of shared
//               memory stages (128-byte swizzle), completion on "full" mbarriers
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (M=128, N=BN, K=16) four times per
//               stage, accumulating in tensor memory; tcgen05.commit releases the stage ("empty") and,
//               after the last k-block, publishes the accumulator ("tmemFull")
//   warps 2-5   epilogue: tcgen05.ld the 128 x BN fp32 accumulator (each warp owns 32 TMEM lanes), hand
//               the accumulator buffer back ("tmemEmpty") and let the Epilogue policy consume the rows
// Tensor memory holds two accumulators (2 x BN columns), so the epilogue of tile i overlaps the
// main loop of tile i+1.  Policies plug in
//   TileOrder   maps the linear tile counter to (mBlock, nBlock) - fused kernels reorder tiles so the
//               data a peer waits for is produced first
//   Gate        is asked before the first TMA load of a tile (all-gather -> GEMM waits for the rows)
//   Epilogue    receives each thread's 32-column fragments
// Every wait is bounded (sm100_ptx.cuh); on expiry the CTA raises *errFlag, drains its copies, frees
// its tensor memory and returns.
#pragma once
#include <cuda_bf16.h>

#include "sm100_ptx.cuh"

namespace hcgemm {
using namespace sm100;

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;     // 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;

template <int BN> struct Config {
    static constexpr int kStages = BN == 256 ? 4 : 6;
    static constexpr int kABytes = kBlockM * kBlockK * 2;
    static constexpr int kBBytes = BN * kBlockK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemCols = 2 * BN;                  // two accumulators
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;
};

struct GemmShape {
    int M, N, K;
    int tilesM, tilesN;
    uint32_t *errFlag;       // device word, set to non-zero when a wait expired
    uint64_t *phase;         // optional phase clocks, kPhaseSlots words per CTA (nanoseconds of the GPU's global timer); NULL = off
    int clusters = 0;        // CTA-pair main loop: pairs that share the tiles (the first `clusters` of the grid); 0 = all of them
};

// Phase clocks of one CTA.  Start / End are time stamps, the others are sums of waiting or working time.
constexpr int kPhaseSlots = 8;
constexpr int kPhaseStart = 0;      // the CTA began
constexpr int kPhaseEnd = 1;        // the CTA left the main loop
constexpr int kPhaseGateWait = 2;   // TMA producer: waiting for rows that another rank sends (all-gather -> GEMM)
constexpr int kPhaseAccWait = 3;    // first epilogue warp: waiting for an accumulator
constexpr int kPhaseTileWait = 4;   // first epilogue warp: waiting for the peers' partial tiles (GEMM -> reduce-scatter)
constexpr int kPhasePushBusy = 5;   // first communication warp: first to last byte of its share of the push
constexpr int kPhasePushEnd = 6;    // first communication warp: time stamp of its last signal
constexpr int kPhaseSignal = 7;     // first communication / epilogue warp: time inside fences and signals

__device__ __forceinline__ uint64_t GlobalTimer()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

struct SharedState {
    uint64_t full[8], empty[8], tmemFull[2], tmemEmpty[2];
    uint32_t tmemBase;
    volatile uint32_t abort;
};

// Extra policies run on the warps after the six GEMM warps.  In the CTA-pair main loop kSmemBytes of shared memory
// (a multiple of 16, zeroed before any role starts) are theirs; epilogue policies with kReportsTiles see it too.
struct NoExtra {
    static constexpr int kSmemBytes = 0;
    __device__ __forceinline__ void operator()(int, int, volatile uint32_t *, uint8_t * = nullptr) const {}
};

// tmA2: optional second tensor map for A; the Gate policy decides per tile which one the producer reads
// (the all-gather fusion reads the caller's own shard in place and the peers' shards from staging).
template <int BN, typename TileOrder, typename Gate, typename Epilogue, typename Extra = NoExtra>
__device__ __forceinline__ void GemmMainLoop(const CUtensorMap *tmA, const CUtensorMap *tmB, const GemmShape &g, TileOrder order, Gate gate,
                                             Epilogue epi, const CUtensorMap *tmA2 = nullptr, Extra extra = Extra())
{
    using Cfg = Config<BN>;
    extern __shared__ uint8_t smemRaw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smemRaw + 1023) & ~(uintptr_t)1023);
    SharedState *st = (SharedState *)(smem + Cfg::kStages * Cfg::kStageBytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int numTiles = g.tilesM * g.tilesN;
    const int kBlocks = (g.K + kBlockK - 1) / kBlockK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::kStages; ++s) { MbarInit(&st->full[s], 1); MbarInit(&st->empty[s], 1); }
        for (int a = 0; a < 2; ++a) { MbarInit(&st->tmemFull[a], 1); MbarInit(&st->tmemEmpty[a], 4); }
        st->abort = 0;
        MbarFenceInit();
        TmaPrefetchDescriptor(tmA);
        TmaPrefetchDescriptor(tmB);
    }
    if (warp == 1) {
        TmemAlloc(&st->tmemBase, Cfg::kTmemCols);
        TmemRelinquish();
    }
    TcFenceBefore();
    __syncthreads();
    TcFenceAfter();
    const uint32_t tmemBase = st->tmemBase;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (ElectOne()) {
            uint32_t it = 0;
            bool alive = true;
            uint32_t lastPhase[8];
            bool issued[8];
            for (int s = 0; s < Cfg::kStages; ++s) { issued[s] = false; lastPhase[s] = 0; }
            for (int t = blockIdx.x; t < numTiles && alive; t += gridDim.x) {
                int mb, nb;
                order(t, g, &mb, &nb);
                int aRow = mb * kBlockM;
                const CUtensorMap *mapA = tmA;
                if (!gate(mb, nb, &st->abort, &aRow, tmA, tmA2, &mapA)) { alive = false; break; }
                for (int kb = 0; kb < kBlocks; ++kb, ++it) {
                    const int s = it % Cfg::kStages;
                    const uint32_t ph = (it / Cfg::kStages) & 1;
                    if (!MbarWait(&st->empty[s], ph ^ 1, &st->abort)) { alive = false; break; }
                    uint8_t *sa = smem + s * Cfg::kStageBytes, *sb = sa + Cfg::kABytes;
                    MbarExpectTx(&st->full[s], Cfg::kStageBytes);
                    TmaLoad2d(sa, mapA, &st->full[s], kb * kBlockK, aRow);
                    TmaLoad2d(sb, tmB, &st->full[s], kb * kBlockK, nb * BN);
                    issued[s] = true;
                    lastPhase[s] = ph;
                }
            }
            if (!alive) {
                // Copies already issued still write into this CTA's shared memory: wait (bounded) until the
                // phase each of them belongs to has completed before the CTA may exit.
                for (int s = 0; s < Cfg::kStages; ++s) {
                    if (!issued[s]) continue;
                    for (uint32_t i = 0; i < (1u << 20) && !MbarTryWait(&st->full[s], lastPhase[s]); ++i) {}
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------------- MMA issuer
        if (ElectOne()) {
            constexpr uint32_t idesc = InstrDescBf16(kBlockM, BN);
            uint32_t it = 0, tileIter = 0;
            bool alive = true;
            for (int t = blockIdx.x; t < numTiles && alive; t += gridDim.x, ++tileIter) {
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
                    for (int k = 0; k < kBlockK / kUmmaK; ++k) {
                        // advance 32 bytes (16 bf16) inside the swizzled row: +2 in 16-byte units
                        MmaBf16(tmemD, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0);
                    }
                    MmaCommit(&st->empty[s]);
                }
                if (alive) MmaCommit(&st->tmemFull[acc]);
            }
        }
    } else if (warp >= 6) {
        // -------------------------------------------------- extra warps (communication roles of fused kernels)
        extra(warp - 6, lane, &st->abort);
    } else {
        // ---------------------------------------------------------------------- epilogue
        const int q = warp & 3;                 // TMEM lane quarter this warp may read
        uint32_t tileIter = 0;
        bool alive = true;
        for (int t = blockIdx.x; t < numTiles && alive; t += gridDim.x, ++tileIter) {
            int mb, nb;
            order(t, g, &mb, &nb);
            const uint32_t acc = tileIter & 1, accPh = (tileIter >> 1) & 1;
            if (!MbarWait(&st->tmemFull[acc], accPh, &st->abort)) { alive = false; break; }
            TcFenceAfter();
            const int row = mb * kBlockM + q * 32 + lane;
            epi.BeginTile(mb, nb, row);
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t frag[32];
                TmemLoad32x32(tmemBase + ((uint32_t)(q * 32) << 16) + acc * BN + c, frag);
                TmemLoadWait();
                epi.Fragment(mb, nb, row, nb * BN + c, frag);
            }
            TcFenceBefore();
            __syncwarp();
            if (lane == 0) MbarArrive(&st->tmemEmpty[acc]);
            epi.EndTile(mb, nb, row);
        }
    }
    TcFenceBefore();
    __syncthreads();
    if (warp == 1) TmemDealloc(tmemBase, Cfg::kTmemCols);
    if (threadIdx.x == 0 && st->abort && g.errFlag) atomicExch(g.errFlag, 1u);
}

// ------------------------------------------------------------------------------ stock policies

// L2-aware rasterisation: tiles are walked in groups of `gm` row blocks, column by column inside a group, so the
// CTAs of one wave (148 tiles) cover about gm x 148/gm tiles and share gm A panels and 148/gm B panels.  With
// B panels twice as tall as A panels the traffic per wave, gm*a + (148/gm)*2a, is smallest near gm = 16; walking
// rows first instead would fetch every B panel once per row block and make large problems HBM bound.
struct GroupedOrder {
    int gm;
    __device__ __forceinline__ void operator()(int t, const GemmShape &g, int *mb, int *nb) const
    {
        const int perGroup = gm * g.tilesN;
        const int group = t / perGroup, rem = t % perGroup;
        const int rowsLeft = g.tilesM - group * gm;
        const int rowsHere = rowsLeft < gm ? rowsLeft : gm;
        *nb = rem / rowsHere;
        *mb = group * gm + rem % rowsHere;
    }
};
struct NoGate {
    __device__ __forceinline__ bool operator()(int, int, volatile uint32_t *, int *, const CUtensorMap *, const CUtensorMap *, const CUtensorMap **) const { return true; }
};

// Writes bf16 rows of C; each thread stores its 32 columns as four 16-byte vectors.
struct StoreBf16 {
    static constexpr bool kStaged = false;
    static constexpr bool kReportsTiles = false;
    __nv_bfloat16 *C;
    int ldc, M, N;
    __device__ __forceinline__ void BeginTile(int, int, int) const {}
    __device__ __forceinline__ void EndTile(int, int, int) const {}
    __device__ __forceinline__ void Fragment(int, int, int row, int col, const uint32_t (&f)[32]) const
    {
        if (row >= M) return;
        __nv_bfloat16 *dst = C + (size_t)row * ldc + col;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            if (col + v * 8 >= N) break;
            uint4 pk;
            uint32_t *pw = (uint32_t *)&pk;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(f[v * 8 + 2 * j]), __uint_as_float(f[v * 8 + 2 * j + 1]));
                pw[j] = *(uint32_t *)&h;
            }
            *(uint4 *)(dst + v * 8) = pk;
        }
    }
};

}  // namespace hcgemm
