// fused_gemm.cu - tensor-parallel GEMMs fused with their collective, one kernel each, the transfer
// moving over NVLink peer memory tile by tile while the tensor cores work on other tiles.
//
// GEMM -> ReduceScatter  (row-parallel linear:  Y[M,N] = sum_r A_r[M,K_r] * B_r[N,K_r]^T, rank q keeps rows q*M/p ..)
//   Rank r computes its partial tiles in an order that cycles through the destinations r+1, r+2, ..., r-1 and takes
//   its own tiles last.  The epilogue of a tile owned by another rank converts the fp32 accumulator to bf16 and
//   stores it into slot r of the owner's staging (remote stores, whole 256-byte row segments).  Every epilogue warp
//   owns 32 rows of the tile (a row group); the operator's sequence number in the flag word of (source rank, tile,
//   row group) on the owner says that the rows have landed.  In the CTA-pair kernel the epilogue warps only count
//   their finished tiles in shared memory and a signaller thread publishes them (see RsSignaller); in the
//   single-CTA kernel each warp publishes its own rows.  Tiles of the rank's own rows: the warp that owns a row group
//   waits for the p-1 flags of that same row group (one lane per source), adds the partials to the accumulator
//   still in registers in ascending rank order (fp32) and writes the final bf16 rows.  There is no separate
//   reduction pass, no CTA-wide barrier on the way and nothing goes through a library collective.
//
// AllGather -> GEMM  (column-parallel linear:  Y_r[M,N_r] = concat_q(x_q)[M,K] * W_r[N_r,K]^T)
//   Extra warps in every CTA push this rank's activation shard into every peer's staging (block-major: block 0 to
//   all peers, then block 1, ...; 32 KB chunks), while the GEMM starts on the local shard.  Finished chunks are
//   counted on this GPU; the thread whose count completes a 128-row block writes the sequence number into the
//   block's flag on the consumer.  In the CTA-pair kernel six warps push and a seventh counts and publishes for
//   them (AgPush::Signal), so the pushing warps never execute a fence.  The TMA producer of a tile whose rows come
//   from rank q waits for that flag, then loads from the local staging copy - TMA never reads peer memory.  Blocks
//   are consumed in the order own, then block i of every source for i = 0, 1, ..., the order in which they arrive.
//
// Flags hold the sequence number of the operator that wrote them (the communicator's launch count, the same on
// every rank and kept on the device) and are compared with >=, so a flag names its call: a fast rank that is
// already in the next call cannot complete a slower rank's wait of this one, nothing has to be reset, shapes may
// change from call to call and a captured launch replays.  Waiting threads poll with relaxed loads and a sleep
// between polls; each flag has one writer and is written once per call.
//
// Both follow the CCL-buffer protocol of the collective kernels (launch parity selects the half, every
// rank waits for every other rank once per call), so they interleave freely with other operators.
// With several ranks sharing one GPU (tests) all ranks run in one cooperative launch, gridDim.y = ranks.
//
// Either operator can also run split in two launches of this library's own kernels (all-gather push kernel, then
// the GEMM reading the staging; GEMM, then the reduce-scatter kernel): the mode argument or HCOMM_FUSED_MODE
// chooses, and shapes that do not fit the fused kernels' tables take the split form by themselves.
//
// Reference counterpart: the MC2 server (framework/device/aicpu_kfc/, framework/op_base/src/op_base_mc2.cc), where
// a matmul kernel posts "tile ready" messages and a control CPU issues the transfers; here the handshake is a flag
// word per tile and both sides live in one kernel.
#include <cuda_runtime.h>

#include <algorithm>

#include "../coll/ops.h"
#include "../comm/comm.h"
#include "../core/log.h"
#include "emu_launch.h"
#include "gemm_api.h"
#include "gemm_sm100.cuh"
#include "gemm_sm100_2sm.cuh"
#include "hcomm_device.cuh"
#include "hcomm_fused.h"

namespace hc {
namespace {

using namespace hcgemm;

constexpr int kFusedThreads = 256;          // reduce-scatter kernels: 6 GEMM warps, the signaller and an idle warp (communication CTAs: 7 forwarding warps + publisher)
constexpr int kAgThreads = 384;             // all-gather kernel on single CTAs: 6 GEMM warps + 6 communication warps
constexpr int kAgPairThreads = 416;         // all-gather kernel on CTA pairs: 6 GEMM warps + 6 pushing warps + the signaller
constexpr size_t kAgChunkBytes = 32 << 10;  // unit of the all-gather push: one warp moves one chunk
// Flag words (u32) inside the HC_OFF_FUSED region of every rank's heap:
//   all-gather:      block b (128 rows of the gathered matrix)           -> kAgFlagBase + b * 8            (own 32-byte sector)
//   reduce-scatter:  (source rank s, tile t of my rows, row group g < 8) -> kRsFlagBase + (s * tilesPer + t) * 8 + g
constexpr int kAgFlagBase = 0;
constexpr int kAgMaxBlocks = 1024;
constexpr int kRsFlagBase = 16384;
constexpr int kRsMaxSrcTiles = 8192;        // nRanks * tiles per rank
static_assert((size_t)(kRsFlagBase + kRsMaxSrcTiles * 8) * 4 <= HC_OFF_TEAM_SYNC - HC_OFF_FUSED, "fused flags outgrew their region");
// Device-local scratch of a communicator (Comm::fusedLocal): chunk counters of the push, the phase clocks, then the ready flags of the outbox.
constexpr size_t kLocalSentWords = kAgMaxBlocks;
constexpr size_t kLocalPhaseWords = 2 * 160 * kPhaseSlots;     // u64, two CTAs per SM pair slot, up to 160 SMs
constexpr int kRsMaxLocalTiles = 4096;                            // tiles of a reduce-scatter whose partial tiles go through the outbox
constexpr size_t kLocalReadyWords = (size_t)kRsMaxLocalTiles * 8;  // u32: (tile, row group) of my partial product is in the outbox
constexpr size_t kLocalReadyOffset = kLocalSentWords * 4 + kLocalPhaseWords * 8;
constexpr size_t kLocalBytes = kLocalReadyOffset + kLocalReadyWords * 4;

struct FusedParams {
    CUtensorMap tmA, tmB, tmA2, tmA2b;   // tmA2 / tmA2b: staging copy of A in CCL half 0 / 1
    GemmShape shape;
    CommDev *dev;
    void *out;
    const void *xLocal;       // AG: this rank's shard; NULL when a separate launch pushes it
    int ldOut;
    int mbPer;                // row blocks per rank (128 rows; 256 in the CTA-pair reduce-scatter)
    int rowsPer;              // rows per rank
    int K;
    uint32_t *sent;           // AG: device-local chunk counters [peer index][block]
    char *outbox;             // RS with communication CTAs: my partial product [M, N] bf16 in local memory
    uint32_t *ready;          // RS with communication CTAs: device-local flags, (tile, row group) is in the outbox
    int orderGroup;           // row blocks per group of the tile order (see RsOrder / AgOrder), at least 1
    int pushWarps;            // AG, CTA-pair kernel: pushing warps per CTA that take part (1..6)
    int signaller;            // AG, CTA-pair kernel: a seventh warp publishes the chunks (1) or every pushing warp its own (0)
};

__device__ __forceinline__ uint32_t *FusedFlag(const CommDev *d, int rank, int idx)
{
    return (uint32_t *)(HcPeerHeap(d, rank) + HC_OFF_FUSED) + idx;
}

// ------------------------------------------------------------------------ GEMM -> ReduceScatter

// Walks `rows` x tilesN tiles in groups of `group` rows, column by column inside a group (the rows of a group share
// B panels, the group's A panels stay in L2 while its columns pass): index -> (row, column).
__host__ __device__ __forceinline__ void GroupedWalk(int index, int rows, int tilesN, int group, int *row, int *col)
{
    const int perGroup = group * tilesN, gi = index / perGroup, r = index - gi * perGroup;
    const int here = rows - gi * group < group ? rows - gi * group : group;       // the last group may be shorter
    *col = r / here;
    *row = gi * group + r % here;
}

// Tile order of a rank: partial tiles for the other ranks first, cycling through the destinations so that the stores
// of the tiles in flight spread over all NVLink destinations at once (a single destination takes a fraction of a GPU's
// outgoing bandwidth), then the rank's own tiles.  Inside a destination: row groups of `group` row blocks, column by
// column; with p - 1 destinations in flight the A panels that are live at once are group x (p - 1), which the host sizes
// for the L2 (a destination's 16 row blocks of K = 14336 at two ranks would not fit).
struct RsOrder {
    int rank, nRanks, mbPer, group;
    __host__ __device__ __forceinline__ void operator()(int t, const GemmShape &g, int *mb, int *nb) const
    {
        const int perDest = mbPer * g.tilesN;
        const int remote = (nRanks - 1) * perDest;
        int q, local;
        if (t < remote) {
            q = (rank + 1 + t % (nRanks - 1)) % nRanks;
            local = t / (nRanks - 1);
        } else {
            q = rank;
            local = t - remote;
        }
        int row;
        GroupedWalk(local, mbPer, g.tilesN, group, &row, nb);
        *mb = q * mbPer + row;
    }
};

// A fence at system scope costs 15 - 20 us while the SM has remote stores in flight (measured on NVLink; it appears
// to wait for all of them, not just the caller's), so the warps that move data never execute one.  In the CTA-pair
// kernels they hand their progress to a signaller warp through shared memory (release / acquire at CTA scope), and
// the signaller publishes whatever has accumulated with ONE fence: the cost is paid off the data path and
// is shared by all tiles (chunks) that completed meanwhile.
constexpr uint32_t kSignallerPolls = 1u << 23;   // x 128 ns of sleep: about a second without progress, then the kernel gives up

__device__ __forceinline__ uint32_t *RsTileFlag(const CommDev *d, int owner, int src, int mbPer, int tilesN, int mb, int nb, int group)
{
    return FusedFlag(d, owner, kRsFlagBase + ((src * mbPer + mb % mbPer) * tilesN + nb) * 8 + group);
}

// TILE_ROWS: 128 (one CTA per tile) or 256 (CTA pair).  A row group is the 32 rows one epilogue warp owns.
// MODE: who publishes a partial tile.  kRsDirect: the epilogue warp itself, after a fence.  kRsSignalled: RsSignaller,
// a warp of the same CTA.  kRsOutbox: the partial tile does not leave the GPU here at all - it goes to a local matrix (the
// outbox) with a local "ready" flag, and the communication CTAs (RsForward) carry it to its owner.
constexpr int kRsDirect = 0, kRsSignalled = 1, kRsOutbox = 2;
template <int BN, int TILE_ROWS, int MODE = kRsDirect>
struct RsEpilogue {
    static constexpr bool kStaged = true;      // the CTA-pair main loop sends partial tiles out as whole 256-byte row segments
    static constexpr bool kReportsTiles = MODE == kRsSignalled;
    static constexpr bool SIGNALLED = MODE == kRsSignalled;
    const CommDev *d;
    __nv_bfloat16 *out;
    int ldOut, N, mbPer, rowsPer, tilesN;
    uint32_t half, seq;
    uint64_t *phase;                           // this CTA's phase clocks or NULL
    char *outbox;                              // kRsOutbox only
    uint32_t *ready;

    __device__ __forceinline__ char *Slot(int owner, int src) const
    {
        return hcdev::CclHalf(d, owner, half) + (size_t)src * rowsPer * N * sizeof(__nv_bfloat16);
    }
    __device__ __forceinline__ uint32_t *TileFlag(int owner, int src, int mb, int nb, int group) const
    {
        return RsTileFlag(d, owner, src, mbPer, tilesN, mb, nb, group);
    }
    __device__ __forceinline__ bool StagedTile(int mb) const { return mb / mbPer != d->rank; }
    // 32 rows x 128 columns of a partial tile, parked in shared memory by the calling warp, go to the owner's staging
    __device__ __forceinline__ void StoreStaged(int mb, int, int rowBase, int colBase, const uint8_t *slab, int lane) const
    {
        const int q = mb / mbPer;
        char *dst = MODE == kRsOutbox ? outbox + ((size_t)rowBase * N + colBase) * sizeof(__nv_bfloat16)
                                      : Slot(q, d->rank) + ((size_t)(rowBase - q * rowsPer) * N + colBase) * sizeof(__nv_bfloat16);
        hcgemm::pair::StageFlushRows(slab, dst, (size_t)N * sizeof(__nv_bfloat16), lane);
    }
    // `row` is the calling thread's row; the warp's 32 rows form row group (row of lane 0 - tile start) / 32.
    __device__ __forceinline__ void BeginTile(int mb, int nb, int row) const
    {
        const int q = mb / mbPer, me = d->rank;
        if (q != me) return;
        // my own rows: every peer's partial of this row group must have landed; lane s waits for source s
        const int lane = threadIdx.x & 31;
        const int group = (row - lane - mb * TILE_ROWS) >> 5;
        const bool clocked = phase && (threadIdx.x >> 5) == 2 && lane == 0;
        const uint64_t t0 = clocked ? GlobalTimer() : 0;
        if (lane < d->nRanks && lane != me) {
            uint64_t waited = 0;
            hcdev::WaitFlagGe32Quiet(d, TileFlag(me, lane, mb, nb, group), seq, (uint32_t)lane, HC_WAIT_TILE_FLAG, (uint32_t)(mb * tilesN + nb), &waited);
        }
        __syncwarp();
        if (clocked) phase[kPhaseTileWait] += GlobalTimer() - t0;      // until the slowest source's flag was seen
    }
    __device__ __forceinline__ void Fragment(int mb, int, int row, int col, const uint32_t (&f)[32]) const
    {
        const int q = mb / mbPer, me = d->rank;
        const int rowLocal = row - q * rowsPer;
        if (q != me) {
            char *dst = Slot(q, me) + ((size_t)rowLocal * N + col) * sizeof(__nv_bfloat16);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                uint4 pk;
                uint32_t *pw = (uint32_t *)&pk;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(f[v * 8 + 2 * j]), __uint_as_float(f[v * 8 + 2 * j + 1]));
                    pw[j] = *(uint32_t *)&h;
                }
                *(uint4 *)(dst + v * 16) = pk;
            }
            return;
        }
        // reduce in ascending rank order, my own accumulator taking its place in the sequence; the partials of up to
        // four peers are fetched together (16 loads in flight per thread) before they are added
        float acc[32];
        bool first = true;
        const int n = d->nRanks;
        for (int base = 0; base < n; base += 4) {
            uint4 pk[4][4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int r = base + k;
                if (r < n && r != me) {
                    const char *src = Slot(me, r) + ((size_t)rowLocal * N + col) * sizeof(__nv_bfloat16);
#pragma unroll
                    for (int v = 0; v < 4; ++v) pk[k][v] = hcdev::Ld16Volatile(src + v * 16);
                }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int r = base + k;
                if (r >= n) break;
                if (r == me) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[j] = first ? __uint_as_float(f[j]) : acc[j] + __uint_as_float(f[j]);
                } else {
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        const __nv_bfloat162 *ph = (const __nv_bfloat162 *)&pk[k][v];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            float2 x = __bfloat1622float2(ph[j]);
                            acc[v * 8 + 2 * j] = first ? x.x : acc[v * 8 + 2 * j] + x.x;
                            acc[v * 8 + 2 * j + 1] = first ? x.y : acc[v * 8 + 2 * j + 1] + x.y;
                        }
                    }
                }
                first = false;
            }
        }
        __nv_bfloat16 *dst = out + (size_t)rowLocal * ldOut + col;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            uint4 pk;
            uint32_t *pw = (uint32_t *)&pk;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 h = __floats2bfloat162_rn(acc[v * 8 + 2 * j], acc[v * 8 + 2 * j + 1]);
                pw[j] = *(uint32_t *)&h;
            }
            *(uint4 *)(dst + v * 8) = pk;
        }
    }
    // The warp's rows of a partial tile are on their way: publish the row group.  The releasing store of lane 0
    // orders the whole warp's stores before the flag (the lanes met at __syncwarp).
    __device__ __forceinline__ void EndTile(int mb, int nb, int row) const
    {
        const int q = mb / mbPer;
        if (SIGNALLED || q == d->rank) return;
        __syncwarp();
        const int lane = threadIdx.x & 31;
        if (MODE == kRsOutbox) {
            // local hand-over to the communication CTAs: release at GPU scope, nothing waits for NVLink
            if (lane == 0) {
                const int group = (row - mb * TILE_ROWS) >> 5;
                asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(ready + ((size_t)mb * tilesN + nb) * 8 + group), "r"(seq) : "memory");
            }
            return;
        }
        if (lane == 0) {
            const int group = (row - mb * TILE_ROWS) >> 5;
            const uint64_t t0 = phase ? GlobalTimer() : 0;
            hcdev::StReleaseSys(TileFlag(q, d->rank, mb, nb, group), seq);
            if (phase && (threadIdx.x >> 5) == 2) phase[kPhaseSignal] += GlobalTimer() - t0;
        }
    }
    // Epilogue warp `quarter` has issued every store of its first `count` tiles (own tiles included).
    __device__ __forceinline__ void TileDone(int quarter, uint32_t count, uint8_t *shared, int lane) const
    {
        __syncwarp();
        if (lane == 0) hcdev::StReleaseCtaShared((uint32_t *)shared + quarter, count);
    }
};

// The signaller of the CTA-pair reduce-scatter kernel: one thread per CTA follows the four epilogue warps' tile counts
// and publishes the row groups of every partial tile all four have stored - one fence for all tiles that completed
// since it last looked, then one flag word per row group.
struct RsSignaller {
    static constexpr int kSmemBytes = 64;
    const CommDev *d;
    RsOrder order;
    const GemmShape *shapePtr;
    int mbPer;
    uint32_t seq;
    uint64_t *phase;
    __device__ __forceinline__ void operator()(int warpInRole, int lane, volatile uint32_t *abortFlag, uint8_t *shared) const
    {
        if (warpInRole != 0 || lane != 0) return;
        const GemmShape &shape = *shapePtr;
        const uint32_t *done = (const uint32_t *)shared;
        const int me = d->rank, numTiles = shape.tilesM * shape.tilesN;
        const int first = (int)pair::ClusterId(), step = shape.clusters > 0 ? shape.clusters : (int)pair::NumClusters(), ctaRank = (int)pair::ClusterCtaRank();
        const int mine = first < numTiles ? (numTiles - first + step - 1) / step : 0;
        int k = 0;
        uint32_t idle = 0;
        uint64_t tSignal = 0;
        while (k < mine) {
            uint32_t c = hcdev::LdAcquireCtaShared(done);
#pragma unroll
            for (int w = 1; w < 4; ++w) { const uint32_t v = hcdev::LdAcquireCtaShared(done + w); c = v < c ? v : c; }
            if ((int)c <= k) {
                if (*abortFlag) return;
                if (++idle > kSignallerPolls) { *abortFlag = 1; return; }
                __nanosleep(128);
                continue;
            }
            idle = 0;
            const uint64_t t0 = phase ? GlobalTimer() : 0;
            bool fenced = false;
            for (int j = k; j < (int)c; ++j) {
                int mb, nb;
                order(first + j * step, shape, &mb, &nb);
                const int q = mb / mbPer;
                if (q == me) continue;
                if (!fenced) { hcdev::FenceAcqRelSys(); fenced = true; }
#pragma unroll
                for (int g = 0; g < 4; ++g) hcdev::StRelaxedSys(RsTileFlag(d, q, me, mbPer, shape.tilesN, mb, nb, ctaRank * 4 + g), seq);
            }
            if (phase && fenced) tSignal += GlobalTimer() - t0;
            k = (int)c;
        }
        if (phase) phase[kPhaseSignal] = tSignal;
    }
};

// Communication CTAs of the reduce-scatter (kRsOutbox): forwarding warps take the (partial tile, row group) units in
// the order the GEMM CTAs produce them, wait for the unit's local ready flag, copy its 32 rows x 256 columns from the
// outbox into this rank's slot on the owner and count it in shared memory; the CTA's last warp publishes the counted
// units - one fence for all that were forwarded since it last looked, then the owner's flag word of each.
// NF forwarding warps per CTA; their global numbers are firstWarp .. firstWarp + NF - 1 of `warps`.
template <int NF>
struct RsForward {
    const CommDev *d;
    RsOrder order;
    const GemmShape *shapePtr;
    int mbPer, rowsPer;
    uint32_t half, seq;
    const char *outbox;
    const uint32_t *ready;
    uint64_t *phase;

    __device__ __forceinline__ int Units() const { return (d->nRanks - 1) * mbPer * shapePtr->tilesN * 8; }   // remote tiles come first in the order
    __device__ __forceinline__ void Forward(int w, int warps, int lane, uint32_t *report, volatile uint32_t *abortFlag) const
    {
        const GemmShape &shape = *shapePtr;
        const int units = Units(), me = d->rank, N = shape.N;
        const size_t pitch = (size_t)N * sizeof(__nv_bfloat16);
        uint32_t forwarded = 0;
        for (int u = w; u < units; u += warps) {
            int mb, nb;
            order(u >> 3, shape, &mb, &nb);
            const int g = u & 7, q = mb / mbPer;
            const uint32_t *flag = ready + ((size_t)mb * shape.tilesN + nb) * 8 + g;
            uint32_t polls = 0;
            for (;;) {
                uint32_t v;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
                if ((int32_t)(v - seq) >= 0) break;
                if (*abortFlag) return;
                if (++polls > kSignallerPolls) { *abortFlag = 1; return; }
                __nanosleep(128);
            }
            const int row0 = mb * kPairM + g * 32;
            const char *src = outbox + ((size_t)row0 * N + (size_t)nb * 256) * sizeof(__nv_bfloat16) + (size_t)lane * 16;
            char *dst = hcdev::CclHalf(d, q, half) + (size_t)me * rowsPer * pitch + ((size_t)(row0 - q * rowsPer) * N + (size_t)nb * 256) * sizeof(__nv_bfloat16) +
                        (size_t)lane * 16;
            // a row of the unit is 512 bytes: one 16-byte access per lane; sixteen rows in flight per lane
#pragma unroll 1
            for (int r0 = 0; r0 < 32; r0 += 16) {
                uint4 v[16];
#pragma unroll
                for (int r = 0; r < 16; ++r) v[r] = hcdev::Ld16Volatile(src + (size_t)(r0 + r) * pitch);
#pragma unroll
                for (int r = 0; r < 16; ++r) hcdev::St16(dst + (size_t)(r0 + r) * pitch, v[r]);
            }
            __syncwarp();
            if (lane == 0) hcdev::StReleaseCtaShared(report, ++forwarded);
        }
    }
    __device__ __forceinline__ void Publish(int firstWarp, int warps, const uint32_t *reports, volatile uint32_t *abortFlag) const
    {
        const GemmShape &shape = *shapePtr;
        const int units = Units(), me = d->rank;
        uint32_t published[NF], total[NF];
        int remaining = 0;
#pragma unroll
        for (int w = 0; w < NF; ++w) {
            published[w] = 0;
            total[w] = firstWarp + w < units ? (uint32_t)((units - (firstWarp + w) + warps - 1) / warps) : 0u;
            remaining += (int)total[w];
        }
        uint32_t idle = 0;
        uint64_t tSignal = 0;
        while (remaining > 0) {
            uint32_t c[NF];
            bool any = false;
#pragma unroll
            for (int w = 0; w < NF; ++w) { c[w] = hcdev::LdAcquireCtaShared(reports + w); any = any || c[w] > published[w]; }
            if (!any) {
                if (*abortFlag) return;
                if (++idle > kSignallerPolls) { *abortFlag = 1; return; }
                __nanosleep(128);
                continue;
            }
            idle = 0;
            const uint64_t t0 = phase ? GlobalTimer() : 0;
            hcdev::FenceAcqRelSys();
#pragma unroll
            for (int w = 0; w < NF; ++w) {
                for (uint32_t k = published[w]; k < c[w]; ++k) {
                    const int u = firstWarp + w + (int)k * warps;
                    int mb, nb;
                    order(u >> 3, shape, &mb, &nb);
                    hcdev::StRelaxedSys(RsTileFlag(d, mb / mbPer, me, mbPer, shape.tilesN, mb, nb, u & 7), seq);
                }
                remaining -= (int)(c[w] - published[w]);
                published[w] = c[w];
            }
            if (phase) tSignal += GlobalTimer() - t0;
        }
        if (phase) { phase[kPhaseSignal] = tSignal; phase[kPhasePushEnd] = GlobalTimer(); }
    }
};

__device__ __forceinline__ uint64_t *PhaseOfCta(const GemmShape &g)
{
    return g.phase ? g.phase + (size_t)blockIdx.x * kPhaseSlots : nullptr;
}

template <int BN>
__global__ void __launch_bounds__(kFusedThreads, 1) GemmReduceScatterKernel(const __grid_constant__ FusedParams own, const FusedParams *table)
{
    const FusedParams &p = table ? table[blockIdx.y] : own;
    const CommDev *d = p.dev;
    const hcdev::LaunchState ls = hcdev::KernelBegin(d);
    RsOrder order{d->rank, d->nRanks, p.mbPer, p.orderGroup};
    RsEpilogue<BN, kBlockM> epi{d, (__nv_bfloat16 *)p.out, p.ldOut, p.shape.N, p.mbPer, p.rowsPer, p.shape.tilesN, ls.half, ls.seq, nullptr, nullptr, nullptr};
    GemmMainLoop<BN>(&p.tmA, &p.tmB, p.shape, order, NoGate(), epi);
    hcdev::KernelEnd(d, ls, 0);
}

// The same on CTA pairs (256 x 256 tiles): row blocks and blocks per rank count 256 rows; a tile has eight row groups.
template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kFusedThreads, 1) GemmReduceScatterPairKernel(const __grid_constant__ FusedParams own, const FusedParams *table)
{
    const FusedParams &p = table ? table[blockIdx.y] : own;
    const CommDev *d = p.dev;
    const hcdev::LaunchState ls = hcdev::KernelBegin(d);
    RsOrder order{d->rank, d->nRanks, p.mbPer, p.orderGroup};
    if constexpr (MODE == kRsOutbox) {
        const int gemmCtas = p.shape.clusters > 0 ? 2 * p.shape.clusters : (int)gridDim.x;
        if ((int)blockIdx.x >= gemmCtas) {
            // communication CTA: seven warps forward, the eighth publishes
            constexpr int NF = kFusedThreads / 32 - 1;
            __shared__ uint32_t reports[NF + 1];
            uint64_t *phase = PhaseOfCta(p.shape);
            if (threadIdx.x <= NF) reports[threadIdx.x] = 0;
            if (threadIdx.x == 0 && phase) phase[kPhaseStart] = GlobalTimer();
            __syncthreads();
            RsForward<NF> fwd{d, order, &p.shape, p.mbPer, p.rowsPer, ls.half, ls.seq, p.outbox, p.ready, phase};
            const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
            const int first = ((int)blockIdx.x - gemmCtas) * NF, warps = ((int)gridDim.x - gemmCtas) * NF;
            volatile uint32_t *abortFlag = &reports[NF];
            if (w < NF) fwd.Forward(first + w, warps, lane, &reports[w], abortFlag);
            else if (lane == 0) fwd.Publish(first, warps, reports, abortFlag);
            __syncthreads();
            if (threadIdx.x == 0) {
                if (*abortFlag && p.shape.errFlag) atomicExch(p.shape.errFlag, 1u);
                if (phase) phase[kPhaseEnd] = GlobalTimer();
            }
            hcdev::KernelEnd(d, ls, 0);
            return;
        }
    }
    RsEpilogue<256, kPairM, MODE> epi{d, (__nv_bfloat16 *)p.out, p.ldOut, p.shape.N, p.mbPer, p.rowsPer, p.shape.tilesN, ls.half, ls.seq, PhaseOfCta(p.shape), p.outbox, p.ready};
    if constexpr (MODE == kRsSignalled) {
        RsSignaller signaller{d, order, &p.shape, p.mbPer, ls.seq, PhaseOfCta(p.shape)};
        GemmMainLoopPair<256, 6>(&p.tmA, &p.tmB, p.shape, order, epi, NoGate(), nullptr, signaller);
    } else {
        GemmMainLoopPair<256, 6>(&p.tmA, &p.tmB, p.shape, order, epi);
    }
    hcdev::KernelEnd(d, ls, 0);
}

// -------------------------------------------------------------------------- AllGather -> GEMM

// Tile order of a rank: tiles of its own rows first, then the other ranks' rows, `group` row blocks of every source at a
// time (blocks i .. i + group - 1 of every source, then the next group), which follows the order in which the push
// delivers them (block-major).  Inside a group: column by column, so its (p - 1) x group A panels stay in L2 while the B
// panels pass once per group; one row block per group (the arrival order exactly) re-reads all of B for every block.
struct AgOrder {
    int rank, nRanks, mbPer, group;
    __host__ __device__ __forceinline__ void operator()(int t, const GemmShape &g, int *mb, int *nb) const
    {
        const int perSrc = mbPer * g.tilesN;
        if (t < perSrc) {
            int row;
            GroupedWalk(t, mbPer, g.tilesN, group * (nRanks - 1) > 0 ? group * (nRanks - 1) : 1, &row, nb);
            *mb = rank * mbPer + row;
            return;
        }
        const int u = t - perSrc, others = nRanks - 1;
        const int perGroup = group * others * g.tilesN, gi = u / perGroup, r = u - gi * perGroup;
        const int here = (mbPer - gi * group < group ? mbPer - gi * group : group) * others;     // rows of this group over all sources
        const int w = r % here;
        const int src = (rank - 1 - w % others + 2 * nRanks) % nRanks;
        *nb = r / here;
        *mb = src * mbPer + gi * group + w / others;
    }
};

struct AgGate {
    const CommDev *d;
    int mbPer;
    uint32_t seq;
    uint64_t *phase;
    __device__ __forceinline__ bool operator()(int mb, int, volatile uint32_t *abortFlag, int *aRow, const CUtensorMap *own, const CUtensorMap *staged,
                                               const CUtensorMap **use) const
    {
        const int src = mb / mbPer;
        if (src == d->rank) {
            *use = own;
            *aRow = (mb % mbPer) * kBlockM;
            return true;
        }
        *use = staged;
        *aRow = mb * kBlockM;
        uint64_t waited = 0;
        if (!hcdev::WaitFlagGe32Quiet(d, FusedFlag(d, d->rank, kAgFlagBase + mb * 8), seq, (uint32_t)src, HC_WAIT_TILE_FLAG, (uint32_t)mb, &waited)) {
            *abortFlag = 1;
            return false;
        }
        if (phase) phase[kPhaseGateWait] += waited;
        // the rows were written by another GPU's ordinary stores; TMA reads through the async proxy
        asm volatile("fence.proxy.async;" ::: "memory");
        return true;
    }
};

// Item `it` of the all-gather push of a rank with p - 1 peers: which 128-row block, which peer (index 0 = the next
// rank), which byte range of the shard.  Items are block-major: all chunks of block 0 for every peer, then block 1, ...
struct AgItem {
    int blk, peerIdx, ch;
    size_t off, len;
};
__host__ __device__ __forceinline__ int AgChunksPerBlock(int K)
{
    const size_t blockBytes = (size_t)kBlockM * K * 2;                          // bf16; a multiple of 2 KB (K is a multiple of 8)
    return (int)((blockBytes + kAgChunkBytes - 1) / kAgChunkBytes);
}
__host__ __device__ __forceinline__ AgItem AgDecode(int it, int nRanks, int K)
{
    const size_t blockBytes = (size_t)kBlockM * K * 2;
    const int chunksPerBlock = AgChunksPerBlock(K), perBlock = (nRanks - 1) * chunksPerBlock;
    AgItem a;
    a.blk = it / perBlock;
    const int rem = it % perBlock;
    a.peerIdx = rem / chunksPerBlock;
    a.ch = rem % chunksPerBlock;
    const size_t inBlock = (size_t)a.ch * kAgChunkBytes;
    a.off = (size_t)a.blk * blockBytes + inBlock;
    a.len = blockBytes - inBlock < kAgChunkBytes ? blockBytes - inBlock : kAgChunkBytes;
    return a;
}

// Communication warps: push my shard to the peers' staging, block-major.  `warps` warps share the work, this one is
// number `w`; its items are w, w + warps, w + 2 * warps, ...  With `report` (a word in shared memory) the warp only
// counts the chunks it has stored there and AgPush::Signal, on another warp of the CTA, publishes them; without, the
// warp fences and counts each chunk itself.
struct AgPush {
    static constexpr int kPushers = 6;         // pushing warps per CTA in the fused CTA-pair kernel, followed by one signaller
    static constexpr int kSmemBytes = 64;
    const CommDev *d;
    const char *x;         // my shard [rowsPer, K] bf16; NULL: nothing to push from this launch
    int mbPer, K;
    uint32_t half, seq;
    uint32_t *sent;
    uint64_t *phase;
    int pushWarps, signaller;

    __device__ __forceinline__ int ChunksPerBlock() const { return AgChunksPerBlock(K); }
    __device__ __forceinline__ int Items() const { return mbPer * (d->nRanks - 1) * ChunksPerBlock(); }
    // Chunk `it` is on the peers' side: count it; the caller has ordered the chunk before the count (fence).  The
    // thread whose count completes a block has seen every chunk of it ordered (fence, atomic on one side - atomic,
    // fence on the other) and names the block on the consumer.
    __device__ __forceinline__ void Count(int it) const
    {
        const int n = d->nRanks, me = d->rank;
        const AgItem a = AgDecode(it, n, K);
        uint32_t *ctr = sent + a.peerIdx * mbPer + a.blk;
        if (atomicAdd(ctr, 1u) + 1u == (uint32_t)ChunksPerBlock()) {
            *(volatile uint32_t *)ctr = 0u;                               // next used by a later launch
            hcdev::FenceAcqRelSys();
            hcdev::StRelaxedSys(FusedFlag(d, (me + 1 + a.peerIdx) % n, kAgFlagBase + (me * mbPer + a.blk) * 8), seq);
        }
    }
    __device__ __forceinline__ void Run(int w, int warps, int lane, uint32_t *report = nullptr, bool clocked = false) const
    {
        if (!x) return;
        const int n = d->nRanks, me = d->rank;
        const size_t blockBytes = (size_t)kBlockM * K * sizeof(__nv_bfloat16);
        const int items = Items();
        clocked = clocked && phase;
        const uint64_t tStart = clocked ? GlobalTimer() : 0;
        uint64_t tSignal = 0;
        uint32_t stored = 0;
        // block-major order: block 0 to every peer (nearest consumer first), then block 1, ...; consecutive warps take
        // consecutive chunks, so the warps in flight write to all peers at once
        for (int it = w; it < items; it += warps) {
            const AgItem a = AgDecode(it, n, K);
            const int peer = (me + 1 + a.peerIdx) % n;
            const size_t len = a.len;
            const char *src = x + a.off;
            char *dst = hcdev::CclHalf(d, peer, half) + (size_t)me * mbPer * blockBytes + a.off;
            // eight 16-byte loads per lane in flight (4 KB per warp and step)
            for (size_t b = (size_t)lane * 16; b < len; b += 32 * 16 * 8) {
                uint4 v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (b + (size_t)u * 512 < len) v[u] = hcdev::Ld16(src + b + (size_t)u * 512);
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (b + (size_t)u * 512 < len) hcdev::St16(dst + b + (size_t)u * 512, v[u]);
            }
            __syncwarp();
            if (lane == 0) {
                if (report) {
                    hcdev::StReleaseCtaShared(report, ++stored);
                } else {
                    const uint64_t t0 = clocked ? GlobalTimer() : 0;
                    hcdev::FenceAcqRelSys();
                    Count(it);
                    if (clocked) tSignal += GlobalTimer() - t0;
                }
            }
        }
        if (clocked && lane == 0) {
            const uint64_t now = GlobalTimer();
            phase[kPhasePushBusy] = now - tStart;
            if (!report) { phase[kPhasePushEnd] = now; phase[kPhaseSignal] = tSignal; }
        }
    }
    // One thread follows the counts of NP pushing warps (global numbers firstWarp .. firstWarp + NP - 1 of `warps`) and
    // counts, after ONE fence, all chunks they have stored since it last looked.
    template <int NP>
    __device__ __forceinline__ void Signal(int firstWarp, int warps, const uint32_t *reports, volatile uint32_t *abortFlag, bool clocked, int active = NP) const
    {
        if (!x) return;
        const int items = Items();
        clocked = clocked && phase;
        uint32_t published[NP], total[NP];
        int remaining = 0;
#pragma unroll
        for (int w = 0; w < NP; ++w) {
            published[w] = 0;
            total[w] = (w < active && firstWarp + w < items) ? (uint32_t)((items - (firstWarp + w) + warps - 1) / warps) : 0u;
            remaining += (int)total[w];
        }
        uint32_t idle = 0;
        uint64_t tSignal = 0;
        while (remaining > 0) {
            uint32_t c[NP];
            bool any = false;
#pragma unroll
            for (int w = 0; w < NP; ++w) { c[w] = hcdev::LdAcquireCtaShared(reports + w); any = any || c[w] > published[w]; }
            if (!any) {
                if (abortFlag && *abortFlag) return;
                if (++idle > kSignallerPolls) { if (abortFlag) *abortFlag = 1; return; }
                __nanosleep(128);
                continue;
            }
            idle = 0;
            const uint64_t t0 = clocked ? GlobalTimer() : 0;
            hcdev::FenceAcqRelSys();
#pragma unroll
            for (int w = 0; w < NP; ++w) {
                for (uint32_t k = published[w]; k < c[w]; ++k) Count(firstWarp + w + (int)k * warps);
                remaining -= (int)(c[w] - published[w]);
                published[w] = c[w];
            }
            if (clocked) tSignal += GlobalTimer() - t0;
        }
        if (clocked) {
            phase[kPhasePushEnd] = GlobalTimer();
            phase[kPhaseSignal] = tSignal;
        }
    }
    // Extra-warp entry of the GEMM main loops.  With shared memory (CTA-pair kernel): kPushers pushing warps and one
    // signaller; without (single-CTA kernel): every extra warp pushes and publishes its own chunks.
    __device__ __forceinline__ void operator()(int warpInRole, int lane, volatile uint32_t *abortFlag, uint8_t *shared = nullptr) const
    {
        if (!shared) {
            const int perCta = (int)(blockDim.x >> 5) - 6;
            Run((int)blockIdx.x * perCta + warpInRole, (int)gridDim.x * perCta, lane);
            return;
        }
        uint32_t *reports = (uint32_t *)shared;
        const int active = pushWarps >= 1 && pushWarps <= kPushers ? pushWarps : kPushers;
        const int first = (int)blockIdx.x * active, warps = (int)gridDim.x * active;
        if (warpInRole < active) Run(first + warpInRole, warps, lane, signaller ? reports + warpInRole : nullptr, warpInRole == 0);
        else if (warpInRole == kPushers && lane == 0 && signaller) Signal<kPushers>(first, warps, reports, abortFlag, true, active);
    }
};

template <int BN>
__global__ void __launch_bounds__(kAgThreads, 1) AllGatherGemmKernel(const __grid_constant__ FusedParams own, const FusedParams *table)
{
    const FusedParams &p = table ? table[blockIdx.y] : own;
    const CommDev *d = p.dev;
    const hcdev::LaunchState ls = hcdev::KernelBegin(d);
    AgOrder order{d->rank, d->nRanks, p.mbPer, p.orderGroup};
    AgGate gate{d, p.mbPer, ls.seq, nullptr};
    AgPush push{d, (const char *)p.xLocal, p.mbPer, p.K, ls.half, ls.seq, p.sent, nullptr, p.pushWarps, p.signaller};
    StoreBf16 epi{(__nv_bfloat16 *)p.out, p.ldOut, p.shape.M, p.shape.N};
    GemmMainLoop<BN>(&p.tmA, &p.tmB, p.shape, order, gate, epi, ls.half ? &p.tmA2b : &p.tmA2, push);
    hcdev::KernelEnd(d, ls, 0);
}

// CTA-pair variant: p.mbPer counts 128-row blocks (gate, push and flags keep that unit), the tile order works
// on 256-row blocks.  BN: tile width (see Config2).
template <int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kAgPairThreads, 1) AllGatherGemmPairKernel(const __grid_constant__ FusedParams own, const FusedParams *table)
{
    const FusedParams &p = table ? table[blockIdx.y] : own;
    const CommDev *d = p.dev;
    const hcdev::LaunchState ls = hcdev::KernelBegin(d);
    const int gemmCtas = p.shape.clusters > 0 ? 2 * p.shape.clusters : (int)gridDim.x;
    if ((int)blockIdx.x >= gemmCtas) {
        // Communication CTA (the last pairs of the grid when the host sets some aside): twelve warps push, the
        // thirteenth publishes; no tile is computed here, so the stores that queue up behind a busy NVLink hold up
        // nobody's operand loads.
        constexpr int NP = kAgPairThreads / 32 - 1;
        __shared__ uint32_t reports[NP + 1];
        uint64_t *phase = PhaseOfCta(p.shape);
        if (threadIdx.x <= NP) reports[threadIdx.x] = 0;
        if (threadIdx.x == 0 && phase) phase[kPhaseStart] = GlobalTimer();
        __syncthreads();
        AgPush push{d, (const char *)p.xLocal, p.mbPer, p.K, ls.half, ls.seq, p.sent, phase, NP, 1};
        const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int first = ((int)blockIdx.x - gemmCtas) * NP, warps = ((int)gridDim.x - gemmCtas) * NP;
        if (w < NP) {
            push.Run(first + w, warps, lane, &reports[w], w == 0);
        } else if (lane == 0) {
            volatile uint32_t *abortFlag = &reports[NP];
            push.Signal<NP>(first, warps, reports, abortFlag, true);
            if (*abortFlag && p.shape.errFlag) atomicExch(p.shape.errFlag, 1u);
        }
        __syncthreads();
        if (threadIdx.x == 0 && phase) phase[kPhaseEnd] = GlobalTimer();
        hcdev::KernelEnd(d, ls, 0);
        return;
    }
    AgOrder order{d->rank, d->nRanks, p.mbPer / 2, p.orderGroup};
    AgGate gate{d, p.mbPer, ls.seq, PhaseOfCta(p.shape)};
    // with communication CTAs the extra warps of the GEMM CTAs have nothing to push
    AgPush push{d, gemmCtas < (int)gridDim.x ? nullptr : (const char *)p.xLocal, p.mbPer, p.K, ls.half, ls.seq, p.sent, PhaseOfCta(p.shape), p.pushWarps, p.signaller};
    StoreBf16 epi{(__nv_bfloat16 *)p.out, p.ldOut, p.shape.M, p.shape.N};
    GemmMainLoopPair<BN, 7>(&p.tmA, &p.tmB, p.shape, order, epi, gate, ls.half ? &p.tmA2b : &p.tmA2, push);
    hcdev::KernelEnd(d, ls, 0);
}

// The push alone, on every SM: first launch of the split form.  It leaves the launch count alone so that the GEMM
// launched next sees the same sequence number and CCL half.  Fifteen warps push, the sixteenth publishes.
constexpr int kPushKernelPushers = 15;
__global__ void __launch_bounds__(512, 1) AllGatherPushKernel(const __grid_constant__ FusedParams own, const FusedParams *table)
{
    __shared__ uint32_t reports[kPushKernelPushers + 1];
    const FusedParams &p = table ? table[blockIdx.y] : own;
    const CommDev *d = p.dev;
    const hcdev::LaunchState ls = hcdev::KernelBegin(d);
    if (threadIdx.x <= kPushKernelPushers) reports[threadIdx.x] = 0;
    __syncthreads();
    AgPush push{d, (const char *)p.xLocal, p.mbPer, p.K, ls.half, ls.seq, p.sent, nullptr, p.pushWarps, p.signaller};
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int first = (int)blockIdx.x * kPushKernelPushers, warps = (int)gridDim.x * kPushKernelPushers;
    if (w < kPushKernelPushers) {
        push.Run(first + w, warps, lane, p.signaller ? &reports[w] : nullptr);
    } else if (lane == 0 && p.signaller) {
        volatile uint32_t *abortFlag = &reports[kPushKernelPushers];
        push.Signal<kPushKernelPushers>(first, warps, reports, abortFlag, false);
        if (*abortFlag && p.shape.errFlag) atomicExch(p.shape.errFlag, 1u);
    }
    hcdev::KernelEnd(d, ls, 0, 0);
}

// --------------------------------------------------------------------------------- host side

std::mutex g_ringMu;

// Device-local scratch of the fused kernels, zeroed once (the push counters return to zero by themselves).
char *FusedLocal(Comm *c)
{
    if (!c->fusedLocal) {
        if (cudaMalloc(&c->fusedLocal, kLocalBytes) != cudaSuccess) { cudaGetLastError(); c->fusedLocal = nullptr; return nullptr; }
        cudaMemset(c->fusedLocal, 0, kLocalBytes);
    }
    return (char *)c->fusedLocal;
}
uint64_t *PhaseBuffer(Comm *c, void *stream)
{
    if (!c->fusedPhaseClocks) return nullptr;
    char *base = FusedLocal(c);
    if (!base) return nullptr;
    uint64_t *ph = (uint64_t *)(base + kLocalSentWords * 4);
    cudaMemsetAsync(ph, 0, kLocalPhaseWords * 8, (cudaStream_t)stream);
    return ph;
}

template <typename KernelT>
void SetSmemOnce(KernelT kernel, int smemBytes)
{
    static std::map<void *, bool> attrSet;
    std::lock_guard<std::mutex> lk(g_ringMu);
    if (!attrSet[(void *)kernel]) {
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smemBytes);
        attrSet[(void *)kernel] = true;
    }
}

template <typename KernelT>
HcclResult LaunchFused(Comm *c, KernelT kernel, int threads, int smemBytes, const FusedParams &hp, int tiles, int opId, void *stream)
{
    SetSmemOnce(kernel, smemBytes);
    if (c->emuSameDevice && c->nRanks > 1) {
        const int ctas = std::max(1, std::min(GemmSmCount() / (int)c->nRanks, tiles));
        return EmuLaunchGeneric(c->identifier + "#fused" + std::to_string(c->group.id), c->nRanks, c->rank, opId, &hp, sizeof(hp), stream,
                                [=](const void *devTable, uint32_t n, void *st) {
                                    FusedParams unused;
                                    memset(&unused, 0, sizeof(unused));
                                    void *args[] = {(void *)&unused, (void *)&devTable};
                                    cudaError_t e = cudaLaunchCooperativeKernel((void *)kernel, dim3(ctas, n, 1), dim3(threads, 1, 1), args, smemBytes, (cudaStream_t)st);
                                    if (e != cudaSuccess) { HCCL_ERROR("fused launch failed: %s", cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
                                    return HCCL_SUCCESS;
                                });
    }
    // the parameter block travels as a kernel argument: no copy to order, nothing for the host to wait for
    const int ctas = std::min(GemmSmCount(), tiles);
    kernel<<<dim3(ctas, 1, 1), threads, smemBytes, (cudaStream_t)stream>>>(hp, (const FusedParams *)nullptr);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { HCCL_ERROR("fused launch failed: %s", cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}

bool PairKernelsEnabled()
{
    static const bool on = [] { const char *e = getenv("HCOMM_GEMM_PAIR"); return !(e && e[0] == '0'); }();
    return on;
}

// Signaller warps (HCOMM_FUSED_SIGNALLER=1 / 0 forces both on / off).  Measured on 8 GPUs at the benchmark shapes: the
// reduce-scatter kernel gains from it (456 us against 465 us, and its epilogue then waits for accumulators instead of
// for fences), the all-gather kernel loses (532 us against 499 us: pushing warps that never fence finish their share
// earlier but disturb the operand loads of the GEMM more while they do), so by default only the reduce-scatter has one.
int SignallerSetting()
{
    static const int v = [] { const char *e = getenv("HCOMM_FUSED_SIGNALLER"); return e ? (e[0] == '0' ? 0 : 1) : -1; }();
    return v;
}
bool RsSignallerEnabled() { return SignallerSetting() != 0; }
bool AgSignallerEnabled() { return SignallerSetting() == 1; }
// CTAs of the all-gather CTA-pair kernel set aside for communication (HCOMM_FUSED_COMM_CTAS, even; 0 = the extra warps
// of every CTA push).
int CommCtas()
{
    static const int v = [] { const char *e = getenv("HCOMM_FUSED_COMM_CTAS"); const int n = e ? atoi(e) : 0; return n > 0 && n <= 64 ? (n + 1) / 2 * 2 : 0; }();
    return v;
}
// The same for the reduce-scatter kernel (HCOMM_FUSED_RS_COMM_CTAS; 0 = the epilogue warps store to the owners themselves).
int RsCommCtas()
{
    static const int v = [] { const char *e = getenv("HCOMM_FUSED_RS_COMM_CTAS"); const int n = e ? atoi(e) : 0; return n > 0 && n <= 64 ? (n + 1) / 2 * 2 : 0; }();
    return v;
}
int PushWarps()
{
    static const int v = [] { const char *e = getenv("HCOMM_FUSED_PUSH_WARPS"); const int n = e ? atoi(e) : 6; return n >= 1 && n <= 6 ? n : 6; }();
    return v;
}

// CTA pairs of `kernel` (compile-time cluster of two) that can be resident at once; 0 when pairs cannot be scheduled.
template <typename KernelT>
int PairCapacityOf(KernelT kernel, int threads, int smemBytes)
{
    static std::map<void *, int> capacity;
    std::lock_guard<std::mutex> lk(g_ringMu);
    auto it = capacity.find((void *)kernel);
    if (it == capacity.end()) {
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smemBytes);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * GemmSmCount(), 1, 1);
        cfg.blockDim = dim3(threads, 1, 1);
        cfg.dynamicSmemBytes = smemBytes;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
        HCCL_INFO("fused CTA-pair kernel %p: %d pairs can be resident", (void *)kernel, n);
        it = capacity.emplace((void *)kernel, n).first;
    }
    return it->second;
}

// Launches a CTA-pair kernel on as many pairs as can be resident at once.
template <typename KernelT>
HcclResult LaunchFusedPair(Comm *c, KernelT kernel, int threads, int smemBytes, const FusedParams &hp, int tiles, void *stream, int pairsWanted = 0)
{
    const int cap = PairCapacityOf(kernel, threads, smemBytes);
    if (cap <= 0 || pairsWanted > cap) return HCCL_E_NOT_SUPPORT;
    const int pairs = pairsWanted > 0 ? pairsWanted : std::min(cap, tiles);
    kernel<<<dim3(2 * pairs, 1, 1), threads, smemBytes, (cudaStream_t)stream>>>(hp, (const FusedParams *)nullptr);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { HCCL_ERROR("fused launch (CTA pairs) failed: %s", cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}

HcclResult CheckFusable(Comm *c, const char *what)
{
    if (c->plat->kind() != PlatKind::CUDA) { RPT_ERR("EI0003", "%s runs on CUDA devices only", what); return HCCL_E_NOT_SUPPORT; }
    if (c->nRanks > HC_KERNEL_MAX_RANKS) return HCCL_E_NOT_SUPPORT;
    int st = c->state.load();
    if (st == (int)CommState::SUSPENDING || st == (int)CommState::SUSPENDED) return HCCL_E_SUSPENDING;
    return HCCL_SUCCESS;
}

// 0 = automatic, 1 = one fused kernel, 2 = two launches of this library's kernels
int ResolveMode(int mode)
{
    if (mode == HCOMM_FUSED_MODE_AUTO) {
        static const int envMode = [] {
            const char *e = getenv("HCOMM_FUSED_MODE");
            if (e && !strcmp(e, "split")) return (int)HCOMM_FUSED_MODE_SPLIT;
            if (e && !strcmp(e, "fused")) return (int)HCOMM_FUSED_MODE_FUSED;
            return (int)HCOMM_FUSED_MODE_AUTO;
        }();
        mode = envMode;
    }
    return mode;
}

}  // namespace

HcclResult LaunchBarrierIfNeeded(Comm *c, void *stream);   // defined in ops.cc

// Tile width of the CTA-pair kernels for an N-column problem with `rowBlocks` 256-row blocks on `pairs` CTA pairs:
// the width (a divisor of N among 256, 224, 192, 160, 128) with the least work in whole waves.
int PickPairTileWidth(int rowBlocks, int N, int pairs)
{
    const int forced = ForcedPairTileWidth();
    if (forced && N % forced == 0 && forced % 32 == 0 && forced >= 128 && forced <= 256) return forced;
    int best = 0;
    long bestCost = 0;
    for (int bn = 256; bn >= 128; bn -= 32) {
        if (N % bn) continue;
        const long tiles = (long)rowBlocks * (N / bn);
        const long waves = (tiles + pairs - 1) / pairs;
        // ties: 224 columns before 256 (measured equal or faster on every shape that both divide: 3584, 7168, 14336 and
        // 28672 columns at K = 8192), anything narrower must win by more than a tie
        const long cost = waves * bn * 8 + (bn == 224 ? 0 : (bn == 256 ? 1 : 32));
        if (!best || cost < bestCost) { best = bn; bestCost = cost; }
    }
    return best;
}

HcclResult FusedGemmReduceScatter(Comm *c, const void *A, const void *B, void *out, int M, int N, int K, int lda, int ldb, int ldOut, void *stream, int mode)
{
    CHK_RET(CheckFusable(c, "GEMM+ReduceScatter"));
    const int p = (int)c->nRanks;
    if (M % (p * kBlockM) != 0 || N % 128 != 0 || K % 8 != 0 || ldOut % 8 != 0) {
        RPT_ERR("EI0003", "GEMM+ReduceScatter needs M divisible by %d, N by 128, K by 8 (M=%d N=%d K=%d)", p * kBlockM, M, N, K);
        return HCCL_E_PARA;
    }
    // a single rank has nobody to exchange with: the plain GEMM (its tile shape tuned per problem) is the whole operator
    if (p == 1 && !c->emuSameDevice) return GemmBf16(A, B, out, M, N, K, lda, ldb, ldOut, stream);
    const int BN = N % 256 == 0 ? 256 : 128;
    const int rowsPer = M / p;
    mode = ResolveMode(mode);
    const bool emu = c->emuSameDevice && c->nRanks > 1;
    constexpr int pairSmem = Config2<256, 6, true, RsSignaller::kSmemBytes>::kSmemBytes;      // enough for every form
    // communication CTAs (the outbox form) need the whole partial product in local memory and a ready flag per tile
    const int commWanted = (p > 1 && mode != HCOMM_FUSED_MODE_SPLIT && (M / kPairM) * (N / 256) <= kRsMaxLocalTiles) ? RsCommCtas() : 0;
    auto pairKernel = commWanted > 0 ? GemmReduceScatterPairKernel<kRsOutbox> : (RsSignallerEnabled() ? GemmReduceScatterPairKernel<kRsSignalled> : GemmReduceScatterPairKernel<kRsDirect>);
    const bool usePair = PairKernelsEnabled() && !emu && rowsPer % kPairM == 0 && N % 256 == 0 && PairCapacityOf(pairKernel, kFusedThreads, pairSmem) > 0;
    const int blockRows = usePair ? kPairM : kBlockM;
    const bool fits = (uint64_t)p * rowsPer * N * 2 <= c->halfBytes && (uint64_t)p * (rowsPer / blockRows) * (N / BN) <= (uint64_t)kRsMaxSrcTiles;
    if (mode == HCOMM_FUSED_MODE_SPLIT || (!fits && !emu && mode == HCOMM_FUSED_MODE_AUTO)) {
        // GEMM into a scratch matrix kept by the communicator, then this library's reduce-scatter kernel
        const size_t need = (size_t)M * N * 2;
        {
            std::lock_guard<std::mutex> lk(c->opMu);
            if (c->fusedTempBytes < need) {
                if (c->fusedTemp) { cudaStreamSynchronize((cudaStream_t)stream); cudaFree(c->fusedTemp); c->fusedTemp = nullptr; c->fusedTempBytes = 0; }
                if (cudaMalloc(&c->fusedTemp, need) != cudaSuccess) { cudaGetLastError(); return HCCL_E_MEMORY; }
                c->fusedTempBytes = need;
            }
        }
        CHK_RET(GemmBf16(A, B, c->fusedTemp, M, N, K, lda, ldb, N, stream));
        if (ldOut != N) { RPT_ERR("EI0003", "the split GEMM+ReduceScatter writes a contiguous result (ldOut %d, N %d)", ldOut, N); return HCCL_E_PARA; }
        OpDesc od;
        od.cmd = HCCL_CMD_REDUCE_SCATTER; od.in = c->fusedTemp; od.out = out; od.count = (uint64_t)rowsPer * N;
        od.dtype = HCCL_DATA_TYPE_BFP16; od.op = HCCL_REDUCE_SUM; od.stream = (Stream)stream;
        return RunOp(c, od);
    }
    if ((uint64_t)p * rowsPer * N * 2 > c->halfBytes) {
        RPT_ERR("EI0003", "GEMM+ReduceScatter staging (%llu MB) exceeds one CCL half (%u MB); raise HCCL_BUFFSIZE", (unsigned long long)((uint64_t)p * rowsPer * N * 2 >> 20), c->cfg.bufferMB);
        return HCCL_E_MEMORY;
    }
    if ((uint64_t)p * (rowsPer / blockRows) * (N / BN) > (uint64_t)kRsMaxSrcTiles) return HCCL_E_NOT_SUPPORT;
    std::lock_guard<std::mutex> lk(c->opMu);
    CHK_RET(LaunchBarrierIfNeeded(c, stream));
    FusedParams hp;
    memset(&hp, 0, sizeof(hp));
    CHK_RET(MakeTensorMap2dBf16(&hp.tmA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, kBlockM, kBlockK));
    CHK_RET(MakeTensorMap2dBf16(&hp.tmB, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, usePair ? 128u : (uint32_t)BN, kBlockK));
    hp.shape.M = M; hp.shape.N = N; hp.shape.K = K; hp.shape.tilesM = M / blockRows; hp.shape.tilesN = N / BN; hp.shape.errFlag = GemmErrorFlag();
    hp.shape.phase = usePair ? PhaseBuffer(c, stream) : nullptr;
    hp.dev = c->devStruct; hp.out = out; hp.ldOut = ldOut; hp.mbPer = rowsPer / blockRows; hp.rowsPer = rowsPer; hp.K = K;
    // A panels live at once: (p - 1) destinations x orderGroup row blocks, sized like the plain GEMM's raster group
    hp.orderGroup = std::min(hp.mbPer, std::max(1, PairGroupRows(K) * (kPairM / blockRows) / std::max(1, p - 1)));
    const int tiles = hp.shape.tilesM * hp.shape.tilesN;
    int pairsWanted = 0;
    if (usePair && commWanted > 0) {
        const int cap = PairCapacityOf(pairKernel, kFusedThreads, pairSmem), commPairs = std::min(commWanted / 2, cap / 2);
        const size_t need = (size_t)M * N * 2;
        if (c->fusedTempBytes < need) {
            if (c->fusedTemp) { cudaStreamSynchronize((cudaStream_t)stream); cudaFree(c->fusedTemp); c->fusedTemp = nullptr; c->fusedTempBytes = 0; }
            if (cudaMalloc(&c->fusedTemp, need) != cudaSuccess) { cudaGetLastError(); return HCCL_E_MEMORY; }
            c->fusedTempBytes = need;
        }
        char *local = FusedLocal(c);
        if (!local) return HCCL_E_MEMORY;
        hp.outbox = (char *)c->fusedTemp;
        hp.ready = (uint32_t *)(local + kLocalReadyOffset);
        hp.shape.clusters = std::min(cap - commPairs, tiles);
        pairsWanted = hp.shape.clusters + commPairs;
    }
    ++c->opSeq;
    c->fusedLastCtas = usePair ? (pairsWanted > 0 ? 2 * pairsWanted : 2 * std::min(PairCapacityOf(pairKernel, kFusedThreads, pairSmem), tiles)) : 0;
    if (usePair) return LaunchFusedPair(c, pairKernel, kFusedThreads, pairSmem, hp, tiles, stream, pairsWanted);
    if (BN == 256) return LaunchFused(c, GemmReduceScatterKernel<256>, kFusedThreads, Config<256>::kSmemBytes, hp, tiles, 9001, stream);
    return LaunchFused(c, GemmReduceScatterKernel<128>, kFusedThreads, Config<128>::kSmemBytes, hp, tiles, 9002, stream);
}

namespace {
template <int BN>
HcclResult LaunchAgPair(Comm *c, const FusedParams &hp, int tiles, void *stream, int pairs)
{
    return LaunchFusedPair(c, AllGatherGemmPairKernel<BN>, kAgPairThreads, Config2<BN, 7, false, AgPush::kSmemBytes>::kSmemBytes, hp, tiles, stream, pairs);
}
}  // namespace

HcclResult FusedAllGatherGemm(Comm *c, const void *x, const void *W, void *out, int Mshard, int N, int K, int ldx, int ldw, int ldOut, void *stream, int mode)
{
    CHK_RET(CheckFusable(c, "AllGather+GEMM"));
    const int p = (int)c->nRanks;
    if (Mshard % kBlockM != 0 || N % 128 != 0 || K % 8 != 0 || ldOut % 8 != 0 || ldx != K) {
        RPT_ERR("EI0003", "AllGather+GEMM needs a contiguous shard with rows divisible by %d, N by 128, K by 8 (rows=%d N=%d K=%d)", kBlockM, Mshard, N, K);
        return HCCL_E_PARA;
    }
    if (p == 1 && !c->emuSameDevice) return GemmBf16(x, W, out, Mshard, N, K, ldx, ldw, ldOut, stream);
    const int M = Mshard * p;
    if ((uint64_t)M * K * 2 > c->halfBytes) {
        RPT_ERR("EI0003", "AllGather+GEMM staging (%llu MB) exceeds one CCL half (%u MB); raise HCCL_BUFFSIZE", (unsigned long long)((uint64_t)M * K * 2 >> 20), c->cfg.bufferMB);
        return HCCL_E_MEMORY;
    }
    if (M / kBlockM > kAgMaxBlocks) return HCCL_E_NOT_SUPPORT;
    mode = ResolveMode(mode);
    std::lock_guard<std::mutex> lk(c->opMu);
    CHK_RET(LaunchBarrierIfNeeded(c, stream));
    FusedParams hp;
    memset(&hp, 0, sizeof(hp));
    // The staging copy of the gathered activations lives in this operator's CCL half; which half is only known on
    // the device (launch parity), so a map is built for each and the kernel picks.
    const bool emu = c->emuSameDevice && c->nRanks > 1;
    const bool usePair = PairKernelsEnabled() && !emu && Mshard % kPairM == 0 && N % 128 == 0 &&
                         PairCapacityOf(AllGatherGemmPairKernel<256>, kAgPairThreads, Config2<256, 7, false, AgPush::kSmemBytes>::kSmemBytes) > 0;
    int BN = N % 256 == 0 ? 256 : 128;
    // pairs that compute tiles: all that can be resident, less the ones set aside for communication
    const int pairCap = usePair ? PairCapacityOf(AllGatherGemmPairKernel<256>, kAgPairThreads, Config2<256, 7, false, AgPush::kSmemBytes>::kSmemBytes) : 0;
    const int commPairs = (usePair && p > 1 && mode != HCOMM_FUSED_MODE_SPLIT) ? std::min(CommCtas() / 2, pairCap / 2) : 0;
    const int gemmPairs = pairCap - commPairs;
    if (usePair) BN = PickPairTileWidth(M / kPairM, N, gemmPairs);
    CHK_RET(MakeTensorMap2dBf16(&hp.tmA, x, (uint64_t)Mshard, (uint64_t)K, (uint64_t)ldx, kBlockM, kBlockK));
    CHK_RET(MakeTensorMap2dBf16(&hp.tmA2, c->CclBuffer(), (uint64_t)M, (uint64_t)K, (uint64_t)K, kBlockM, kBlockK));
    CHK_RET(MakeTensorMap2dBf16(&hp.tmA2b, c->CclBuffer() + c->halfBytes, (uint64_t)M, (uint64_t)K, (uint64_t)K, kBlockM, kBlockK));
    CHK_RET(MakeTensorMap2dBf16(&hp.tmB, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, usePair ? (uint32_t)(BN / 2) : (uint32_t)BN, kBlockK));
    hp.shape.M = M; hp.shape.N = N; hp.shape.K = K; hp.shape.tilesM = M / (usePair ? kPairM : kBlockM); hp.shape.tilesN = N / BN; hp.shape.errFlag = GemmErrorFlag();
    hp.shape.phase = usePair ? PhaseBuffer(c, stream) : nullptr;
    hp.dev = c->devStruct; hp.out = out; hp.ldOut = ldOut; hp.mbPer = Mshard / kBlockM; hp.rowsPer = Mshard; hp.K = K; hp.xLocal = x;
    {
        const int blocksPerSrc = usePair ? Mshard / kPairM : Mshard / kBlockM;
        hp.orderGroup = std::min(blocksPerSrc, std::max(1, PairGroupRows(K) * (usePair ? 1 : 2) / std::max(1, p - 1)));
    }
    char *local = FusedLocal(c);
    if (!local) return HCCL_E_MEMORY;
    hp.sent = (uint32_t *)local;
    hp.pushWarps = PushWarps(); hp.signaller = AgSignallerEnabled() ? 1 : 0;
    ++c->opSeq;
    const int tiles = hp.shape.tilesM * hp.shape.tilesN;
    if (mode == HCOMM_FUSED_MODE_SPLIT && !emu && p > 1) {
        // first launch: the push on the whole GPU; the GEMM launched next waits for the peers' flags like the fused form
        AllGatherPushKernel<<<dim3(GemmSmCount(), 1, 1), 512, 0, (cudaStream_t)stream>>>(hp, (const FusedParams *)nullptr);
        if (cudaGetLastError() != cudaSuccess) return HCCL_E_RUNTIME;
        hp.xLocal = nullptr;
    }
    if (usePair) {
        // with communication pairs the grid is always full: the first `clusters` pairs share the tiles, the rest push
        if (commPairs > 0) hp.shape.clusters = std::min(gemmPairs, tiles);
        c->fusedLastCtas = commPairs > 0 ? 2 * (hp.shape.clusters + commPairs) : 2 * std::min(pairCap, tiles);
        switch (BN) {
            case 256: return LaunchAgPair<256>(c, hp, tiles, stream, c->fusedLastCtas / 2);
            case 224: return LaunchAgPair<224>(c, hp, tiles, stream, c->fusedLastCtas / 2);
            case 192: return LaunchAgPair<192>(c, hp, tiles, stream, c->fusedLastCtas / 2);
            case 160: return LaunchAgPair<160>(c, hp, tiles, stream, c->fusedLastCtas / 2);
            default: return LaunchAgPair<128>(c, hp, tiles, stream, c->fusedLastCtas / 2);
        }
    }
    c->fusedLastCtas = 0;
    if (BN == 256) return LaunchFused(c, AllGatherGemmKernel<256>, kAgThreads, Config<256>::kSmemBytes, hp, tiles, 9003, stream);
    return LaunchFused(c, AllGatherGemmKernel<128>, kAgThreads, Config<128>::kSmemBytes, hp, tiles, 9004, stream);
}

// Clears the device-local scratch after a suspension (a call that was cut short leaves counts behind).
void FusedResetLocal(Comm *c)
{
    if (c->fusedLocal) cudaMemset(c->fusedLocal, 0, kLocalBytes);
}

}  // namespace hc

extern "C" {

int HcommFusedGemmReduceScatterBf16(HcclComm comm, const void *A, const void *B, void *out, int M, int N, int K, int lda, int ldb, int ldOut, void *stream)
{
    hc::Comm *c = hc::AsComm(comm);
    if (!c) return HCCL_E_PTR;
    return (int)hc::FusedGemmReduceScatter(c, A, B, out, M, N, K, lda, ldb, ldOut, stream, HCOMM_FUSED_MODE_AUTO);
}

int HcommFusedAllGatherGemmBf16(HcclComm comm, const void *x, const void *W, void *out, int Mshard, int N, int K, int ldx, int ldw, int ldOut, void *stream)
{
    hc::Comm *c = hc::AsComm(comm);
    if (!c) return HCCL_E_PTR;
    return (int)hc::FusedAllGatherGemm(c, x, W, out, Mshard, N, K, ldx, ldw, ldOut, stream, HCOMM_FUSED_MODE_AUTO);
}

int HcommFusedGemmReduceScatterBf16Mode(HcclComm comm, const void *A, const void *B, void *out, int M, int N, int K, int lda, int ldb, int ldOut, void *stream, int mode)
{
    hc::Comm *c = hc::AsComm(comm);
    if (!c) return HCCL_E_PTR;
    return (int)hc::FusedGemmReduceScatter(c, A, B, out, M, N, K, lda, ldb, ldOut, stream, mode);
}

int HcommFusedAllGatherGemmBf16Mode(HcclComm comm, const void *x, const void *W, void *out, int Mshard, int N, int K, int ldx, int ldw, int ldOut, void *stream, int mode)
{
    hc::Comm *c = hc::AsComm(comm);
    if (!c) return HCCL_E_PTR;
    return (int)hc::FusedAllGatherGemm(c, x, W, out, Mshard, N, K, ldx, ldw, ldOut, stream, mode);
}

// Tile t of the fused kernels' schedules, evaluated on the host: kind 0 = GEMM -> reduce-scatter, 1 = all-gather -> GEMM;
// `mbPer` row blocks per rank, `tilesN` tile columns, `group` row blocks per group.  The kernels run the same functions;
// tests check on the CPU that every schedule visits every tile once and in the order the flags are produced.
int HcommToolFusedTileOrder(int kind, int rank, int nRanks, int mbPer, int tilesN, int group, int t, int *mb, int *nb)
{
    if (!mb || !nb || nRanks < 1 || rank < 0 || rank >= nRanks || mbPer < 1 || tilesN < 1 || group < 1 || t < 0 || t >= nRanks * mbPer * tilesN) return HCCL_E_PARA;
    hcgemm::GemmShape g;
    g.M = g.N = g.K = 0; g.tilesM = nRanks * mbPer; g.tilesN = tilesN; g.errFlag = nullptr; g.phase = nullptr;
    if (kind == 0) hc::RsOrder{rank, nRanks, mbPer, group}(t, g, mb, nb);
    else hc::AgOrder{rank, nRanks, mbPer, group}(t, g, mb, nb);
    return HCCL_SUCCESS;
}

// Item `item` of the all-gather push (see AgDecode), evaluated on the host; *items receives the number of items of a rank.
int HcommToolFusedPushItem(int nRanks, int mbPer, int K, int item, int *items, int *blk, int *peerIdx, unsigned long long *off, unsigned long long *len)
{
    if (nRanks < 2 || mbPer < 1 || K < 8 || K % 8) return HCCL_E_PARA;
    const int total = mbPer * (nRanks - 1) * hc::AgChunksPerBlock(K);
    if (items) *items = total;
    if (item < 0 || item >= total) return item == -1 ? HCCL_SUCCESS : HCCL_E_PARA;
    const hc::AgItem a = hc::AgDecode(item, nRanks, K);
    if (blk) *blk = a.blk;
    if (peerIdx) *peerIdx = a.peerIdx;
    if (off) *off = a.off;
    if (len) *len = a.len;
    return HCCL_SUCCESS;
}

// Phase clocks of the CTA-pair fused kernels: when on, every call records per CTA when it started and ended and how long
// its roles waited (the slots are listed in gemm_sm100.cuh).  Costs a few clock reads per tile; off by default.
int HcommFusedSetPhaseClocks(HcclComm comm, int on)
{
    hc::Comm *c = hc::AsComm(comm);
    if (!c) return HCCL_E_PTR;
    c->fusedPhaseClocks = on != 0;
    return HCCL_SUCCESS;
}

// Copies the clocks of the most recent fused call (after the caller synchronised its stream): `words` receives
// ctas x 8 values, *ctas the number of CTAs that call ran on.
int HcommFusedGetPhaseClocks(HcclComm comm, uint64_t *words, int maxCtas, int *ctas)
{
    hc::Comm *c = hc::AsComm(comm);
    if (!c || !words || !ctas) return HCCL_E_PTR;
    *ctas = 0;
    if (!c->fusedLocal || !c->fusedLastCtas) return HCCL_SUCCESS;
    const int n = std::min(maxCtas, c->fusedLastCtas);
    if (cudaMemcpy(words, (char *)c->fusedLocal + hc::kLocalSentWords * 4, (size_t)n * hcgemm::kPhaseSlots * 8, cudaMemcpyDeviceToHost) != cudaSuccess) return HCCL_E_RUNTIME;
    *ctas = n;
    return HCCL_SUCCESS;
}

}  // extern "C"
