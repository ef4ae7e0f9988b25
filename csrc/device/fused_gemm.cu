// fused_gemm.cu - tensor-parallel GEMMs fused with their collective, one kernel each, the transfer
// moving over NVLink peer memory tile by tile while the tensor cores work on other tiles.
//
// GEMM -> ReduceScatter  (row-parallel linear:  Y[M,N] = sum_r A_r[M,K_r] * B_r[N,K_r]^T, rank q keeps rows q*M/p ..)
//   Rank r computes its partial tiles in destination order r+1, r+2, ..., r-1, r.  The epilogue of a
//   tile owned by another rank converts the fp32 accumulator to bf16 and stores it straight into slot r of
//   the owner's staging (remote stores), then bumps that tile's arrival counter on the owner.  Tiles of
//   the rank's own rows come last: their epilogue waits until the p-1 partials have arrived, adds them
//   to the accumulator still in registers in ascending rank order (fp32) and writes the final bf16 rows.
//   There is no separate reduction pass and nothing goes through a library collective.
//
// AllGather -> GEMM  (column-parallel linear:  Y_r[M,N_r] = concat_q(x_q)[M,K] * W_r[N_r,K]^T)
//   Two extra warps per CTA push this rank's activation shard into every peer's staging (nearest consumer
//   first, 32 KB chunks, one arrival counter per 128-row block), while the GEMM starts on the local
//   shard.  The TMA producer of a tile whose rows come from rank q waits for that block's counter, then
//   loads from the local staging copy - TMA never reads peer memory.  Blocks are consumed in the order
//   own, r-1, r-2, ... which is the order in which peers send them.
//
// Both follow the CCL-buffer protocol of the collective kernels (launch parity selects the half, every
// rank waits for every other rank once per call), so they interleave freely with other operators.
// Arrival counters only grow: the host keeps the value each counter reaches in the next call and passes the table.
// With several ranks sharing one GPU (tests) all ranks run in one cooperative launch, gridDim.y = ranks.
#include <cuda_runtime.h>

#include <algorithm>

#include "../comm/comm.h"
#include "../core/log.h"
#include "emu_launch.h"
#include "gemm_api.h"
#include "gemm_sm100.cuh"
#include "gemm_sm100_2sm.cuh"
#include "hcomm_device.cuh"

namespace hc {
namespace {

using namespace hcgemm;

constexpr int kFusedThreads = 256;          // 6 GEMM warps + 2 communication warps
constexpr int kRsFlagBase = 0;              // u32 indices inside HC_OFF_FUSED
constexpr int kAgFlagBase = 4096;
constexpr size_t kAgChunkBytes = 32 << 10;  // unit of the all-gather push: one warp moves one chunk, then bumps the block's counter
constexpr int kFlagCount = 8192;

struct FusedParams {
    CUtensorMap tmA, tmB, tmA2, tmA2b;   // tmA2 / tmA2b: staging copy of A in CCL half 0 / 1
    GemmShape shape;
    CommDev *dev;
    void *out;
    const void *xLocal;       // AG: this rank's shard
    int ldOut;
    int mbPer;                // 128-row blocks per rank
    const uint32_t *expect;   // per arrival counter: the value that means "complete" in this call (indexed like the counters)
    int rowsPer;              // rows per rank
    int K;
};

__device__ __forceinline__ uint32_t *FusedFlag(const CommDev *d, int rank, int idx)
{
    return (uint32_t *)(HcPeerHeap(d, rank) + HC_OFF_FUSED) + idx;
}
__device__ __forceinline__ void RedReleaseSysAdd32(uint32_t *p, uint32_t v)
{
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void EpilogueBarrier()   // the four epilogue warps only
{
    asm volatile("bar.sync 1, 128;" ::: "memory");
}

// ------------------------------------------------------------------------ GEMM -> ReduceScatter

struct RsOrder {
    int rank, nRanks, mbPer;
    __device__ __forceinline__ void operator()(int t, const GemmShape &g, int *mb, int *nb) const
    {
        const int perDest = mbPer * g.tilesN;
        const int i = t / perDest, local = t % perDest;
        const int q = (rank + 1 + i) % nRanks;
        *mb = q * mbPer + local % mbPer;      // column by column inside a destination: its row blocks share B panels
        *nb = local / mbPer;
    }
};

template <int BN>
struct RsEpilogue {
    static constexpr bool kStaged = true;      // the CTA-pair main loop sends partial tiles out as whole 256-byte row segments
    const CommDev *d;
    __nv_bfloat16 *out;
    int ldOut, N, mbPer, rowsPer, tilesN;
    uint32_t half;
    const uint32_t *expect;
    volatile uint32_t *abortFlag;

    __device__ __forceinline__ char *Slot(int owner, int src) const
    {
        return hcdev::CclHalf(d, owner, half) + (size_t)src * rowsPer * N * sizeof(__nv_bfloat16);
    }
    __device__ __forceinline__ bool StagedTile(int mb) const { return mb / mbPer != d->rank; }
    // 32 rows x 128 columns of a partial tile, parked in shared memory by the calling warp, go to the owner's staging
    __device__ __forceinline__ void StoreStaged(int mb, int, int rowBase, int colBase, const uint8_t *slab, int lane) const
    {
        const int q = mb / mbPer;
        char *dst = Slot(q, d->rank) + ((size_t)(rowBase - q * rowsPer) * N + colBase) * sizeof(__nv_bfloat16);
        hcgemm::pair::StageFlushRows(slab, dst, (size_t)N * sizeof(__nv_bfloat16), lane);
    }
    __device__ __forceinline__ void BeginTile(int mb, int nb, int) const
    {
        const int q = mb / mbPer;
        if (q != d->rank) return;
        // my own rows: every peer's partial of this tile must have landed
        const int idx = kRsFlagBase + (mb % mbPer) * tilesN + nb;
        if ((threadIdx.x & 31) == 0) hcdev::WaitFlagGe32(d, FusedFlag(d, d->rank, idx), expect[idx], 0, HC_WAIT_TILE_FLAG, (uint32_t)idx);
        __syncwarp();
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
    __device__ __forceinline__ void EndTile(int mb, int nb, int) const
    {
        const int q = mb / mbPer;
        if (q == d->rank) return;
        EpilogueBarrier();                       // all 128 epilogue threads have issued their stores
        if (threadIdx.x == 64) {                 // first thread of the first epilogue warp
            __threadfence_system();
            RedReleaseSysAdd32(FusedFlag(d, q, kRsFlagBase + (mb % mbPer) * tilesN + nb), 1u);
        }
    }
};

template <int BN>
__global__ void __launch_bounds__(kFusedThreads, 1) GemmReduceScatterKernel(const FusedParams *table)
{
    const FusedParams &p = table[blockIdx.y];
    const CommDev *d = p.dev;
    const hcdev::LaunchState ls = hcdev::KernelBegin(d);
    RsOrder order{d->rank, d->nRanks, p.mbPer};
    RsEpilogue<BN> epi{d, (__nv_bfloat16 *)p.out, p.ldOut, p.shape.N, p.mbPer, p.rowsPer, p.shape.tilesN, ls.half, p.expect, nullptr};
    GemmMainLoop<BN>(&p.tmA, &p.tmB, p.shape, order, NoGate(), epi);
    hcdev::KernelEnd(d, ls, 0);
}

// The same on CTA pairs (256 x 256 tiles): tile row blocks, blocks per rank and the epilogue's arrival counters are
// per 256-row block; both CTAs of a pair write their half of a partial tile and each bumps the counter once.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kFusedThreads, 1) GemmReduceScatterPairKernel(const FusedParams *table)
{
    const FusedParams &p = table[blockIdx.y];
    const CommDev *d = p.dev;
    const hcdev::LaunchState ls = hcdev::KernelBegin(d);
    RsOrder order{d->rank, d->nRanks, p.mbPer};
    RsEpilogue<256> epi{d, (__nv_bfloat16 *)p.out, p.ldOut, p.shape.N, p.mbPer, p.rowsPer, p.shape.tilesN, ls.half, p.expect, nullptr};
    GemmMainLoopPair<256, 6>(&p.tmA, &p.tmB, p.shape, order, epi);
    hcdev::KernelEnd(d, ls, 0);
}

// -------------------------------------------------------------------------- AllGather -> GEMM

struct AgOrder {
    int rank, nRanks, mbPer;
    __device__ __forceinline__ void operator()(int t, const GemmShape &g, int *mb, int *nb) const
    {
        const int perSrc = mbPer * g.tilesN;
        const int j = t / perSrc, local = t % perSrc;
        const int src = (rank - j + nRanks) % nRanks;
        *mb = src * mbPer + local % mbPer;
        *nb = local / mbPer;
    }
};

struct AgGate {
    const CommDev *d;
    int mbPer;
    const uint32_t *expect;
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
        const int idx = kAgFlagBase + mb;
        if (!hcdev::WaitFlagGe32(d, FusedFlag(d, d->rank, idx), expect[idx], (uint32_t)src, HC_WAIT_TILE_FLAG, (uint32_t)idx)) {
            *abortFlag = 1;
            return false;
        }
        // the rows were written by another GPU's ordinary stores; TMA reads through the async proxy
        asm volatile("fence.proxy.async;" ::: "memory");
        return true;
    }
};

// Communication warps: push my shard to the peers' staging, nearest consumer first.
struct AgPush {
    const CommDev *d;
    const char *x;         // my shard [rowsPer, K] bf16
    int mbPer, K;
    uint32_t half;
    __device__ __forceinline__ void operator()(int warpInRole, int lane, volatile uint32_t *) const
    {
        const int n = d->nRanks, me = d->rank;
        const size_t rowBytes = (size_t)K * sizeof(__nv_bfloat16);
        const size_t blockBytes = (size_t)kBlockM * rowBytes;                     // a multiple of 2 KB (K is a multiple of 8)
        const int chunksPerBlock = (int)((blockBytes + kAgChunkBytes - 1) / kAgChunkBytes);
        const int perPeer = mbPer * chunksPerBlock;
        const int items = (n - 1) * perPeer;
        const int warps = gridDim.x * 2;
        // peer-major order: everything for the nearest consumer first; consecutive warps take consecutive chunks
        for (int it = blockIdx.x * 2 + warpInRole; it < items; it += warps) {
            const int peerIdx = it / perPeer, rem = it % perPeer;
            const int blk = rem / chunksPerBlock, ch = rem % chunksPerBlock;
            const int peer = (me + 1 + peerIdx) % n;
            const size_t off = (size_t)blk * blockBytes + (size_t)ch * kAgChunkBytes;
            const size_t len = blockBytes - (size_t)ch * kAgChunkBytes < kAgChunkBytes ? blockBytes - (size_t)ch * kAgChunkBytes : kAgChunkBytes;
            const char *src = x + off;
            char *dst = hcdev::CclHalf(d, peer, half) + (size_t)me * mbPer * blockBytes + off;
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
                __threadfence_system();
                RedReleaseSysAdd32(FusedFlag(d, peer, kAgFlagBase + me * mbPer + blk), 1u);
            }
        }
    }
};

template <int BN>
__global__ void __launch_bounds__(kFusedThreads, 1) AllGatherGemmKernel(const FusedParams *table)
{
    const FusedParams &p = table[blockIdx.y];
    const CommDev *d = p.dev;
    const hcdev::LaunchState ls = hcdev::KernelBegin(d);
    AgOrder order{d->rank, d->nRanks, p.mbPer};
    AgGate gate{d, p.mbPer, p.expect};
    AgPush push{d, (const char *)p.xLocal, p.mbPer, p.K, ls.half};
    StoreBf16 epi{(__nv_bfloat16 *)p.out, p.ldOut, p.shape.M, p.shape.N};
    GemmMainLoop<BN>(&p.tmA, &p.tmB, p.shape, order, gate, epi, ls.half ? &p.tmA2b : &p.tmA2, push);
    hcdev::KernelEnd(d, ls, 0);
}

// CTA-pair variant: p.mbPer counts 128-row blocks (gate, push and counters keep that unit), the tile order works
// on 256-row blocks.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kFusedThreads, 1) AllGatherGemmPairKernel(const FusedParams *table)
{
    const FusedParams &p = table[blockIdx.y];
    const CommDev *d = p.dev;
    const hcdev::LaunchState ls = hcdev::KernelBegin(d);
    AgOrder order{d->rank, d->nRanks, p.mbPer / 2};
    AgGate gate{d, p.mbPer, p.expect};
    AgPush push{d, (const char *)p.xLocal, p.mbPer, p.K, ls.half};
    StoreBf16 epi{(__nv_bfloat16 *)p.out, p.ldOut, p.shape.M, p.shape.N};
    GemmMainLoopPair<256, 7>(&p.tmA, &p.tmB, p.shape, order, epi, gate, ls.half ? &p.tmA2b : &p.tmA2, push);
    hcdev::KernelEnd(d, ls, 0);
}

// --------------------------------------------------------------------------------- host side

std::mutex g_ringMu;

FusedParams *ParamSlot(Comm *c)
{
    if (!c->fusedParamRing) cudaMalloc(&c->fusedParamRing, sizeof(FusedParams) * 64);
    FusedParams *p = (FusedParams *)c->fusedParamRing + c->fusedParamNext;
    c->fusedParamNext = (c->fusedParamNext + 1) % 64;
    return p;
}

// Adds `units` to the expected value of counters [lo, hi) and returns a device table (indexed like the counters) that
// holds the new values for that range; the copy is ordered on the operator's stream.
const uint32_t *ExpectTable(Comm *c, int lo, int hi, uint32_t units, void *stream, int skipLo = 0, int skipHi = 0)
{
    if (c->fusedExpect.empty()) c->fusedExpect.assign(kFlagCount, 0u);
    if (!c->fusedExpectRing && cudaMalloc(&c->fusedExpectRing, sizeof(uint32_t) * kFlagCount * 16) != cudaSuccess) return nullptr;
    for (int i = lo; i < hi; ++i)
        if (i < skipLo || i >= skipHi) c->fusedExpect[i] += units;      // [skipLo, skipHi): counters nobody bumps in this call
    uint32_t *slot = (uint32_t *)c->fusedExpectRing + (size_t)c->fusedExpectNext * kFlagCount;
    c->fusedExpectNext = (c->fusedExpectNext + 1) % 16;
    if (cudaMemcpyAsync(slot + lo, c->fusedExpect.data() + lo, sizeof(uint32_t) * (size_t)(hi - lo), cudaMemcpyHostToDevice, (cudaStream_t)stream) != cudaSuccess) return nullptr;
    return slot;
}

template <typename KernelT>
HcclResult LaunchFused(Comm *c, KernelT kernel, int smemBytes, const FusedParams &hp, int tiles, int opId, void *stream)
{
    static std::map<void *, bool> attrSet;
    {
        std::lock_guard<std::mutex> lk(g_ringMu);
        if (!attrSet[(void *)kernel]) {
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smemBytes);
            attrSet[(void *)kernel] = true;
        }
    }
    if (c->emuSameDevice && c->nRanks > 1) {
        const int ctas = std::max(1, std::min(GemmSmCount() / (int)c->nRanks, tiles));
        return EmuLaunchGeneric(c->identifier + "#fused" + std::to_string(c->group.id), c->nRanks, c->rank, opId, &hp, sizeof(hp), stream,
                                [=](const void *devTable, uint32_t n, void *st) {
                                    void *args[] = {(void *)&devTable};
                                    cudaError_t e = cudaLaunchCooperativeKernel((void *)kernel, dim3(ctas, n, 1), dim3(kFusedThreads, 1, 1), args, smemBytes, (cudaStream_t)st);
                                    if (e != cudaSuccess) { HCCL_ERROR("fused launch failed: %s", cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
                                    return HCCL_SUCCESS;
                                });
    }
    FusedParams *slot = ParamSlot(c);
    cudaError_t e = cudaMemcpyAsync(slot, &hp, sizeof(hp), cudaMemcpyHostToDevice, (cudaStream_t)stream);
    if (e != cudaSuccess) return HCCL_E_RUNTIME;
    const int ctas = std::min(GemmSmCount(), tiles);
    kernel<<<dim3(ctas, 1, 1), kFusedThreads, smemBytes, (cudaStream_t)stream>>>(slot);
    e = cudaGetLastError();
    if (e != cudaSuccess) { HCCL_ERROR("fused launch failed: %s", cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}

bool PairKernelsEnabled()
{
    static const bool on = [] { const char *e = getenv("HCOMM_GEMM_PAIR"); return !(e && e[0] == '0'); }();
    return on;
}

// CTA pairs of `kernel` (compile-time cluster of two) that can be resident at once; 0 when pairs cannot be scheduled.
template <typename KernelT>
int PairCapacityOf(KernelT kernel)
{
    constexpr int smemBytes = Config2<256, 7>::kSmemBytes;      // = Config2<256, 6, true>::kSmemBytes
    static_assert(Config2<256, 7>::kSmemBytes == Config2<256, 6, true>::kSmemBytes, "both fused pair kernels use the same shared-memory size");
    static std::map<void *, int> capacity;
    std::lock_guard<std::mutex> lk(g_ringMu);
    auto it = capacity.find((void *)kernel);
    if (it == capacity.end()) {
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smemBytes);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * GemmSmCount(), 1, 1);
        cfg.blockDim = dim3(kFusedThreads, 1, 1);
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
HcclResult LaunchFusedPair(Comm *c, KernelT kernel, const FusedParams &hp, int tiles, void *stream)
{
    constexpr int smemBytes = Config2<256, 7>::kSmemBytes;
    const int cap = PairCapacityOf(kernel);
    if (cap <= 0) return HCCL_E_NOT_SUPPORT;
    FusedParams *slot = ParamSlot(c);
    if (cudaMemcpyAsync(slot, &hp, sizeof(hp), cudaMemcpyHostToDevice, (cudaStream_t)stream) != cudaSuccess) return HCCL_E_RUNTIME;
    const int pairs = std::min(cap, tiles);
    kernel<<<dim3(2 * pairs, 1, 1), kFusedThreads, smemBytes, (cudaStream_t)stream>>>(slot);
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

}  // namespace

HcclResult LaunchBarrierIfNeeded(Comm *c, void *stream);   // defined in ops.cc

HcclResult FusedGemmReduceScatter(Comm *c, const void *A, const void *B, void *out, int M, int N, int K, int lda, int ldb, int ldOut, void *stream)
{
    CHK_RET(CheckFusable(c, "GEMM+ReduceScatter"));
    const int p = (int)c->nRanks;
    if (M % (p * kBlockM) != 0 || N % 128 != 0 || K % 8 != 0 || ldOut % 8 != 0) {
        RPT_ERR("EI0003", "GEMM+ReduceScatter needs M divisible by %d, N by 128, K by 8 (M=%d N=%d K=%d)", p * kBlockM, M, N, K);
        return HCCL_E_PARA;
    }
    const int BN = N % 256 == 0 ? 256 : 128;
    const int rowsPer = M / p;
    if ((uint64_t)p * rowsPer * N * 2 > c->halfBytes) {
        RPT_ERR("EI0003", "GEMM+ReduceScatter staging (%llu MB) exceeds one CCL half (%u MB); raise HCCL_BUFFSIZE", (unsigned long long)((uint64_t)p * rowsPer * N * 2 >> 20), c->cfg.bufferMB);
        return HCCL_E_MEMORY;
    }
    if ((rowsPer / kBlockM) * (N / BN) > 4096) return HCCL_E_NOT_SUPPORT;
    std::lock_guard<std::mutex> lk(c->opMu);
    CHK_RET(LaunchBarrierIfNeeded(c, stream));
    FusedParams hp;
    memset(&hp, 0, sizeof(hp));
    const bool usePair = PairKernelsEnabled() && !(c->emuSameDevice && c->nRanks > 1) && rowsPer % kPairM == 0 && N % 256 == 0 &&
                         PairCapacityOf(GemmReduceScatterPairKernel) > 0;
    CHK_RET(MakeTensorMap2dBf16(&hp.tmA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, kBlockM, kBlockK));
    CHK_RET(MakeTensorMap2dBf16(&hp.tmB, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, usePair ? 128u : (uint32_t)BN, kBlockK));
    const int blockRows = usePair ? kPairM : kBlockM;
    hp.shape.M = M; hp.shape.N = N; hp.shape.K = K; hp.shape.tilesM = M / blockRows; hp.shape.tilesN = N / BN; hp.shape.errFlag = GemmErrorFlag();
    hp.dev = c->devStruct; hp.out = out; hp.ldOut = ldOut; hp.mbPer = rowsPer / blockRows; hp.rowsPer = rowsPer; hp.K = K;
    // every peer bumps a tile's counter once per CTA that wrote part of it (two CTAs share a tile in the pair kernel)
    hp.expect = ExpectTable(c, kRsFlagBase, kRsFlagBase + hp.mbPer * hp.shape.tilesN, (uint32_t)(p - 1) * (usePair ? 2u : 1u), stream);
    if (!hp.expect) return HCCL_E_RUNTIME;
    ++c->opSeq;
    const int tiles = hp.shape.tilesM * hp.shape.tilesN;
    if (usePair) {
        return LaunchFusedPair(c, GemmReduceScatterPairKernel, hp, tiles, stream);
    }
    if (BN == 256) return LaunchFused(c, GemmReduceScatterKernel<256>, Config<256>::kSmemBytes, hp, tiles, 9001, stream);
    return LaunchFused(c, GemmReduceScatterKernel<128>, Config<128>::kSmemBytes, hp, tiles, 9002, stream);
}

HcclResult FusedAllGatherGemm(Comm *c, const void *x, const void *W, void *out, int Mshard, int N, int K, int ldx, int ldw, int ldOut, void *stream)
{
    CHK_RET(CheckFusable(c, "AllGather+GEMM"));
    const int p = (int)c->nRanks;
    if (Mshard % kBlockM != 0 || N % 128 != 0 || K % 8 != 0 || ldOut % 8 != 0 || ldx != K) {
        RPT_ERR("EI0003", "AllGather+GEMM needs a contiguous shard with rows divisible by %d, N by 128, K by 8 (rows=%d N=%d K=%d)", kBlockM, Mshard, N, K);
        return HCCL_E_PARA;
    }
    const int BN = N % 256 == 0 ? 256 : 128;
    const int M = Mshard * p;
    if ((uint64_t)M * K * 2 > c->halfBytes) {
        RPT_ERR("EI0003", "AllGather+GEMM staging (%llu MB) exceeds one CCL half (%u MB); raise HCCL_BUFFSIZE", (unsigned long long)((uint64_t)M * K * 2 >> 20), c->cfg.bufferMB);
        return HCCL_E_MEMORY;
    }
    if (M / kBlockM > 4096) return HCCL_E_NOT_SUPPORT;
    std::lock_guard<std::mutex> lk(c->opMu);
    CHK_RET(LaunchBarrierIfNeeded(c, stream));
    FusedParams hp;
    memset(&hp, 0, sizeof(hp));
    // The staging copy of the gathered activations lives in this operator's CCL half; which half is only known on
    // the device (launch parity), so a map is built for each and the kernel picks.
    const bool usePair = PairKernelsEnabled() && !(c->emuSameDevice && c->nRanks > 1) && Mshard % kPairM == 0 && N % 256 == 0 &&
                         PairCapacityOf(AllGatherGemmPairKernel) > 0;
    CHK_RET(MakeTensorMap2dBf16(&hp.tmA, x, (uint64_t)Mshard, (uint64_t)K, (uint64_t)ldx, kBlockM, kBlockK));
    CHK_RET(MakeTensorMap2dBf16(&hp.tmA2, c->CclBuffer(), (uint64_t)M, (uint64_t)K, (uint64_t)K, kBlockM, kBlockK));
    CHK_RET(MakeTensorMap2dBf16(&hp.tmA2b, c->CclBuffer() + c->halfBytes, (uint64_t)M, (uint64_t)K, (uint64_t)K, kBlockM, kBlockK));
    CHK_RET(MakeTensorMap2dBf16(&hp.tmB, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, usePair ? 128u : (uint32_t)BN, kBlockK));
    hp.shape.M = M; hp.shape.N = N; hp.shape.K = K; hp.shape.tilesM = M / (usePair ? kPairM : kBlockM); hp.shape.tilesN = N / BN; hp.shape.errFlag = GemmErrorFlag();
    hp.dev = c->devStruct; hp.out = out; hp.ldOut = ldOut; hp.mbPer = Mshard / kBlockM; hp.rowsPer = Mshard; hp.K = K; hp.xLocal = x;
    const uint64_t blockBytes = (uint64_t)kBlockM * K * 2;
    hp.expect = ExpectTable(c, kAgFlagBase, kAgFlagBase + M / kBlockM, (uint32_t)((blockBytes + kAgChunkBytes - 1) / kAgChunkBytes), stream,
                            kAgFlagBase + (int)c->rank * (Mshard / kBlockM), kAgFlagBase + ((int)c->rank + 1) * (Mshard / kBlockM));   // my own blocks are not sent to me
    if (!hp.expect) return HCCL_E_RUNTIME;
    ++c->opSeq;
    const int tiles = hp.shape.tilesM * hp.shape.tilesN;
    if (usePair) {
        return LaunchFusedPair(c, AllGatherGemmPairKernel, hp, tiles, stream);
    }
    if (BN == 256) return LaunchFused(c, AllGatherGemmKernel<256>, Config<256>::kSmemBytes, hp, tiles, 9003, stream);
    return LaunchFused(c, AllGatherGemmKernel<128>, Config<128>::kSmemBytes, hp, tiles, 9004, stream);
}

}  // namespace hc

extern "C" {

int HcommFusedGemmReduceScatterBf16(HcclComm comm, const void *A, const void *B, void *out, int M, int N, int K, int lda, int ldb, int ldOut, void *stream)
{
    hc::Comm *c = hc::AsComm(comm);
    if (!c) return HCCL_E_PTR;
    return (int)hc::FusedGemmReduceScatter(c, A, B, out, M, N, K, lda, ldb, ldOut, stream);
}

int HcommFusedAllGatherGemmBf16(HcclComm comm, const void *x, const void *W, void *out, int Mshard, int N, int K, int ldx, int ldw, int ldOut, void *stream)
{
    hc::Comm *c = hc::AsComm(comm);
    if (!c) return HCCL_E_PTR;
    return (int)hc::FusedAllGatherGemm(c, x, W, out, Mshard, N, K, ldx, ldw, ldOut, stream);
}

}  // extern "C"
