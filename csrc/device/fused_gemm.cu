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
//   first, 32-row pieces, one arrival counter per 128-row block), while the GEMM starts on the local
//   shard.  The TMA producer of a tile whose rows come from rank q waits for that block's counter, then
//   loads from the local staging copy - TMA never reads peer memory.  Blocks are consumed in the order
//   own, r-1, r-2, ... which is the order in which peers send them.
//
// Both follow the CCL-buffer protocol of the collective kernels (launch parity selects the half, every
// rank waits for every other rank once per call), so they interleave freely with other operators.
// Arrival counters only grow: the value expected in call number s is s * (pieces per block).
// With several ranks sharing one GPU (tests) all ranks run in one cooperative launch, gridDim.y = ranks.
#include <cuda_runtime.h>

#include <algorithm>

#include "../comm/comm.h"
#include "../core/log.h"
#include "emu_launch.h"
#include "gemm_api.h"
#include "gemm_sm100.cuh"
#include "hcomm_device.cuh"

namespace hc {
namespace {

using namespace hcgemm;

constexpr int kFusedThreads = 256;          // 6 GEMM warps + 2 communication warps
constexpr int kRsFlagBase = 0;              // u32 indices inside HC_OFF_FUSED
constexpr int kAgFlagBase = 4096;
constexpr int kAgParts = 4;                 // 32-row pieces per 128-row block

struct FusedParams {
    CUtensorMap tmA, tmB, tmA2, tmA2b;   // tmA2 / tmA2b: staging copy of A in CCL half 0 / 1
    GemmShape shape;
    CommDev *dev;
    void *out;
    const void *xLocal;       // AG: this rank's shard
    int ldOut;
    int mbPer;                // 128-row blocks per rank
    uint32_t expected;        // arrival-counter value that means "complete" in this call
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
    const CommDev *d;
    __nv_bfloat16 *out;
    int ldOut, N, mbPer, rowsPer, tilesN;
    uint32_t half, expected;
    volatile uint32_t *abortFlag;

    __device__ __forceinline__ char *Slot(int owner, int src) const
    {
        return hcdev::CclHalf(d, owner, half) + (size_t)src * rowsPer * N * sizeof(__nv_bfloat16);
    }
    __device__ __forceinline__ void BeginTile(int mb, int nb, int) const
    {
        const int q = mb / mbPer;
        if (q != d->rank) return;
        // my own rows: every peer's partial of this tile must have landed
        const int idx = kRsFlagBase + (mb % mbPer) * tilesN + nb;
        if ((threadIdx.x & 31) == 0) hcdev::WaitFlagGe32(d, FusedFlag(d, d->rank, idx), expected, 0, HC_WAIT_TILE_FLAG, (uint32_t)idx);
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
        // reduce in ascending rank order, my own accumulator taking its place in the sequence
        float acc[32];
        bool first = true;
        for (int r = 0; r < d->nRanks; ++r) {
            if (r == me) {
#pragma unroll
                for (int j = 0; j < 32; ++j) acc[j] = first ? __uint_as_float(f[j]) : acc[j] + __uint_as_float(f[j]);
            } else {
                const char *src = Slot(me, r) + ((size_t)rowLocal * N + col) * sizeof(__nv_bfloat16);
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    uint4 pk = hcdev::Ld16Volatile(src + v * 16);
                    const __nv_bfloat162 *ph = (const __nv_bfloat162 *)&pk;
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
    RsEpilogue<BN> epi{d, (__nv_bfloat16 *)p.out, p.ldOut, p.shape.N, p.mbPer, p.rowsPer, p.shape.tilesN, ls.half, p.expected, nullptr};
    GemmMainLoop<BN>(&p.tmA, &p.tmB, p.shape, order, NoGate(), epi);
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
    uint32_t expected;
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
        if (!hcdev::WaitFlagGe32(d, FusedFlag(d, d->rank, idx), expected, (uint32_t)src, HC_WAIT_TILE_FLAG, (uint32_t)idx)) {
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
        const int items = (n - 1) * mbPer * kAgParts;
        const int warps = gridDim.x * 2;
        const size_t rowBytes = (size_t)K * sizeof(__nv_bfloat16);
        const size_t pieceBytes = (size_t)(kBlockM / kAgParts) * rowBytes;
        for (int it = blockIdx.x * 2 + warpInRole; it < items; it += warps) {
            const int peerIdx = it / (mbPer * kAgParts), rem = it % (mbPer * kAgParts);
            const int blk = rem / kAgParts, part = rem % kAgParts;
            const int peer = (me + 1 + peerIdx) % n;
            const size_t off = ((size_t)blk * kBlockM + (size_t)part * (kBlockM / kAgParts)) * rowBytes;
            const char *src = x + off;
            char *dst = hcdev::CclHalf(d, peer, half) + (size_t)me * mbPer * kBlockM * rowBytes + off;
            for (size_t b = (size_t)lane * 16; b < pieceBytes; b += 32 * 16 * 4) {
                uint4 v0 = hcdev::Ld16(src + b), v1, v2, v3;
                const bool h1 = b + 512 < pieceBytes, h2 = b + 1024 < pieceBytes, h3 = b + 1536 < pieceBytes;
                if (h1) v1 = hcdev::Ld16(src + b + 512);
                if (h2) v2 = hcdev::Ld16(src + b + 1024);
                if (h3) v3 = hcdev::Ld16(src + b + 1536);
                hcdev::St16(dst + b, v0);
                if (h1) hcdev::St16(dst + b + 512, v1);
                if (h2) hcdev::St16(dst + b + 1024, v2);
                if (h3) hcdev::St16(dst + b + 1536, v3);
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
    AgGate gate{d, p.mbPer, p.expected};
    AgPush push{d, (const char *)p.xLocal, p.mbPer, p.K, ls.half};
    StoreBf16 epi{(__nv_bfloat16 *)p.out, p.ldOut, p.shape.M, p.shape.N};
    GemmMainLoop<BN>(&p.tmA, &p.tmB, p.shape, order, gate, epi, ls.half ? &p.tmA2b : &p.tmA2, push);
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
    CHK_RET(MakeTensorMap2dBf16(&hp.tmA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, kBlockM, kBlockK));
    CHK_RET(MakeTensorMap2dBf16(&hp.tmB, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, (uint32_t)BN, kBlockK));
    hp.shape.M = M; hp.shape.N = N; hp.shape.K = K; hp.shape.tilesM = M / kBlockM; hp.shape.tilesN = N / BN; hp.shape.errFlag = GemmErrorFlag();
    hp.dev = c->devStruct; hp.out = out; hp.ldOut = ldOut; hp.mbPer = rowsPer / kBlockM; hp.rowsPer = rowsPer; hp.K = K;
    hp.expected = ++c->fusedRsSeq * (uint32_t)(p - 1);
    ++c->opSeq;
    const int tiles = hp.shape.tilesM * hp.shape.tilesN;
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
    CHK_RET(MakeTensorMap2dBf16(&hp.tmA, x, (uint64_t)Mshard, (uint64_t)K, (uint64_t)ldx, kBlockM, kBlockK));
    CHK_RET(MakeTensorMap2dBf16(&hp.tmA2, c->CclBuffer(), (uint64_t)M, (uint64_t)K, (uint64_t)K, kBlockM, kBlockK));
    CHK_RET(MakeTensorMap2dBf16(&hp.tmA2b, c->CclBuffer() + c->halfBytes, (uint64_t)M, (uint64_t)K, (uint64_t)K, kBlockM, kBlockK));
    CHK_RET(MakeTensorMap2dBf16(&hp.tmB, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, (uint32_t)BN, kBlockK));
    hp.shape.M = M; hp.shape.N = N; hp.shape.K = K; hp.shape.tilesM = M / kBlockM; hp.shape.tilesN = N / BN; hp.shape.errFlag = GemmErrorFlag();
    hp.dev = c->devStruct; hp.out = out; hp.ldOut = ldOut; hp.mbPer = Mshard / kBlockM; hp.rowsPer = Mshard; hp.K = K; hp.xLocal = x;
    hp.expected = ++c->fusedAgSeq * (uint32_t)kAgParts;
    ++c->opSeq;
    const int tiles = hp.shape.tilesM * hp.shape.tilesN;
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
