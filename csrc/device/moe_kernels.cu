// moe_kernels.cu - expert-parallel all-to-all for mixture-of-experts layers: dispatch (tokens to the
// ranks that own their experts, quantised on the fly to fp8 e4m3 with one fp32 scale per 128 values) and
// combine (expert outputs back to the token's rank with the gate-weighted sum fused).  One kernel each;
// all traffic is remote stores into symmetric buffers.  The reference only offers AlltoAll(V/VC) for this
// (pkg_inc/legacy/hccl/hccl_inner.h:55-66); routing, quantisation and the weighted sum are fused here.
//
// Dispatch, rank r - two ordinary launches (no CTA of a launch waits for another CTA of it, so they can share the GPU
// with expert GEMMs on other streams):
//   route    (1 CTA)  histogram of the experts its tokens chose, the counts published to the rank that owns each expert,
//                     one cross-rank barrier, the per-expert offsets of this rank's own experts for its grouped GEMM
//   dispatch (N CTAs) every CTA reads the owners' count tables and derives, for each expert, where this rank's rows
//                     start in the owner's receive buffer (rows are grouped by expert, inside an expert by source rank);
//                     one warp per token: load 7168 bf16, per 128-value block absmax -> scale -> e4m3, lanes 0..k-1
//                     claim the rows of the token's k experts in parallel (local atomics), then the k rows, scales and
//                     origins leave back to back; each CTA ends with one cross-rank barrier with its namesakes
// Combine, rank r (owner of experts) - two ordinary launches:
//   send  one warp per received row: the bf16 expert output goes to slot (token, k) of the token's rank; cross-rank barrier
//   sum   one warp per local token: out = sum_k gate[k] * slot(token, k) over the k that were sent, fp32 accumulation
//
// Device scratch (beyond inputs and outputs): numExperts u32 row cursors (second half of a 2 * numExperts table), cleared
// by the route launch.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <map>

#include "../comm/comm.h"
#include "../core/log.h"
#include "emu_launch.h"
#include "hccl/hccl_sym_win.h"
#include "hcomm_res.h"
#include "hcomm_device.cuh"
#include "hcomm_moe.h"

namespace hc {
namespace {

namespace cg = cooperative_groups;
using namespace hcdev;

constexpr int kMaxExperts = 1024;
constexpr int kBlock = 128;            // quantisation block

struct MoeParams {
    CommDev *dev;
    char *peerBuf[HC_KERNEL_MAX_RANKS];   // symmetric buffer of every rank as mapped here
    MoeLayout lay;
    // dispatch
    const __nv_bfloat16 *x;
    const int32_t *topkIdx;
    int numTokens;
    uint32_t *scratch;                    // [2 * numExperts]: histogram, row cursors (zero between calls)
    // combine
    const __nv_bfloat16 *y;
    const float *gates;
    __nv_bfloat16 *out;
    uint32_t *overflow;                   // device word: rows that did not fit the receive capacity
};

__device__ __forceinline__ uint32_t *Counts(const MoeParams &p, int rank) { return (uint32_t *)(p.peerBuf[rank] + p.lay.offCounts); }
__device__ __forceinline__ uint8_t *Rows(const MoeParams &p, int rank) { return (uint8_t *)(p.peerBuf[rank] + p.lay.offRows); }
__device__ __forceinline__ float *Scales(const MoeParams &p, int rank) { return (float *)(p.peerBuf[rank] + p.lay.offScales); }
__device__ __forceinline__ uint64_t *Origin(const MoeParams &p, int rank) { return (uint64_t *)(p.peerBuf[rank] + p.lay.offOrigin); }
__device__ __forceinline__ uint32_t *ExpertOffsets(const MoeParams &p, int rank) { return (uint32_t *)(p.peerBuf[rank] + p.lay.offExpertOffsets); }
__device__ __forceinline__ __nv_bfloat16 *Comb(const MoeParams &p, int rank) { return (__nv_bfloat16 *)(p.peerBuf[rank] + p.lay.offCombine); }
// one byte per (token, k) of the LOCAL tokens: 1 when dispatch sent that row, 0 when the expert index was out of range
// (masked) or the owner's receive capacity was exhausted; combine leaves such rows out of the sum
__device__ __forceinline__ uint8_t *Valid(const MoeParams &p, int rank) { return (uint8_t *)(p.peerBuf[rank] + p.lay.offValid); }

// Dispatch, first launch (one CTA per rank): routing histogram, counts published to the experts' owners, one cross-rank
// barrier, the offsets of this rank's own experts, row cursors cleared for the second launch.
__global__ void __launch_bounds__(1024) MoeRouteKernel(const MoeParams *table)
{
    const MoeParams &p = table[blockIdx.y];
    const CommDev *d = p.dev;
    const LaunchState ls = KernelBegin(d);
    const int n = d->nRanks, me = d->rank;
    const int E = p.lay.numExperts, El = E / n, K = p.lay.topk;
    const int tid = threadIdx.x;
    __shared__ uint32_t sHist[kMaxExperts], sTot[kMaxExperts];
    uint32_t *cursor = p.scratch + E;
    for (int e = tid; e < E; e += blockDim.x) { sHist[e] = 0; cursor[e] = 0; }
    __syncthreads();
    for (int i = tid; i < p.numTokens * K; i += blockDim.x) {
        int e = p.topkIdx[i];
        if (e >= 0 && e < E) atomicAdd(&sHist[e], 1u);
    }
    __syncthreads();
    for (int e = tid; e < E; e += blockDim.x) Counts(p, e / El)[me * El + (e % El)] = sHist[e];
    CrossRankBarrier(d, ls.epoch0 + 1);
    // the offsets of my own experts for the grouped GEMM that follows (the table may be overwritten by a peer's next
    // dispatch as soon as the second launch's barrier is passed, so derive them now): one thread per local expert sums
    // its column, thread 0 turns the sums into a prefix
    for (int el = tid; el < El; el += blockDim.x) {
        const volatile uint32_t *c = Counts(p, me);
        uint32_t sum = 0;
        for (int s = 0; s < n; ++s) sum += c[s * El + el];
        sTot[el] = sum;
    }
    __syncthreads();
    if (tid == 0) {
        // every entry is clamped to the receive capacity: a grouped GEMM that walks [off[el], off[el + 1]) never leaves the buffer
        const uint32_t capRows = (uint32_t)p.lay.maxRecvRows;
        uint32_t acc = 0;
        uint32_t *off = ExpertOffsets(p, me);
        for (int el = 0; el < El; ++el) {
            off[el] = acc < capRows ? acc : capRows;
            acc += sTot[el];
        }
        off[El] = acc < capRows ? acc : capRows;
    }
    KernelEnd(d, ls, 1, 0);
}

// Dispatch, second launch (any number of CTAs, an ordinary launch that can share the GPU with expert GEMMs): every CTA
// derives from the owners' count tables where this rank's rows of each expert start, then quantises and sends its
// tokens, one warp per token, and meets its namesakes on the other ranks once all of its rows are on their way.
__global__ void __launch_bounds__(512) MoeDispatchKernel(const MoeParams *table)
{
    const MoeParams &p = table[blockIdx.y];
    const CommDev *d = p.dev;
    const LaunchState ls = KernelBegin(d);
    const int n = d->nRanks, me = d->rank;
    const int E = p.lay.numExperts, El = E / n, K = p.lay.topk, H = p.lay.hidden;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int warpsPerCta = blockDim.x >> 5;
    __shared__ uint32_t sBase[kMaxExperts], sTot[kMaxExperts];
    uint32_t *cursor = p.scratch + E;

    // where do my rows of expert e start at its owner?  before them: all rows of the owner's earlier experts,
    // and the rows of this expert that come from lower ranks.  One thread per expert fetches that expert's n
    // counts from the owner (independent loads, one NVLink round trip), then the prefix runs on shared memory.
    for (int e = tid; e < E; e += blockDim.x) {
        const int owner = e / El, el = e % El;
        const volatile uint32_t *c = Counts(p, owner);
        uint32_t total = 0, below = 0;
        for (int s = 0; s < n; ++s) {
            const uint32_t v = c[s * El + el];
            total += v;
            if (s < me) below += v;
        }
        sTot[e] = total;
        sBase[e] = below;
    }
    __syncthreads();
    for (int e = tid; e < E; e += blockDim.x) {
        const int first = (e / El) * El;
        uint32_t base = 0;
        for (int e2 = first; e2 < e; ++e2) base += sTot[e2];
        sBase[e] += base;       // only this thread touches sBase[e]; sTot is read-only here
    }
    __syncthreads();

    // quantise and send, one warp per token
    const int chunks = H / 16;                       // 16 values (32 bytes in, 16 bytes out) per lane step
    const int blocksPerRow = H / kBlock;
    for (int t = blockIdx.x * warpsPerCta + warp; t < p.numTokens; t += gridDim.x * warpsPerCta) {
        // lane k claims the row of the token's k-th expert while the other lanes already load the token
        int myExpert = -1;
        uint32_t mySlot = 0xffffffffu;
        if (lane < K) {
            myExpert = p.topkIdx[t * K + lane];
            if (myExpert >= 0 && myExpert < E) {
                mySlot = sBase[myExpert] + atomicAdd(&cursor[myExpert], 1u);
                if (mySlot >= (uint32_t)p.lay.maxRecvRows) { atomicAdd(p.overflow, 1u); mySlot = 0xffffffffu; }
            }
            Valid(p, me)[t * K + lane] = mySlot != 0xffffffffu ? 1 : 0;
        }
        const __nv_bfloat16 *src = p.x + (size_t)t * H;
        uint4 q[16];                                 // up to 16 chunks per lane: hidden <= 8192; fully unrolled so that they stay in registers
        float sc[16];
#pragma unroll
        for (int nq = 0; nq < 16; ++nq) {
            const int c = lane + 32 * nq;
            if (c >= chunks) break;
            const uint4 a = *(const uint4 *)(src + c * 16), b = *(const uint4 *)(src + c * 16 + 8);
            float v[16];
            const __nv_bfloat162 *pa = (const __nv_bfloat162 *)&a, *pb = (const __nv_bfloat162 *)&b;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 fa = __bfloat1622float2(pa[j]), fb = __bfloat1622float2(pb[j]);
                v[2 * j] = fa.x; v[2 * j + 1] = fa.y; v[8 + 2 * j] = fb.x; v[8 + 2 * j + 1] = fb.y;
            }
            float amax = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
            // the 8 lanes that share a 128-value block sit next to each other
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
            const float scale = fmaxf(amax, 1e-4f) / 448.0f;   // values are divided (not multiplied by a reciprocal): bit-exact with x / scale
            sc[nq] = scale;
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j] / scale, v[4 * j + 1] / scale), __NV_SATFINITE, __NV_E4M3);
                __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * j + 2] / scale, v[4 * j + 3] / scale), __NV_SATFINITE, __NV_E4M3);
                w[j] = (uint32_t)lo | ((uint32_t)hi << 16);
            }
            q[nq] = make_uint4(w[0], w[1], w[2], w[3]);
        }
        // the token's rows leave back to back: nothing but stores between the first and the last
        for (int k = 0; k < K; ++k) {
            const int e = __shfl_sync(0xffffffffu, myExpert, k);
            const uint32_t slot = __shfl_sync(0xffffffffu, mySlot, k);
            if (slot == 0xffffffffu) continue;
            const int owner = e / El;
            uint8_t *row = Rows(p, owner) + (size_t)slot * H;
            float *srow = Scales(p, owner) + (size_t)slot * blocksPerRow;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int c = lane + 32 * i;
                if (c >= chunks) break;
                *(uint4 *)(row + c * 16) = q[i];
                if ((lane & 7) == 0) srow[c / 8] = sc[i];
            }
            if (lane == 0) Origin(p, owner)[slot] = ((uint64_t)me << 32) | (uint32_t)(t * K + k);
        }
    }
    // all rows of this CTA are on their way; once every local CTA has passed its barrier (= the kernel has ended) all
    // CTAs of all ranks have sent
    CrossRankBarrier(d, ls.epoch0 + 1);
    KernelEnd(d, ls, 1);
}

// Combine, first launch: every expert output row goes home, into slot (token, k) of the token's rank; each CTA then
// meets its namesakes on the other ranks.  When the kernel has ended on a rank, every rank's rows for it have landed.
__global__ void __launch_bounds__(512) MoeCombineSendKernel(const MoeParams *table)
{
    const MoeParams &p = table[blockIdx.y];
    const CommDev *d = p.dev;
    const LaunchState ls = KernelBegin(d);
    const int n = d->nRanks, me = d->rank;
    const int El = p.lay.numExperts / n, H = p.lay.hidden;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warpsPerCta = blockDim.x >> 5;
    const int rows = (int)ExpertOffsets(p, me)[El];
    const int vecs = H / 8;                          // 16-byte vectors of bf16 per row
    for (int r = blockIdx.x * warpsPerCta + warp; r < rows; r += gridDim.x * warpsPerCta) {
        const uint64_t o = Origin(p, me)[r];
        const int src = (int)(o >> 32);
        const uint32_t tk = (uint32_t)o;
        const uint4 *in = (const uint4 *)(p.y + (size_t)r * H);
        uint4 *dst = (uint4 *)(Comb(p, src) + (size_t)tk * H);
        // eight loads of the row in flight per lane, then their stores back to back
        for (int v0 = lane; v0 < vecs; v0 += 32 * 8) {
            uint4 buf[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (v0 + 32 * u < vecs) buf[u] = in[v0 + 32 * u];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (v0 + 32 * u < vecs) dst[v0 + 32 * u] = buf[u];
        }
    }
    CrossRankBarrier(d, ls.epoch0 + 1);
    KernelEnd(d, ls, 1);
}

// Combine, second launch (local): gate-weighted sum of the K landing slots of every local token, fp32 accumulation.
__global__ void __launch_bounds__(512) MoeCombineSumKernel(const MoeParams *table)
{
    const MoeParams &p = table[blockIdx.y];
    const int me = p.dev->rank;
    const int K = p.lay.topk, H = p.lay.hidden;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warpsPerCta = blockDim.x >> 5;
    const int vecs = H / 8;
    for (int t = blockIdx.x * warpsPerCta + warp; t < p.numTokens; t += gridDim.x * warpsPerCta) {
        float g[16];
        bool live[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            live[k] = k < K && Valid(p, me)[t * K + k] != 0;
            g[k] = live[k] ? p.gates[t * K + k] : 0.f;
        }
        for (int v = lane; v < vecs; v += 32) {
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            // eight rows of this column at a time: eight independent loads in flight (fully unrolled: registers, not local memory)
#pragma unroll
            for (int kb = 0; kb < 16; kb += 8) {
                if (kb >= K) break;
                uint4 pk[8];
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    if (live[kb + k]) pk[k] = Ld16Volatile((const char *)(Comb(p, me) + ((size_t)t * K + kb + k) * H) + (size_t)v * 16);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    if (!live[kb + k]) continue;            // nothing was sent for this (token, k): the slot holds an older step's row
                    const __nv_bfloat162 *ph = (const __nv_bfloat162 *)&pk[k];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float2 f = __bfloat1622float2(ph[j]);
                        acc[2 * j] += g[kb + k] * f.x;
                        acc[2 * j + 1] += g[kb + k] * f.y;
                    }
                }
            }
            uint4 outv;
            uint32_t *pw = (uint32_t *)&outv;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
                pw[j] = *(uint32_t *)&h;
            }
            *(uint4 *)((char *)(p.out + (size_t)t * H) + (size_t)v * 16) = outv;
        }
    }
}

struct MoeCtx {
    Comm *comm;
    MoeLayout lay;
    void *buf = nullptr;          // local symmetric buffer
    HcclCommSymWindow win = nullptr;
    char *peer[HC_KERNEL_MAX_RANKS] = {nullptr};
    uint32_t *scratch = nullptr;
    uint32_t *staticScratch = nullptr;   // device address of the built-in counter table on this exchange's GPU
    int device = -1;                     // the GPU this exchange was created on
    uint32_t *overflow = nullptr;
    MoeParams *devParams = nullptr;
    int nextParam = 0;
};
std::mutex g_mu;
std::map<void *, MoeCtx *> g_ctx;

uint64_t Align256(uint64_t v) { return (v + 255) & ~255ull; }

// CTAs of the data-moving launches: all SMs unless HCOMM_MOE_CTAS leaves some to kernels running beside them.
int MoeCtas(int sms)
{
    static const int forced = [] { const char *e = getenv("HCOMM_MOE_CTAS"); return e ? atoi(e) : 0; }();
    return forced > 0 ? std::min(forced, HC_MAX_CTAS) : std::min(sms, HC_MAX_CTAS);
}

// One launch of `kernel` with `ctas` CTAs of `threads` threads (ctas <= 0: the data-moving default).  Ordinary launches:
// nothing in these kernels waits for another CTA of the same launch.  Ranks that share a GPU (tests) are merged into one
// cooperative launch, because their kernels wait for each other.
HcclResult LaunchMoe(MoeCtx *m, void *kernel, const MoeParams &hp, int id, void *stream, int ctas = 0, int threads = 512)
{
    Comm *c = m->comm;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (c->emuSameDevice && c->nRanks > 1) {
        const int perRank = ctas > 0 ? ctas : std::max(1, sms / (int)c->nRanks);
        return EmuLaunchGeneric(c->identifier + "#moe" + std::to_string(c->group.id), c->nRanks, c->rank, id, &hp, sizeof(hp), stream,
                                [=](const void *devTable, uint32_t n, void *st) {
                                    void *args[] = {(void *)&devTable};
                                    cudaError_t e = cudaLaunchCooperativeKernel(kernel, dim3(perRank, n, 1), dim3(threads, 1, 1), args, 0, (cudaStream_t)st);
                                    if (e != cudaSuccess) { HCCL_ERROR("MoE launch failed: %s", cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
                                    return HCCL_SUCCESS;
                                });
    }
    MoeParams *slot = m->devParams + m->nextParam;
    m->nextParam = (m->nextParam + 1) % 32;
    if (cudaMemcpyAsync(slot, &hp, sizeof(hp), cudaMemcpyHostToDevice, (cudaStream_t)stream) != cudaSuccess) return HCCL_E_RUNTIME;
    void *args[] = {(void *)&slot};
    cudaError_t e = cudaLaunchKernel(kernel, dim3(ctas > 0 ? ctas : MoeCtas(sms), 1, 1), dim3(threads, 1, 1), args, 0, (cudaStream_t)stream);
    if (e != cudaSuccess) { HCCL_ERROR("MoE launch failed: %s", cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}

}  // namespace

HcclResult LaunchBarrierIfNeeded(Comm *c, void *stream);

}  // namespace hc

using namespace hc;

// ------------------------------------------------------------------ built-in scratch of HcommMoeDispatchStaticScratch
//
// The dispatch kernel counts rows per expert in a small table of global-memory counters.  HcommMoeDispatch keeps
// that table in a cudaMalloc'ed block owned by the exchange object.  HcommMoeDispatchStaticScratch runs the SAME kernel
// with the table placed in the array below, which is part of this library's device image, so that nothing on its path
// asks any allocator for memory - neither the CUDA runtime's nor a framework's caching one.
//
// It exists for callers that must not allocate at the moment they dispatch:
//   * a serving process whose memory pool has already claimed all of the GPU, where a late cudaMalloc fails;
//   * a step in which other streams (or other ranks' kernels waiting on this rank) are in flight, where the
//     implicit device-wide synchronisation of cudaMalloc / cudaFree stalls them or lengthens a peer's wait;
//   * code that owns no handle it could hang a buffer on and would otherwise allocate and free around each call.
//
// Limits and rules:
//   * at most kStaticScratchExperts experts (2 counters each, kStaticScratchBytes of device memory per process and
//     GPU, reserved when the library is loaded); larger exchanges are refused with HCCL_E_PARA;
//   * the array's device address is looked up (cudaGetSymbolAddress) by HcommMoeCreate, which runs at set-up on the
//     exchange's GPU; the dispatch call itself does no look-up, and it refuses (HCCL_E_PARA, before anything is queued)
//     a call made while another device is current - the address belongs to the exchange's GPU only;
//   * the array is shared by every call from this process on the same GPU and keeps whatever the previous call
//     left (a call that ran out of time leaves counts behind); each call therefore zeroes the part it uses, on
//     the caller's stream, before the kernel runs;
//   * because the array is shared, two calls that overlap in time on one GPU (different streams, different
//     exchange objects) race on it: keep calls of this entry point ordered one after another per GPU;
//   * ranks of one process that share a GPU (the single-GPU test arrangement) are refused: their launches are
//     merged through a table that is created on demand, which this entry point promises not to do.
constexpr int kStaticScratchExperts = 256;
constexpr size_t kStaticScratchBytes = sizeof(uint32_t) * 2 * kStaticScratchExperts;
static __device__ __align__(256) uint32_t g_staticDispatchScratch[2 * kStaticScratchExperts];

// Device address of the table on the CURRENT device (in host code the array's name is only a stand-in for it).
static uint32_t *ResolveStaticScratch()
{
    uint32_t *ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void **)&ptr, g_staticDispatchScratch);
    if (e != cudaSuccess || !ptr) {
        HCCL_WARNING("built-in dispatch scratch: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        cudaGetLastError();
        return nullptr;
    }
    return ptr;
}

extern "C" {

// Collective: every rank allocates the same symmetric buffer and maps its peers'.
int HcommMoeCreate(HcclComm comm, int numExperts, int topk, int hidden, int maxTokens, float capacityFactor, void **handle, MoeLayout *layoutOut)
{
    Comm *c = AsComm(comm);
    if (!c || !handle) return HCCL_E_PTR;
    if (c->plat->kind() != PlatKind::CUDA || c->nRanks > HC_KERNEL_MAX_RANKS) return HCCL_E_NOT_SUPPORT;
    const int n = (int)c->nRanks;
    if (numExperts <= 0 || numExperts > kMaxExperts || numExperts % n || topk <= 0 || topk > 16 || hidden % 512 || hidden > 8192 || maxTokens <= 0) {
        RPT_ERR("EI0003", "MoE geometry not supported: experts %d (multiple of %d, <= %d), top-k %d (<= 16), hidden %d (multiple of 512, <= 8192)", numExperts, n, kMaxExperts, topk, hidden);
        return HCCL_E_PARA;
    }
    MoeCtx *m = new MoeCtx();
    m->comm = c;
    MoeLayout &L = m->lay;
    L.numExperts = numExperts; L.topk = topk; L.hidden = hidden; L.maxTokens = maxTokens;
    L.maxRecvRows = (int)std::max<int64_t>(1, (int64_t)((double)maxTokens * topk * (capacityFactor > 0 ? capacityFactor : 2.0)));
    uint64_t off = 0;
    L.offCounts = off; off = Align256(off + (uint64_t)n * (numExperts / n) * 4);
    L.offExpertOffsets = off; off = Align256(off + (uint64_t)(numExperts / n + 1) * 4);
    L.offOrigin = off; off = Align256(off + (uint64_t)L.maxRecvRows * 8);
    L.offScales = off; off = Align256(off + (uint64_t)L.maxRecvRows * (hidden / 128) * 4);
    L.offRows = off; off = Align256(off + (uint64_t)L.maxRecvRows * hidden);
    L.offCombine = off; off = Align256(off + (uint64_t)maxTokens * topk * hidden * 2);
    L.offValid = off; off = Align256(off + (uint64_t)maxTokens * topk);
    L.totalBytes = off;
    HcclResult r = (HcclResult)HcommMemAlloc(&m->buf, L.totalBytes);
    if (r != HCCL_SUCCESS) { delete m; return r; }
    cudaMemset(m->buf, 0, L.offOrigin);
    r = HcclCommSymWinRegister(comm, m->buf, L.totalBytes, &m->win, 0);
    if (r != HCCL_SUCCESS) { HcommMemFree(m->buf); delete m; return r; }
    for (int q = 0; q < n; ++q) {
        void *pp = nullptr;
        HcclSymWinGetPeerPointer(m->win, 0, (uint32_t)q, &pp);
        m->peer[q] = (char *)pp;
    }
    cudaMalloc(&m->scratch, sizeof(uint32_t) * 2 * numExperts);
    cudaMemset(m->scratch, 0, sizeof(uint32_t) * 2 * numExperts);
    cudaMalloc(&m->overflow, sizeof(uint32_t));
    cudaMemset(m->overflow, 0, sizeof(uint32_t));
    cudaMalloc(&m->devParams, sizeof(MoeParams) * 32);
    cudaGetDevice(&m->device);
    m->staticScratch = ResolveStaticScratch();       // set-up time, the exchange's GPU is current
    cudaFuncAttributes fa;
    cudaFuncGetAttributes(&fa, MoeRouteKernel);
    cudaFuncGetAttributes(&fa, MoeDispatchKernel);
    cudaFuncGetAttributes(&fa, MoeCombineSendKernel);
    cudaFuncGetAttributes(&fa, MoeCombineSumKernel);
    cudaDeviceSynchronize();
    *handle = m;
    if (layoutOut) *layoutOut = L;
    std::lock_guard<std::mutex> lk(g_mu);
    g_ctx[m] = m;
    return HCCL_SUCCESS;
}

int HcommMoeDestroy(void *handle)
{
    MoeCtx *m = (MoeCtx *)handle;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (!g_ctx.erase(handle)) return HCCL_E_NOT_FOUND;
    }
    cudaDeviceSynchronize();
    HcclCommSymWinDeregister(m->win);
    HcommMemFree(m->buf);
    cudaFree(m->scratch); cudaFree(m->overflow); cudaFree(m->devParams);
    delete m;
    return HCCL_SUCCESS;
}

// Local addresses of the receive-side arrays (valid after a dispatch on the same stream).
int HcommMoeGetBuffers(void *handle, void **rows, void **scales, void **origin, void **expertOffsets, void **combine)
{
    MoeCtx *m = (MoeCtx *)handle;
    if (!m) return HCCL_E_PTR;
    char *b = (char *)m->buf;
    if (rows) *rows = b + m->lay.offRows;
    if (scales) *scales = b + m->lay.offScales;
    if (origin) *origin = b + m->lay.offOrigin;
    if (expertOffsets) *expertOffsets = b + m->lay.offExpertOffsets;
    if (combine) *combine = b + m->lay.offCombine;
    return HCCL_SUCCESS;
}

static void FillCommon(MoeCtx *m, MoeParams &hp)
{
    memset(&hp, 0, sizeof(hp));
    hp.dev = m->comm->devStruct;
    for (uint32_t q = 0; q < m->comm->nRanks; ++q) hp.peerBuf[q] = m->peer[q];
    hp.lay = m->lay;
    hp.scratch = m->scratch;
    hp.overflow = m->overflow;
}

int HcommMoeDispatch(void *handle, const void *x, const int32_t *topkIdx, int numTokens, void *stream)
{
    MoeCtx *m = (MoeCtx *)handle;
    if (!m || !x || !topkIdx) return HCCL_E_PTR;
    if (numTokens < 0 || numTokens > m->lay.maxTokens) return HCCL_E_PARA;
    Comm *c = m->comm;
    std::lock_guard<std::mutex> lk(c->opMu);
    int st = c->state.load();
    if (st == (int)CommState::SUSPENDING || st == (int)CommState::SUSPENDED) return HCCL_E_SUSPENDING;
    CHK_RET(LaunchBarrierIfNeeded(c, stream));
    MoeParams hp;
    FillCommon(m, hp);
    hp.x = (const __nv_bfloat16 *)x; hp.topkIdx = topkIdx; hp.numTokens = numTokens;
    ++c->opSeq;
    CHK_RET(LaunchMoe(m, (void *)MoeRouteKernel, hp, 9100, stream, 1, 1024));
    return LaunchMoe(m, (void *)MoeDispatchKernel, hp, 9101, stream);
}

int HcommMoeCombine(void *handle, const void *y, const float *gates, void *out, int numTokens, void *stream)
{
    MoeCtx *m = (MoeCtx *)handle;
    if (!m || !y || !gates || !out) return HCCL_E_PTR;
    if (numTokens < 0 || numTokens > m->lay.maxTokens) return HCCL_E_PARA;
    Comm *c = m->comm;
    std::lock_guard<std::mutex> lk(c->opMu);
    int st = c->state.load();
    if (st == (int)CommState::SUSPENDING || st == (int)CommState::SUSPENDED) return HCCL_E_SUSPENDING;
    CHK_RET(LaunchBarrierIfNeeded(c, stream));
    MoeParams hp;
    FillCommon(m, hp);
    hp.y = (const __nv_bfloat16 *)y; hp.gates = gates; hp.out = (__nv_bfloat16 *)out; hp.numTokens = numTokens;
    ++c->opSeq;
    CHK_RET(LaunchMoe(m, (void *)MoeCombineSendKernel, hp, 9102, stream));
    return LaunchMoe(m, (void *)MoeCombineSumKernel, hp, 9104, stream);
}

// ------------------------------------------------------------------ dispatch without any allocation
//
// See the comment at g_staticDispatchScratch (top of the host section) for what this entry point is for and its rules.
int HcommMoeDispatchStaticScratch(void *handle, const void *x, const int32_t *topkIdx, int numTokens, void *stream)
{
    MoeCtx *m = (MoeCtx *)handle;
    if (!m || !x || !topkIdx) return HCCL_E_PTR;
    if (numTokens < 0 || numTokens > m->lay.maxTokens) return HCCL_E_PARA;
    Comm *c = m->comm;
    if (m->lay.numExperts > kStaticScratchExperts) {
        RPT_ERR("EI0003", "HcommMoeDispatchStaticScratch serves at most %d experts (%zu bytes of built-in scratch); this exchange has %d - use HcommMoeDispatch",
                kStaticScratchExperts, kStaticScratchBytes, m->lay.numExperts);
        return HCCL_E_PARA;
    }
    if (c->emuSameDevice && c->nRanks > 1) {
        RPT_ERR("EI0003", "HcommMoeDispatchStaticScratch does not serve several ranks of one process on one GPU - use HcommMoeDispatch");
        return HCCL_E_NOT_SUPPORT;
    }
    // The table's address belongs to the GPU the exchange was created on; with another device current the launch
    // below would go elsewhere.  Checked before anything is queued or counted.
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev != m->device) {
        RPT_ERR("EI0003", "HcommMoeDispatchStaticScratch called with device %d current; the exchange lives on device %d", dev, m->device);
        return HCCL_E_PARA;
    }
    if (!m->staticScratch) {
        RPT_ERR("EI0003", "the built-in dispatch scratch could not be resolved when this exchange was created - use HcommMoeDispatch");
        return HCCL_E_NOT_SUPPORT;
    }
    std::lock_guard<std::mutex> lk(c->opMu);
    int st = c->state.load();
    if (st == (int)CommState::SUSPENDING || st == (int)CommState::SUSPENDED) return HCCL_E_SUSPENDING;
    CHK_RET(LaunchBarrierIfNeeded(c, stream));
    // the kernel expects both counter rows at zero and the array may hold a previous call's leftovers
    if (cudaMemsetAsync(m->staticScratch, 0, sizeof(uint32_t) * 2 * (size_t)m->lay.numExperts, (cudaStream_t)stream) != cudaSuccess) {
        HCCL_ERROR("built-in dispatch scratch: clearing failed: %s", cudaGetErrorString(cudaGetLastError()));
        return HCCL_E_RUNTIME;
    }
    MoeParams hp;
    FillCommon(m, hp);
    hp.scratch = m->staticScratch;
    hp.x = (const __nv_bfloat16 *)x; hp.topkIdx = topkIdx; hp.numTokens = numTokens;
    ++c->opSeq;
    CHK_RET(LaunchMoe(m, (void *)MoeRouteKernel, hp, 9105, stream, 1, 1024));
    return LaunchMoe(m, (void *)MoeDispatchKernel, hp, 9103, stream);
}

// Rows dropped because a rank received more than its capacity since the last call (clears the counter).
int HcommMoeTakeOverflow(void *handle)
{
    MoeCtx *m = (MoeCtx *)handle;
    if (!m) return -1;
    uint32_t v = 0, zero = 0;
    cudaMemcpy(&v, m->overflow, 4, cudaMemcpyDeviceToHost);
    if (v) cudaMemcpy(m->overflow, &zero, 4, cudaMemcpyHostToDevice);
    return (int)v;
}

}  // extern "C"
