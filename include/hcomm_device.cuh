// hcomm_device.cuh - device-side primitive library of the SM engine (public: kernels written by users of the
// library include it, the library's own kernels are built from it).
//
// These are the __device__ forms of the verbs in hcomm_primitives.h, written against peer pointers
// into the symmetric heap: system-scope release/acquire flag accesses, bounded waits that record
// where they gave up instead of hanging, a cross-rank barrier between same-index CTAs, vectorised
// copy / reduce loops, and the NVLS multimem wrappers.  Every collective kernel, the schedule
// interpreter and the fused GEMM kernels are built from them.
//
// Reference counterpart: the AscendC base class of the AIV kernels
// (algorithm/base/alg_aiv_template/aiv_communication_base.h:696-1137: CpGM2GM, Record/Wait,
// Record1vN/WaitNv1, head/tail counters) - with the difference that no wait here is unbounded.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "hcomm_comm_dev.h"
#include "hccl/hccl_types.h"

namespace hcdev {

#ifdef HCOMM_DEBUG_BOUNDS
static __device__ const CommDev *g_hcBoundsDev = nullptr;     // communicator of the kernel that began last (one copy per translation unit)
#endif

// ------------------------------------------------------------------------------ flag accesses

__device__ __forceinline__ void StReleaseSys(uint32_t *p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t LdAcquireSys(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void StReleaseSys64(uint64_t *p, uint64_t v)
{
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t LdAcquireSys64(const uint64_t *p)
{
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t LdRelaxedSys(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void StRelaxedSys(uint32_t *p, uint32_t v)
{
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void FenceAcqRelSys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
// Hand-off inside a CTA through a word in shared memory: the writer's earlier accesses (and those it has observed, e.g.
// its warp's after __syncwarp) are ordered before whatever the reader does after it has seen the value.
__device__ __forceinline__ void StReleaseCtaShared(uint32_t *p, uint32_t v)
{
    asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(p)), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t LdAcquireCtaShared(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"((uint32_t)__cvta_generic_to_shared(p)) : "memory");
    return v;
}
__device__ __forceinline__ void RedReleaseSysAdd64(uint64_t *p, uint64_t v)
{
    asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t GlobalTimerNs()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool Aborted(const CommDev *d) { return *(volatile uint32_t *)d->abortWord != 0; }

// Records the first expired wait of the communicator and raises the abort word.
static __device__ __noinline__ void ReportTimeout(const CommDev *d, uint32_t peer, uint32_t kind, uint32_t slot, uint64_t expected,
                                           uint64_t seen)
{
    if (atomicExch_system(&d->status->valid, 1u) == 0u) {
        d->status->rank = (uint32_t)d->rank; d->status->peer = peer; d->status->kind = kind; d->status->slot = slot;
        d->status->block = blockIdx.x; d->status->expected = expected; d->status->seen = seen; d->status->seq = d->opCounters[0];
    }
    *(volatile uint32_t *)d->abortWord = 1u;
    __threadfence_system();
}

// Spins until *flag reaches `target` (wrap-safe), the abort word is raised, or the time budget ends.  The first polls
// come back to back (a barrier between ranks that arrive together costs no more than before); a wait that lasts longer
// sleeps between polls, so that a kernel waiting for a late peer leaves the memory system to the kernels beside it.
__device__ __forceinline__ bool WaitFlagGe32(const CommDev *d, const uint32_t *flag, uint32_t target, uint32_t peer, uint32_t kind,
                                             uint32_t slot)
{
    uint32_t seen = LdAcquireSys(flag);
    if ((int32_t)(seen - target) >= 0) return true;
    uint64_t start = GlobalTimerNs();
    uint32_t ns = 0;
    for (uint32_t it = 1;; ++it) {
        seen = LdAcquireSys(flag);
        if ((int32_t)(seen - target) >= 0) return true;
        if (it >= 128) { if (ns < 512) ns += 32; __nanosleep(ns); }
        if ((it & 63) == 0) {
            if (Aborted(d)) return false;
            if (GlobalTimerNs() - start > d->timeoutNs) { ReportTimeout(d, peer, kind, slot, target, seen); return false; }
        }
    }
}
// The same wait for flags that are polled next to busy tensor-core and copy warps: relaxed loads with a growing
// sleep between them (a poll costs one L2 access and nothing else), and one acquire fence once the value is there.
// `waitedNs`, when given, is increased by the time spent here.
__device__ __forceinline__ bool WaitFlagGe32Quiet(const CommDev *d, const uint32_t *flag, uint32_t target, uint32_t peer, uint32_t kind,
                                                  uint32_t slot, uint64_t *waitedNs = nullptr)
{
    uint32_t seen = LdRelaxedSys(flag);
    if ((int32_t)(seen - target) < 0) {
        const uint64_t start = GlobalTimerNs();
        uint32_t ns = 32;
        for (uint32_t it = 1;; ++it) {
            __nanosleep(ns);
            if (ns < 512) ns *= 2;
            seen = LdRelaxedSys(flag);
            if ((int32_t)(seen - target) >= 0) break;
            if ((it & 31) == 0) {
                if (Aborted(d)) return false;
                if (GlobalTimerNs() - start > d->timeoutNs) { ReportTimeout(d, peer, kind, slot, target, seen); return false; }
            }
        }
        if (waitedNs) *waitedNs += GlobalTimerNs() - start;
    }
    FenceAcqRelSys();
    return true;
}
__device__ __forceinline__ bool WaitFlagGe64(const CommDev *d, const uint64_t *flag, uint64_t target, uint32_t peer, uint32_t kind,
                                             uint32_t slot)
{
    uint64_t seen = LdAcquireSys64(flag);
    if (seen >= target) return true;
    uint64_t start = GlobalTimerNs();
    uint32_t ns = 0;
    for (uint32_t it = 1;; ++it) {
        seen = LdAcquireSys64(flag);
        if (seen >= target) return true;
        if (it >= 128) { if (ns < 512) ns += 32; __nanosleep(ns); }
        if ((it & 63) == 0) {
            if (Aborted(d)) return false;
            if (GlobalTimerNs() - start > d->timeoutNs) { ReportTimeout(d, peer, kind, slot, target, seen); return false; }
        }
    }
}

// Barrier between CTA `blockIdx.x` of every rank.  Writes issued by any thread of the CTA before the
// call are visible to the peers' CTAs after they leave it (bar.sync orders them before the
// signalling threads' system-scope release stores).
__device__ __forceinline__ void CrossRankBarrier(const CommDev *d, uint32_t epoch)
{
    __syncthreads();
    const int t = threadIdx.x;
    if (t < d->nRanks) {
        uint32_t *theirs = (uint32_t *)(HcPeerHeap(d, t) + HC_OFF_BARRIER) + (uint64_t)blockIdx.x * HC_MAX_RANKS + d->rank;
        StReleaseSys(theirs, epoch);
        const uint32_t *mine = (const uint32_t *)(HcPeerHeap(d, d->rank) + HC_OFF_BARRIER) + (uint64_t)blockIdx.x * HC_MAX_RANKS + t;
        WaitFlagGe32(d, mine, epoch, (uint32_t)t, HC_WAIT_BARRIER, blockIdx.x);
    }
    __syncthreads();
}

// Same barrier, arrival announced through the NVLS multicast alias: one multimem.st lands in every rank's slot.
// Used after multimem data stores - a unicast flag write takes another route through the fabric and may overtake
// multicast data, a multicast flag write from the same SM follows it.
__device__ __forceinline__ void CrossRankBarrierMc(const CommDev *d, uint32_t epoch)
{
    __syncthreads();
    const int t = threadIdx.x;
    if (t == 0) {
        uint32_t *slot = (uint32_t *)(d->mcBase + HC_OFF_BARRIER) + (uint64_t)blockIdx.x * HC_MAX_RANKS + d->rank;
        asm volatile("multimem.st.release.sys.global.u32 [%0], %1;" ::"l"(slot), "r"(epoch) : "memory");
    }
    if (t < d->nRanks) {
        const uint32_t *mine = (const uint32_t *)(HcPeerHeap(d, d->rank) + HC_OFF_BARRIER) + (uint64_t)blockIdx.x * HC_MAX_RANKS + t;
        WaitFlagGe32(d, mine, epoch, (uint32_t)t, HC_WAIT_BARRIER, blockIdx.x);
    }
    __syncthreads();
}

// Kernel prologue / epilogue: read the epoch and CCL half, count the launch when the last CTA ends.
struct LaunchState {
    uint32_t epoch0;
    uint32_t half;
    uint32_t seq;      // operators launched on this communicator so far + 1: the same on every rank, never zero in a flag's lifetime
};
static_assert(sizeof(CommDev) <= HC_DEV_COUNTERS_OFFSET, "CommDev outgrew its slot");
__device__ __forceinline__ uint32_t *DevCounters(const CommDev *d) { return (uint32_t *)((char *)d + HC_DEV_COUNTERS_OFFSET); }
__device__ __forceinline__ unsigned long long *DevOpCounters(const CommDev *d) { return (unsigned long long *)((char *)d + HC_DEV_OPCOUNTERS_OFFSET); }
__device__ __forceinline__ LaunchState KernelBegin(const CommDev *d)
{
    LaunchState s;
    const uint32_t *ctr = DevCounters(d);
    s.epoch0 = *(volatile const uint32_t *)&ctr[0];
#ifdef HCOMM_DEBUG_BOUNDS
    g_hcBoundsDev = d;
#endif
    s.seq = *(volatile const uint32_t *)&ctr[1] + 1u;
    s.half = (s.seq - 1u) & 1u;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        if (d->profile) {
            // device-side timestamps of the last kernels, read by the host (HcclDiagGetKernelTimes); only when profiling
            // is on, because the returning atomic sits on the first CTA's critical path
            const unsigned long long seq = atomicAdd(&DevOpCounters(d)[0], 1ull);
            unsigned long long *slot = (unsigned long long *)((char *)d + HC_DEV_TIMES_OFFSET) + 2 * (seq % HC_DEV_TIME_SLOTS);
            slot[0] = GlobalTimerNs();
            slot[1] = 0;
        } else {
            atomicAdd(&DevOpCounters(d)[0], 1ull);
        }
    }
    return s;
}
__device__ __forceinline__ void KernelEnd(const CommDev *d, const LaunchState &s, uint32_t barriersUsed, uint32_t halvesUsed = 1)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t *ctr = DevCounters(d);
        __threadfence();
        uint32_t done = atomicAdd(&ctr[2], 1u);
        if (done == gridDim.x - 1) {
            *(volatile uint32_t *)&ctr[0] = s.epoch0 + barriersUsed;
            *(volatile uint32_t *)&ctr[1] = *(volatile uint32_t *)&ctr[1] + halvesUsed;
            *(volatile uint32_t *)&ctr[2] = 0u;
            if (d->profile) {
                const unsigned long long seq = atomicAdd(&DevOpCounters(d)[1], 1ull);
                ((unsigned long long *)((char *)d + HC_DEV_TIMES_OFFSET))[2 * (seq % HC_DEV_TIME_SLOTS) + 1] = GlobalTimerNs();
            } else {
                atomicAdd(&DevOpCounters(d)[1], 1ull);
            }
        }
    }
}
__device__ __forceinline__ char *CclHalf(const CommDev *d, int rank, uint32_t half)
{
    return HcPeerHeap(d, rank) + d->bufOffset + (uint64_t)half * d->halfBytes;
}

// ----------------------------------------------------------------------------- element algebra

template <typename T> struct AccOf { using type = T; };
template <> struct AccOf<__half> { using type = float; };
template <> struct AccOf<__nv_bfloat16> { using type = float; };

template <typename A> __device__ __forceinline__ A Combine(int op, A a, A b)
{
    switch (op) {
        case HCCL_REDUCE_SUM: return a + b;
        case HCCL_REDUCE_PROD: return a * b;
        case HCCL_REDUCE_MAX: return a > b ? a : b;
        default: return a < b ? a : b;
    }
}
template <typename T> __device__ __forceinline__ typename AccOf<T>::type Widen(T v) { return (typename AccOf<T>::type)v; }
template <> __device__ __forceinline__ float Widen<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float Widen<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T Narrow(typename AccOf<T>::type v) { return (T)v; }
template <> __device__ __forceinline__ __half Narrow<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 Narrow<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <typename A> __device__ __forceinline__ A ScaleAcc(A a, float) { return a; }
template <> __device__ __forceinline__ float ScaleAcc<float>(float a, float s) { return a * s; }
template <> __device__ __forceinline__ double ScaleAcc<double>(double a, float s) { return a * (double)s; }

// 16 bytes of T.
template <typename T> struct Pack {
    static constexpr int N = 16 / sizeof(T);
    union { uint4 v; T e[N]; };
};

__device__ __forceinline__ uint4 Ld16(const void *p) { return *(const uint4 *)p; }
__device__ __forceinline__ void St16(void *p, uint4 v) { *(uint4 *)p = v; }
// Loads that bypass L1: data written by another GPU must not be served from a stale line.
__device__ __forceinline__ uint4 Ld16Volatile(const void *p)
{
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// Copies n bytes dst <- src with all CTAs of the grid taking interleaved 16-byte vectors.  Both
// pointers must be 16-byte aligned; the (n % 16) tail is moved bytewise by CTA 0.
__device__ __forceinline__ void GridCopy16(char *dst, const char *src, uint64_t n)
{
    const uint64_t nvec = n >> 4;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    // eight independent 16-byte loads per thread in flight: the copy is latency bound with the few CTAs it gets
    for (; i + 7 * stride < nvec; i += 8 * stride) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = Ld16Volatile(src + ((i + u * stride) << 4));
#pragma unroll
        for (int u = 0; u < 8; ++u) St16(dst + ((i + u * stride) << 4), v[u]);
    }
    for (; i < nvec; i += stride) St16(dst + (i << 4), Ld16Volatile(src + (i << 4)));
    if (blockIdx.x == 0) {
        const uint64_t tail0 = nvec << 4;
        for (uint64_t b = tail0 + threadIdx.x; b < n; b += blockDim.x) dst[b] = *(volatile const char *)(src + b);
    }
}
// The same partition for any alignment: thread i moves the 16 bytes at offset 16 i as elements of `esz` bytes (1, 2, 4
// or 8), and CTA 0 the (n % 16) tail.  Two phases of one kernel therefore agree on which CTA owns which bytes even
// when only one of them may use vector accesses (say staging -> user buffer at an odd displacement); the per-CTA
// barriers between phases order nothing else.
__device__ __forceinline__ void GridCopyElems(char *dst, const char *src, uint64_t n, uint32_t esz)
{
    const uint64_t nvec = n >> 4;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        char *pd = dst + (i << 4);
        const char *ps = src + (i << 4);
        switch (esz) {
            case 8: {
                uint64_t v[2];
#pragma unroll
                for (int j = 0; j < 2; ++j) v[j] = ((volatile const uint64_t *)ps)[j];
#pragma unroll
                for (int j = 0; j < 2; ++j) ((uint64_t *)pd)[j] = v[j];
                break;
            }
            case 4: {
                uint32_t v[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = ((volatile const uint32_t *)ps)[j];
#pragma unroll
                for (int j = 0; j < 4; ++j) ((uint32_t *)pd)[j] = v[j];
                break;
            }
            case 2: {
                uint16_t v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = ((volatile const uint16_t *)ps)[j];
#pragma unroll
                for (int j = 0; j < 8; ++j) ((uint16_t *)pd)[j] = v[j];
                break;
            }
            default: {
                char v[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = ((volatile const char *)ps)[j];
#pragma unroll
                for (int j = 0; j < 16; ++j) pd[j] = v[j];
                break;
            }
        }
    }
    if (blockIdx.x == 0) {
        const uint64_t tail0 = nvec << 4;
        for (uint64_t b = tail0 + threadIdx.x; b < n; b += blockDim.x) dst[b] = *(volatile const char *)(src + b);
    }
}
// ---------------------------------------------------------------------- debug build: bounds checks
//
// Compiled with -DHCOMM_DEBUG_BOUNDS every grid copy and reduction first checks the ranges it was given: an address
// inside the symmetric heap's address span must stay inside its rank's heap, and a range that starts in a CCL half must
// end in the same half.  A violation is recorded in the communicator's status block (kind HC_WAIT_BOUNDS: peer = rank
// whose heap was addressed, slot = low 32 bits of the offset, expected = limit, seen = end of the range), the abort
// word is raised and the access is skipped - nothing traps.  The checks know the communicator of the kernel that
// called KernelBegin last on this GPU, which is enough for the test runs they are meant for.
#ifdef HCOMM_DEBUG_BOUNDS
static __device__ __noinline__ bool BoundsOk(const void *p, uint64_t n)
{
    const CommDev *d = g_hcBoundsDev;
    if (!d || n == 0) return true;
    const char *c = (const char *)p;
    const char *base = d->heapBase;
    if (c < base || c >= base + (uint64_t)d->nRanks * d->heapStride) return true;        // not heap memory: a caller's buffer
    const uint64_t off = (uint64_t)(c - base) % d->heapStride, heapBytes = (uint64_t)d->heapMB << 20;
    uint64_t limit = heapBytes;
    if (off >= d->bufOffset && off < d->bufOffset + 2 * d->halfBytes) limit = d->bufOffset + ((off - d->bufOffset) / d->halfBytes + 1) * d->halfBytes;
    if (off + n <= limit) return true;
    ReportTimeout(d, (uint32_t)((uint64_t)(c - base) / d->heapStride), HC_WAIT_BOUNDS, (uint32_t)off, limit, off + n);
    return false;
}
#define HC_BOUNDS_OR_RETURN(p, n) do { if (!hcdev::BoundsOk((p), (n))) return; } while (0)
#else
#define HC_BOUNDS_OR_RETURN(p, n) do { } while (0)
#endif

// Picks the widest legal path.
__device__ __forceinline__ void GridCopy(char *dst, const char *src, uint64_t n, uint32_t esz)
{
    if (n == 0 || dst == src) return;
    HC_BOUNDS_OR_RETURN(dst, n);
    HC_BOUNDS_OR_RETURN(src, n);
    if ((((uintptr_t)dst | (uintptr_t)src) & 15) == 0) GridCopy16(dst, src, n);
    else {
        uint32_t w = esz;
        while (w < 8 && ((((uintptr_t)dst | (uintptr_t)src | n) & (2 * w - 1)) == 0)) w *= 2;
        GridCopyElems(dst, src, n, w);
    }
}

// ------------------------------------------------------------------------------ NVLS multimem

template <typename T> struct Multimem;
template <> struct Multimem<float> {
    __device__ static __forceinline__ uint4 LdReduceAdd(const void *mc)
    {
        uint4 v;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
        return v;
    }
};
template <> struct Multimem<__nv_bfloat16> {
    __device__ static __forceinline__ uint4 LdReduceAdd(const void *mc)
    {
        uint4 v;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
        return v;
    }
};
template <> struct Multimem<__half> {
    __device__ static __forceinline__ uint4 LdReduceAdd(const void *mc)
    {
        uint4 v;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
        return v;
    }
};
__device__ __forceinline__ void MultimemSt16(void *mc, uint4 v)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ------------------------------------------------------------------- channels, for user kernels
//
// HcclChannelGetDeviceView(comm, channel, &view) hands a kernel what it needs to talk to the channel's peer: the peer's
// heap as mapped on this GPU, the notify words in both directions and the place of the communication buffer.  The
// calls below are the device forms of the host verbs of hcomm_primitives.h (record / wait on a channel notify, the
// peer's communication buffer for writes and reads).  Notify words only grow: the kernel's caller keeps, per slot, how
// many records it has consumed so far and passes the value to wait for (the host engines do the same bookkeeping).
// Reference counterpart: the device-side channel entities (pkg_inc/hcomm/hcomm_res_entity_defs.h:19-190) and the
// seven-step kernel recipe of docs/zh/comm_op_dev_guide/aiv_comm_op_dev/task_sched.md:25-60.
struct ChannelView {
    char *peerHeap;
    uint64_t *remoteNotify;   // where my records land (in the peer's memory)
    uint64_t *localNotify;    // where the peer's records land (in my memory)
    uint32_t notifyNum;
    uint32_t remoteRank;
    uint64_t cclOffset, cclBytes;
};
// The peer's communication buffer (both halves) as this GPU addresses it.
__device__ __forceinline__ char *ChannelPeerBuffer(const ChannelView *ch) { return ch->peerHeap + ch->cclOffset; }
// Everything the calling thread (and, after a __syncthreads, its CTA) stored before becomes visible to the peer before the record.
__device__ __forceinline__ void ChannelNotifyRecord(const ChannelView *ch, uint32_t slot)
{
    RedReleaseSysAdd64(ch->remoteNotify + slot, 1ull);
}
// Waits until the peer has recorded `expected` times on `slot` or `budgetNs` have passed; false = gave up.
__device__ __forceinline__ bool ChannelNotifyWait(const ChannelView *ch, uint32_t slot, uint64_t expected, uint64_t budgetNs)
{
    const uint64_t *flag = ch->localNotify + slot;
    if (LdAcquireSys64(flag) >= expected) return true;
    const uint64_t start = GlobalTimerNs();
    uint32_t ns = 32;
    for (;;) {
        if (LdAcquireSys64(flag) >= expected) return true;
        if (GlobalTimerNs() - start > budgetNs) return false;
        __nanosleep(ns);
        if (ns < 1024) ns *= 2;
    }
}
// CTA-wide copy of n bytes (both pointers 16-byte aligned, n a multiple of 16); either side may be peer memory.
__device__ __forceinline__ void BlockCopy16(char *dst, const char *src, uint64_t n)
{
    for (uint64_t i = (uint64_t)threadIdx.x * 16; i < n; i += (uint64_t)blockDim.x * 16) St16(dst + i, Ld16Volatile(src + i));
}

}  // namespace hcdev
