// coll_kernels.cu - the specialised collective kernels of the SM and NVLS engines (sm_100a).
//
// Design (all kernels):
//   * CTA b of rank r only ever depends on CTA b of the other ranks: data is partitioned among CTAs
//     by interleaved 16-byte vectors with the same (gridDim, blockDim) on every rank, and phases are
//     separated by CrossRankBarrier between same-index CTAs.  CTAs therefore pipeline naturally:
//     one CTA may be gathering while another still reduces.
//   * Staging lives in this operator's half of the CCL buffer (launch parity), every kernel contains
//     at least one barrier that all ranks wait on, so a rank can be at most one operator ahead of a
//     peer and never overwrites staging that is still being read.
//   * Traffic pattern: "push" (remote stores, posted, one NVLink traversal) for scatter phases,
//     "pull" (remote loads straight into the caller's output) for gather phases, so neither input
//     nor output has to be registered and no extra copy pass over HBM is needed.
//   * Reductions add the ranks' contributions in ascending rank order with fp32 accumulation for
//     16-bit floats: every rank computes bit-identical results and results do not depend on timing
//     (what the reference calls deterministic mode, aiv_all_reduce_deter_910b_*.h).
//   * A scale factor and the narrowing cast are applied in the reduce phase (fused scale/cast).
//
// Kernel inventory and the reference kernels they replace (alg_aiv_template/...):
//   AllReduceOneShot    aiv_all_reduce_910b_smalldata.h, A5 aiv_all_reduce_mesh_1d_oneshot.h
//   AllReduceTwoShot    aiv_all_reduce_910b_middata.h / bigdata.h, A5 mesh_1D_twoshot
//   AllReduceNvls       (no AIV analogue; replaces the CCU in-fabric reduce programs)
//   ReduceScatter(V)    aiv_reduce_scatter_910b_{small,mid,big}data.h, aiv_reduce_scatter_v_910b_*.h
//   AllGather(V)        aiv_all_gather_910b_{small,big}data.h, aiv_all_gather_v_910b_*.h
//   AlltoAll(V/VC)      aiv_all_to_all_910b_smalldata.h, aiv_all_to_all_v_910b.h, ..._vc_910b_*.h
//   Broadcast*          aiv_broadcast_910b_{small,big}data.h
//   Reduce / Scatter / Gather   A5 aiv_reduce_mesh_1d.h, aiv_scatter_mesh_1d.h (+ gather)
//   Send / Recv         A5 aiv_send_mesh_1D.h / aiv_recv_mesh_1D.h
#include <cuda_runtime.h>

#include "../alg/ir.h"
#include "../core/log.h"
#include "coll_kernels.h"
#include "hcomm_device.cuh"

namespace hc {
using namespace hcdev;

#define HC_ARGS const CollArgs &a = (emu != nullptr) ? emu[blockIdx.y] : byval; const CommDev *d = a.dev

namespace {

template <typename T, bool VEC> struct Chunk;
template <typename T> struct Chunk<T, true> {
    static constexpr int N = 16 / sizeof(T);
    union { uint4 v; T e[N]; };
    __device__ __forceinline__ void Load(const char *p) { v = Ld16Volatile(p); }
    __device__ __forceinline__ void Store(char *p) const { St16(p, v); }
};
// Buffers that are not 16-byte aligned: the same 16-byte chunks (by offset from the start of the range), moved element
// by element through the bit pattern.  Both forms give chunk i to the same thread, so two phases of a kernel agree on
// which CTA owns which bytes even when only one of them can use vector accesses - the per-CTA barriers rely on that.
template <int BYTES> struct BitsOf;
template <> struct BitsOf<1> { using type = unsigned char; };
template <> struct BitsOf<2> { using type = unsigned short; };
template <> struct BitsOf<4> { using type = unsigned int; };
template <> struct BitsOf<8> { using type = unsigned long long; };
template <typename T> struct Chunk<T, false> {
    static constexpr int N = 16 / sizeof(T);
    using B = typename BitsOf<sizeof(T)>::type;
    union { uint4 v; T e[N]; B b[N]; };
    __device__ __forceinline__ void Load(const char *p)
    {
#pragma unroll
        for (int j = 0; j < N; ++j) b[j] = ((volatile const B *)p)[j];
    }
    __device__ __forceinline__ void Store(char *p) const
    {
#pragma unroll
        for (int j = 0; j < N; ++j) ((B *)p)[j] = b[j];
    }
};

// dst[k][i] = scale * (src[0][i] op src[1][i] op ... op src[n-1][i]) for every destination k (local or remote) and
// nElems elements, contributions combined in index order (the same order on every rank: results are bit-identical).
// Grid-interleaved by chunks of Chunk::N elements.  A thread keeps M x U 16-byte loads in flight: M sources of U
// chunks; with few ranks U grows so that the bytes in flight per thread stay the same (NVLink and HBM latency are
// hidden by memory-level parallelism, not by occupancy: these kernels run with few CTAs next to compute kernels).
template <typename T, bool VEC, int M, int U>
__device__ __forceinline__ void ReduceLoop(const char *const *src, int n, char *const *dst, int nd, uint64_t nElems, int op, int useScale, float scale)
{
    using A = typename AccOf<T>::type;
    using C = Chunk<T, VEC>;
    constexpr int N = C::N;
    constexpr uint64_t CB = (uint64_t)N * sizeof(T);
    const uint64_t nChunks = nElems / N;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nChunks; i += U * stride) {
        A acc[U][N];
        for (int base = 0; base < n; base += M) {
            C buf[U][M];
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int k = 0; k < M; ++k)
                    if (base + k < n && i + u * stride < nChunks) buf[u][k].Load(src[base + k] + (i + u * stride) * CB);
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int k = 0; k < M; ++k) {
                    if (base + k < n) {
                        if (base + k == 0) {
#pragma unroll
                            for (int j = 0; j < N; ++j) acc[u][j] = Widen<T>(buf[u][k].e[j]);
                        } else {
#pragma unroll
                            for (int j = 0; j < N; ++j) acc[u][j] = Combine<A>(op, acc[u][j], Widen<T>(buf[u][k].e[j]));
                        }
                    }
                }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (i + u * stride < nChunks) {
                C out;
#pragma unroll
                for (int j = 0; j < N; ++j) out.e[j] = Narrow<T>(useScale ? ScaleAcc<A>(acc[u][j], scale) : acc[u][j]);
                for (int k = 0; k < nd; ++k) out.Store(dst[k] + (i + u * stride) * CB);
            }
        }
    }
    if (blockIdx.x == 0) {   // ragged end: fewer elements than one chunk
        for (uint64_t e = nChunks * N + threadIdx.x; e < nElems; e += blockDim.x) {
            const uint64_t off = e * sizeof(T);
            A acc = Widen<T>(*(volatile const T *)(src[0] + off));
            for (int r = 1; r < n; ++r) acc = Combine<A>(op, acc, Widen<T>(*(volatile const T *)(src[r] + off)));
            T v = Narrow<T>(useScale ? ScaleAcc<A>(acc, scale) : acc);
            for (int k = 0; k < nd; ++k) *(T *)(dst[k] + off) = v;
        }
    }
}
// Not inlined: a kernel calls it from several places (per window, staged and zero-copy forms) and the four loop
// variants inside would otherwise be replicated at each call site, which cost the callers half their registers.
template <typename T>
static __device__ __noinline__ void ReduceFanOut(const char *const *src, int n, char *const *dst, int nd, uint64_t nElems, int op, int useScale, float scale)
{
    uintptr_t bits = 0;
    for (int r = 0; r < n; ++r) { HC_BOUNDS_OR_RETURN(src[r], nElems * sizeof(T)); bits |= (uintptr_t)src[r]; }
    for (int k = 0; k < nd; ++k) { HC_BOUNDS_OR_RETURN(dst[k], nElems * sizeof(T)); bits |= (uintptr_t)dst[k]; }
    if ((bits & 15) == 0) {
        if (n <= 2) ReduceLoop<T, true, 2, 4>(src, n, dst, nd, nElems, op, useScale, scale);
        else if (n <= 4) ReduceLoop<T, true, 4, 2>(src, n, dst, nd, nElems, op, useScale, scale);
        else ReduceLoop<T, true, 8, 1>(src, n, dst, nd, nElems, op, useScale, scale);
    } else {
        ReduceLoop<T, false, 8, 1>(src, n, dst, nd, nElems, op, useScale, scale);
    }
}
// One or two destinations (dst2 may be null).
template <typename T>
__device__ __forceinline__ void ReduceAuto(const char *const *src, int n, char *dst1, char *dst2, uint64_t nElems, int op, int useScale, float scale)
{
    char *dst[2] = {dst1, dst2};
    ReduceFanOut<T>(src, n, dst, dst2 ? 2 : 1, nElems, op, useScale, scale);
}

// Element range of slice q when `count` elements are cut into slices of `S`.
__device__ __forceinline__ void SliceRange(uint64_t count, uint64_t S, int q, uint64_t *beg, uint64_t *len)
{
    uint64_t b = (uint64_t)q * S;
    *beg = b < count ? b : count;
    uint64_t e = b + S < count ? b + S : count;
    *len = e > *beg ? e - *beg : 0;
}

__device__ __forceinline__ uint32_t MaybePreBarrier(const CommDev *d, const CollArgs &a, const LaunchState &ls)
{
    if (!a.preBarrier) return 0;
    CrossRankBarrier(d, ls.epoch0 + 1);
    return 1;
}

// Operands larger than the staging walk it in windows of a.winElems elements inside ONE launch; window w works in CCL
// half (first half + w) & 1.  CTAs only ever wait for their namesakes on the other ranks, so CTAs drift apart and the
// copy-in of one window, the reduction of another and the copy-out of a third overlap - the counter-chasing pipeline
// of the reference's big-data kernels (aiv_all_reduce_910b_bigdata.h:90-165,262-289) without its progress counters.
// A half is reused two windows later; by then every peer's namesake CTA has passed a barrier that follows its last
// access to it (the same argument that lets consecutive operators alternate halves).
struct Window {
    uint32_t index, half;
    uint64_t off, cnt;       // elements
};
__device__ __forceinline__ uint32_t WindowCount(const CollArgs &a, uint64_t total)
{
    if (a.winElems == 0 || total <= a.winElems) return 1;
    return (uint32_t)((total + a.winElems - 1) / a.winElems);
}
__device__ __forceinline__ Window WindowAt(const CollArgs &a, const LaunchState &ls, uint32_t w, uint64_t total)
{
    Window x;
    x.index = w;
    x.half = (ls.half + w) & 1u;
    const uint64_t W = (a.winElems == 0 || total <= a.winElems) ? total : a.winElems;
    x.off = (uint64_t)w * W;
    x.cnt = total - x.off < W ? total - x.off : W;
    return x;
}
// Elements per slice when `cnt` elements are cut into n slices of whole 16-byte vectors.
__device__ __forceinline__ uint64_t SliceElems(uint64_t cnt, int n, uint32_t esz)
{
    const uint64_t per = (cnt + n - 1) / n, q = esz >= 16 ? 1 : 16 / esz;
    return (per + q - 1) / q * q;
}

// ------------------------------------------------------------------------------------ AllReduce

// count <= sliceElems; staging: n slots of sliceElems elements.
template <typename T>
__global__ void __launch_bounds__(512) KAllReduceOneShot(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const LaunchState ls = KernelBegin(d);
    uint32_t used = MaybePreBarrier(d, a, ls);
    const int n = d->nRanks, me = d->rank;
    const uint64_t bytes = a.count * sizeof(T), slotBytes = a.sliceElems * sizeof(T);
    for (int i = 1; i < n; ++i) {
        int q = (me + i) % n;
        GridCopy(CclHalf(d, q, ls.half) + (uint64_t)me * slotBytes, (const char *)a.in, bytes, sizeof(T));
    }
    CrossRankBarrier(d, ls.epoch0 + (++used));
    const char *src[HC_KERNEL_MAX_RANKS];
    for (int r = 0; r < n; ++r) src[r] = (r == me) ? (const char *)a.in : CclHalf(d, me, ls.half) + (uint64_t)r * slotBytes;
    ReduceAuto<T>(src, n, (char *)a.out, nullptr, a.count, a.op, a.useScale, a.scale);
    KernelEnd(d, ls, used);
}

// Staging: 2n slots of S elements: [0,n) partial slices arriving from the peers, [n,2n) reduced slices
// arriving from their owners.  A window holds at most n * S elements.  NVLink carries data in the first two phases
// (partials out, then reduced slices out while they are being computed); the last phase is a local copy.
// One window of the two-shot all-reduce.  Out of line and fed with values only (no reference to the argument block):
// inlined into the window loop, the body's loads of the argument block were hoisted and kept alive across the loop,
// which cost the kernel its registers (spills in the copy and reduction loops).
template <typename T>
__device__ __forceinline__ void AllReduceTwoShotBody(const CommDev *d, const char *in, char *out, uint32_t half, uint64_t cnt, uint64_t S, uint32_t epoch,
                                                     int op, int useScale, float scale)
{
    const int n = d->nRanks, me = d->rank;
    const uint64_t slotBytes = S * sizeof(T);
    uint64_t beg, len;
    // scatter: my copy of slice q goes to slot `me` of rank q
    for (int i = 1; i < n; ++i) {
        int q = (me + i) % n;
        SliceRange(cnt, S, q, &beg, &len);
        GridCopy(CclHalf(d, q, half) + (uint64_t)me * slotBytes, in + beg * sizeof(T), len * sizeof(T), sizeof(T));
    }
    CrossRankBarrier(d, epoch);
    // reduce my slice in rank order; the result goes to my output and to slot n+me of every peer
    SliceRange(cnt, S, me, &beg, &len);
    {
        const char *src[HC_KERNEL_MAX_RANKS];
        char *dst[HC_KERNEL_MAX_RANKS];
        for (int r = 0; r < n; ++r) src[r] = (r == me) ? in + beg * sizeof(T) : CclHalf(d, me, half) + (uint64_t)r * slotBytes;
        int nd = 0;
        dst[nd++] = out + beg * sizeof(T);
        for (int i = 1; i < n; ++i) dst[nd++] = CclHalf(d, (me + i) % n, half) + (uint64_t)(n + me) * slotBytes;
        ReduceFanOut<T>(src, n, dst, nd, len, op, useScale, scale);
    }
    CrossRankBarrier(d, epoch + 1);
    // the other slices have landed in my staging: copy them out
    for (int i = 1; i < n; ++i) {
        int q = (me + i) % n;
        SliceRange(cnt, S, q, &beg, &len);
        GridCopy(out + beg * sizeof(T), CclHalf(d, me, half) + (uint64_t)(n + q) * slotBytes, len * sizeof(T), sizeof(T));
    }
}
template <typename T>
static __device__ __noinline__ void AllReduceTwoShotWindow(const CommDev *d, const char *in, char *out, uint32_t half, uint64_t cnt, uint64_t S, uint32_t epoch,
                                                           int op, int useScale, float scale)
{
    AllReduceTwoShotBody<T>(d, in, out, half, cnt, S, epoch, op, useScale, scale);
}
// The operand fits one window (the common case): the body is inlined, nothing is kept across a loop.
template <typename T>
__global__ void __launch_bounds__(512) KAllReduceTwoShot(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const LaunchState ls = KernelBegin(d);
    uint32_t used = MaybePreBarrier(d, a, ls);
    AllReduceTwoShotBody<T>(d, (const char *)a.in, (char *)a.out, ls.half, a.count, a.sliceElems, ls.epoch0 + used + 1, a.op, a.useScale, a.scale);
    KernelEnd(d, ls, used + 2);
}
// Operands beyond one window: the same body, called once per window.
template <typename T>
__global__ void __launch_bounds__(512, 1) KAllReduceTwoShotWin(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const LaunchState ls = KernelBegin(d);
    uint32_t used = MaybePreBarrier(d, a, ls);
    const uint32_t nWin = WindowCount(a, a.count);
    for (uint32_t w = 0; w < nWin; ++w) {
        const Window x = WindowAt(a, ls, w, a.count);
        const uint64_t S = nWin == 1 && a.sliceElems ? a.sliceElems : SliceElems(x.cnt, d->nRanks, sizeof(T));
        AllReduceTwoShotWindow<T>(d, (const char *)a.in + x.off * sizeof(T), (char *)a.out + x.off * sizeof(T), x.half, x.cnt, S, ls.epoch0 + used + 1, a.op,
                                  a.useScale, a.scale);
        used += 2;
    }
    KernelEnd(d, ls, used, nWin);
}

// In-switch reduction.  count*sizeof(T) <= halfBytes; the vector lives in the symmetric half,
// multimem.ld_reduce pulls the sum of all ranks' copies, multimem.st replicates it to all of them.
//
// Which thread touches which 16-byte vector is the same in all three phases: vector i belongs to grid thread
// i % (gridDim * blockDim) - the rule of GridCopy - and, in the reduce phase, to rank (i / (gridDim * blockDim)) % n.
// The per-CTA barriers between the phases pair CTA b of one rank with CTA b of the others, so a vector must never
// change its CTA index from one phase to the next.  The ragged last vector (bytes % 16) belongs to CTA 0 of every
// rank in the copies and to rank 0's CTA 0 in the reduce phase.
template <typename T>
__device__ __forceinline__ uint4 ScaleVec(uint4 v, float scale)
{
    Pack<T> p; p.v = v;
#pragma unroll
    for (int j = 0; j < Pack<T>::N; ++j) p.e[j] = Narrow<T>(Widen<T>(p.e[j]) * scale);
    return p.v;
}
// Reduces, through the switch, the vectors [0, nvec) of `mc` that this rank owns (see above) and hands each sum to sink(i, v).
template <typename T, typename Sink>
__device__ __forceinline__ void NvlsReduceOwned(const char *mc, uint64_t nvec, int n, int me, int useScale, float scale, Sink sink)
{
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, step = (uint64_t)n * stride;
    // A switch round trip takes microseconds: four independent 16-byte reductions per thread are kept in flight.
    constexpr int kUnroll = 4;
    uint64_t i = (uint64_t)me * stride + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + (kUnroll - 1) * step < nvec; i += kUnroll * step) {
        uint4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) v[u] = Multimem<T>::LdReduceAdd(mc + ((i + u * step) << 4));
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) sink(i + u * step, useScale ? ScaleVec<T>(v[u], scale) : v[u]);
    }
    for (; i < nvec; i += step) {
        uint4 v = Multimem<T>::LdReduceAdd(mc + (i << 4));
        sink(i, useScale ? ScaleVec<T>(v, scale) : v);
    }
}

template <typename T>
__global__ void __launch_bounds__(512) KAllReduceNvls(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const LaunchState ls = KernelBegin(d);
    uint32_t used = MaybePreBarrier(d, a, ls);
    const int n = d->nRanks, me = d->rank;
    if (a.inMc && a.outMc) {
        // Registered buffers (both inside a window with a multicast alias): the switch reads the ranks' inputs in place
        // and writes every rank's output in place; nothing is staged.  First barrier: every rank's input is final (its
        // stream has reached this operator).  Last barrier: nobody reuses its input or reads its output before every
        // rank has finished pulling / storing.
        const uint64_t bytes = a.count * sizeof(T), nvec = bytes >> 4;
        CrossRankBarrier(d, ls.epoch0 + (++used));
        char *omc = (char *)a.outMc;
        NvlsReduceOwned<T>((const char *)a.inMc, nvec, n, me, a.useScale, a.scale, [&](uint64_t i, uint4 v) { MultimemSt16(omc + (i << 4), v); });
        if ((bytes & 15) && blockIdx.x == 0 && threadIdx.x < (bytes & 15) / sizeof(T)) {
            // ragged tail (fewer than 16 bytes): every rank reduces it for itself from the peers' inputs with plain loads
            const uint64_t e = (nvec << 4) / sizeof(T) + threadIdx.x;
            typename AccOf<T>::type acc = Widen<T>(*(volatile const T *)((const char *)a.inPeer[0] + e * sizeof(T)));
            for (int r = 1; r < n; ++r) acc = Combine<typename AccOf<T>::type>(a.op, acc, Widen<T>(*(volatile const T *)((const char *)a.inPeer[r] + e * sizeof(T))));
            ((T *)a.out)[e] = Narrow<T>(a.useScale ? ScaleAcc<typename AccOf<T>::type>(acc, a.scale) : acc);
        }
        __threadfence_system();
        CrossRankBarrierMc(d, ls.epoch0 + (++used));
        KernelEnd(d, ls, used, 0);
        return;
    }
    const uint32_t nWin = WindowCount(a, a.count);
    for (uint32_t w = 0; w < nWin; ++w) {
        const Window x = WindowAt(a, ls, w, a.count);
        const uint64_t bytes = x.cnt * sizeof(T);
        char *mine = CclHalf(d, me, x.half);
        GridCopy(mine, (const char *)a.in + x.off * sizeof(T), bytes, sizeof(T));
        CrossRankBarrier(d, ls.epoch0 + (++used));
        {
            char *mc = d->mcBase + d->bufOffset + (uint64_t)x.half * d->halfBytes;
            const uint64_t nvec = bytes >> 4;
            NvlsReduceOwned<T>(mc, nvec, n, me, a.useScale, a.scale, [&](uint64_t i, uint4 v) { MultimemSt16(mc + (i << 4), v); });
            if ((bytes & 15) && me == 0 && blockIdx.x == 0 && threadIdx.x == 0) {
                // the padding bytes of the last vector are whatever the half held on each rank: harmless, they are not copied out
                uint4 v = Multimem<T>::LdReduceAdd(mc + (nvec << 4));
                MultimemSt16(mc + (nvec << 4), a.useScale ? ScaleVec<T>(v, a.scale) : v);
            }
            // Multicast stores travel through the switch; the barrier's release by another thread of the CTA does not
            // cover them, so every thread fences its own before the CTA signals.
            __threadfence_system();
        }
        CrossRankBarrierMc(d, ls.epoch0 + (++used));
        GridCopy((char *)a.out + x.off * sizeof(T), mine, bytes, sizeof(T));
    }
    KernelEnd(d, ls, used, nWin);
}

// The same for a large operand that is not registered, as a software pipeline over windows: while window w is reduced
// and replicated through the switch in one CCL half, the same threads copy the result of window w - 1 out of the other
// half and the input of window w + 1 into it.  The link-bound phase and the two HBM-bound copies then run at the same
// time instead of one after the other, and there is one cross-rank barrier per window instead of two.
//   * A "row" is n * gridsize vectors; thread g of the grid owns column g of every row: it reduces the vector of
//     sub-row `me` (the ownership rule above) and copies the vectors of all n sub-rows.  A vector keeps its thread, hence
//     its CTA, in every phase, which is what the per-CTA barriers need.
//   * Copy-out and copy-in of the other half touch the same addresses: a thread reads a vector's old contents (result
//     of window w - 1) before it overwrites them (input of window w + 1).
//   * The barrier at the end of step w orders: results of w on every rank before anyone copies them out (step w + 1);
//     input of w + 1 on every rank before anyone reduces it; everybody's reads of half (w & 1) before window w + 2
//     is copied into it.
// Needs count * sizeof(T) and the window to be whole 16-byte vectors (the host checks).  The reference's big-data
// all-reduce (aiv_all_reduce_910b_bigdata.h:90-165,262-289) overlaps the same three stages with progress counters.
template <typename T>
__global__ void __launch_bounds__(512) KAllReduceNvlsPipe(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const LaunchState ls = KernelBegin(d);
    uint32_t used = MaybePreBarrier(d, a, ls);
    const int n = d->nRanks, me = d->rank;
    const uint32_t nWin = WindowCount(a, a.count);
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t rowVecs = (uint64_t)n * stride;
    {
        const Window x0 = WindowAt(a, ls, 0, a.count);
        GridCopy(CclHalf(d, me, x0.half), (const char *)a.in + x0.off * sizeof(T), x0.cnt * sizeof(T), sizeof(T));
    }
    CrossRankBarrier(d, ls.epoch0 + (++used));
    for (uint32_t w = 0; w < nWin; ++w) {
        const Window x = WindowAt(a, ls, w, a.count);
        char *mc = d->mcBase + d->bufOffset + (uint64_t)x.half * d->halfBytes;
        char *other = CclHalf(d, me, x.half ^ 1u);
        const uint64_t nvec = (x.cnt * sizeof(T)) >> 4;
        uint64_t ovec = 0, ivec = 0;
        char *outp = nullptr;
        const char *inp = nullptr;
        if (w > 0) {
            const Window xo = WindowAt(a, ls, w - 1, a.count);
            ovec = (xo.cnt * sizeof(T)) >> 4;
            outp = (char *)a.out + xo.off * sizeof(T);
        }
        if (w + 1 < nWin) {
            const Window xi = WindowAt(a, ls, w + 1, a.count);
            ivec = (xi.cnt * sizeof(T)) >> 4;
            inp = (const char *)a.in + xi.off * sizeof(T);
        }
        uint64_t most = nvec > ovec ? nvec : ovec;
        if (ivec > most) most = ivec;
        for (uint64_t row = 0; row < most; row += rowVecs) {
            const uint64_t base = row + g, mine = base + (uint64_t)me * stride;
            uint4 red = make_uint4(0, 0, 0, 0);
            if (mine < nvec) red = Multimem<T>::LdReduceAdd(mc + (mine << 4));          // in flight while the copies run
            for (int r0 = 0; r0 < n; r0 += 4) {
                uint4 o[4], c[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint64_t idx = base + (uint64_t)(r0 + u) * stride;
                    if (r0 + u < n && idx < ovec) o[u] = Ld16Volatile(other + (idx << 4));
                    if (r0 + u < n && idx < ivec) c[u] = Ld16Volatile(inp + (idx << 4));
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint64_t idx = base + (uint64_t)(r0 + u) * stride;
                    if (r0 + u < n && idx < ovec) St16(outp + (idx << 4), o[u]);
                    if (r0 + u < n && idx < ivec) St16(other + (idx << 4), c[u]);
                }
            }
            if (mine < nvec) MultimemSt16(mc + (mine << 4), a.useScale ? ScaleVec<T>(red, a.scale) : red);
        }
        __threadfence_system();      // multicast stores travel through the switch: every thread fences its own
        CrossRankBarrierMc(d, ls.epoch0 + (++used));
    }
    {
        const Window xl = WindowAt(a, ls, nWin - 1, a.count);
        GridCopy((char *)a.out + xl.off * sizeof(T), CclHalf(d, me, xl.half), xl.cnt * sizeof(T), sizeof(T));
    }
    KernelEnd(d, ls, used, nWin);
}

// Column window [c0, c0 + cap) of a block of `cnt` elements: how many of its elements fall inside.
__device__ __forceinline__ uint64_t InWindow(uint64_t cnt, uint64_t c0, uint64_t cap)
{
    const uint64_t hi = cnt < c0 + cap ? cnt : c0 + cap;
    return hi > c0 ? hi - c0 : 0;
}

// In-switch reduce-scatter: every rank parks (a window of) its n blocks in its half, then rank r pulls the sum of
// block r through the switch straight into its output.  Blocks are whole 16-byte vectors (count * sizeof(T) % 16 == 0,
// checked by the host).  With a registered input that has a multicast alias nothing is parked at all.
// Replaces the in-fabric reduce-scatter programs of the reference (alg_ccu_context/.../reduce_scatter mesh1d).
template <typename T>
__device__ __forceinline__ void NvlsPullBlock(const char *mc, char *out, uint64_t vecs, int useScale, float scale)
{
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    constexpr int kUnroll = 4;
    for (; j + (kUnroll - 1) * stride < vecs; j += kUnroll * stride) {
        uint4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) v[u] = Multimem<T>::LdReduceAdd(mc + ((j + u * stride) << 4));
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) St16(out + ((j + u * stride) << 4), useScale ? ScaleVec<T>(v[u], scale) : v[u]);
    }
    for (; j < vecs; j += stride) {
        uint4 v = Multimem<T>::LdReduceAdd(mc + (j << 4));
        St16(out + (j << 4), useScale ? ScaleVec<T>(v, scale) : v);
    }
}
template <typename T>
__global__ void __launch_bounds__(512) KReduceScatterNvls(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const LaunchState ls = KernelBegin(d);
    uint32_t used = MaybePreBarrier(d, a, ls);
    const int n = d->nRanks, me = d->rank;
    if (a.inMc) {
        CrossRankBarrier(d, ls.epoch0 + (++used));           // every rank's input is final
        NvlsPullBlock<T>((const char *)a.inMc + (uint64_t)me * a.count * sizeof(T), (char *)a.out, a.count * sizeof(T) >> 4, a.useScale, a.scale);
        CrossRankBarrier(d, ls.epoch0 + (++used));           // nobody reuses its input while a peer still pulls from it
        KernelEnd(d, ls, used, 0);
        return;
    }
    const uint64_t cap = a.sliceElems;                       // elements of every block per window: n * cap * sizeof(T) <= half
    const uint32_t nWin = (uint32_t)((a.count + cap - 1) / cap);
    for (uint32_t w = 0; w < nWin; ++w) {
        const uint32_t half = (ls.half + w) & 1u;
        const uint64_t c0 = (uint64_t)w * cap, len = InWindow(a.count, c0, cap), slotBytes = len * sizeof(T);
        char *mine = CclHalf(d, me, half);
        // slot q of my half = my contribution to block q; vector j of a slot belongs to grid thread j % (grid size) in both phases
        for (int q = 0; q < n; ++q) GridCopy(mine + (uint64_t)q * slotBytes, (const char *)a.in + ((uint64_t)q * a.count + c0) * sizeof(T), slotBytes, sizeof(T));
        CrossRankBarrier(d, ls.epoch0 + (++used));
        const char *mc = d->mcBase + d->bufOffset + (uint64_t)half * d->halfBytes;
        NvlsPullBlock<T>(mc + (uint64_t)me * slotBytes, (char *)a.out + c0 * sizeof(T), slotBytes >> 4, a.useScale, a.scale);
        // this half is written again two windows (or two operators) from now; a barrier that every rank reaches only
        // after leaving this loop lies in between
    }
    KernelEnd(d, ls, used, nWin);
}

// Input: n blocks; block q has sendCounts[q] elements at sendDispls[q]; output sendCounts[me] elements.
// Staging: n slots of sliceElems elements; longer blocks travel in column windows of sliceElems (a.count = longest block).
// One column window of the reduce-scatter: block q of this rank's input starts at in + dspBytes[q] and has lenBytes[q]
// bytes inside the window.  Out of line and fed with values only, like AllReduceTwoShotWindow.
template <typename T>
__device__ __forceinline__ void ReduceScatterBody(const CommDev *d, const char *in, char *out, const uint64_t *dspBytes, const uint64_t *lenBytes, uint32_t half,
                                                  uint64_t slotBytes, uint32_t epoch, int op, int useScale, float scale)
{
    const int n = d->nRanks, me = d->rank;
    for (int i = 1; i < n; ++i) {
        int q = (me + i) % n;
        GridCopy(CclHalf(d, q, half) + (uint64_t)me * slotBytes, in + dspBytes[q], lenBytes[q], sizeof(T));
    }
    CrossRankBarrier(d, epoch);
    const char *src[HC_KERNEL_MAX_RANKS];
    for (int r = 0; r < n; ++r) src[r] = (r == me) ? in + dspBytes[me] : CclHalf(d, me, half) + (uint64_t)r * slotBytes;
    ReduceAuto<T>(src, n, out, nullptr, lenBytes[me] / sizeof(T), op, useScale, scale);
}
template <typename T>
static __device__ __noinline__ void ReduceScatterWindow(const CommDev *d, const char *in, char *out, const uint64_t *dspBytes, const uint64_t *lenBytes, uint32_t half,
                                                        uint64_t slotBytes, uint32_t epoch, int op, int useScale, float scale)
{
    ReduceScatterBody<T>(d, in, out, dspBytes, lenBytes, half, slotBytes, epoch, op, useScale, scale);
}
// Every block fits a staging slot (the common case): one window, body inlined.
template <typename T>
__global__ void __launch_bounds__(512) KReduceScatter(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const LaunchState ls = KernelBegin(d);
    uint32_t used = MaybePreBarrier(d, a, ls);
    const int n = d->nRanks;
    uint64_t dsp[HC_KERNEL_MAX_RANKS], len[HC_KERNEL_MAX_RANKS];
    for (int q = 0; q < n; ++q) { dsp[q] = a.sendDispls[q] * sizeof(T); len[q] = a.sendCounts[q] * sizeof(T); }
    ReduceScatterBody<T>(d, (const char *)a.in, (char *)a.out, dsp, len, ls.half, a.sliceElems * sizeof(T), ls.epoch0 + (++used), a.op, a.useScale, a.scale);
    KernelEnd(d, ls, used);
}
// Registered input: the peers' blocks are read where they are - no staging, one pass.
template <typename T>
__global__ void __launch_bounds__(512) KReduceScatterInPlace(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const LaunchState ls = KernelBegin(d);
    uint32_t used = MaybePreBarrier(d, a, ls);
    const int n = d->nRanks, me = d->rank;
    CrossRankBarrier(d, ls.epoch0 + (++used));           // every rank's input is final
    const char *src[HC_KERNEL_MAX_RANKS];
    for (int r = 0; r < n; ++r) src[r] = (const char *)a.inPeer[r] + a.sendDispls[me] * sizeof(T);
    ReduceAuto<T>(src, n, (char *)a.out, nullptr, a.sendCounts[me], a.op, a.useScale, a.scale);
    CrossRankBarrier(d, ls.epoch0 + (++used));           // nobody reuses its input while a peer still reads it
    KernelEnd(d, ls, used, 0);
}
// Blocks longer than a staging slot: column windows of sliceElems, the body called once per window.
template <typename T>
__global__ void __launch_bounds__(512, 1) KReduceScatterWin(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const LaunchState ls = KernelBegin(d);
    uint32_t used = MaybePreBarrier(d, a, ls);
    const int n = d->nRanks;
    const uint64_t cap = a.sliceElems;
    uint32_t nWin = (uint32_t)((a.count + cap - 1) / cap);
    if (nWin == 0) nWin = 1;
    for (uint32_t w = 0; w < nWin; ++w) {
        const uint64_t c0 = (uint64_t)w * cap;
        uint64_t dsp[HC_KERNEL_MAX_RANKS], len[HC_KERNEL_MAX_RANKS];
        for (int q = 0; q < n; ++q) {
            dsp[q] = (a.sendDispls[q] + c0) * sizeof(T);
            len[q] = InWindow(a.sendCounts[q], c0, cap) * sizeof(T);
        }
        ReduceScatterWindow<T>(d, (const char *)a.in, (char *)a.out + c0 * sizeof(T), dsp, len, (ls.half + w) & 1u, cap * sizeof(T), ls.epoch0 + (++used), a.op,
                               a.useScale, a.scale);
    }
    KernelEnd(d, ls, used, nWin);
}

// --------------------------------------------------------------------------------------- Reduce

template <typename T>
__global__ void __launch_bounds__(512) KReduce(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const LaunchState ls = KernelBegin(d);
    uint32_t used = MaybePreBarrier(d, a, ls);
    const int n = d->nRanks, me = d->rank;
    const uint64_t S = a.sliceElems, slotBytes = S * sizeof(T);
    uint64_t beg, len;
    for (int i = 1; i < n; ++i) {
        int q = (me + i) % n;
        SliceRange(a.count, S, q, &beg, &len);
        GridCopy(CclHalf(d, q, ls.half) + (uint64_t)me * slotBytes, (const char *)a.in + beg * sizeof(T), len * sizeof(T), sizeof(T));
    }
    CrossRankBarrier(d, ls.epoch0 + (++used));
    SliceRange(a.count, S, me, &beg, &len);
    char *red = CclHalf(d, me, ls.half) + (uint64_t)n * slotBytes;
    {
        const char *src[HC_KERNEL_MAX_RANKS];
        for (int r = 0; r < n; ++r) src[r] = (r == me) ? (const char *)a.in + beg * sizeof(T) : CclHalf(d, me, ls.half) + (uint64_t)r * slotBytes;
        ReduceAuto<T>(src, n, red, me == a.root ? (char *)a.out + beg * sizeof(T) : nullptr, len, a.op, a.useScale, a.scale);
    }
    CrossRankBarrier(d, ls.epoch0 + (++used));
    if (me == a.root) {
        for (int i = 1; i < n; ++i) {
            int q = (me + i) % n;
            SliceRange(a.count, S, q, &beg, &len);
            GridCopy((char *)a.out + beg * sizeof(T), CclHalf(d, q, ls.half) + (uint64_t)n * slotBytes, len * sizeof(T), sizeof(T));
        }
    }
    KernelEnd(d, ls, used);
}

// ------------------------------------------------------------------------- byte-moving kernels

// AllGather(V): my block has recvCounts[me] elements and lands at recvDispls[q] of everyone's output (counts in
// elements of elemSize bytes).  Blocks longer than the staging (sliceElems elements) travel in column windows
// (a.count = longest block).  With a registered input (a.inPeer set) the peers' blocks are pulled from where they are.
__global__ void __launch_bounds__(512) KAllGather(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const LaunchState ls = KernelBegin(d);
    uint32_t used = MaybePreBarrier(d, a, ls);
    const int n = d->nRanks, me = d->rank;
    const uint64_t es = a.elemSize;
    if (a.inPeer[0]) {
        CrossRankBarrier(d, ls.epoch0 + (++used));           // every rank's input is final
        for (int i = 0; i < n; ++i) {
            int q = (me + i) % n;
            GridCopy((char *)a.out + a.recvDispls[q] * es, (const char *)a.inPeer[q], a.recvCounts[q] * es, a.elemSize);
        }
        CrossRankBarrier(d, ls.epoch0 + (++used));           // nobody reuses its input while a peer still reads it
        KernelEnd(d, ls, used, 0);
        return;
    }
    const uint64_t cap = a.sliceElems;
    uint32_t nWin = (uint32_t)((a.count + cap - 1) / cap);
    if (nWin == 0) nWin = 1;
    for (uint32_t w = 0; w < nWin; ++w) {
        const uint32_t half = (ls.half + w) & 1u;
        const uint64_t c0 = (uint64_t)w * cap;
        const char *in = (const char *)a.in + c0 * es;
        const uint64_t mineBytes = InWindow(a.recvCounts[me], c0, cap) * es;
        GridCopy(CclHalf(d, me, half), in, mineBytes, a.elemSize);
        CrossRankBarrier(d, ls.epoch0 + (++used));
        GridCopy((char *)a.out + (a.recvDispls[me] + c0) * es, in, mineBytes, a.elemSize);
        for (int i = 1; i < n; ++i) {
            int q = (me + i) % n;
            GridCopy((char *)a.out + (a.recvDispls[q] + c0) * es, CclHalf(d, q, half), InWindow(a.recvCounts[q], c0, cap) * es, a.elemSize);
        }
    }
    KernelEnd(d, ls, used, nWin);
}

// All-gather through the switch: every rank stores its block ONCE to the multicast alias and the switch replicates it
// into all ranks' memory, so a GPU sends 1/(n-1) of what the unicast form sends.  Equal blocks of whole 16-byte
// vectors from a 16-byte aligned input (checked by the host).  With a registered output that has a multicast alias the
// blocks land in the output itself; otherwise in the staging half (windows of sliceElems elements per rank) and a
// local copy follows.  Replaces the in-fabric all-gather programs of the reference (alg_ccu_context/.../all_gather mesh1d).
__device__ __forceinline__ void NvlsStoreBlock(char *mc, const char *src, uint64_t vecs)
{
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; j + 3 * stride < vecs; j += 4 * stride) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = Ld16(src + ((j + u * stride) << 4));
#pragma unroll
        for (int u = 0; u < 4; ++u) MultimemSt16(mc + ((j + u * stride) << 4), v[u]);
    }
    for (; j < vecs; j += stride) MultimemSt16(mc + (j << 4), Ld16(src + (j << 4)));
    __threadfence_system();      // multicast stores are fenced by the thread that issued them
}
__global__ void __launch_bounds__(512) KAllGatherNvls(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const LaunchState ls = KernelBegin(d);
    uint32_t used = MaybePreBarrier(d, a, ls);
    const int n = d->nRanks, me = d->rank;
    const uint64_t es = a.elemSize, blockBytes = a.count * es;
    if (a.outMc) {
        CrossRankBarrier(d, ls.epoch0 + (++used));           // every rank has left whatever last touched its output
        NvlsStoreBlock((char *)a.outMc + (uint64_t)me * blockBytes, (const char *)a.in, blockBytes >> 4);
        CrossRankBarrierMc(d, ls.epoch0 + (++used));
        KernelEnd(d, ls, used, 0);
        return;
    }
    const uint64_t cap = a.sliceElems;                       // elements per rank and window: n * cap * es <= half
    const uint32_t nWin = (uint32_t)((a.count + cap - 1) / cap);
    for (uint32_t w = 0; w < nWin; ++w) {
        const uint32_t half = (ls.half + w) & 1u;
        const uint64_t c0 = (uint64_t)w * cap, slotBytes = InWindow(a.count, c0, cap) * es;
        char *mc = d->mcBase + d->bufOffset + (uint64_t)half * d->halfBytes;
        // Peers read this half (their copy-out of two windows / operators ago) only before a barrier that I have passed.
        NvlsStoreBlock(mc + (uint64_t)me * slotBytes, (const char *)a.in + c0 * es, slotBytes >> 4);
        CrossRankBarrierMc(d, ls.epoch0 + (++used));
        for (int i = 0; i < n; ++i) {
            int q = (me + i) % n;
            GridCopy((char *)a.out + ((uint64_t)q * a.count + c0) * es, CclHalf(d, me, half) + (uint64_t)q * slotBytes, slotBytes, a.elemSize);
        }
    }
    KernelEnd(d, ls, used, nWin);
}

// AlltoAll(V/VC): block for rank q has sendCounts[q] elements at sendDispls[q]; block from rank r has
// recvCounts[r] elements at recvDispls[r].  Blocks longer than a staging slot (sliceElems) travel in
// column windows; consecutive windows alternate between the two CCL halves.  With variable counts
// (a.root != 0) no rank knows the longest block of the job, so the ranks first agree on it in-kernel:
// everyone publishes its own maximum (a.count) in every peer's meta slot, one barrier, take the max.
__global__ void __launch_bounds__(512) KAlltoAll(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const LaunchState ls = KernelBegin(d);
    uint32_t used = MaybePreBarrier(d, a, ls);
    const int n = d->nRanks, me = d->rank;
    const uint64_t es = a.elemSize, cap = a.sliceElems, slotBytes = cap * es;
    uint64_t gmax = a.count;
    if (a.root != 0) {
        if ((int)threadIdx.x < n) ((volatile uint64_t *)(HcPeerHeap(d, threadIdx.x) + HC_OFF_META))[me] = a.count;
        CrossRankBarrier(d, ls.epoch0 + (++used));
        const volatile uint64_t *meta = (const volatile uint64_t *)(HcPeerHeap(d, me) + HC_OFF_META);
        for (int r = 0; r < n; ++r) { uint64_t v = meta[r]; gmax = v > gmax ? v : gmax; }
    }
    uint32_t nWin = (uint32_t)((gmax + cap - 1) / cap);
    if (nWin == 0) nWin = 1;
    for (uint32_t w = 0; w < nWin; ++w) {
        const uint32_t half = (ls.half + w) & 1u;
        const uint64_t col0 = (uint64_t)w * cap, col1 = col0 + cap;
        auto window = [&](uint64_t cnt) { uint64_t hi = cnt < col1 ? cnt : col1; return hi > col0 ? hi - col0 : (uint64_t)0; };
        for (int i = 1; i < n; ++i) {
            int q = (me + i) % n;
            GridCopy(CclHalf(d, q, half) + (uint64_t)me * slotBytes, (const char *)a.in + (a.sendDispls[q] + col0) * es, window(a.sendCounts[q]) * es, a.elemSize);
        }
        GridCopy((char *)a.out + (a.recvDispls[me] + col0) * es, (const char *)a.in + (a.sendDispls[me] + col0) * es, window(a.sendCounts[me]) * es, a.elemSize);
        CrossRankBarrier(d, ls.epoch0 + (++used));
        for (int i = 1; i < n; ++i) {
            int r = (me + n - i) % n;
            GridCopy((char *)a.out + (a.recvDispls[r] + col0) * es, CclHalf(d, me, half) + (uint64_t)r * slotBytes, window(a.recvCounts[r]) * es, a.elemSize);
        }
    }
    KernelEnd(d, ls, used, nWin);
}

// Broadcast, root pushes the whole buffer to every peer's staging.
__global__ void __launch_bounds__(512) KBroadcastPush(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const LaunchState ls = KernelBegin(d);
    uint32_t used = MaybePreBarrier(d, a, ls);
    const int n = d->nRanks, me = d->rank;
    const uint64_t bytes = a.count * a.elemSize;
    if (me == a.root) {
        for (int i = 1; i < n; ++i) GridCopy(CclHalf(d, (me + i) % n, ls.half), (const char *)a.in, bytes, a.elemSize);
        GridCopy((char *)a.out, (const char *)a.in, bytes, a.elemSize);
    }
    CrossRankBarrier(d, ls.epoch0 + (++used));
    if (me != a.root) GridCopy((char *)a.out, CclHalf(d, me, ls.half), bytes, a.elemSize);
    KernelEnd(d, ls, used);
}

// Broadcast as scatter + all-gather: the root sends slice q to rank q only; everyone then pulls
// slice q from rank q.  The root's outbound traffic is one buffer instead of n-1.
__global__ void __launch_bounds__(512) KBroadcastTwoShot(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const LaunchState ls = KernelBegin(d);
    uint32_t used = MaybePreBarrier(d, a, ls);
    const int n = d->nRanks, me = d->rank;
    const uint64_t es = a.elemSize, S = a.sliceElems;
    uint64_t beg, len;
    if (me == a.root) {
        for (int i = 0; i < n; ++i) {
            int q = (me + i) % n;
            SliceRange(a.count, S, q, &beg, &len);
            GridCopy(CclHalf(d, q, ls.half), (const char *)a.in + beg * es, len * es, a.elemSize);
        }
        GridCopy((char *)a.out, (const char *)a.in, a.count * es, a.elemSize);
    }
    CrossRankBarrier(d, ls.epoch0 + (++used));
    if (me != a.root) {
        for (int i = 0; i < n; ++i) {
            int q = (me + i) % n;
            SliceRange(a.count, S, q, &beg, &len);
            GridCopy((char *)a.out + beg * es, CclHalf(d, q, ls.half), len * es, a.elemSize);
        }
    }
    KernelEnd(d, ls, used);
}

// Broadcast through the switch: the root stores once to the multicast alias, the switch replicates.
__global__ void __launch_bounds__(512) KBroadcastNvls(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const LaunchState ls = KernelBegin(d);
    uint32_t used = MaybePreBarrier(d, a, ls);
    const int me = d->rank;
    const uint64_t bytes = a.count * a.elemSize;
    CrossRankBarrier(d, ls.epoch0 + (++used));   // everyone has left the previous use of this half
    if (me == a.root) {
        char *mc = d->mcBase + d->bufOffset + (uint64_t)ls.half * d->halfBytes;
        const char *src = (const char *)a.in;
        const uint64_t nvec = bytes >> 4, stride = (uint64_t)gridDim.x * blockDim.x;
        if (((uintptr_t)src & 15) == 0) {
            for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) MultimemSt16(mc + (i << 4), Ld16(src + (i << 4)));
            if (blockIdx.x == 0 && threadIdx.x == 0 && (bytes & 15)) {   // last partial vector: zero-padded
                Pack<char> p; p.v = make_uint4(0, 0, 0, 0);
                for (uint64_t b = 0; b < (bytes & 15); ++b) p.e[b] = src[(nvec << 4) + b];
                MultimemSt16(mc + (nvec << 4), p.v);
            }
        } else {
            for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < ((bytes + 15) >> 4); i += stride) {
                Pack<char> p; p.v = make_uint4(0, 0, 0, 0);
                for (int b = 0; b < 16; ++b) if ((i << 4) + b < bytes) p.e[b] = src[(i << 4) + b];
                MultimemSt16(mc + (i << 4), p.v);
            }
        }
        GridCopy((char *)a.out, src, bytes, a.elemSize);
        __threadfence_system();   // multicast stores are fenced by the thread that issued them
    }
    CrossRankBarrierMc(d, ls.epoch0 + (++used));
    if (me != a.root) GridCopy((char *)a.out, CclHalf(d, me, ls.half), bytes, a.elemSize);
    KernelEnd(d, ls, used);
}

// Scatter: root's block q (count elements each) goes to rank q.
__global__ void __launch_bounds__(512) KScatter(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const LaunchState ls = KernelBegin(d);
    uint32_t used = MaybePreBarrier(d, a, ls);
    const int n = d->nRanks, me = d->rank;
    const uint64_t bytes = a.count * a.elemSize;
    if (me == a.root) {
        for (int i = 1; i < n; ++i) {
            int q = (me + i) % n;
            GridCopy(CclHalf(d, q, ls.half), (const char *)a.in + (uint64_t)q * bytes, bytes, a.elemSize);
        }
        GridCopy((char *)a.out, (const char *)a.in + (uint64_t)me * bytes, bytes, a.elemSize);
    }
    CrossRankBarrier(d, ls.epoch0 + (++used));
    if (me != a.root) GridCopy((char *)a.out, CclHalf(d, me, ls.half), bytes, a.elemSize);
    KernelEnd(d, ls, used);
}

// Gather: every rank pushes its block into slot `me` of the root.
__global__ void __launch_bounds__(512) KGather(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const LaunchState ls = KernelBegin(d);
    uint32_t used = MaybePreBarrier(d, a, ls);
    const int n = d->nRanks, me = d->rank;
    const uint64_t bytes = a.count * a.elemSize, slotBytes = a.sliceElems * a.elemSize;
    if (me != a.root) GridCopy(CclHalf(d, a.root, ls.half) + (uint64_t)me * slotBytes, (const char *)a.in, bytes, a.elemSize);
    CrossRankBarrier(d, ls.epoch0 + (++used));
    if (me == a.root) {
        GridCopy((char *)a.out + (uint64_t)me * bytes, (const char *)a.in, bytes, a.elemSize);
        for (int i = 1; i < n; ++i) {
            int r = (me + i) % n;
            GridCopy((char *)a.out + (uint64_t)r * bytes, CclHalf(d, me, ls.half) + (uint64_t)r * slotBytes, bytes, a.elemSize);
        }
    }
    KernelEnd(d, ls, used);
}

__global__ void __launch_bounds__(512) KBarrier(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const LaunchState ls = KernelBegin(d);
    CrossRankBarrier(d, ls.epoch0 + 1);
    KernelEnd(d, ls, 1);
}

// ---------------------------------------------------------------------------------- Send / Recv
//
// The landing area of (receiver, sender) is two sub-slots; chunk k uses sub-slot k%2.  Two 64-bit
// counters per ordered pair live in the receiver's / sender's control region:
//   data[receiver][sender]   chunks written so far (sender increments, release)
//   ack [sender][receiver]   chunks consumed so far (receiver increments, release)
// Both only grow over the life of the communicator; the host passes their values before this call.
// These kernels involve two ranks only, so they touch neither the barrier epoch nor the CCL halves.

__device__ __forceinline__ uint64_t *P2pWord(const CommDev *d, int owner, int other, int which)
{
    return (uint64_t *)(HcPeerHeap(d, owner) + HC_OFF_P2P) + (uint64_t)other * 8 + which;
}

// Chunk completion inside one kernel is tracked with a device-local counter per (direction, peer) instead of a
// grid-wide barrier, so these kernels are ordinary launches: a send and a receive kernel of the same rank must be
// able to run side by side (each waits for the other GPU), which cooperative launches do not promise.
// CTAs of one kernel can be at most one chunk apart from each other (chunk k+2 reuses the sub-slot of chunk k and
// needs its acknowledgement, which needs every CTA to have finished chunk k), so two counters per (direction, peer),
// selected by chunk parity, are enough; the last CTA to finish a chunk resets the counter and signals the peer.
__device__ __forceinline__ uint32_t *P2pDone(const CommDev *d, int dir, int peer, uint64_t chunk)
{
    return d->blocksDone + 6 + ((dir * HC_KERNEL_MAX_RANKS + peer) * 2 + (int)(chunk & 1));
}

__device__ __forceinline__ bool LastCtaOfChunk(uint32_t *counter)
{
    __shared__ uint32_t isLast;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        uint32_t old = atomicAdd(counter, 1u);
        isLast = (old == gridDim.x - 1) ? 1u : 0u;
        if (isLast) { *(volatile uint32_t *)counter = 0u; __threadfence(); }
    }
    __syncthreads();
    return isLast != 0;
}

__global__ void __launch_bounds__(512) KSend(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const int me = d->rank, dst = a.peer;
    const uint64_t bytes = a.count * a.elemSize, sub = a.p2pSlotBytes / 2;
    const uint64_t nChunks = bytes == 0 ? 0 : (bytes + sub - 1) / sub;
    char *land = HcPeerHeap(d, dst) + a.p2pOffset + (uint64_t)me * a.p2pSlotBytes;
    for (uint64_t k = 0; k < nChunks; ++k) {
        const uint64_t global = a.p2pDataBase + k;            // ordinal of this chunk on the pair
        if (global >= 2) {                                     // sub-slot reuse: chunk global-2 must be consumed
            if (threadIdx.x == 0) WaitFlagGe64(d, P2pWord(d, me, dst, 1), global - 1, (uint32_t)dst, HC_WAIT_CHAN_NOTIFY, 1);
            __syncthreads();
        }
        const uint64_t off = k * sub, len = (bytes - off < sub) ? bytes - off : sub;
        GridCopy(land + (global & 1) * sub, (const char *)a.in + off, len, a.elemSize);
        if (LastCtaOfChunk(P2pDone(d, 0, dst, global)) && threadIdx.x == 0) RedReleaseSysAdd64(P2pWord(d, dst, me, 0), 1);
    }
}

__global__ void __launch_bounds__(512) KRecv(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const int me = d->rank, src = a.peer;
    const uint64_t bytes = a.count * a.elemSize, sub = a.p2pSlotBytes / 2;
    const uint64_t nChunks = bytes == 0 ? 0 : (bytes + sub - 1) / sub;
    const char *land = HcPeerHeap(d, me) + a.p2pOffset + (uint64_t)src * a.p2pSlotBytes;
    for (uint64_t k = 0; k < nChunks; ++k) {
        const uint64_t global = a.p2pDataBase + k;
        if (threadIdx.x == 0) WaitFlagGe64(d, P2pWord(d, me, src, 0), global + 1, (uint32_t)src, HC_WAIT_CHAN_NOTIFY, 0);
        __syncthreads();
        const uint64_t off = k * sub, len = (bytes - off < sub) ? bytes - off : sub;
        GridCopy((char *)a.out + off, land + (global & 1) * sub, len, a.elemSize);
        if (LastCtaOfChunk(P2pDone(d, 1, src, global)) && threadIdx.x == 0) RedReleaseSysAdd64(P2pWord(d, src, me, 1), 1);
    }
}

// ------------------------------------------------------------------------ small messages (LL)

// Flag-in-data exchange: every 8 bytes written to a peer hold 4 bytes of payload and the 4-byte tag of this launch,
// so the receiver needs no barrier - it polls the words themselves (8-byte writes are not torn).  The tag is the
// communicator's launch count + 1: it is the same on all ranks, grows with every operator and the area is used for
// nothing else, so a word can never show this launch's tag before this launch's sender wrote it.  Slots alternate
// with the launch parity; a slot is rewritten two launches later, which a sender can only reach after the receiver
// has sent - hence finished reading - in between (every rank receives from every rank in all four collectives).
//
// a.peer selects the collective; a.count = elements per block:
//   LL_ALLREDUCE       every rank sends its whole vector to all peers, out = sum in rank order of in_r[0..count)
//   LL_ALLGATHER       block = my contribution, out[r*count ..] = block of rank r
//   LL_ALLTOALL        in[q*count ..] goes to rank q, out[r*count ..] comes from rank r
//   LL_REDUCE_SCATTER  in[q*count ..] goes to rank q, out = sum in rank order of the blocks addressed to me
// Blocks are whole aligned 16-byte vectors of at most HC_LL_MAX_PAYLOAD bytes, or (a.root != 0) tiny blocks of any length
// and alignment that are moved byte by byte.
__device__ __forceinline__ char *LlSlot(const CommDev *d, int owner, uint32_t parity, int src)
{
    return HcPeerHeap(d, owner) + d->llOffset + ((uint64_t)parity * HC_KERNEL_MAX_RANKS + (uint64_t)src) * HC_LL_SLOT_BYTES;
}
__device__ __forceinline__ void LlStore(char *slot, uint64_t vec, uint4 v, uint32_t tag)
{
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(slot + vec * 32), "r"(v.x), "r"(tag), "r"(v.y), "r"(tag) : "memory");
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(slot + vec * 32 + 16), "r"(v.z), "r"(tag), "r"(v.w), "r"(tag) : "memory");
}
// Spins until both halves of vector `vec` carry `tag`; false when the wait was given up.
__device__ __forceinline__ bool LlLoad(const CommDev *d, const char *slot, uint64_t vec, uint32_t tag, int src, uint4 *out)
{
    uint64_t start = 0;
    for (uint32_t it = 0;; ++it) {
        const uint4 a = Ld16Volatile(slot + vec * 32), b = Ld16Volatile(slot + vec * 32 + 16);
        if (a.y == tag && a.w == tag && b.y == tag && b.w == tag) {
            *out = make_uint4(a.x, a.z, b.x, b.z);
            return true;
        }
        if ((it & 63) == 63) {
            if (Aborted(d)) return false;
            if (start == 0) start = GlobalTimerNs();
            else if (GlobalTimerNs() - start > d->timeoutNs) { ReportTimeout(d, (uint32_t)src, HC_WAIT_TILE_FLAG, (uint32_t)vec, tag, a.y); return false; }
        }
    }
}

// 16 bytes of a block that may end inside the vector or start at any address: assembled from single bytes, missing
// bytes read as zero (tiny messages only; whole aligned vectors use Ld16 / St16).
__device__ __forceinline__ uint4 LlLoadBytes(const char *base, uint64_t vec, uint64_t blockBytes)
{
    union { uint4 v; unsigned char b[16]; } u;
    u.v = make_uint4(0, 0, 0, 0);
    const uint64_t off = vec << 4;
#pragma unroll
    for (int j = 0; j < 16; ++j)
        if (off + j < blockBytes) u.b[j] = *(volatile const unsigned char *)(base + off + j);
    return u.v;
}
__device__ __forceinline__ void LlStoreBytes(char *base, uint64_t vec, uint64_t blockBytes, uint4 val)
{
    union { uint4 v; unsigned char b[16]; } u;
    u.v = val;
    const uint64_t off = vec << 4;
#pragma unroll
    for (int j = 0; j < 16; ++j)
        if (off + j < blockBytes) base[off + j] = (char)u.b[j];
}

template <typename T>
__global__ void __launch_bounds__(512) KSmallLL(const __grid_constant__ CollArgs byval, const CollArgs *emu)
{
    HC_ARGS;
    const LaunchState ls = KernelBegin(d);
    const uint32_t tag = *(volatile const uint32_t *)&DevCounters(d)[1] + 1u;
    const int n = d->nRanks, me = d->rank, mode = a.peer;
    const bool reducing = mode == LL_ALLREDUCE || mode == LL_REDUCE_SCATTER;
    const uint64_t blockBytes = a.count * (reducing ? sizeof(T) : (uint64_t)a.elemSize);
    const uint64_t nvec = (blockBytes + 15) >> 4;
    // a.root != 0: the block is not made of whole aligned 16-byte vectors (the host sets it for tiny messages)
    const bool bytewise = a.root != 0;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, first = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool perPeerInput = mode == LL_ALLTOALL || mode == LL_REDUCE_SCATTER;
    // send
    for (int i = 1; i < n; ++i) {
        const int q = (me + i) % n;
        const char *src = (const char *)a.in + (perPeerInput ? (uint64_t)q * blockBytes : 0);
        char *slot = LlSlot(d, q, ls.half, me);
        for (uint64_t v = first; v < nvec; v += stride) LlStore(slot, v, bytewise ? LlLoadBytes(src, v, blockBytes) : Ld16(src + (v << 4)), tag);
    }
    // receive
    const char *own = (const char *)a.in + (perPeerInput ? (uint64_t)me * blockBytes : 0);
    if (reducing) {
        using A = typename AccOf<T>::type;
        constexpr int N = Pack<T>::N;
        for (uint64_t v = first; v < nvec; v += stride) {
            A acc[N];
            bool ok = true;
            for (int r = 0; r < n && ok; ++r) {
                Pack<T> p;
                if (r == me) p.v = bytewise ? LlLoadBytes(own, v, blockBytes) : Ld16(own + (v << 4));
                else ok = LlLoad(d, LlSlot(d, me, ls.half, r), v, tag, r, &p.v);
                if (r == 0) {
#pragma unroll
                    for (int j = 0; j < N; ++j) acc[j] = Widen<T>(p.e[j]);
                } else {
#pragma unroll
                    for (int j = 0; j < N; ++j) acc[j] = Combine<A>(a.op, acc[j], Widen<T>(p.e[j]));
                }
            }
            if (!ok) break;
            Pack<T> o;
#pragma unroll
            for (int j = 0; j < N; ++j) o.e[j] = Narrow<T>(a.useScale ? ScaleAcc<A>(acc[j], a.scale) : acc[j]);
            if (bytewise) LlStoreBytes((char *)a.out, v, blockBytes, o.v);
            else St16((char *)a.out + (v << 4), o.v);
        }
    } else {
        for (uint64_t v = first; v < nvec; v += stride) {
            if (bytewise) LlStoreBytes((char *)a.out + (uint64_t)me * blockBytes, v, blockBytes, LlLoadBytes(own, v, blockBytes));
            else St16((char *)a.out + (uint64_t)me * blockBytes + (v << 4), Ld16(own + (v << 4)));
        }
        for (int i = 1; i < n; ++i) {
            const int r = (me + n - i) % n;
            const char *slot = LlSlot(d, me, ls.half, r);
            bool ok = true;
            for (uint64_t v = first; v < nvec && ok; v += stride) {
                uint4 val;
                ok = LlLoad(d, slot, v, tag, r, &val);
                if (ok) {
                    if (bytewise) LlStoreBytes((char *)a.out + (uint64_t)r * blockBytes, v, blockBytes, val);
                    else St16((char *)a.out + (uint64_t)r * blockBytes + (v << 4), val);
                }
            }
            if (!ok) break;
        }
    }
    KernelEnd(d, ls, 0);
}

// ------------------------------------------------------------------- schedule interpreter (sm-ir)

// Runs this rank's program of a Schedule (ring, halving-doubling, Bruck, pairwise, tree ... templates) in one launch.
// Every CTA walks the whole program; of each slice it moves the 2048-element blocks b with b % gridDim.x == blockIdx.x,
// counted from the start of the slice, so the same elements belong to the same CTA index on every rank whatever the
// alignment of the buffers, and POST / WAIT can be per-CTA: CTA i signals CTA i of the peer through notify words
// [cta][from][slot] in the control region and consumes posts with device-resident counters (they survive the launch,
// a wait expects one more post than the previous wait on that word).  Primitives run in program order, which is the
// order the host engine runs them in on one stream.
// Moves (or reduces into dst) n elements.  CTA c owns the blocks b with b % gridDim.x == c, a block being kIrBlock
// elements counted from the start of the slice (so ownership does not depend on buffer alignment and is the same in every
// primitive of a program).  A CTA walks its blocks kIrUnroll at a time: every thread keeps one 16-byte load (two when it
// reduces) per block of the batch in flight, which is what hides NVLink and HBM latency with the few CTAs these
// kernels run on.
constexpr uint64_t kIrBlock = 4096;
constexpr int kIrUnroll = 4;
template <typename T> struct IrBits { using type = T; };
template <> struct IrBits<__half> { using type = unsigned short; };
template <> struct IrBits<__nv_bfloat16> { using type = unsigned short; };
template <typename T>
__device__ __forceinline__ T IrCombineBits(int op, typename IrBits<T>::type d, typename IrBits<T>::type s)
{
    using A = typename AccOf<T>::type;
    T dv, sv;
    memcpy(&dv, &d, sizeof(T)); memcpy(&sv, &s, sizeof(T));
    return Narrow<T>(Combine<A>(op, Widen<T>(dv), Widen<T>(sv)));
}
template <typename T>
__device__ __forceinline__ void IrMove(char *dst, const char *src, uint64_t n, bool reduce, int op)
{
    using A = typename AccOf<T>::type;
    using B = typename IrBits<T>::type;
    constexpr int N = Pack<T>::N;
    HC_BOUNDS_OR_RETURN(dst, n * sizeof(T));
    HC_BOUNDS_OR_RETURN(src, n * sizeof(T));
    const uint64_t nBlocks = (n + kIrBlock - 1) / kIrBlock;
    const bool aligned = ((((uintptr_t)src | (uintptr_t)dst) & 15) == 0) && (kIrBlock * sizeof(T)) % 16 == 0;
    for (uint64_t b0 = blockIdx.x; b0 < nBlocks; b0 += (uint64_t)kIrUnroll * gridDim.x) {
        if (aligned) {
            // vectors of the batch's blocks, thread-strided inside each block
            constexpr uint64_t kVecs = kIrBlock / N;
            for (uint64_t v = threadIdx.x; v < kVecs; v += blockDim.x) {
                Pack<T> s[kIrUnroll], t[kIrUnroll];
                bool live[kIrUnroll];
#pragma unroll
                for (int u = 0; u < kIrUnroll; ++u) {
                    const uint64_t b = b0 + (uint64_t)u * gridDim.x, e = b * kIrBlock + v * N;
                    live[u] = b < nBlocks && e + N <= n;
                    if (live[u]) {
                        s[u].v = Ld16Volatile(src + e * sizeof(T));
                        if (reduce) t[u].v = Ld16Volatile(dst + e * sizeof(T));
                    }
                }
#pragma unroll
                for (int u = 0; u < kIrUnroll; ++u) {
                    if (!live[u]) continue;
                    const uint64_t e = (b0 + (uint64_t)u * gridDim.x) * kIrBlock + v * N;
                    if (reduce) {
#pragma unroll
                        for (int j = 0; j < N; ++j) s[u].e[j] = Narrow<T>(Combine<A>(op, Widen<T>(t[u].e[j]), Widen<T>(s[u].e[j])));
                    }
                    St16(dst + e * sizeof(T), s[u].v);
                }
            }
        }
        // elements no vector covered: everything when the buffers are not 16-byte aligned, else the ragged end of the slice
        for (int u = 0; u < kIrUnroll; ++u) {
            const uint64_t b = b0 + (uint64_t)u * gridDim.x;
            if (b >= nBlocks) break;
            const uint64_t e0 = b * kIrBlock, cnt = n - e0 < kIrBlock ? n - e0 : kIrBlock;
            const uint64_t done = aligned ? cnt / N * N : 0;
            for (uint64_t e = e0 + done + threadIdx.x; e < e0 + cnt; e += blockDim.x) {
                B sb = *(volatile const B *)(src + e * sizeof(T));
                if (reduce) {
                    const B db = *(volatile const B *)(dst + e * sizeof(T));
                    T r = IrCombineBits<T>(op, db, sb);
                    memcpy(&sb, &r, sizeof(T));
                }
                *(B *)(dst + e * sizeof(T)) = sb;
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(512) KIrInterp(const __grid_constant__ IrArgs byval, const IrArgs *emu)
{
    const IrArgs &a = (emu != nullptr) ? emu[blockIdx.y] : byval;
    const CommDev *d = a.dev;
    const LaunchState ls = KernelBegin(d);
    uint32_t used = 0;
    if (a.preBarrier) CrossRankBarrier(d, ls.epoch0 + (++used));
    const int me = d->rank;
    const DevPrim *prims = (const DevPrim *)a.prims;
    const uint32_t esz = a.elemSize;
    auto Word = [&](int owner, int from, uint32_t slot) {
        return (uint64_t *)(HcPeerHeap(d, owner) + HC_OFF_IR_NOTIFY) + ((uint64_t)blockIdx.x * HC_IR_RANKS + (uint64_t)from) * HC_IR_NOTIFY + slot;
    };
    auto Count = [&](uint32_t buf, uint32_t slice) -> uint64_t {      // elements of a slice inside the column window
        const IrLayoutDev &L = a.lay[buf];
        const uint64_t b0 = (uint64_t)slice * L.sliceCount;
        uint64_t cnt = b0 >= L.total ? 0 : (L.total - b0 < L.sliceCount ? L.total - b0 : L.sliceCount);
        if (cnt <= a.col0) return 0;
        return (cnt < a.col1 ? cnt : a.col1) - a.col0;
    };
    auto Addr = [&](uint32_t buf, uint32_t slice, int rank) -> char * {
        if (buf == 2) return CclHalf(d, rank, ls.half) + (uint64_t)slice * a.cap * esz;
        char *base = buf == 0 ? (char *)a.in : (char *)a.out;
        return base + ((uint64_t)slice * a.lay[buf].sliceCount + a.col0) * esz;
    };
    bool alive = true;
    for (uint32_t i = 0; i < a.nPrims && alive; ++i) {
        const DevPrim p = prims[i];
        switch (p.op) {
            case 6: {   // POST
                __syncthreads();
                if (threadIdx.x == 0) {
                    __threadfence_system();
                    RedReleaseSysAdd64(Word(p.peer, me, p.notify), 1ull);
                }
                break;
            }
            case 7: {   // WAIT
                __shared__ int okFlag;
                if (threadIdx.x == 0) {
                    uint64_t *consumed = d->irConsumed + ((uint64_t)blockIdx.x * HC_IR_RANKS + (uint64_t)p.peer) * HC_IR_NOTIFY + p.notify;
                    const uint64_t expect = *consumed + 1;
                    *consumed = expect;
                    okFlag = WaitFlagGe64(d, Word(me, p.peer, p.notify), expect, (uint32_t)p.peer, HC_WAIT_CHAN_NOTIFY, p.notify) ? 1 : 0;
                }
                __syncthreads();
                alive = okFlag != 0;
                __syncthreads();
                break;
            }
            case 8: break;   // NOP
            default: {
                const bool remoteDst = p.op == 2 || p.op == 3, remoteSrc = p.op == 4 || p.op == 5;
                const bool reduce = p.op == 1 || p.op == 3 || p.op == 5;
                const int srcRank = remoteSrc ? p.peer : me, dstRank = remoteDst ? p.peer : me;
                for (uint32_t s = 0; s < p.nSlices; ++s) {
                    const uint64_t n = Count(p.lenBuf, p.lenSlice + s);
                    if (n == 0) continue;
                    const char *src = Addr(p.srcBuf, p.srcSlice + s, srcRank);
                    char *dst = Addr(p.dstBuf, p.dstSlice + s, dstRank);
                    if (reduce || src != dst) IrMove<T>(dst, src, n, reduce, a.op);
                }
                // later primitives of this CTA may read what other threads of the CTA just wrote
                __syncthreads();
            }
        }
    }
    KernelEnd(d, ls, used);
}

template <typename K> struct KernelOf { K fn; };

template <template <typename> class Dummy = AccOf>
void *ReduceKernelFor(int kind, int dtype)
{
#define HC_PICK(KERNEL)                                                                                             \
    switch (dtype) {                                                                                                \
        case HCCL_DATA_TYPE_FP32: return (void *)KERNEL<float>; case HCCL_DATA_TYPE_FP16: return (void *)KERNEL<__half>;                   \
        case HCCL_DATA_TYPE_BFP16: return (void *)KERNEL<__nv_bfloat16>; case HCCL_DATA_TYPE_FP64: return (void *)KERNEL<double>;          \
        case HCCL_DATA_TYPE_INT8: return (void *)KERNEL<int8_t>; case HCCL_DATA_TYPE_INT16: return (void *)KERNEL<int16_t>;                \
        case HCCL_DATA_TYPE_INT32: return (void *)KERNEL<int32_t>; case HCCL_DATA_TYPE_INT64: return (void *)KERNEL<long long>;            \
        case HCCL_DATA_TYPE_UINT8: return (void *)KERNEL<uint8_t>; case HCCL_DATA_TYPE_UINT16: return (void *)KERNEL<uint16_t>;            \
        case HCCL_DATA_TYPE_UINT32: return (void *)KERNEL<uint32_t>; case HCCL_DATA_TYPE_UINT64: return (void *)KERNEL<unsigned long long>; \
        default: return nullptr;                                                                                    \
    }
    switch (kind) {
        case FK_ALLREDUCE_ONESHOT: HC_PICK(KAllReduceOneShot)
        case FK_ALLREDUCE_TWOSHOT: HC_PICK(KAllReduceTwoShot)
        case FK_REDUCE_SCATTER: HC_PICK(KReduceScatter)
        case FK_ALLREDUCE_TWOSHOT_WIN: HC_PICK(KAllReduceTwoShotWin)
        case FK_REDUCE_SCATTER_WIN: HC_PICK(KReduceScatterWin)
        case FK_REDUCE_SCATTER_INPLACE: HC_PICK(KReduceScatterInPlace)
        case FK_REDUCE: HC_PICK(KReduce)
        case FK_SMALL_LL: HC_PICK(KSmallLL)
        case FK_ALLREDUCE_NVLS:
            switch (dtype) {
                case HCCL_DATA_TYPE_FP32: return (void *)KAllReduceNvls<float>;
                case HCCL_DATA_TYPE_FP16: return (void *)KAllReduceNvls<__half>;
                case HCCL_DATA_TYPE_BFP16: return (void *)KAllReduceNvls<__nv_bfloat16>;
                default: return nullptr;
            }
        case FK_ALLREDUCE_NVLS_PIPE:
            switch (dtype) {
                case HCCL_DATA_TYPE_FP32: return (void *)KAllReduceNvlsPipe<float>;
                case HCCL_DATA_TYPE_FP16: return (void *)KAllReduceNvlsPipe<__half>;
                case HCCL_DATA_TYPE_BFP16: return (void *)KAllReduceNvlsPipe<__nv_bfloat16>;
                default: return nullptr;
            }
        case FK_REDUCE_SCATTER_NVLS:
            switch (dtype) {
                case HCCL_DATA_TYPE_FP32: return (void *)KReduceScatterNvls<float>;
                case HCCL_DATA_TYPE_FP16: return (void *)KReduceScatterNvls<__half>;
                case HCCL_DATA_TYPE_BFP16: return (void *)KReduceScatterNvls<__nv_bfloat16>;
                default: return nullptr;
            }
        default: return nullptr;
    }
#undef HC_PICK
}

void *KernelFor(int kind, int dtype)
{
    switch (kind) {
        case FK_ALLGATHER: return (void *)KAllGather;
        case FK_ALLGATHER_NVLS: return (void *)KAllGatherNvls;
        case FK_ALLTOALL: return (void *)KAlltoAll;
        case FK_BROADCAST_PUSH: return (void *)KBroadcastPush;
        case FK_BROADCAST_TWOSHOT: return (void *)KBroadcastTwoShot;
        case FK_BROADCAST_NVLS: return (void *)KBroadcastNvls;
        case FK_SCATTER: return (void *)KScatter;
        case FK_GATHER: return (void *)KGather;
        case FK_SEND: return (void *)KSend;
        case FK_RECV: return (void *)KRecv;
        case FK_BARRIER: return (void *)KBarrier;
        default: return ReduceKernelFor<>(kind, dtype);
    }
}

}  // namespace

// With lazy module loading the first launch of a kernel may have to wait for running kernels; a kernel that spins
// on a peer which in turn waits for a not-yet-loaded kernel of this process would stall until its time budget ends.
// Loading every kernel up front (function attributes force the load) removes that dependency.
void PreloadFastKernels()
{
    static const int dtypes[] = {HCCL_DATA_TYPE_FP32, HCCL_DATA_TYPE_FP16, HCCL_DATA_TYPE_BFP16, HCCL_DATA_TYPE_FP64, HCCL_DATA_TYPE_INT8, HCCL_DATA_TYPE_INT16,
                                 HCCL_DATA_TYPE_INT32, HCCL_DATA_TYPE_INT64, HCCL_DATA_TYPE_UINT8, HCCL_DATA_TYPE_UINT16, HCCL_DATA_TYPE_UINT32, HCCL_DATA_TYPE_UINT64};
    for (int k = 0; k < FK_COUNT; ++k)
        for (int dt : dtypes) {
            void *fn = KernelFor(k, dt);
            cudaFuncAttributes attr;
            if (fn) cudaFuncGetAttributes(&attr, fn);
        }
    for (int dt : dtypes) {
        void *fn = IrKernelFor(dt);
        cudaFuncAttributes attr;
        if (fn) cudaFuncGetAttributes(&attr, fn);
    }
    cudaGetLastError();
}

const char *FastKindName(int32_t k)
{
    static const char *names[] = {"AllReduceOneShot", "AllReduceTwoShot", "AllReduceNvls", "ReduceScatter", "AllGather", "AlltoAll",
                                  "BroadcastPush", "BroadcastTwoShot", "BroadcastNvls", "Reduce", "Scatter", "Gather", "Send", "Recv", "Barrier", "SmallLL",
                                  "ReduceScatterNvls", "AllGatherNvls", "AllReduceTwoShotWindows", "ReduceScatterWindows", "ReduceScatterInPlace", "AllReduceNvlsPipeline"};
    return (k >= 0 && k < FK_COUNT) ? names[k] : "?";
}

uint32_t FastKindBarriers(int32_t kind, int preBarrier)
{
    uint32_t k = 1;
    switch (kind) {
        case FK_ALLREDUCE_TWOSHOT: case FK_ALLREDUCE_NVLS: case FK_REDUCE: case FK_BROADCAST_NVLS: k = 2; break;   // per window
        case FK_SEND: case FK_RECV: case FK_SMALL_LL: return 0;
        default: k = 1;
    }
    return k + (preBarrier ? 1 : 0);
}

int FastMaxCoResidentCtas(int32_t kind, int threads, int ranksOnDevice)
{
    void *fn = KernelFor(kind, HCCL_DATA_TYPE_FP32);
    if (!fn) return 0;
    int perSm = 0, dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, fn, threads, 0) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    int total = perSm * sms;
    return ranksOnDevice > 0 ? total / ranksOnDevice : total;
}

HcclResult LaunchFastKernel(const FastLaunch &l)
{
    void *fn = KernelFor(l.kind, l.args.dtype);
    if (!fn) {
        HCCL_ERROR("no %s kernel for data type %d", FastKindName(l.kind), l.args.dtype);
        return HCCL_E_NOT_SUPPORT;
    }
    dim3 grid((unsigned)l.ctas, (unsigned)(l.emuTable ? l.emuRanks : 1), 1), block((unsigned)l.threads, 1, 1);
    CollArgs args = l.args;
    const CollArgs *emu = l.emuTable;
    void *params[] = {(void *)&args, (void *)&emu};
    cudaError_t e;
    // Cooperative launch guarantees that all CTAs are resident at once: required whenever CTAs wait
    // for CTAs of the same launch (shared-GPU emulation, grid.sync in send/recv).
    bool coop = l.emuTable != nullptr;
    if (coop) e = cudaLaunchCooperativeKernel(fn, grid, block, params, 0, (cudaStream_t)l.stream);
    else e = cudaLaunchKernel(fn, grid, block, params, 0, (cudaStream_t)l.stream);
    if (e != cudaSuccess) {
        HCCL_ERROR("launch of %s (%d CTAs x %d threads, %d ranks) failed: %s", FastKindName(l.kind), l.ctas, l.threads, grid.y, cudaGetErrorString(e));
        return HCCL_E_RUNTIME;
    }
    return HCCL_SUCCESS;
}


void *IrKernelFor(int dtype)
{
    switch (dtype) {
        case HCCL_DATA_TYPE_FP32: return (void *)KIrInterp<float>; case HCCL_DATA_TYPE_FP16: return (void *)KIrInterp<__half>;
        case HCCL_DATA_TYPE_BFP16: return (void *)KIrInterp<__nv_bfloat16>; case HCCL_DATA_TYPE_FP64: return (void *)KIrInterp<double>;
        case HCCL_DATA_TYPE_INT8: return (void *)KIrInterp<int8_t>; case HCCL_DATA_TYPE_INT16: return (void *)KIrInterp<int16_t>;
        case HCCL_DATA_TYPE_INT32: return (void *)KIrInterp<int32_t>; case HCCL_DATA_TYPE_INT64: return (void *)KIrInterp<long long>;
        case HCCL_DATA_TYPE_UINT8: return (void *)KIrInterp<uint8_t>; case HCCL_DATA_TYPE_UINT16: return (void *)KIrInterp<uint16_t>;
        case HCCL_DATA_TYPE_UINT32: return (void *)KIrInterp<uint32_t>; case HCCL_DATA_TYPE_UINT64: return (void *)KIrInterp<unsigned long long>;
        default: return nullptr;
    }
}

HcclResult LaunchIrKernel(const IrArgs &args, int ctas, void *stream, const IrArgs *emuTable, int emuRanks)
{
    void *fn = IrKernelFor(args.dtype);
    if (!fn) return HCCL_E_NOT_SUPPORT;
    dim3 grid((unsigned)ctas, (unsigned)(emuTable ? emuRanks : 1), 1), block(512, 1, 1);
    IrArgs a = args;
    const IrArgs *emu = emuTable;
    void *params[] = {(void *)&a, (void *)&emu};
    cudaError_t e = emuTable ? cudaLaunchCooperativeKernel(fn, grid, block, params, 0, (cudaStream_t)stream)
                             : cudaLaunchKernel(fn, grid, block, params, 0, (cudaStream_t)stream);
    if (e != cudaSuccess) {
        HCCL_ERROR("launch of the schedule interpreter (%d CTAs, %d ranks) failed: %s", ctas, grid.y, cudaGetErrorString(e));
        return HCCL_E_RUNTIME;
    }
    return HCCL_SUCCESS;
}

}  // namespace hc
