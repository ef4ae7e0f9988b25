/* hcomm_moe.h - expert-parallel exchange for mixture-of-experts layers: dispatch (tokens to the ranks that own their
 * experts, quantised to fp8 e4m3 with one fp32 scale per 128 values on the way) and combine (expert outputs back to the
 * token's rank with the gate-weighted sum fused).  The reference library offers AlltoAll(V/VC) for this
 * (pkg_inc/legacy/hccl/hccl_inner.h:55-66); routing, quantisation and the weighted sum are fused here.
 * `stream` is a cudaStream_t; functions return an HcclResult value. */
#pragma once
#include <stdint.h>

#include "hccl/hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif
// Offsets are relative to the start of each rank's buffer; the layout is identical on all ranks.
struct MoeLayout {
    int32_t numExperts, topk, hidden, maxTokens, maxRecvRows, reserved;
    uint64_t offCounts;          // u32 [nRanks][expertsPerRank]      rows each source sends to each local expert
    uint64_t offExpertOffsets;   // u32 [expertsPerRank + 1]          start row of every local expert, last = total
    uint64_t offOrigin;          // u64 [maxRecvRows]                 (source rank << 32) | (token * topk + k)
    uint64_t offScales;          // f32 [maxRecvRows][hidden / 128]
    uint64_t offRows;            // fp8 e4m3 [maxRecvRows][hidden]
    uint64_t offCombine;         // bf16 [maxTokens][topk][hidden]    landing area of the combine step
    uint64_t totalBytes;
    uint64_t offValid;           // u8 [maxTokens][topk]              1 = dispatch sent this (token, k), 0 = masked or dropped
};
#ifndef __cplusplus
typedef struct MoeLayout MoeLayout;
#endif

/* Collective: every rank allocates the same symmetric buffer (capacityFactor x maxTokens x topk receive rows; <= 0 means 2)
 * and maps its peers'.  numExperts a multiple of the rank count (<= 1024), topk <= 16, hidden a multiple of 512 (<= 8192). */
int HcommMoeCreate(HcclComm comm, int numExperts, int topk, int hidden, int maxTokens, float capacityFactor, void **handle, MoeLayout *layoutOut);
int HcommMoeDestroy(void *handle);
/* Local addresses of the receive-side arrays (valid after a dispatch on the same stream). */
int HcommMoeGetBuffers(void *handle, void **rows, void **scales, void **origin, void **expertOffsets, void **combine);
/* x: bf16 [numTokens][hidden]; topkIdx: int32 [numTokens][topk], an index outside [0, numExperts) masks that choice. */
int HcommMoeDispatch(void *handle, const void *x, const int32_t *topkIdx, int numTokens, void *stream);
/* y: bf16 expert outputs in receive-row order; gates: f32 [numTokens][topk]; out: bf16 [numTokens][hidden]. */
int HcommMoeCombine(void *handle, const void *y, const float *gates, void *out, int numTokens, void *stream);
/* Rows dropped because a rank received more than its capacity since the last call (clears the counter). */
int HcommMoeTakeOverflow(void *handle);

// HcommMoeDispatch with the kernel's per-expert counters kept in an array built into the library's device image
// rather than in allocated memory: the call allocates nothing, on the device or through any library.  Same
// arguments and results as HcommMoeDispatch.  This entry point has no counterpart in the reference library.
// Up to 256 experts (2 KB of built-in scratch per process and GPU); larger exchanges return HCCL_E_PARA.
// All calls on one GPU share the array: it is cleared at the start of every call, and calls that overlap in time
// race on it.  The array's address is resolved by HcommMoeCreate (set-up time); the call must be made with the
// exchange's GPU current and is refused with HCCL_E_PARA otherwise.
int HcommMoeDispatchStaticScratch(void *handle, const void *x, const int32_t *topkIdx, int numTokens, void *stream);
#ifdef __cplusplus
}
#endif
