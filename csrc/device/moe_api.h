// moe_api.h - geometry of the symmetric buffer used by the MoE dispatch / combine kernels.
#pragma once
#include <stdint.h>

extern "C" {
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
};

// HcommMoeDispatch with the kernel's per-expert counters kept in an array built into the library's device image
// rather than in allocated memory: the call allocates nothing, on the device or through any library.  Same
// arguments and results as HcommMoeDispatch.  This entry point has no counterpart in the reference library.
// Up to 256 experts (2 KB of built-in scratch per process and GPU); larger exchanges return HCCL_E_PARA.
// All calls on one GPU share the array: it is cleared at the start of every call, and calls that overlap in time
// race on it.  The first call on a device resolves the array's address; make it before any stream capture.
int HcommMoeDispatchStaticScratch(void *handle, const void *x, const int32_t *topkIdx, int numTokens, void *stream);
}
