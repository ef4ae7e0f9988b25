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
}
