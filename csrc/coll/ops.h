// ops.h - operator front end: validation, group deferral, selection, dispatch to an engine.
#pragma once
#include <functional>
#include <vector>

#include "../alg/selector.h"
#include "../comm/comm.h"

namespace hc {

struct OpDesc {
    HcclCMDType cmd = HCCL_CMD_INVALID;
    const void *in = nullptr;
    void *out = nullptr;
    uint64_t count = 0;
    HcclDataType dtype = HCCL_DATA_TYPE_FP32;
    HcclReduceOp op = HCCL_REDUCE_SUM;
    uint32_t root = 0;
    uint32_t peer = 0;
    Stream stream = nullptr;
    bool useScale = false;
    float scale = 1.0f;
    // variable-count collectives, in elements, length nRanks (all-to-all VC: nRanks*nRanks in sendCounts)
    std::vector<uint64_t> sendCounts, sendDispls, recvCounts, recvDispls;
    std::vector<HcclSendRecvItem> batch;
};

// Runs (or, inside HcclGroupStart/End, queues) one operator.
HcclResult SubmitOp(Comm *c, const OpDesc &d);
// Executes immediately; used by SubmitOp and by HcclGroupEnd.
HcclResult RunOp(Comm *c, const OpDesc &d);
uint64_t OpDataVolume(const Comm *c, const OpDesc &d);

// Group bookkeeping (thread local).
bool GroupActive();
void GroupQueue(std::function<HcclResult()> job, uint64_t volume, bool isP2p, Comm *c, const OpDesc *p2p);

// Parsed per-communicator algorithm configuration (cached on the communicator name).
const AlgoConfig &AlgoConfigOf(Comm *c);

// Launches one specialised kernel for this rank, handling the shared-GPU rendezvous.
struct FastLaunch;
HcclResult LaunchForRank(Comm *c, FastLaunch &l);

}  // namespace hc
