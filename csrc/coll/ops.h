// ops.h - operator front end: validation, group deferral, selection, dispatch to an engine.
#pragma once
#include <atomic>
#include <condition_variable>
#include <functional>
#include <mutex>
#include <thread>
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
// Executes immediately; used by SubmitOp and by HcclGroupEnd.  With operator retry on, an operator that ends with an
// expired wait is run again by the retry rounds before the caller sees a result.
HcclResult RunOp(Comm *c, const OpDesc &d);
// The same for a caller that already holds the communicator's operator lock (the retry agent).
HcclResult RunOpLocked(Comm *c, const OpDesc &d);

// Operator retry (retry.cc): per-communicator state of the agent thread.
struct RetryState {
    uint32_t maxCnt = 1, holdMs = 5000, intervalMs = 1000;
    Bootstrap::Group group;                  // the agents' own gather group on the control plane
    std::thread agent;
    std::atomic<bool> stop{false};
    // last operator issued on this communicator (guarded by the operator lock)
    OpDesc lastOp;
    uint64_t lastSeq = 0;
    bool lastValid = false;
    // request / verdict hand-over between the caller and the agent
    std::mutex mu;
    std::condition_variable cv;
    bool requested = false;
    uint64_t verdictSeq = 0, servedSeq = 0;
    int verdict = 0;
    std::atomic<uint64_t> requests{0}, rounds{0}, succeeded{0}, failed{0};   // read by HcclCommGetOpRetryStats from any thread
};
void RetryNoteOp(Comm *c, const OpDesc &d);
HcclResult RetryAfterTimeout(Comm *c, uint64_t seq);
uint64_t OpDataVolume(const Comm *c, const OpDesc &d);

// Group bookkeeping (thread local).
bool GroupActive();
void GroupQueue(std::function<HcclResult()> job, uint64_t volume, bool isP2p, Comm *c, const OpDesc *p2p);

// Parsed per-communicator algorithm configuration (cached on the communicator name).
const AlgoConfig &AlgoConfigOf(Comm *c);

// What the communicator would do with such an operator: the selector's choice and the CTAs its kernel would use.
HcclResult DescribeSelection(Comm *c, HcclCMDType cmd, uint64_t count, HcclDataType dtype, HcclReduceOp op, bool variableCounts, Selection *sel, int *ctas);

// Launches one specialised kernel for this rank, handling the shared-GPU rendezvous.
struct FastLaunch;
HcclResult LaunchForRank(Comm *c, FastLaunch &l);

}  // namespace hc
