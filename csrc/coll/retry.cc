// retry.cc - operator retry: when an operator ends with an expired wait, the ranks agree over the control plane to
// run it again instead of failing the communicator.
//
// Roles (reference: framework/cluster_maintenance/recovery/operator_retry/hccl_op_retry_pub.h:30-65 - a server state
// machine on the root and an agent on every rank, opretry_agent.cc, opretry_base.cc):
//   * every rank runs an AGENT thread per communicator that has retry switched on.  The agent watches the
//     communicator's abort word (a device-side wait that ran out raises it) and listens for the server's commands;
//   * rank 0's agent is also the SERVER: it takes retry requests from any rank and drives the rounds.
//
// One round, started by a request {operator ordinal, command, count, data type} of a rank whose wait expired:
//   1. the server sends the round's command to every agent;
//   2. each agent takes the communicator's operator lock (no new operator starts), raises its own abort word so that
//      waits still in flight on its GPU return, and drains its stream;                                 [stop]
//   3. the agents exchange the identity of the last operator each of them issued; the round goes on only if all of
//      them name the operator of the request and that operator can be run again (its input was not overwritten: an
//      in-place reduction cannot);                                                                      [check]
//   4. every rank clears the flag pages, epochs and counters (what HcclCommResume does);                [clear]
//   5. every agent issues the saved operator again on its stream and waits for it;                      [retry]
//   6. the outcomes are exchanged: all good -> the round succeeded; otherwise the server starts another round after
//      IntervalTime, up to MaxCnt rounds, and then declares HCCL_E_OPRETRY_FAIL on every rank.
// A caller that got HCCL_E_TIMEOUT from an operator (host engines report it synchronously) is parked until the verdict;
// on the CUDA engines the failure is asynchronous and the verdict replaces the asynchronous error.
// Nothing here touches a GPU except through the ordinary operator path; the faults it is tested with are made on the
// host (a withheld flag write in the simulator, a rank that arrives late).
#include <unistd.h>

#include <chrono>
#include <cstring>

#include "../core/env.h"
#include "../core/log.h"
#include "ops.h"

namespace hc {

namespace {

constexpr uint64_t kTagReq = 0x52540001ull, kTagCmd = 0x52540002ull;

struct Identity {
    uint64_t seq;
    uint32_t cmd, dtype;
    uint64_t count;
    uint32_t retryable, attempt;
};

uint64_t Tag(const Comm *c, uint64_t t) { return ((uint64_t)c->group.id << 32) | t; }

Blob ToBlob(const Identity &id)
{
    Blob b(sizeof(id));
    memcpy(b.data(), &id, sizeof(id));
    return b;
}
bool FromBlob(const Blob &b, Identity *id)
{
    if (b.size() != sizeof(*id)) return false;
    memcpy(id, b.data(), sizeof(*id));
    return true;
}

// "MaxCnt:3,HoldTime:5000,IntervalTime:1000"
void ParseParams(const std::string &s, RetryState *r)
{
    size_t pos = 0;
    while (pos < s.size()) {
        size_t comma = s.find(',', pos);
        std::string kv = s.substr(pos, comma == std::string::npos ? std::string::npos : comma - pos);
        size_t colon = kv.find(':');
        if (colon != std::string::npos) {
            std::string k = kv.substr(0, colon);
            long v = strtol(kv.c_str() + colon + 1, nullptr, 10);
            if (v >= 0) {
                if (k == "MaxCnt") r->maxCnt = (uint32_t)std::max(1L, std::min(v, 10L));
                else if (k == "HoldTime") r->holdMs = (uint32_t)v;
                else if (k == "IntervalTime") r->intervalMs = (uint32_t)v;
            }
        }
        if (comma == std::string::npos) break;
        pos = comma + 1;
    }
}

// The reference's switch is "L0:1, L1:0, L2:0" (per network level) or a plain 0 / 1.
bool ParseEnable(const std::string &s)
{
    if (s.empty()) return false;
    if (s.find("L0:1") != std::string::npos || s.find("L1:1") != std::string::npos || s.find("L2:1") != std::string::npos) return true;
    return s == "1" || s == "true" || s == "TRUE";
}

bool Retryable(const OpDesc &d)
{
    switch (d.cmd) {
        case HCCL_CMD_ALLREDUCE: case HCCL_CMD_REDUCE: case HCCL_CMD_REDUCE_SCATTER: case HCCL_CMD_REDUCE_SCATTER_V:
            return d.in != d.out;                      // an in-place reduction has consumed its input
        case HCCL_CMD_ALLGATHER: case HCCL_CMD_ALLGATHER_V: case HCCL_CMD_ALLTOALL: case HCCL_CMD_ALLTOALLV: case HCCL_CMD_ALLTOALLVC:
        case HCCL_CMD_BROADCAST: case HCCL_CMD_SCATTER: case HCCL_CMD_GATHER: case HCCL_CMD_BARRIER:
            return true;
        default: return false;                         // point-to-point traffic involves two ranks only: not handled by the rounds
    }
}

Identity IdentityOf(Comm *c)
{
    RetryState *r = c->retry.get();
    Identity id{};
    id.seq = r->lastSeq; id.cmd = (uint32_t)r->lastOp.cmd; id.dtype = (uint32_t)r->lastOp.dtype; id.count = r->lastOp.count;
    id.retryable = r->lastValid && Retryable(r->lastOp) ? 1u : 0u;
    return id;
}

// Steps 2-6 on one rank.  Returns the round's outcome as every rank computes it: 0 good, 1 run another round, 2 failed.
int RunRound(Comm *c, const Identity &req)
{
    RetryState *r = c->retry.get();
    Platform *P = c->plat;
    std::unique_lock<std::mutex> op(c->opMu);
    ++r->rounds;
    // stop
    __atomic_store_n(c->abortWord, 1u, __ATOMIC_RELEASE);
    if (P->kind() == PlatKind::CUDA && r->lastValid && r->lastOp.stream) P->StreamSync(r->lastOp.stream);
    // check
    Identity mine = IdentityOf(c);
    std::vector<Blob> all;
    if (c->boot->AllGather(r->group, ToBlob(mine), &all, (int)r->holdMs + 2000) != HCCL_SUCCESS) return 2;
    bool same = true;
    for (auto &b : all) {
        Identity o;
        if (!FromBlob(b, &o) || o.seq != req.seq || o.cmd != req.cmd || o.dtype != req.dtype || o.count != req.count || !o.retryable) same = false;
    }
    if (!same) {
        HCCL_ERROR("operator retry: the ranks do not agree on operator #%llu (%s x %llu) or it cannot be run again", (unsigned long long)req.seq,
                   CmdName((HcclCMDType)req.cmd), (unsigned long long)req.count);
        return 2;
    }
    // clear
    if (CommClearSyncState(c, r->group) != HCCL_SUCCESS) return 2;
    // retry
    OpDesc again = r->lastOp;
    HcclResult rc = RunOpLocked(c, again);
    if (rc == HCCL_SUCCESS && P->kind() == PlatKind::CUDA && again.stream) P->StreamSync(again.stream);
    bool good = rc == HCCL_SUCCESS && __atomic_load_n(c->abortWord, __ATOMIC_ACQUIRE) == 0;
    r->lastSeq = req.seq;                                   // the re-issue stands for the same operator
    Blob ok(1, good ? 1 : 0);
    if (c->boot->AllGather(r->group, ok, &all, (int)c->TimeoutMs() + 5000) != HCCL_SUCCESS) return 2;
    for (auto &b : all)
        if (b.empty() || !b[0]) good = false;
    HCCL_RUN_INFO("operator retry: round %u of operator #%llu %s on rank %u", req.attempt, (unsigned long long)req.seq, good ? "succeeded" : "did not complete", c->rank);
    return good ? 0 : 1;
}

void Verdict(Comm *c, uint64_t seq, int outcome)
{
    RetryState *r = c->retry.get();
    {
        std::lock_guard<std::mutex> lk(r->mu);
        r->verdictSeq = seq;
        r->verdict = outcome;
        r->requested = false;
        if (outcome == 0) ++r->succeeded; else ++r->failed;
    }
    r->cv.notify_all();
    if (outcome != 0) {
        // the failure that the rounds could not cure becomes the communicator's error
        std::lock_guard<std::mutex> op(c->opMu);
        CommSetAsyncError(c, HCCL_E_OPRETRY_FAIL);
    }
}

void SendRequest(Comm *c)
{
    RetryState *r = c->retry.get();
    Identity id;
    {
        std::lock_guard<std::mutex> lk(r->mu);
        if (r->requested) return;
        r->requested = true;
        ++r->requests;
    }
    {
        std::lock_guard<std::mutex> op(c->opMu);
        id = IdentityOf(c);
    }
    c->boot->Send(c->worldRanks[0], Tag(c, kTagReq), ToBlob(id));
}

void AgentLoop(Comm *c)
{
    RetryState *r = c->retry.get();
    const uint32_t n = c->nRanks;
    while (!r->stop.load()) {
        // without the hub there are no rounds: its calls return at once, so do not spin on them
        if (c->boot->HubGone()) { usleep(50000); continue; }
        // a wait that ran out on this rank's GPU (the host engines report theirs to the caller, who asks)
        if (c->plat->kind() == PlatKind::CUDA && c->abortWord && __atomic_load_n(c->abortWord, __ATOMIC_ACQUIRE) != 0 &&
            c->state.load() == (int)CommState::READY && c->asyncError.load() == 0)
            SendRequest(c);
        if (c->rank == 0) {
            // server: one request starts the rounds; requests of other ranks for the same operator are duplicates
            Identity req{};
            bool have = false;
            for (uint32_t q = 0; q < n && !have; ++q) {
                Blob b;
                if (c->boot->Recv(c->worldRanks[q], Tag(c, kTagReq), &b, q + 1 == n ? 20 : 0) == HCCL_SUCCESS && FromBlob(b, &req)) have = true;
            }
            if (have && req.seq > r->servedSeq) {
                r->servedSeq = req.seq;
                // HoldTime: give the other ranks' waits the time to run out by themselves before everything is stopped
                for (uint32_t waited = 0; waited < r->holdMs && !r->stop.load(); waited += 20) usleep(20000);
                for (uint32_t attempt = 1; attempt <= r->maxCnt && !r->stop.load(); ++attempt) {
                    req.attempt = attempt;
                    for (uint32_t q = 0; q < n; ++q) c->boot->Send(c->worldRanks[q], Tag(c, kTagCmd), ToBlob(req));
                    // the server's own agent half takes the command from its inbox like everyone else
                    Blob b;
                    Identity cmd;
                    int outcome = 2;
                    if (c->boot->Recv(c->worldRanks[0], Tag(c, kTagCmd), &b, 5000) == HCCL_SUCCESS && FromBlob(b, &cmd)) outcome = RunRound(c, cmd);
                    if (outcome == 1 && attempt < r->maxCnt) {
                        for (uint32_t waited = 0; waited < r->intervalMs && !r->stop.load(); waited += 20) usleep(20000);
                        continue;
                    }
                    Verdict(c, req.seq, outcome == 0 ? 0 : 2);
                    break;
                }
            }
            // drain duplicates of operators already served
        } else {
            Blob b;
            Identity cmd;
            if (c->boot->Recv(c->worldRanks[0], Tag(c, kTagCmd), &b, 50) == HCCL_SUCCESS && FromBlob(b, &cmd)) {
                int outcome = RunRound(c, cmd);
                if (outcome == 1 && cmd.attempt < r->maxCnt) continue;      // the server sends the next round's command
                Verdict(c, cmd.seq, outcome == 0 ? 0 : 2);
            }
        }
    }
}

}  // namespace

void RetrySetup(Comm *c)
{
    const EnvConfig &env = EnvConfig::Get();
    bool enable = env.opRetryEnable.value != 0;
    if (!c->cfg.retryEnable.empty()) enable = ParseEnable(c->cfg.retryEnable);
    if (!enable || c->nRanks < 2 || !c->boot) return;
    std::unique_ptr<RetryState> r(new RetryState());
    r->maxCnt = 1; r->holdMs = 5000; r->intervalMs = 1000;
    ParseParams(env.opRetryParams.value, r.get());
    if (!c->cfg.retryParams.empty()) ParseParams(c->cfg.retryParams, r.get());
    r->group = c->boot->MakeGroup(c->group.id | 0x40000000u, c->group.ranks);
    c->retry = std::move(r);
    c->retry->agent = std::thread(AgentLoop, c);
    HCCL_INFO("operator retry on for \"%s\": MaxCnt %u HoldTime %u ms IntervalTime %u ms", c->cfg.name.c_str(), c->retry->maxCnt, c->retry->holdMs, c->retry->intervalMs);
}

void RetryTeardown(Comm *c)
{
    if (!c->retry) return;
    c->retry->stop.store(true);
    c->retry->cv.notify_all();
    if (c->retry->agent.joinable()) c->retry->agent.join();
    c->retry.reset();
}

// Remembers what was issued (the caller holds the operator lock).
void RetryNoteOp(Comm *c, const OpDesc &d)
{
    if (!c->retry) return;
    c->retry->lastOp = d;
    c->retry->lastSeq = c->opSeq;
    c->retry->lastValid = true;
}

// Called by an operator's caller after HCCL_E_TIMEOUT, without the operator lock: asks for a retry and waits for the verdict.
HcclResult RetryAfterTimeout(Comm *c, uint64_t seq)
{
    RetryState *r = c->retry.get();
    if (!r) return HCCL_E_TIMEOUT;
    {
        std::lock_guard<std::mutex> op(c->opMu);
        if (!r->lastValid || !Retryable(r->lastOp)) {
            CommSetAsyncError(c, HCCL_E_TIMEOUT);       // nothing to run again: the expired wait is the communicator's error
            return HCCL_E_TIMEOUT;
        }
    }
    SendRequest(c);
    std::unique_lock<std::mutex> lk(r->mu);
    const auto budget = std::chrono::milliseconds((uint64_t)r->holdMs + (uint64_t)r->maxCnt * ((uint64_t)c->TimeoutMs() + r->intervalMs + 10000));
    if (!r->cv.wait_for(lk, budget, [&] { return r->verdictSeq >= seq || r->stop.load(); })) return HCCL_E_OPRETRY_FAIL;
    return r->verdict == 0 ? HCCL_SUCCESS : HCCL_E_OPRETRY_FAIL;
}

}  // namespace hc
