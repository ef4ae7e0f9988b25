// dfx_api.cc - hooks that callers register with the library (exception callbacks, operator descriptions, a
// profiling sink), the profiling report entry points, operator-retry statistics and the extended entry points of
// the reference's "ex" / "expt" headers.
//
// Reference counterparts: pkg_inc/hcomm/hcomm_exception.h:78 (callback registry fed by the task-exception handler,
// src/base_comm/dfx), pkg_inc/hccl/hcomm_diag.h:40-55 and pkg_inc/hccl/hccl_diag.h:29-51 (reports to the profiler
// plug-in), pkg_inc/legacy/hccl/hccl_ex.h:206-232, pkg_inc/hccl/hccl_res_expt.h:44-99, hcomm_primitives_expt.h:32.
// Here the raw material is the wait-status block that an expired device wait fills in and the operator ring.
#include <time.h>

#include <cstring>
#include <mutex>
#include <vector>

#include "../coll/ops.h"
#include "../comm/comm.h"
#include "../core/log.h"
#include "hccl/hccl.h"
#include "hccl/hccl_dfx.h"
#include "hccl/hccl_sym_win.h"
#include "hcomm_res.h"

using namespace hc;

namespace hc {
ThreadRes *AsThread(ThreadHandle h);     // prim/primitives.cc
}

namespace {

struct ExceptionCb { HcommExceptionCallback cb; void *user; };
std::mutex g_dfxMu;
std::vector<ExceptionCb> g_exceptionCbs;
HcclProfilingSink g_sink = nullptr;
void *g_sinkUser = nullptr;

uint64_t NowNs()
{
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}

void Emit(int kind, const char *group, const char *name, uint64_t b, uint64_t e)
{
    HcclProfilingSink sink;
    void *user;
    {
        std::lock_guard<std::mutex> lk(g_dfxMu);
        sink = g_sink; user = g_sinkUser;
    }
    if (sink) sink(kind, group ? group : "", name ? name : "", b, e, user);
}

}  // namespace

namespace hc {

void DfxFireException(Comm *c, HcclResult err)
{
    std::vector<ExceptionCb> cbs;
    {
        std::lock_guard<std::mutex> lk(g_dfxMu);
        cbs = g_exceptionCbs;
    }
    HcommExceptionInfo info;
    memset(&info, 0, sizeof(info));
    info.header.version = 1; info.header.magicWord = 0x0f0f0f0f; info.header.size = sizeof(info);
    info.taskId = (uint32_t)c->opSeq;
    info.retCode = (uint32_t)err;
    info.expandInfo.type = HCOMM_EXCEPTION_INVALID;
    if (c->waitStatus && c->waitStatus->valid) {
        info.expandInfo.type = HCOMM_EXCEPTION_NVLINK_WAIT;
        info.expandInfo.detail.waitInfo = *c->waitStatus;
    }
    // the caller's description of the operator, in its own words
    if (c->userOpInfoFormatter && !c->userOpInfo.empty()) {
        char text[512] = "";
        c->userOpInfoFormatter(c->userOpInfo.data(), text, sizeof(text));
        text[sizeof(text) - 1] = 0;
        HCCL_ERROR("communicator \"%s\": operator in flight when the failure was recorded: %s", c->cfg.name.c_str(), text);
    }
    for (auto &e : cbs) e.cb(&info, e.user);
}

void DfxReportOp(Comm *c, const char *name, uint64_t beginNs, uint64_t endNs) { Emit(0, c->cfg.name.c_str(), name, beginNs, endNs); }

}  // namespace hc

extern "C" {

int32_t HcommExceptionRegisterCallback(HcommExceptionCallback cb, void *userData)
{
    if (!cb) return HCCL_E_PTR;
    std::lock_guard<std::mutex> lk(g_dfxMu);
    for (auto &e : g_exceptionCbs)
        if (e.cb == cb) { e.user = userData; return HCCL_SUCCESS; }
    g_exceptionCbs.push_back({cb, userData});
    return HCCL_SUCCESS;
}

int32_t HcommExceptionUnregisterCallback(HcommExceptionCallback cb)
{
    std::lock_guard<std::mutex> lk(g_dfxMu);
    for (auto it = g_exceptionCbs.begin(); it != g_exceptionCbs.end(); ++it)
        if (it->cb == cb) { g_exceptionCbs.erase(it); return HCCL_SUCCESS; }
    return HCCL_E_NOT_FOUND;
}

HcclResult HcommRegOpInfo(const char *commId, void *opInfo, size_t size)
{
    CHK_PTR_NULL(commId); CHK_PTR_NULL(opInfo);
    if (size == 0 || size > 65536) return HCCL_E_PARA;
    Comm *c = RegistryFind(commId);
    if (!c) return HCCL_E_NOT_FOUND;
    std::lock_guard<std::mutex> lk(c->diagMu);
    c->userOpInfo.assign((uint8_t *)opInfo, (uint8_t *)opInfo + size);
    return HCCL_SUCCESS;
}

HcclResult HcommRegOpTaskException(const char *commId, HcommGetOpInfoCallback callback)
{
    CHK_PTR_NULL(commId);
    Comm *c = RegistryFind(commId);
    if (!c) return HCCL_E_NOT_FOUND;
    std::lock_guard<std::mutex> lk(c->diagMu);
    c->userOpInfoFormatter = callback;
    return HCCL_SUCCESS;
}

HcclResult HcclProfilingSetSink(HcclProfilingSink sink, void *userData)
{
    std::lock_guard<std::mutex> lk(g_dfxMu);
    g_sink = sink; g_sinkUser = userData;
    return HCCL_SUCCESS;
}

uint64_t HcommGetProfilingSysCycleTime(void) { return NowNs(); }

HcclResult HcclProfilingReportOp(HcclComm comm, uint64_t beginTime)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    const uint64_t now = NowNs();
    char name[64] = "operator";
    {
        std::lock_guard<std::mutex> lk(c->diagMu);
        if (c->userOpInfo.size() >= sizeof(HcclDfxOpInfo)) {
            const HcclDfxOpInfo *oi = (const HcclDfxOpInfo *)c->userOpInfo.data();
            snprintf(name, sizeof(name), "%.63s", oi->algTag);
        }
        // external operators (built on the channel / primitive API) appear in the same ring as the library's own
        HcclOpRecord &r = c->opRing[c->opRingNext % c->opRing.size()];
        memset(&r, 0, sizeof(r));
        r.seq = c->opSeq; r.cmdType = HCCL_CMD_INVALID;
        snprintf(r.algName, sizeof(r.algName), "%.47s", name);
        r.hostStartNs = beginTime; r.hostEndNs = now;
        ++c->opRingNext;
    }
    Emit(0, c->cfg.name.c_str(), name, beginTime, now);
    return HCCL_SUCCESS;
}

HcclResult HcclReportAicpuKernel(HcclComm comm, uint64_t beginTime, char *kernelName)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    Emit(1, c->cfg.name.c_str(), kernelName ? kernelName : "kernel", beginTime, NowNs());
    return HCCL_SUCCESS;
}

HcclResult HcclReportAivKernel(HcclComm comm, uint64_t beginTime)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    Emit(1, c->cfg.name.c_str(), "sm kernel", beginTime, NowNs());
    return HCCL_SUCCESS;
}

HcclResult HcclDfxRegOpInfoByCommId(char *commId, void *hcclDfxOpInfo)
{
    CHK_PTR_NULL(commId); CHK_PTR_NULL(hcclDfxOpInfo);
    return HcommRegOpInfo(commId, hcclDfxOpInfo, sizeof(HcclDfxOpInfo));
}

HcclResult HcommProfilingReportDeviceOp(const char *groupname)
{
    CHK_PTR_NULL(groupname);
    const uint64_t now = NowNs();
    Emit(3, groupname, "device operator", now, now);
    return HCCL_SUCCESS;
}

HcclResult HcommProfilingReportKernelStartTask(uint64_t thread, const char *groupname)
{
    CHK_PTR_NULL(groupname);
    char name[48];
    snprintf(name, sizeof(name), "thread %llx", (unsigned long long)thread);
    const uint64_t now = NowNs();
    Emit(1, groupname, name, now, 0);
    return HCCL_SUCCESS;
}

HcclResult HcommProfilingReportKernelEndTask(uint64_t thread, const char *groupname)
{
    CHK_PTR_NULL(groupname);
    char name[48];
    snprintf(name, sizeof(name), "thread %llx", (unsigned long long)thread);
    const uint64_t now = NowNs();
    Emit(2, groupname, name, 0, now);
    return HCCL_SUCCESS;
}

HcclResult HcclCommGetOpRetryStats(HcclComm comm, HcclOpRetryStats *stats)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(stats);
    memset(stats, 0, sizeof(*stats));
    RetryState *r = c->retry.get();
    if (!r) return HCCL_SUCCESS;
    std::lock_guard<std::mutex> lk(r->mu);
    stats->enabled = 1; stats->maxCnt = r->maxCnt; stats->holdTimeMs = r->holdMs; stats->intervalMs = r->intervalMs;
    stats->requests = r->requests.load(); stats->rounds = r->rounds.load(); stats->succeeded = r->succeeded.load(); stats->failed = r->failed.load();
    return HCCL_SUCCESS;
}

// ------------------------------------------------------------------------- extended entry points

HcclResult HcclGetTopoDesc(HcclComm comm, HcclTopoDescs *topoDescs, uint32_t topoSize)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(topoDescs);
    if (topoSize == 0) return HCCL_E_PARA;
    // level 0: the NVLink domain, every family of the algorithm layer can be forced there
    // (bit order of HcclAlgoType: ring 0, pipeline 1, fullmesh 2, H-D_R 3, pairwise 4, NHR 5, NHR_V1 6, NB 7)
    topoDescs[0].algSets = 0xffu;
    topoDescs[0].rankSize = c->nRanks;
    for (uint32_t l = 1; l < topoSize; ++l) { topoDescs[l].algSets = 0; topoDescs[l].rankSize = 1; }   // one node: the upper levels are trivial
    return HCCL_SUCCESS;
}

HcclResult HcclCommRegister(HcclComm comm, void *addr, uint64_t size, void **handle, uint32_t flag)
{
    CHK_PTR_NULL(handle);
    HcclCommSymWindow w = nullptr;
    HcclResult r = HcclCommSymWinRegister(comm, addr, size, &w, flag);
    *handle = w;
    return r;
}
HcclResult HcclCommDeregister(HcclComm comm, void *handle)
{
    (void)comm;
    return HcclCommSymWinDeregister((HcclCommSymWindow)handle);
}
// Registration already exchanged the window with every rank of the communicator; this checks the peer list.
HcclResult HcclCommExchangeMem(HcclComm comm, void *windowHandle, uint32_t *peerRanks, uint32_t peerRankNum)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(windowHandle);
    if (peerRankNum && !peerRanks) return HCCL_E_PTR;
    for (uint32_t i = 0; i < peerRankNum; ++i) {
        void *p = nullptr;
        if (peerRanks[i] >= c->nRanks) return HCCL_E_PARA;
        CHK_RET(HcclSymWinGetPeerPointer((HcclCommSymWindow)windowHandle, 0, peerRanks[i], &p));
    }
    return HCCL_SUCCESS;
}

HcclResult HcclGetRemoteIpcHcclBuf(HcclComm comm, uint64_t remoteRank, void **addr, uint64_t *size)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(addr); CHK_PTR_NULL(size);
    if (remoteRank >= c->nRanks) return HCCL_E_PARA;
    *addr = c->PeerHeap((uint32_t)remoteRank) + HC_CTRL_BYTES;
    *size = 2 * c->halfBytes;
    return HCCL_SUCCESS;
}

HcclResult HcclDevMemAcquire(HcclComm comm, const char *memTag, uint64_t *size, void **addr, bool *newCreated)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(memTag); CHK_PTR_NULL(size); CHK_PTR_NULL(addr);
    std::lock_guard<std::mutex> lk(c->resMu);
    auto it = c->taggedDevMem.find(memTag);
    if (it != c->taggedDevMem.end()) {
        *addr = it->second.first; *size = it->second.second;
        if (newCreated) *newCreated = false;
        return HCCL_SUCCESS;
    }
    if (*size == 0) return HCCL_E_PARA;
    void *p = nullptr;
    CHK_RET(c->plat->DevAlloc(*size, &p));
    c->plat->MemsetSync(p, 0, *size);
    c->taggedDevMem[memTag] = {p, *size};
    *addr = p;
    if (newCreated) *newCreated = true;
    return HCCL_SUCCESS;
}

HcclResult HcclThreadExportToCommEngine(HcclComm comm, uint32_t threadNum, const ThreadHandle *threads, CommEngine dstCommEngine, ThreadHandle *exportedThreads)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(threads); CHK_PTR_NULL(exportedThreads);
    if (dstCommEngine == COMM_ENGINE_CCU) return HCCL_E_NOT_SUPPORT;
    for (uint32_t i = 0; i < threadNum; ++i) {
        if (!AsThread(threads[i])) return HCCL_E_PARA;
        exportedThreads[i] = threads[i];     // every engine here drives the same CUDA stream and notify words
    }
    return HCCL_SUCCESS;
}

int32_t HcclTaskRegister(HcclComm comm, const char *msgTag, HcclTaskCallback cb)
{
    Comm *c = AsComm(comm);
    if (!c || !msgTag || !cb) return HCCL_E_PTR;
    std::lock_guard<std::mutex> lk(c->resMu);
    c->taskCallbacks[msgTag] = cb;
    return HCCL_SUCCESS;
}
int32_t HcclTaskUnRegister(HcclComm comm, const char *msgTag)
{
    Comm *c = AsComm(comm);
    if (!c || !msgTag) return HCCL_E_PTR;
    std::lock_guard<std::mutex> lk(c->resMu);
    return c->taskCallbacks.erase(msgTag) ? HCCL_SUCCESS : HCCL_E_NOT_FOUND;
}
// Queues the registered callback on `stream`: it runs on a host thread once everything queued before it has finished.
int32_t HcclTaskNotify(HcclComm comm, const char *msgTag, uint64_t arg0, int32_t arg1, aclrtStream stream)
{
    Comm *c = AsComm(comm);
    if (!c || !msgTag) return HCCL_E_PTR;
    HcclTaskCallback *cb = nullptr;
    {
        std::lock_guard<std::mutex> lk(c->resMu);
        auto it = c->taskCallbacks.find(msgTag);
        if (it == c->taskCallbacks.end()) return HCCL_E_NOT_FOUND;
        cb = it->second;
    }
    return (int32_t)c->plat->HostFuncAsync([cb, arg0, arg1] { cb(arg0, arg1); }, c->plat->kind() == PlatKind::SIM ? nullptr : stream);
}

HcclResult HcclCommAddExchangeInfo(HcclComm comm, const void *data, uint32_t length)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(data);
    if (length == 0 || length > 4096) return HCCL_E_PARA;
    std::lock_guard<std::mutex> lk(c->resMu);
    c->exchangeInfo.insert(c->exchangeInfo.end(), (const uint8_t *)data, (const uint8_t *)data + length);
    return HCCL_SUCCESS;
}
// Collective on first use after a change: gathers every rank's bytes over the control plane.
HcclResult HcclCommGetExchangeInfo(HcclComm comm, uint32_t rank, void *data, uint32_t capacity, uint32_t *length)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(length);
    if (rank >= c->nRanks) return HCCL_E_PARA;
    if (c->peerExchangeInfo.empty()) {
        Blob mine;
        {
            std::lock_guard<std::mutex> lk(c->resMu);
            mine = c->exchangeInfo;
        }
        std::vector<Blob> all;
        CHK_RET(c->boot->AllGather(c->group, mine, &all));
        std::lock_guard<std::mutex> lk(c->resMu);
        c->peerExchangeInfo.assign(all.begin(), all.end());
    }
    const auto &b = c->peerExchangeInfo[rank];
    *length = (uint32_t)b.size();
    if (data) {
        if (capacity < b.size()) return HCCL_E_MEMORY;
        memcpy(data, b.data(), b.size());
    }
    return HCCL_SUCCESS;
}
HcclResult HcclCommResetExchangeInfo(HcclComm comm)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    std::lock_guard<std::mutex> lk(c->resMu);
    c->exchangeInfo.clear();
    c->peerExchangeInfo.clear();
    return HCCL_SUCCESS;
}

int32_t HcommThreadJoin(ThreadHandle thread, uint32_t timeout)
{
    ThreadRes *t = AsThread(thread);
    if (!t) return HCCL_E_PTR;
    if (!t->stream || !t->plat) return HCCL_SUCCESS;
    (void)timeout;      // device-side waits carry their own limits, so a stream always drains
    return (int32_t)t->plat->StreamSync(t->stream);
}

}  // extern "C"
