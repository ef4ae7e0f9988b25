// comm_api.cc - C entry points for communicator life cycle, configuration and fault handling
// (declared in include/hccl/hccl_comm.h).
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <thread>

#include "../coll/ops.h"
#include "../comm/comm.h"
#include "../core/env.h"
#include "../core/log.h"
#include "../core/net.h"
#include "hccl/hccl.h"
#include "hccl/hccl_comm.h"

using namespace hc;

namespace {

std::mutex g_hubMu;
// Rendezvous servers started by HcclGetRootInfo, keyed by identifier, until a communicator adopts them.
std::map<std::string, std::shared_ptr<BootstrapHub>> g_pendingHubs;
std::atomic<int> g_processDeterministic{-1};

struct StateCb {
    std::string name;
    HcclCommStateCallback cb;
    void *args;
};
std::mutex g_cbMu;
std::vector<StateCb> g_stateCbs;

void FireState(Comm *c, HcclCommStatePhase phase)
{
    std::vector<StateCb> cbs;
    {
        std::lock_guard<std::mutex> lk(g_cbMu);
        cbs = g_stateCbs;
    }
    for (auto &s : cbs) s.cb((HcclComm)c, phase, s.args);
}

HcclResult InitWithRoot(uint32_t nRanks, const RootHandle &root, uint32_t rank, const HcclCommConfig *config, HcclComm *comm)
{
    if (nRanks == 0 || rank >= nRanks) {
        RPT_ERR("EI0003", "rank %u is outside a communicator of %u ranks", rank, nRanks);
        return HCCL_E_PARA;
    }
    Platform *plat = DefaultPlatform();
    if (!plat) return HCCL_E_NOT_SUPPORT;
    int device = plat->CurrentDevice();
    if (plat->kind() == PlatKind::CUDA) CHK_RET(plat->SetDevice(device));
    auto boot = std::make_shared<Bootstrap>();
    std::vector<Blob> table;
    CHK_RET(boot->Connect(root, rank, nRanks, MakeRankRecord(plat, device, rank), &table));
    CommInitArgs args;
    args.plat = plat;
    args.device = device;
    args.boot = boot;
    {
        std::lock_guard<std::mutex> lk(g_hubMu);
        auto it = g_pendingHubs.find(root.identifier);
        if (it != g_pendingHubs.end() && rank == 0) {
            args.hub = it->second;
            g_pendingHubs.erase(it);
        }
    }
    args.group = boot->WorldGroup();
    args.memberInfo = table;
    args.config = config;
    args.defaultName = root.identifier;
    Comm *c = nullptr;
    HcclResult r = CommCreate(args, &c);
    if (r != HCCL_SUCCESS) {
        boot->Close();
        return r;
    }
    if (g_processDeterministic.load() >= 0 && !(config && config->hcclDeterministic != HCCL_COMM_DETERMINISTIC_CONFIG_NOT_SET))
        c->cfg.deterministic = (uint32_t)g_processDeterministic.load();
    *comm = (HcclComm)c;
    return HCCL_SUCCESS;
}

}  // namespace

extern "C" {

HcclResult HcclGetRootInfo(HcclRootInfo *rootInfo)
{
    CHK_PTR_NULL(rootInfo);
    static_assert(sizeof(RootHandle) <= HCCL_ROOT_INFO_BYTES, "root handle must fit the ticket");
    auto hub = std::make_shared<BootstrapHub>();
    CHK_RET(hub->Start(net::PickLocalIp(), 0, ""));
    memset(rootInfo->internal, 0, sizeof(rootInfo->internal));
    memcpy(rootInfo->internal, &hub->handle(), sizeof(RootHandle));
    std::lock_guard<std::mutex> lk(g_hubMu);
    g_pendingHubs[hub->handle().identifier] = hub;
    return HCCL_SUCCESS;
}

HcclResult HcclCommInitRootInfoConfig(uint32_t nRanks, const HcclRootInfo *rootInfo, uint32_t rank, const HcclCommConfig *config,
                                      HcclComm *comm)
{
    CHK_PTR_NULL(rootInfo);
    CHK_PTR_NULL(comm);
    RootHandle root;
    memcpy(&root, rootInfo->internal, sizeof(root));
    if (GroupActive()) {
        // Deferred bring-up inside a group: several communicators can rendezvous concurrently at GroupEnd.
        HcclCommConfig cfgCopy;
        bool hasCfg = config != nullptr;
        if (hasCfg) cfgCopy = *config;
        GroupQueue([=]() { return InitWithRoot(nRanks, root, rank, hasCfg ? &cfgCopy : nullptr, comm); }, 0, false, nullptr, nullptr);
        return HCCL_SUCCESS;
    }
    return InitWithRoot(nRanks, root, rank, config, comm);
}

HcclResult HcclCommInitRootInfo(uint32_t nRanks, const HcclRootInfo *rootInfo, uint32_t rank, HcclComm *comm)
{
    return HcclCommInitRootInfoConfig(nRanks, rootInfo, rank, nullptr, comm);
}

HcclResult HcclCommInitClusterInfoConfig(const char *clusterInfo, uint32_t rank, HcclCommConfig *config, HcclComm *comm)
{
    CHK_PTR_NULL(clusterInfo);
    CHK_PTR_NULL(comm);
    RankTable table;
    std::string err;
    HcclResult r = table.LoadFile(clusterInfo, &err);
    if (r != HCCL_SUCCESS) {
        RPT_ERR("EI0004", "rank table %s rejected: %s", clusterInfo, err.c_str());
        return r;
    }
    if (rank >= table.size()) {
        RPT_ERR("EI0004", "rank %u is not in the rank table (%u ranks)", rank, table.size());
        return HCCL_E_PARA;
    }
    // Rank 0 hosts the rendezvous at an address every rank derives from the table alone.
    const EnvConfig &env = EnvConfig::Get();
    std::string ip = table.ranks[0].hostIp.empty() ? (table.ranks[0].deviceIp.empty() ? "127.0.0.1" : table.ranks[0].deviceIp) : table.ranks[0].hostIp;
    if (table.ServerCount() == 1) ip = env.ifIp.value.empty() ? "127.0.0.1" : env.ifIp.value;
    int port = (env.ifBasePort.fromEnv ? env.ifBasePort.value : 60000) + (int)(table.Crc() % 16);
    RootHandle root;
    memset(&root, 0, sizeof(root));
    snprintf(root.ip, sizeof(root.ip), "%s", ip.c_str());
    root.port = (uint32_t)port;
    root.magic = kRootHandleMagic;
    root.version = 1;
    snprintf(root.identifier, sizeof(root.identifier), "ranktable_%08x_%d", table.Crc(), port);
    if (rank == 0) {
        auto hub = std::make_shared<BootstrapHub>();
        // The port follows from the table, so the hub of an earlier communicator from a table with the same port (or
        // from this one) may still be winding down there: try for a few seconds before giving up.
        r = hub->Start(ip, port, root.identifier);
        for (int attempt = 0; r != HCCL_SUCCESS && attempt < 50; ++attempt) {
            usleep(100000);
            hub = std::make_shared<BootstrapHub>();
            r = hub->Start(ip, port, root.identifier);
        }
        if (r != HCCL_SUCCESS) {
            RPT_ERR("EI0019", "rank 0 cannot listen on %s:%d for the rank-table rendezvous (set HCCL_IF_BASE_PORT to move it)", ip.c_str(), port);
            return r;
        }
        std::lock_guard<std::mutex> lk(g_hubMu);
        g_pendingHubs[root.identifier] = hub;
    }
    r = InitWithRoot(table.size(), root, rank, config, comm);
    if (r != HCCL_SUCCESS) return r;
    // The table in the file is authoritative for layers and addresses; what the rendezvous measured must agree on devices.
    Comm *c = AsComm(*comm);
    for (uint32_t i = 0; i < table.size(); ++i) {
        if (c->plat->kind() == PlatKind::CUDA && table.ranks[i].deviceId != c->table.ranks[i].deviceId)
            HCCL_WARNING("rank %u runs on device %d but the rank table says %d", i, c->table.ranks[i].deviceId, table.ranks[i].deviceId);
        table.ranks[i].platKind = c->table.ranks[i].platKind;
        table.ranks[i].pid = c->table.ranks[i].pid;
        table.ranks[i].fabricClique = c->table.ranks[i].fabricClique;
    }
    c->table = table;
    c->graph.Build(table, rank);
    return HCCL_SUCCESS;
}

HcclResult HcclCommInitClusterInfo(const char *clusterInfo, uint32_t rank, HcclComm *comm)
{
    return HcclCommInitClusterInfoConfig(clusterInfo, rank, nullptr, comm);
}

HcclResult HcclCommInitAll(uint32_t ndev, int32_t *devices, HcclComm *comms)
{
    CHK_PTR_NULL(devices);
    CHK_PTR_NULL(comms);
    if (ndev == 0) return HCCL_E_PARA;
    Platform *plat = DefaultPlatform();
    if (!plat) return HCCL_E_NOT_SUPPORT;
    if (plat->kind() == PlatKind::CUDA) {
        for (uint32_t i = 0; i < ndev; ++i)
            for (uint32_t j = 0; j < i; ++j)
                if (devices[i] == devices[j] && devices[0] != devices[i]) {
                    RPT_ERR("EI0003", "HcclCommInitAll: device %d is listed twice", devices[i]);
                    return HCCL_E_PARA;
                }
    }
    HcclRootInfo info;
    CHK_RET(HcclGetRootInfo(&info));
    std::vector<HcclResult> results(ndev, HCCL_SUCCESS);
    std::vector<std::thread> th;
    for (uint32_t i = 0; i < ndev; ++i) {
        th.emplace_back([&, i] {
            HcclResult r = plat->SetDevice(devices[i]);
            if (r == HCCL_SUCCESS) r = HcclCommInitRootInfo(ndev, &info, i, &comms[i]);
            results[i] = r;
        });
    }
    for (auto &t : th) t.join();
    for (auto r : results)
        if (r != HCCL_SUCCESS) return r;
    return HCCL_SUCCESS;
}

HcclResult HcclCreateSubCommConfig(HcclComm *comm, uint32_t rankNum, uint32_t *rankIds, uint64_t subCommId, uint32_t subCommRankId,
                                   HcclCommConfig *config, HcclComm *subComm)
{
    CHK_PTR_NULL(comm);
    CHK_PTR_NULL(subComm);
    Comm *parent = AsComm(*comm);
    CHK_PTR_NULL(parent);
    // A rank that is not a member passes rankIds == NULL (or 0xffffffff as its sub rank) and gets no communicator.
    if (rankIds == nullptr || subCommRankId == 0xffffffffu) {
        *subComm = nullptr;
        return HCCL_SUCCESS;
    }
    if (rankNum == 0 || rankNum > parent->nRanks || subCommRankId >= rankNum) return HCCL_E_PARA;
    std::vector<uint32_t> world;
    std::vector<Blob> info;
    for (uint32_t i = 0; i < rankNum; ++i) {
        if (rankIds[i] >= parent->nRanks) {
            RPT_ERR("EI0003", "sub communicator member %u is outside the parent (%u ranks)", rankIds[i], parent->nRanks);
            return HCCL_E_PARA;
        }
        for (uint32_t j = 0; j < i; ++j)
            if (rankIds[j] == rankIds[i]) return HCCL_E_PARA;
        world.push_back(parent->worldRanks[rankIds[i]]);
        RankTable one;
        one.version = "boot";
        RankEntry e = parent->table.ranks[rankIds[i]];
        e.rankId = 0;
        e.levels.clear();
        one.ranks.push_back(e);
        info.push_back(one.Serialize());
    }
    if (rankIds[subCommRankId] != parent->rank) {
        RPT_ERR("EI0003", "subCommRankId %u does not name the calling rank", subCommRankId);
        return HCCL_E_PARA;
    }
    CommInitArgs args;
    args.plat = parent->plat;
    args.device = parent->device;
    args.boot = parent->boot;
    // group id: derived from the caller's id and the member list so that unrelated sub groups never share tags
    uint32_t gid = Crc32(world.data(), world.size() * 4, (uint32_t)(subCommId * 2654435761u + 1));
    if (gid == 0) gid = 1;
    args.group = parent->boot->MakeGroup(gid, world);
    args.memberInfo = info;
    args.config = config;
    args.defaultName = parent->cfg.name + "_sub" + std::to_string(subCommId);
    Comm *c = nullptr;
    CHK_RET(CommCreate(args, &c));
    if (!(config && config->hcclDeterministic != HCCL_COMM_DETERMINISTIC_CONFIG_NOT_SET)) c->cfg.deterministic = parent->cfg.deterministic;
    *subComm = (HcclComm)c;
    return HCCL_SUCCESS;
}

HcclResult HcclCommDestroy(HcclComm comm)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    FireState(c, HCCL_COMM_STATE_PHASE_DESTROY_PRE);
    {
        std::lock_guard<std::mutex> lk(c->opMu);
        if (c->plat->kind() == PlatKind::CUDA) {
            // everything this communicator launched must have left the GPU before its memory goes away
            for (auto &t : c->threads)
                if (t->stream && t->ownsStream) c->plat->StreamSync(t->stream);
            for (auto s : c->auxStreams) c->plat->StreamSync(s);
        }
    }
    CommDestroy(c);
    FireState(nullptr, HCCL_COMM_STATE_PHASE_DESTROY_POST);
    return HCCL_SUCCESS;
}

HcclResult HcclSetConfig(HcclConfig config, union HcclConfigValue configValue)
{
    if (config != HCCL_DETERMINISTIC) return HCCL_E_NOT_SUPPORT;
    if (configValue.value < 0 || configValue.value > 2) return HCCL_E_PARA;
    g_processDeterministic.store(configValue.value);
    // operators of other threads may be reading the setting right now
    RegistryForEach([&](Comm *c) { __atomic_store_n(&c->cfg.deterministic, (uint32_t)configValue.value, __ATOMIC_RELAXED); });
    return HCCL_SUCCESS;
}

HcclResult HcclGetConfig(HcclConfig config, union HcclConfigValue *configValue)
{
    CHK_PTR_NULL(configValue);
    if (config != HCCL_DETERMINISTIC) return HCCL_E_NOT_SUPPORT;
    int v = g_processDeterministic.load();
    configValue->value = v >= 0 ? v : EnvConfig::Get().deterministic.value;
    return HCCL_SUCCESS;
}

HcclResult HcclGetCommName(HcclComm comm, char *commName)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    CHK_PTR_NULL(commName);
    snprintf(commName, COMM_NAME_MAX_LENGTH, "%s", c->cfg.name.c_str());
    return HCCL_SUCCESS;
}

HcclResult HcclCommGetHandleWithName(const char *commName, HcclComm *comm)
{
    CHK_PTR_NULL(commName);
    CHK_PTR_NULL(comm);
    Comm *c = RegistryFind(commName);
    if (!c) return HCCL_E_NOT_FOUND;
    *comm = (HcclComm)c;
    return HCCL_SUCCESS;
}

HcclResult HcclGetRankSize(HcclComm comm, uint32_t *rankSize)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    CHK_PTR_NULL(rankSize);
    *rankSize = c->nRanks;
    return HCCL_SUCCESS;
}

HcclResult HcclGetRankId(HcclComm comm, uint32_t *rank)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    CHK_PTR_NULL(rank);
    *rank = c->rank;
    return HCCL_SUCCESS;
}

HcclResult HcclGetCommAsyncError(HcclComm comm, HcclResult *asyncError)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    CHK_PTR_NULL(asyncError);
    CommPollDeviceStatus(c);
    int e = c->asyncError.load();
    if (e == 0 && c->boot) {
        if (c->boot->RemoteError() != HCCL_SUCCESS) e = HCCL_E_REMOTE;
        else {
            // a member of this communicator stopped answering heartbeats or went away (ranks that are lost but do not
            // belong to it - a communicator over the survivors of its parent - do not count)
            const uint64_t lost = c->boot->LostMask();
            for (uint32_t w : c->worldRanks)
                if (w < 64 && ((lost >> w) & 1)) e = HCCL_E_REMOTE;
        }
        if (e == 0 && c->boot->HubGone()) e = HCCL_E_REMOTE;    // rank 0's process, which hosts the hub, is gone
    }
    *asyncError = (HcclResult)e;
    return HCCL_SUCCESS;
}

const char *HcclGetErrorString(HcclResult code)
{
    switch (code) {
        case HCCL_SUCCESS: return "no error";
        case HCCL_E_PARA: return "parameter error";
        case HCCL_E_PTR: return "empty pointer";
        case HCCL_E_MEMORY: return "memory error";
        case HCCL_E_INTERNAL: return "internal error";
        case HCCL_E_NOT_SUPPORT: return "not support feature";
        case HCCL_E_NOT_FOUND: return "not found specific resource";
        case HCCL_E_UNAVAIL: return "resource unavailable";
        case HCCL_E_SYSCALL: return "call system interface error";
        case HCCL_E_TIMEOUT: return "timeout";
        case HCCL_E_OPEN_FILE_FAILURE: return "open file fail";
        case HCCL_E_TCP_CONNECT: return "tcp connect fail";
        case HCCL_E_ROCE_CONNECT: return "roce connect fail";
        case HCCL_E_TCP_TRANSFER: return "tcp transfer fail";
        case HCCL_E_ROCE_TRANSFER: return "roce transfer fail";
        case HCCL_E_RUNTIME: return "call runtime api fail";
        case HCCL_E_DRV: return "call driver api fail";
        case HCCL_E_PROFILING: return "call profiling api fail";
        case HCCL_E_CCE: return "call cce api fail";
        case HCCL_E_NETWORK: return "call network api fail";
        case HCCL_E_AGAIN: return "try again";
        case HCCL_E_REMOTE: return "error cqe";
        case HCCL_E_SUSPENDING: return "error communicator suspending";
        case HCCL_E_OPRETRY_FAIL: return "retry constraint";
        case HCCL_E_OOM: return "out of memory";
        case HCCL_E_IN_STATUS: return "the error information is in the status";
        default: return "unknown error";
    }
}

uint32_t HcclGetCommConfigCapability(void)
{
    return (1u << HCCL_COMM_CONFIG_BUFFER_SIZE) | (1u << HCCL_COMM_CONFIG_DETERMINISTIC) | (1u << HCCL_COMM_CONFIG_COMM_NAME) |
           (1u << HCCL_COMM_CONFIG_OP_EXPANSION_MODE) | (1u << HCCL_COMM_CONFIG_SUPPORT_INIT_BY_ENV) | (1u << HCCL_COMM_CONFIG_WORLD_RANKID) |
           (1u << HCCL_COMM_CONFIG_JOBID) | (1u << HCCL_COMM_CONFIG_ACLGRAPH_ZEROCOPY_ENABLE) | (1u << HCCL_COMM_CONFIG_EXEC_TIMEOUT) |
           (1u << HCCL_COMM_CONFIG_ALGO) | (1u << HCCL_COMM_CONFIG_RETRY) | (1u << HCCL_COMM_CONFIG_BUFFER_NAME);
}

HcclResult HcclConfigGetInfo(HcclComm comm, HcclConfigType cfgType, uint32_t infoLen, void *info)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    CHK_PTR_NULL(info);
    if (cfgType == HCCL_CONFIG_TYPE_OP_EXPANSION_MODE) {
        if (infoLen < sizeof(HcclOpExpansionMode)) return HCCL_E_PARA;
        // translate the communicator setting into the query enum
        static const HcclOpExpansionMode map[] = {HCCL_OP_EXPANSION_MODE_AIV, HCCL_OP_EXPANSION_MODE_HOST, HCCL_OP_EXPANSION_MODE_HOST_TS,
                                                  HCCL_OP_EXPANSION_MODE_AIV, HCCL_OP_EXPANSION_AIV_ONLY, HCCL_OP_EXPANSION_MODE_CCU_MS,
                                                  HCCL_OP_EXPANSION_MODE_CCU_SCHED};
        HcclOpExpansionMode m = c->plat->kind() == PlatKind::SIM ? HCCL_OP_EXPANSION_MODE_HOST : map[c->cfg.opExpansionMode % 7];
        memcpy(info, &m, sizeof(m));
        return HCCL_SUCCESS;
    }
    if (cfgType == HCCL_CONFIG_TYPE_HCCL_ALGO) {
        std::string s = c->cfg.algo.empty() ? "auto" : c->cfg.algo;
        if (infoLen < s.size() + 1) return HCCL_E_PARA;
        memcpy(info, s.c_str(), s.size() + 1);
        return HCCL_SUCCESS;
    }
    return HCCL_E_NOT_SUPPORT;
}

// ------------------------------------------------------------------------------ fault handling

HcclResult HcclCommSuspend(HcclComm comm)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    int expected = (int)CommState::READY;
    if (!c->state.compare_exchange_strong(expected, (int)CommState::SUSPENDING)) {
        return expected == (int)CommState::SUSPENDED ? HCCL_SUCCESS : HCCL_E_PARA;
    }
    // Stop launching: taking the operator lock waits for the launch in progress; raising the abort word makes
    // every device-side wait of operators already on the GPU return.
    std::lock_guard<std::mutex> lk(c->opMu);
    __atomic_store_n(c->abortWord, 1u, __ATOMIC_RELEASE);
    if (c->plat->kind() == PlatKind::CUDA) {
        for (auto &t : c->threads)
            if (t->stream && t->ownsStream) c->plat->StreamSync(t->stream);
        for (auto s : c->auxStreams) c->plat->StreamSync(s);
    }
    c->state.store((int)CommState::SUSPENDED);
    HCCL_RUN_INFO("communicator \"%s\" rank %u suspended", c->cfg.name.c_str(), c->rank);
    return HCCL_SUCCESS;
}

}  // extern "C"

namespace hc {
// Collective (two barriers on `g`): puts every synchronisation value of the communicator back to its initial state -
// flag pages, device counters, host-side expectations, the abort word and the recorded failure.  The caller holds
// the operator lock and nothing of this communicator is in flight on any rank.
HcclResult CommClearSyncState(Comm *c, Bootstrap::Group &g)
{
    Platform *P = c->plat;
    CHK_RET(c->boot->Barrier(g));            // everyone is quiescent
    CHK_RET(P->MemsetSync(c->LocalHeap(), 0, HC_CTRL_BYTES));
    CHK_RET(P->MemsetSync(c->LocalHeap() + c->llOffset, 0, c->llBytes));
    CHK_RET(P->MemsetSync(c->devCounters, 0, 128 * sizeof(uint32_t)));
    CHK_RET(P->MemsetSync(c->devIrCounters, 0, 2ull * HC_IR_MAX_CTAS * HC_IR_RANKS * HC_IR_NOTIFY * sizeof(uint64_t)));
    std::fill(c->chanWaited.begin(), c->chanWaited.end(), 0);
    std::fill(c->p2pSent.begin(), c->p2pSent.end(), 0);
    std::fill(c->p2pRecvd.begin(), c->p2pRecvd.end(), 0);
    for (auto &ch : c->channels) std::fill(ch->waited.begin(), ch->waited.end(), 0);
    for (auto &t : c->threads) {
        std::fill(t->waited.begin(), t->waited.end(), 0);
        if (t->notify) memset(t->notify, 0, t->notifyNum * sizeof(uint64_t));
    }
    c->hostLaunches = 0;
    c->lastOpOnHost = true;
    if (P->kind() == PlatKind::CUDA) FusedResetLocal(c);
    memset(c->waitStatus, 0, sizeof(HcclDeviceWaitStatus));
    __atomic_store_n(c->abortWord, 0u, __ATOMIC_RELEASE);
    c->asyncError.store(0);
    c->boot->ClearRemoteError();
    CHK_RET(c->boot->Barrier(g));            // nobody signals into a page that is still being cleared
    return HCCL_SUCCESS;
}
}  // namespace hc

extern "C" {

// Collective over the ranks that are still alive: clears the flag pages and counters so that the
// next operator starts from a consistent state, then reopens the communicator.
HcclResult HcclCommResume(HcclComm comm)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    if (c->state.load() != (int)CommState::SUSPENDED) {
        RPT_ERR("EI0003", "HcclCommResume on a communicator that is not suspended");
        return HCCL_E_PARA;
    }
    FireState(c, HCCL_COMM_STATE_PHASE_RESUME_PRE);
    std::lock_guard<std::mutex> lk(c->opMu);
    CHK_RET(CommClearSyncState(c, c->group));
    c->state.store((int)CommState::READY);
    FireState(c, HCCL_COMM_STATE_PHASE_RESUME_POST);
    HCCL_RUN_INFO("communicator \"%s\" rank %u resumed", c->cfg.name.c_str(), c->rank);
    return HCCL_SUCCESS;
}

HcclResult HcclCommRecover(HcclComm comm, uint32_t timeoutSec, HcclComm *newComm, uint32_t *newSize, uint32_t *oldRanks)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(newComm);
    if (!c->boot) return HCCL_E_NOT_SUPPORT;
    if (timeoutSec == 0) timeoutSec = (uint32_t)EnvConfig::Get().connectTimeoutSec.value;
    const int64_t deadline = net::NowMs() + (int64_t)timeoutSec * 1000;
    constexpr uint8_t kProbe = 'P', kTicket = 'T';
    struct Ticket { uint8_t kind; uint8_t pad[3]; uint32_t count; HcclRootInfo info; };      // followed by `count` old ranks
    std::vector<uint32_t> members;          // old ranks of the new communicator, ascending
    HcclRootInfo info;
    for (;;) {
        if (net::NowMs() >= deadline) { RPT_ERR("EI0015", "HcclCommRecover: the survivors of \"%s\" did not find each other within %u s", c->cfg.name.c_str(), timeoutSec); return HCCL_E_TIMEOUT; }
        uint64_t lost = c->boot->LostMask();
        if (c->boot->HubGone()) lost |= 1ull;                   // the hub lives in world rank 0's process
        std::vector<uint32_t> alive;
        for (uint32_t i = 0; i < c->nRanks; ++i)
            if (c->worldRanks[i] >= 64 || !((lost >> c->worldRanks[i]) & 1)) alive.push_back(i);
        if (alive.empty() || std::find(alive.begin(), alive.end(), c->rank) == alive.end()) return HCCL_E_INTERNAL;
        const uint32_t leader = alive[0];
        if (leader == c->rank) {
            // who of them answers on its local socket right now?  (a rank that is gone refuses the connection)
            members.assign(1, c->rank);
            for (uint32_t i : alive)
                if (i != c->rank && c->boot->SendDirect(c->worldRanks[i], Blob(1, kProbe)) == HCCL_SUCCESS) members.push_back(i);
            std::sort(members.begin(), members.end());
            CHK_RET(HcclGetRootInfo(&info));
            Blob msg(sizeof(Ticket) + members.size() * 4);
            Ticket t;
            memset(&t, 0, sizeof(t));
            t.kind = kTicket; t.count = (uint32_t)members.size(); t.info = info;
            memcpy(msg.data(), &t, sizeof(t));
            memcpy(msg.data() + sizeof(t), members.data(), members.size() * 4);
            for (uint32_t i : members)
                if (i != c->rank) CHK_RET(c->boot->SendDirect(c->worldRanks[i], msg));
            break;
        }
        Blob msg;
        HcclResult r = c->boot->RecvDirect(c->worldRanks[leader], &msg, 500);
        if (r == HCCL_E_TIMEOUT) continue;                      // look at the lost set again: the leader may be gone as well
        if (r != HCCL_SUCCESS) return r;
        if (msg.size() < sizeof(Ticket) || msg[0] != kTicket) continue;      // a probe
        Ticket t;
        memcpy(&t, msg.data(), sizeof(t));
        if (msg.size() != sizeof(Ticket) + (size_t)t.count * 4 || t.count == 0 || t.count > c->nRanks) return HCCL_E_INTERNAL;
        members.resize(t.count);
        memcpy(members.data(), msg.data() + sizeof(t), (size_t)t.count * 4);
        info = t.info;
        break;
    }
    auto me = std::find(members.begin(), members.end(), c->rank);
    if (me == members.end()) { RPT_ERR("EI0015", "HcclCommRecover: rank %u is not among the survivors the leader found", c->rank); return HCCL_E_INTERNAL; }
    HcclCommConfig cfg;
    HcclCommConfigInit(&cfg);
    snprintf(cfg.hcclCommName, sizeof(cfg.hcclCommName), "%.100s_recovered", c->cfg.name.c_str());
    cfg.hcclBufferSize = c->cfg.bufferMB;
    cfg.hcclDeterministic = __atomic_load_n(&c->cfg.deterministic, __ATOMIC_RELAXED);
    cfg.hcclOpExpansionMode = c->cfg.opExpansionMode;
    cfg.hcclExecTimeOut = c->cfg.execTimeoutSec;
    snprintf(cfg.hcclAlgo, sizeof(cfg.hcclAlgo), "%s", c->cfg.algo.c_str());
    snprintf(cfg.hcclRetryEnable, sizeof(cfg.hcclRetryEnable), "%s", c->cfg.retryEnable.c_str());
    snprintf(cfg.hcclRetryParams, sizeof(cfg.hcclRetryParams), "%s", c->cfg.retryParams.c_str());
    CHK_RET(HcclCommInitRootInfoConfig((uint32_t)members.size(), &info, (uint32_t)(me - members.begin()), &cfg, newComm));
    if (newSize) *newSize = (uint32_t)members.size();
    if (oldRanks) memcpy(oldRanks, members.data(), members.size() * 4);
    HCCL_RUN_INFO("communicator \"%s\": %zu of %u ranks go on as \"%s\", this one as rank %u", c->cfg.name.c_str(), members.size(), c->nRanks, cfg.hcclCommName,
                  (uint32_t)(me - members.begin()));
    return HCCL_SUCCESS;
}

HcclResult HcclCommRegCommStateCallback(const char *regName, HcclCommStateCallback cb, void *args)
{
    CHK_PTR_NULL(regName);
    std::lock_guard<std::mutex> lk(g_cbMu);
    for (auto it = g_stateCbs.begin(); it != g_stateCbs.end(); ++it)
        if (it->name == regName) { g_stateCbs.erase(it); break; }
    if (cb) g_stateCbs.push_back({regName, cb, args});
    return HCCL_SUCCESS;
}

HcclResult HcclCommGetStatus(const char *commId, HcclCommStatus *status)
{
    CHK_PTR_NULL(commId);
    CHK_PTR_NULL(status);
    Comm *c = RegistryFind(commId);
    if (!c) {
        *status = HCCL_COMM_STATUS_INVALID;
        return HCCL_E_NOT_FOUND;
    }
    int st = c->state.load();
    *status = st == (int)CommState::READY ? HCCL_COMM_STATUS_READY : (st == (int)CommState::DESTROYED ? HCCL_COMM_STATUS_INVALID : HCCL_COMM_STATUS_SUSPENDING);
    return HCCL_SUCCESS;
}

// One NVSwitch node has a single path between two GPUs, so there is no backup port to move to; the
// call validates its arguments and reports that nothing can change.
HcclResult HcclCommWorkingDevNicSet(HcclComm comm, uint32_t *ranks, bool *useBackup, uint32_t nRanks)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    CHK_PTR_NULL(ranks);
    CHK_PTR_NULL(useBackup);
    for (uint32_t i = 0; i < nRanks; ++i) {
        if (ranks[i] >= c->nRanks) return HCCL_E_PARA;
        if (useBackup[i]) return HCCL_E_NOT_SUPPORT;
    }
    return HCCL_SUCCESS;
}

HcclResult HcclBarrier(HcclComm comm, aclrtStream stream)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    OpDesc d;
    d.cmd = HCCL_CMD_BARRIER;
    d.stream = stream;
    d.count = 1;
    return SubmitOp(c, d);
}

}  // extern "C"
