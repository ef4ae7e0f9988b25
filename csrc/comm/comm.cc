#include "comm.h"

#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <fstream>

#include "../alg/selector.h"
#include "../core/env.h"
#include "../core/log.h"
#include "../device/coll_kernels.h"
#include "../topo/nvml_topo.h"

namespace hc {

namespace {

std::mutex g_regMu;
std::map<std::string, Comm *> g_registry;

std::string HostIdentity()
{
    char host[128] = {0};
    gethostname(host, sizeof(host) - 1);
    std::string id = host;
    std::ifstream f("/proc/sys/kernel/random/boot_id");
    std::string boot;
    if (f && std::getline(f, boot)) id += "-" + boot.substr(0, 8);
    return id;
}

uint64_t AlignUp(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

}  // namespace

Blob MakeRankRecord(Platform *plat, int device, uint32_t rank)
{
    RankTable t;
    t.version = "boot";
    RankEntry e;
    e.rankId = 0;
    e.deviceId = device;
    e.localId = -1;
    e.serverId = HostIdentity();
    e.hostIp = net::PickLocalIp();
    e.pid = (uint32_t)getpid();
    e.platKind = (uint32_t)plat->kind();
    if (plat->kind() == PlatKind::CUDA) {
        std::vector<GpuTopoInfo> gpus;
        if (ProbeLocalGpus(&gpus) == HCCL_SUCCESS && device >= 0 && (size_t)device < gpus.size()) {
            e.busId = gpus[device].busId;
            e.nvlinkCount = gpus[device].activeLinks;
            e.fabricClique = gpus[device].fabricClique;
        }
    }
    (void)rank;
    t.ranks.push_back(e);
    return t.Serialize();
}

HcclResult ResolveConfig(const HcclCommConfig *cfg, const std::string &defaultName, ResolvedConfig *out)
{
    const EnvConfig &env = EnvConfig::Get();
    ResolvedConfig r;
    r.bufferMB = env.buffSizeMB.value;
    r.deterministic = (uint32_t)env.deterministic.value;
    r.opExpansionMode = (uint32_t)env.opExpansionMode.value;
    r.execTimeoutSec = env.execTimeoutSec.value;
    r.algo = env.algo.value;
    r.name = defaultName;
    r.symStrideGB = env.symStrideGB.value > 0 ? (uint64_t)env.symStrideGB.value : HCCL_DEFAULT_SYMMETRIC_MEMORY_STRIDE;
    if (cfg) {
        struct Header { size_t size; uint32_t magic; uint32_t version; uint64_t reserved; };
        const Header *h = (const Header *)cfg;
        if (h->magic != HCCL_COMM_CONFIG_MAGIC_WORD) {
            RPT_ERR("EI0003", "HcclCommConfig was not initialised with HcclCommConfigInit (magic 0x%x)", h->magic);
            return HCCL_E_PARA;
        }
        if (h->version > HCCL_COMM_CONFIG_VERSION) HCCL_WARNING("HcclCommConfig version %u is newer than %u; extra fields ignored", h->version, (unsigned)HCCL_COMM_CONFIG_VERSION);
        // Fields appear in the struct in the order versions introduced them; only read what the caller's size covers.
        auto covers = [&](const void *field, size_t len) { return (size_t)((const char *)field - (const char *)cfg) + len <= h->size; };
        if (covers(&cfg->hcclBufferSize, 4) && cfg->hcclBufferSize != HCCL_COMM_BUFFSIZE_CONFIG_NOT_SET) {
            if (cfg->hcclBufferSize == 0) { RPT_ERR("EI0003", "hcclBufferSize must be at least 1 MB"); return HCCL_E_PARA; }
            r.bufferMB = cfg->hcclBufferSize;
        }
        if (covers(&cfg->hcclDeterministic, 4) && cfg->hcclDeterministic != HCCL_COMM_DETERMINISTIC_CONFIG_NOT_SET) {
            if (cfg->hcclDeterministic > 2) { RPT_ERR("EI0003", "hcclDeterministic must be 0, 1 or 2"); return HCCL_E_PARA; }
            r.deterministic = cfg->hcclDeterministic;
        }
        if (covers(cfg->hcclCommName, COMM_NAME_MAX_LENGTH) && cfg->hcclCommName[0]) r.name = std::string(cfg->hcclCommName, strnlen(cfg->hcclCommName, COMM_NAME_MAX_LENGTH));
        if (covers(cfg->hcclUdi, UDI_MAX_LENGTH) && cfg->hcclUdi[0]) r.udi = std::string(cfg->hcclUdi, strnlen(cfg->hcclUdi, UDI_MAX_LENGTH));
        if (covers(&cfg->hcclOpExpansionMode, 4) && cfg->hcclOpExpansionMode != 0) {
            if (cfg->hcclOpExpansionMode > 6) { RPT_ERR("EI0003", "hcclOpExpansionMode %u is not defined", cfg->hcclOpExpansionMode); return HCCL_E_PARA; }
            r.opExpansionMode = cfg->hcclOpExpansionMode;
        }
        if (covers(&cfg->hcclWorldRankID, 4)) r.worldRankId = cfg->hcclWorldRankID;
        if (covers(&cfg->hcclJobID, 8)) r.jobId = cfg->hcclJobID;
        if (covers(&cfg->aclGraphZeroCopyEnable, 1)) r.graphZeroCopy = cfg->aclGraphZeroCopyEnable;
        if (covers(&cfg->hcclExecTimeOut, 4) && cfg->hcclExecTimeOut != HCCL_COMM_EXECTIMEOUT_CONFIG_NOT_SET) r.execTimeoutSec = cfg->hcclExecTimeOut;
        if (covers(cfg->hcclAlgo, HCCL_COMM_ALGO_MAX_LENGTH) && cfg->hcclAlgo[0]) r.algo = std::string(cfg->hcclAlgo, strnlen(cfg->hcclAlgo, HCCL_COMM_ALGO_MAX_LENGTH));
        if (covers(cfg->hcclRetryEnable, HCCL_COMM_RETRY_ENABLE_MAX_LENGTH) && cfg->hcclRetryEnable[0]) r.retryEnable = cfg->hcclRetryEnable;
        if (covers(cfg->hcclRetryParams, HCCL_COMM_RETRY_PARAMS_MAX_LENGTH) && cfg->hcclRetryParams[0]) r.retryParams = cfg->hcclRetryParams;
        if (covers(cfg->hcclBufferName, BUFFER_NAME_MAX_LENGTH) && cfg->hcclBufferName[0]) r.bufferName = cfg->hcclBufferName;
        if (covers(&cfg->hcclSymWinMaxMemSizePerRank, 8) && cfg->hcclSymWinMaxMemSizePerRank != 0) r.symStrideGB = cfg->hcclSymWinMaxMemSizePerRank;
    }
    if (r.execTimeoutSec < 0) { RPT_ERR("EI0003", "the execution timeout (%d s) must not be negative", r.execTimeoutSec); return HCCL_E_PARA; }
    if (!r.algo.empty()) {
        // a setting that does not parse is refused here, where the caller sees it, not ignored at the first operator
        AlgoConfig probe;
        std::string why;
        if (!probe.Parse(r.algo, &why)) {
            RPT_ERR("EI0003", "algorithm configuration \"%s\" (hcclAlgo / HCCL_ALGO): %s", r.algo.c_str(), why.c_str());
            return HCCL_E_PARA;
        }
    }
    *out = r;
    return HCCL_SUCCESS;
}

HcclResult RegistryAdd(Comm *c)
{
    std::lock_guard<std::mutex> lk(g_regMu);
    // Several ranks of one process (threads as ranks) share a name; key them by name#rank.
    std::string key = c->cfg.name + "#" + std::to_string(c->rank);
    if (g_registry.count(key)) {
        RPT_ERR("EI0003", "a communicator named \"%s\" already exists for rank %u in this process", c->cfg.name.c_str(), c->rank);
        return HCCL_E_PARA;
    }
    g_registry[key] = c;
    return HCCL_SUCCESS;
}

void RegistryRemove(Comm *c)
{
    std::lock_guard<std::mutex> lk(g_regMu);
    g_registry.erase(c->cfg.name + "#" + std::to_string(c->rank));
}

Comm *RegistryFind(const std::string &name)
{
    std::lock_guard<std::mutex> lk(g_regMu);
    for (auto &kv : g_registry)
        if (kv.second->cfg.name == name) return kv.second;
    return nullptr;
}

void RegistryForEach(const std::function<void(Comm *)> &fn)
{
    std::vector<Comm *> all;
    {
        std::lock_guard<std::mutex> lk(g_regMu);
        for (auto &kv : g_registry) all.push_back(kv.second);
    }
    for (Comm *c : all) fn(c);
}

static HcclResult SetupHeap(Comm *c)
{
    Platform *P = c->plat;
    const uint32_t n = c->nRanks, me = c->rank;
    const uint64_t gran = P->Granularity();
    c->halfBytes = (uint64_t)c->cfg.bufferMB << 20;
    c->p2pSlotBytes = 4ull << 20;
    c->p2pOffset = HC_CTRL_BYTES + 2 * c->halfBytes;
    c->llOffset = c->p2pOffset + (uint64_t)n * c->p2pSlotBytes;
    c->llBytes = 2ull * HC_KERNEL_MAX_RANKS * HC_LL_SLOT_BYTES;
    c->heapBytes = AlignUp(c->llOffset + c->llBytes, gran);
    c->p2pSent.assign(n, 0);
    c->p2pRecvd.assign(n, 0);
    c->heapStride = c->heapBytes;
    CHK_RET(P->PhysAlloc(c->heapBytes, &c->heapPhys));
    void *base = nullptr;
    CHK_RET(P->VaReserve(c->heapStride * n, &base));
    c->heapBase = (char *)base;
    c->peerPhys.assign(n, PhysMem());
    CHK_RET(P->Map(c->heapBase + (uint64_t)me * c->heapStride, c->heapPhys, c->heapBytes));
    CHK_RET(P->MemsetSync(c->LocalHeap(), 0, HC_CTRL_BYTES));
    CHK_RET(P->MemsetSync(c->LocalHeap() + c->llOffset, 0, c->llBytes));     // tags in this area only ever grow from zero

    // Hand my block to every peer, take theirs.  Tag = communicator group id and a fixed purpose code.
    const uint64_t tag = ((uint64_t)c->group.id << 32) | 0x48454150u;  // "HEAP"
    for (uint32_t i = 1; i < n; ++i) {
        uint32_t q = (me + i) % n;
        int fd = -1;
        CHK_RET(P->PhysExportFd(c->heapPhys, &fd));
        HcclResult r = c->boot->SendFd(c->worldRanks[q], tag, fd);
        ::close(fd);
        CHK_RET(r);
    }
    for (uint32_t i = 1; i < n; ++i) {
        uint32_t q = (me + n - i) % n;
        int fd = -1;
        HcclResult r = c->boot->RecvFd(c->worldRanks[q], tag, &fd);
        if (r != HCCL_SUCCESS) {
            RPT_ERR("EI0006", "rank %u did not receive the memory handle of rank %u", me, q);
            return r;
        }
        r = P->PhysImportFd(fd, c->heapBytes, &c->peerPhys[q]);
        ::close(fd);
        CHK_RET(r);
        CHK_RET(P->Map(c->heapBase + (uint64_t)q * c->heapStride, c->peerPhys[q], c->heapBytes));
    }
    // Nobody may signal into a control region that its owner has not cleared yet.
    CHK_RET(c->boot->Barrier(c->group));
    return HCCL_SUCCESS;
}

static void SetupMulticast(Comm *c)
{
    Platform *P = c->plat;
    const uint32_t n = c->nRanks;
    bool want = P->kind() == PlatKind::CUDA && EnvConfig::Get().nvlsEnable.value != 0 && n > 1 && !c->emuSameDevice &&
                c->graph.SingleNvlinkDomain() && P->MulticastSupported();
    // Every step is followed by an agreement round so that all ranks keep or drop NVLS together.
    auto agree = [&](bool ok) {
        std::vector<Blob> all;
        Blob mine(1, ok ? 1 : 0);
        if (c->boot->AllGather(c->group, mine, &all) != HCCL_SUCCESS) return false;
        for (auto &b : all)
            if (b.empty() || !b[0]) return false;
        return true;
    };
    if (!agree(want)) return;
    const uint64_t tag = ((uint64_t)c->group.id << 32) | 0x4d434153u;  // "MCAS"
    bool ok = true;
    if (c->rank == 0) {
        ok = P->McCreate(c->heapBytes, (int)n, &c->mcPhys) == HCCL_SUCCESS;
        for (uint32_t q = 1; q < n && ok; ++q) {
            int fd = -1;
            ok = P->PhysExportFd(c->mcPhys, &fd) == HCCL_SUCCESS && c->boot->SendFd(c->worldRanks[q], tag, fd) == HCCL_SUCCESS;
            if (fd >= 0) ::close(fd);
        }
    }
    if (!agree(ok)) { if (c->mcPhys.bytes) P->PhysRelease(&c->mcPhys); return; }
    if (c->rank != 0) {
        int fd = -1;
        ok = c->boot->RecvFd(c->worldRanks[0], tag, &fd) == HCCL_SUCCESS && P->PhysImportFd(fd, c->heapBytes, &c->mcPhys) == HCCL_SUCCESS;
        if (fd >= 0) ::close(fd);
    }
    ok = ok && P->McAddDevice(c->mcPhys) == HCCL_SUCCESS;
    if (!agree(ok)) { if (c->mcPhys.bytes) P->PhysRelease(&c->mcPhys); return; }
    ok = P->McBind(c->mcPhys, 0, c->heapPhys, c->heapBytes) == HCCL_SUCCESS;
    c->mcBound = ok;
    void *va = nullptr;
    ok = ok && P->VaReserve(c->heapBytes, &va) == HCCL_SUCCESS && P->Map(va, c->mcPhys, c->heapBytes) == HCCL_SUCCESS;
    if (!agree(ok)) {
        HCCL_WARNING("NVLS multicast could not be set up on every rank; continuing without it");
        if (c->mcBound) { P->McUnbind(c->mcPhys, 0, c->heapBytes); c->mcBound = false; }
        if (c->mcPhys.bytes) P->PhysRelease(&c->mcPhys);
        return;
    }
    c->mcBase = (char *)va;
    HCCL_INFO("rank %u: NVLS multicast alias of the heap at %p", c->rank, va);
}

static HcclResult SetupDeviceState(Comm *c)
{
    Platform *P = c->plat;
    void *p = nullptr;
    // one block: [CommDev | launch counters | head/tail counters], see comm_dev.h
    CHK_RET(P->DevAlloc(HC_DEV_BLOCK_BYTES, &p));
    CHK_RET(P->MemsetSync(p, 0, HC_DEV_BLOCK_BYTES));
    c->devStruct = (CommDev *)p;
    c->devCounters = (uint32_t *)((char *)p + HC_DEV_COUNTERS_OFFSET);
    c->opCounters = (uint64_t *)((char *)p + HC_DEV_OPCOUNTERS_OFFSET);
    size_t irBytes = 2ull * HC_IR_MAX_CTAS * HC_IR_RANKS * HC_IR_NOTIFY * sizeof(uint64_t);
    CHK_RET(P->DevAlloc(irBytes, &p));
    c->devIrCounters = (uint64_t *)p;
    CHK_RET(P->MemsetSync(p, 0, irBytes));
    CHK_RET(P->HostAlloc(4096, &p));
    memset(p, 0, 4096);
    c->abortWord = (uint32_t *)p;
    c->waitStatus = (HcclDeviceWaitStatus *)((char *)p + 64);

    CommDev &d = c->hostDev;
    d.rank = (int32_t)c->rank;
    d.nRanks = (int32_t)c->nRanks;
    d.heapBase = c->heapBase;
    d.heapStride = c->heapStride;
    d.mcBase = c->mcBase;
    d.bufOffset = HC_CTRL_BYTES;
    d.halfBytes = c->halfBytes;
    d.epoch = c->devCounters;
    d.launches = c->devCounters + 1;
    d.blocksDone = c->devCounters + 2;
    d.irConsumed = c->devIrCounters + (size_t)HC_IR_MAX_CTAS * HC_IR_RANKS * HC_IR_NOTIFY;
    d.abortWord = c->abortWord;
    d.status = c->waitStatus;
    d.opCounters = c->opCounters;
    d.timeoutNs = (uint64_t)c->TimeoutMs() * 1000000ull;
    d.llOffset = c->llOffset;
    d.heapMB = (uint32_t)((c->heapBytes + (1u << 20) - 1) >> 20);
    static_assert(sizeof(CommDev) <= HC_DEV_COUNTERS_OFFSET, "CommDev outgrew its slot");
    CHK_RET(P->MemcpySync(c->devStruct, &d, sizeof(CommDev)));
    return HCCL_SUCCESS;
}

HcclResult CommCreate(const CommInitArgs &args, Comm **out)
{
    std::unique_ptr<Comm> c(new Comm());
    c->plat = args.plat;
    c->boot = args.boot;
    c->hub = args.hub;
    c->group = args.group;
    c->worldRanks = args.group.ranks;
    c->rank = args.group.myIndex;
    c->nRanks = (uint32_t)args.group.ranks.size();
    c->identifier = args.boot->identifier();
    if (c->nRanks > HC_MAX_RANKS) {
        RPT_ERR("EI0014", "communicators of more than %d ranks are not supported (asked for %u)", HC_MAX_RANKS, c->nRanks);
        return HCCL_E_NOT_SUPPORT;
    }
    c->device = args.device >= 0 ? args.device : c->plat->CurrentDevice();
    CHK_RET(ResolveConfig(args.config, args.defaultName, &c->cfg));

    // Rank table from the member records.
    c->table.version = "boot";
    for (uint32_t i = 0; i < c->nRanks; ++i) {
        RankTable one;
        if (i >= args.memberInfo.size() || one.Deserialize(args.memberInfo[i]) != HCCL_SUCCESS || one.ranks.size() != 1) {
            HCCL_ERROR("rank record of member %u is unreadable", i);
            return HCCL_E_INTERNAL;
        }
        RankEntry e = one.ranks[0];
        e.rankId = i;
        e.levels.clear();
        e.localId = -1;
        c->table.ranks.push_back(e);
    }
    std::string err;
    HcclResult r = c->table.Normalize(&err);
    if (r != HCCL_SUCCESS) {
        RPT_ERR("EI0014", "rank table built at rendezvous is inconsistent: %s", err.c_str());
        return r;
    }
    c->table.version = "2.0";
    CHK_RET(c->graph.Build(c->table, c->rank));
    for (uint32_t i = 0; i < c->nRanks; ++i) {
        if (c->table.ranks[i].platKind != (uint32_t)c->plat->kind()) {
            RPT_ERR("EI0014", "rank %u runs on another platform kind than rank %u", i, c->rank);
            return HCCL_E_PARA;
        }
        if (c->plat->kind() == PlatKind::CUDA && c->table.ranks[i].serverId != c->table.ranks[c->rank].serverId) {
            RPT_ERR("EI0014", "rank %u is on another host; this build connects GPUs of one NVLink domain", i);
            return HCCL_E_NOT_SUPPORT;
        }
        for (uint32_t j = 0; j < i; ++j) {
            const RankEntry &a = c->table.ranks[i], &b = c->table.ranks[j];
            if (c->plat->kind() == PlatKind::CUDA && a.serverId == b.serverId && a.deviceId == b.deviceId) c->emuSameDevice = true;
        }
    }
    if (c->emuSameDevice) {
        for (uint32_t i = 1; i < c->nRanks; ++i)
            if (c->table.ranks[i].pid != c->table.ranks[0].pid || c->table.ranks[i].deviceId != c->table.ranks[0].deviceId) {
                RPT_ERR("EI0014", "ranks may share a GPU only when all ranks are threads of one process on that one GPU");
                return HCCL_E_NOT_SUPPORT;
            }
    }
    c->chanWaited.assign((size_t)HC_MAX_RANKS * HC_CHAN_NOTIFY, 0);
    c->opRing.resize(256);

    if (c->plat->kind() == PlatKind::CUDA) { PreloadFastKernels(); PreloadPlatformKernels(); }
    CHK_RET(SetupHeap(c.get()));
    SetupMulticast(c.get());
    CHK_RET(SetupDeviceState(c.get()));
    CHK_RET(RegistryAdd(c.get()));
    CHK_RET(c->boot->Barrier(c->group));
    HCCL_RUN_INFO("communicator \"%s\" ready: rank %u/%u on %s device %d, CCL buffer 2x%u MB, NVLS %s, %s", c->cfg.name.c_str(), c->rank,
                  c->nRanks, c->plat->name(), c->device, c->cfg.bufferMB, c->mcBase ? "on" : "off", c->graph.Describe().c_str());
    RetrySetup(c.get());
    *out = c.release();
    return HCCL_SUCCESS;
}

Comm::~Comm()
{
    if (!plat) return;
    magic = 0;
    for (auto &t : threads) {
        if (t->ownsStream && t->stream) plat->StreamDestroy(t->stream);
        if (t->ownsNotify && t->notify) plat->HostFree(t->notify);
    }
    for (auto s : auxStreams) plat->StreamDestroy(s);
    for (auto &kv : engineCtxs) {
        if (kv.second.engine == COMM_ENGINE_AIV || kv.second.engine == COMM_ENGINE_CCU) plat->DevFree(kv.second.ptr);
        else free(kv.second.ptr);
    }
    for (auto &ch : channels)
        if (ch->devView) plat->DevFree(ch->devView);
    for (auto &w : windows) {
        if (w->kind == Window::VMM) {
            for (uint32_t r = 0; r < w->peerPtr.size(); ++r)
                if (r != rank && w->peerPtr[r]) plat->Unmap((char *)w->vaBase + (size_t)r * w->mapStride, w->mapStride);
            for (auto &ph : w->imported) plat->PhysRelease(&ph);
            if (w->vaBase) plat->VaFree(w->vaBase, w->vaBytes);
            if (w->mcVa) { plat->Unmap(w->mcVa, w->mcBytes); plat->VaFree(w->mcVa, w->mcBytes); }
            if (w->mcBound) plat->McUnbind(w->mcPhys, 0, w->mcBytes);
            if (w->mcPhys.bytes) plat->PhysRelease(&w->mcPhys);
        } else if (w->kind == Window::IPC) {
            for (void *b : w->ipcBases)
                if (b) plat->IpcClose(b);
        }
    }
    if (mcBase) { plat->Unmap(mcBase, heapBytes); plat->VaFree(mcBase, heapBytes); }
    if (mcBound) plat->McUnbind(mcPhys, 0, heapBytes);
    if (mcPhys.bytes) plat->PhysRelease(&mcPhys);
    if (heapBase) {
        for (uint32_t r = 0; r < nRanks; ++r) {
            if (r == rank || (r < peerPhys.size() && peerPhys[r].bytes)) plat->Unmap(heapBase + (uint64_t)r * heapStride, heapBytes);
        }
        for (auto &ph : peerPhys)
            if (ph.bytes) plat->PhysRelease(&ph);
        plat->VaFree(heapBase, heapStride * nRanks);
    }
    if (heapPhys.bytes) plat->PhysRelease(&heapPhys);
    if (fusedLocal) plat->DevFree(fusedLocal);
    if (fusedTemp) plat->DevFree(fusedTemp);
    if (irPrimRing) plat->DevFree(irPrimRing);
    if (devStruct) plat->DevFree(devStruct);
    if (devIrCounters) plat->DevFree(devIrCounters);
    if (abortWord) plat->HostFree(abortWord);
}

namespace {
// Communicators whose HcclCommDestroy has returned although other ranks had not arrived yet (see CommDestroy); keyed by
// rendezvous identifier and group.  They are freed by the rank of this process whose own barrier completes.
std::mutex g_parkedMu;
std::map<std::string, std::vector<Comm *>> g_parked;

std::string FamilyKey(const Comm *c) { return c->identifier + "/" + std::to_string(c->group.id); }

// Another rank of the same communicator lives in this process and has not entered its destroy yet.
bool HasLiveSibling(const Comm *c)
{
    const std::string key = FamilyKey(c);
    std::lock_guard<std::mutex> lk(g_regMu);
    for (auto &kv : g_registry)
        if (kv.second != c && FamilyKey(kv.second) == key) return true;
    return false;
}

void Release(Comm *c)
{
    std::shared_ptr<Bootstrap> boot = c->boot;
    std::shared_ptr<BootstrapHub> hub = c->hub;
    bool world = c->group.id == 0;
    delete c;
    if (world && boot) boot->Close();
    // the hub (if this process owns it) ends when every agent has said goodbye
}
}  // namespace

// Peers must stop touching a rank's heap before it disappears, so destruction meets the other ranks in a barrier.  When
// several ranks of the communicator are objects of one process and one thread destroys them one after the other
// (the usual way after HcclCommInitAll), the first call cannot wait for ranks whose destroy only that same thread will
// ever call.  Such a rank says that it has arrived, waits briefly, and if the others are not there yet its resources
// are parked; the rank of this process that sees the barrier complete frees them with its own.
void CommDestroy(Comm *c)
{
    if (!c) return;
    RetryTeardown(c);
    RegistryRemove(c);
    bool met = true;
    if (c->boot && c->state.load() != (int)CommState::DESTROYED) {
        uint64_t ticket = 0;
        if (c->boot->BarrierArrive(c->group, &ticket) == HCCL_SUCCESS) {
            const bool siblings = HasLiveSibling(c);
            HcclResult r = c->boot->BarrierWait(ticket, siblings ? 50 : 10000, siblings);
            met = !(siblings && r == HCCL_E_TIMEOUT);
        }
    }
    c->state.store((int)CommState::DESTROYED);
    const std::string key = FamilyKey(c);
    if (!met) {
        c->magic = 0x5a4f4d42;           // the handle is dead for the caller
        std::lock_guard<std::mutex> lk(g_parkedMu);
        g_parked[key].push_back(c);
        return;
    }
    std::vector<Comm *> parked;
    {
        std::lock_guard<std::mutex> lk(g_parkedMu);
        auto it = g_parked.find(key);
        if (it != g_parked.end()) { parked.swap(it->second); g_parked.erase(it); }
    }
    Platform *plat = c->plat;
    const int device = c->device;
    Release(c);
    for (Comm *z : parked) {
        if (plat) plat->SetDevice(z->device);
        Release(z);
    }
    if (plat && !parked.empty()) plat->SetDevice(device);
}

Window *FindWindow(Comm *c, const void *ptr, uint64_t bytes, uint64_t *offset)
{
    std::lock_guard<std::mutex> lk(c->resMu);
    for (auto &w : c->windows) {
        const char *b = (const char *)w->localAddr;
        if ((const char *)ptr >= b && (const char *)ptr + bytes <= b + w->size) {
            if (offset) *offset = (uint64_t)((const char *)ptr - b);
            return w.get();
        }
    }
    return nullptr;
}

void CommSetAsyncError(Comm *c, HcclResult err)
{
    int expected = 0;
    if (c->asyncError.compare_exchange_strong(expected, (int)err)) {
        HCCL_ERROR("communicator \"%s\" rank %u: asynchronous error %d", c->cfg.name.c_str(), c->rank, (int)err);
        if (c->boot) c->boot->NotifyError(err);
        DfxFireException(c, err);
    }
}

HcclResult CommPollDeviceStatus(Comm *c)
{
    if (c->abortWord && __atomic_load_n(c->abortWord, __ATOMIC_ACQUIRE) != 0) {
        const HcclDeviceWaitStatus &s = *c->waitStatus;
        RPT_ERR("EI0002", "rank %u gave up waiting for rank %u (kind %u slot %u block %u): expected %llu, saw %llu, operator #%llu", s.rank,
                s.peer, s.kind, s.slot, s.block, (unsigned long long)s.expected, (unsigned long long)s.seen, (unsigned long long)s.seq);
        // with operator retry on, the retry rounds own the failure: it becomes the communicator's error only if they give up
        if (!c->retry) CommSetAsyncError(c, HCCL_E_TIMEOUT);
        return HCCL_E_TIMEOUT;
    }
    return HCCL_SUCCESS;
}

}  // namespace hc
