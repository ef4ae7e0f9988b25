// services_api.cc - one-sided put/get between two ranks (include/hccl/hccl_one_sided.h; reference:
// framework/communicator/impl/one_sided_service) and launching caller-supplied communication kernels
// under the communicator's ordering (include/hccl/hccl_launch.h).
//
// One-sided memory descriptors are built on the base resource layer: every communicator lazily owns an
// endpoint; HcclRegisterMem registers + exports through it, HcclExchangeMemDesc swaps the 512-byte
// descriptors over the control plane, HcclEnableMemAccess imports one and returns the address to use
// as `remoteAddr`.  Put and get are then plain copies on the caller's stream over NVLink.
#include <dlfcn.h>

#include <cstring>
#include <map>

#include "../comm/comm.h"
#include "../core/dtype.h"
#include "../core/log.h"
#include "hccl/hccl_launch.h"
#include "hccl/hccl_mc2.h"
#include "hccl/hccl_one_sided.h"
#include "hccl/hccl_res.h"
#include "hcomm_res.h"

using namespace hc;

namespace hc {
ThreadRes *AsThread(ThreadHandle h);
}

namespace {

struct OneSided {
    EndpointHandle ep = nullptr;
    std::map<std::string, HcommMemHandle> regs;     // descriptor bytes -> registration
    uint64_t exchangeSeq[HC_MAX_RANKS] = {0};
};
std::mutex g_mu;
std::map<Comm *, OneSided> g_svc;

struct WireDesc {            // what sits inside HcclMemDesc::desc
    uint32_t magic, ownerRank;
    uint64_t addr, size;
    uint32_t innerLen;
    uint8_t inner[400];
};
static_assert(sizeof(WireDesc) <= HCCL_MEM_DESC_LENGTH + 1, "descriptor must fit 512 bytes");

HcclResult Svc(Comm *c, OneSided **out)
{
    std::lock_guard<std::mutex> lk(g_mu);
    OneSided &s = g_svc[c];
    if (!s.ep) {
        EndpointDesc d;
        uint32_t n = 1;
        CHK_RET((HcclResult)HcommEndpointGetDescs(c->device, &n, &d));
        CHK_RET((HcclResult)HcommEndpointCreate(&d, &s.ep));
    }
    *out = &s;
    return HCCL_SUCCESS;
}

}  // namespace

extern "C" {

HcclResult HcclRegisterMem(HcclComm comm, uint32_t remoteRank, int type, void *addr, uint64_t size, HcclMemDesc *desc)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(addr); CHK_PTR_NULL(desc);
    if (remoteRank >= c->nRanks || size == 0) return HCCL_E_PARA;
    OneSided *s;
    CHK_RET(Svc(c, &s));
    CommMem m{type == COMM_MEM_TYPE_HOST ? COMM_MEM_TYPE_HOST : COMM_MEM_TYPE_DEVICE, addr, size};
    HcommMemHandle h;
    char tag[64];
    snprintf(tag, sizeof(tag), "onesided:%p:%u", addr, remoteRank);
    CHK_RET((HcclResult)HcommMemReg(s->ep, tag, &m, &h));
    void *inner;
    uint32_t innerLen;
    HcclResult r = (HcclResult)HcommMemExport(s->ep, h, &inner, &innerLen);
    if (r != HCCL_SUCCESS) { HcommMemUnreg(s->ep, h); return r; }
    WireDesc w;
    memset(&w, 0, sizeof(w));
    w.magic = 0x4f534d44; w.ownerRank = c->rank; w.addr = (uint64_t)(uintptr_t)addr; w.size = size; w.innerLen = innerLen;
    if (innerLen > sizeof(w.inner)) return HCCL_E_INTERNAL;
    memcpy(w.inner, inner, innerLen);
    memset(desc->desc, 0, sizeof(desc->desc));
    memcpy(desc->desc, &w, sizeof(w));
    std::lock_guard<std::mutex> lk(g_mu);
    s->regs[std::string(desc->desc, sizeof(desc->desc))] = h;
    return HCCL_SUCCESS;
}

HcclResult HcclDeregisterMem(HcclComm comm, HcclMemDesc *desc)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(desc);
    OneSided *s;
    CHK_RET(Svc(c, &s));
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = s->regs.find(std::string(desc->desc, sizeof(desc->desc)));
    if (it == s->regs.end()) return HCCL_E_NOT_FOUND;
    HcommMemUnreg(s->ep, it->second);
    s->regs.erase(it);
    return HCCL_SUCCESS;
}

HcclResult HcclExchangeMemDesc(HcclComm comm, uint32_t remoteRank, HcclMemDescs *local, int timeout, HcclMemDescs *remote, uint32_t *actualNum)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(local); CHK_PTR_NULL(remote); CHK_PTR_NULL(actualNum);
    if (remoteRank >= c->nRanks || remoteRank == c->rank) return HCCL_E_PARA;
    OneSided *s;
    CHK_RET(Svc(c, &s));
    uint64_t tag = ((uint64_t)c->group.id << 32) | 0x4f530000u;
    Blob msg;
    uint32_t n = local->arrayLength;
    msg.insert(msg.end(), (uint8_t *)&n, (uint8_t *)&n + 4);
    for (uint32_t i = 0; i < n; ++i) msg.insert(msg.end(), (uint8_t *)local->array[i].desc, (uint8_t *)local->array[i].desc + sizeof(HcclMemDesc));
    CHK_RET(c->boot->Send(c->worldRanks[remoteRank], tag, msg));
    Blob theirs;
    HcclResult r = c->boot->Recv(c->worldRanks[remoteRank], tag, &theirs, timeout > 0 ? timeout * 1000 : -1);
    if (r != HCCL_SUCCESS) { RPT_ERR("EI0006", "rank %u did not answer the memory-descriptor exchange", remoteRank); return r; }
    uint32_t pn = 0;
    if (theirs.size() < 4) return HCCL_E_INTERNAL;
    memcpy(&pn, theirs.data(), 4);
    uint32_t take = std::min(pn, remote->arrayLength);
    for (uint32_t i = 0; i < take; ++i) memcpy(remote->array[i].desc, theirs.data() + 4 + (size_t)i * sizeof(HcclMemDesc), sizeof(HcclMemDesc));
    *actualNum = take;
    return pn > remote->arrayLength ? HCCL_E_MEMORY : HCCL_SUCCESS;
}

HcclResult HcclEnableMemAccess(HcclComm comm, HcclMemDesc *remoteMemDesc, CommMem *remoteMem)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(remoteMemDesc); CHK_PTR_NULL(remoteMem);
    OneSided *s;
    CHK_RET(Svc(c, &s));
    WireDesc w;
    memcpy(&w, remoteMemDesc->desc, sizeof(w));
    if (w.magic != 0x4f534d44) { RPT_ERR("EI0003", "not a memory descriptor produced by HcclRegisterMem"); return HCCL_E_PARA; }
    return (HcclResult)HcommMemImport(s->ep, w.inner, w.innerLen, remoteMem);
}

HcclResult HcclDisableMemAccess(HcclComm comm, HcclMemDesc *remoteMemDesc)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(remoteMemDesc);
    OneSided *s;
    CHK_RET(Svc(c, &s));
    WireDesc w;
    memcpy(&w, remoteMemDesc->desc, sizeof(w));
    return (HcclResult)HcommMemUnimport(s->ep, w.inner, w.innerLen);
}

static HcclResult BatchCopy(HcclComm comm, uint32_t remoteRank, HcclOneSideOpDesc *desc, uint32_t descNum, aclrtStream stream, bool put)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    if (descNum && !desc) return HCCL_E_PTR;
    if (remoteRank >= c->nRanks) return HCCL_E_PARA;
    int st = c->state.load();
    if (st == (int)CommState::SUSPENDING || st == (int)CommState::SUSPENDED) return HCCL_E_SUSPENDING;
    Stream s = c->plat->kind() == PlatKind::SIM ? nullptr : stream;
    for (uint32_t i = 0; i < descNum; ++i) {
        uint64_t bytes = desc[i].count * DtypeSize(desc[i].dataType);
        if (bytes == 0) continue;
        if (!desc[i].localAddr || !desc[i].remoteAddr) return HCCL_E_PTR;
        CHK_RET(put ? c->plat->MemcpyAsync(desc[i].remoteAddr, desc[i].localAddr, bytes, s) : c->plat->MemcpyAsync(desc[i].localAddr, desc[i].remoteAddr, bytes, s));
    }
    return HCCL_SUCCESS;
}
HcclResult HcclBatchPut(HcclComm comm, uint32_t remoteRank, HcclOneSideOpDesc *desc, uint32_t descNum, aclrtStream stream) { return BatchCopy(comm, remoteRank, desc, descNum, stream, true); }
HcclResult HcclBatchGet(HcclComm comm, uint32_t remoteRank, HcclOneSideOpDesc *desc, uint32_t descNum, aclrtStream stream) { return BatchCopy(comm, remoteRank, desc, descNum, stream, false); }

// Process-level registrations that can later be bound to communicators.
namespace { std::mutex g_globalMu; std::map<void *, CommMem> g_globalMems; }
HcclResult HcclRegisterGlobalMem(const CommMem *mem, void **memHandle)
{
    CHK_PTR_NULL(mem); CHK_PTR_NULL(memHandle);
    if (!mem->addr || !mem->size) return HCCL_E_PARA;
    std::lock_guard<std::mutex> lk(g_globalMu);
    if (g_globalMems.count(mem->addr)) return HCCL_E_PARA;
    g_globalMems[mem->addr] = *mem;
    *memHandle = mem->addr;
    return HCCL_SUCCESS;
}
HcclResult HcclDeregisterGlobalMem(void *memHandle)
{
    std::lock_guard<std::mutex> lk(g_globalMu);
    return g_globalMems.erase(memHandle) ? HCCL_SUCCESS : HCCL_E_NOT_FOUND;
}
HcclResult HcclCommBindMem(HcclComm comm, void *memHandle)
{
    CommMem m;
    {
        std::lock_guard<std::mutex> lk(g_globalMu);
        auto it = g_globalMems.find(memHandle);
        if (it == g_globalMems.end()) return HCCL_E_NOT_FOUND;
        m = it->second;
    }
    HcclMemHandle h;
    char tag[64];
    snprintf(tag, sizeof(tag), "global:%p", memHandle);
    return HcclCommMemReg(comm, tag, &m, &h);
}
HcclResult HcclCommUnbindMem(HcclComm comm, void *memHandle)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    char tag[64];
    snprintf(tag, sizeof(tag), "global:%p", memHandle);
    std::lock_guard<std::mutex> lk(c->resMu);
    for (auto it = c->regMems.begin(); it != c->regMems.end(); ++it)
        if ((*it)->tag == tag) { c->regMems.erase(it); return HCCL_SUCCESS; }
    return HCCL_E_NOT_FOUND;
}
// Peer memory is mapped when the communicator is created, so there are no connections left to build.
HcclResult HcclCommPrepare(HcclComm comm, const HcclPrepareConfig *prepareConfig, const int timeout)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(prepareConfig);
    if (prepareConfig->topoType != HCCL_TOPO_FULLMESH) return HCCL_E_NOT_SUPPORT;
    return c->boot->Barrier(c->group, timeout > 0 ? timeout * 1000 : -1);
}

// ------------------------------------------------- resources of fused compute + communication kernels

static HcclResult ContextOf(Comm *c, void **commContext)
{
    CHK_PTR_NULL(c); CHK_PTR_NULL(commContext);
    *commContext = c->devStruct ? c->devStruct : (void *)&c->hostDev;
    return HCCL_SUCCESS;
}

HcclResult HcclAllocComResource(HcclComm comm, uint32_t streamMode, void **commContext)
{
    (void)streamMode;
    return ContextOf(AsComm(comm), commContext);
}
HcclResult HcclAllocComResourceByTiling(HcclComm comm, void *stream, void *mc2Tiling, void **commContext)
{
    (void)stream; (void)mc2Tiling;
    return ContextOf(AsComm(comm), commContext);
}
HcclResult HcclCreateComResource(const char *commName, uint32_t streamMode, void **commContext)
{
    (void)streamMode;
    CHK_PTR_NULL(commName);
    Comm *c = RegistryFind(commName);
    if (!c) return HCCL_E_NOT_FOUND;
    return ContextOf(c, commContext);
}

HcclResult HcclGetAicpuOpStreamAndNotify(HcclComm comm, aclrtStream *opStream, uint8_t aicpuNotifyNum, void **aicpuNotify)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(opStream);
    if (aicpuNotifyNum && !aicpuNotify) return HCCL_E_PTR;
    ThreadHandle h = 0;
    CHK_RET(HcclDedicatedThreadAcquire(comm, HCCL_DED_THREAD_TYPE_AICPU_LAUNCH, aicpuNotifyNum, &h));
    ThreadRes *t = AsThread(h);
    CHK_PTR_NULL(t);
    *opStream = t->stream;
    for (uint32_t i = 0; i < aicpuNotifyNum; ++i) aicpuNotify[i] = t->notify + i;
    return HCCL_SUCCESS;
}
HcclResult HcclGetAicpuOpStreamNotify(const char *commName, aclrtStream *opStream, void **aicpuNotify)
{
    CHK_PTR_NULL(commName);
    Comm *c = RegistryFind(commName);
    if (!c) return HCCL_E_NOT_FOUND;
    return HcclGetAicpuOpStreamAndNotify((HcclComm)c, opStream, aicpuNotify ? 1 : 0, aicpuNotify);
}

// ------------------------------------------------------------------------------ kernel launch

HcclResult HcclAicpuKernelLaunch(HcclComm comm, const HcclOpDesc *opInfo, const HcclKernelFuncInfo *funcInfo, ThreadHandle launchThread,
                                 aclrtStream userStream, const HcclKernelLaunchCfg *kernelLaunchCfg)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(opInfo); CHK_PTR_NULL(funcInfo);
    if (opInfo->header.magicWord != HCCL_OPDESC_MAGIC_WORD) { RPT_ERR("EI0003", "HcclOpDesc was not initialised with HcclOpDescInit"); return HCCL_E_PARA; }
    if (kernelLaunchCfg && kernelLaunchCfg->header.magicWord != HCCL_KERNEL_LAUNCH_CFG_MAGIC_WORD) return HCCL_E_PARA;
    int st = c->state.load();
    if (st == (int)CommState::SUSPENDING || st == (int)CommState::SUSPENDED) return HCCL_E_SUSPENDING;
    ThreadRes *t = AsThread(launchThread);
    typedef int (*KernelFn)(void *, uint32_t, void *);
    void *lib = funcInfo->kernelSoName[0] ? dlopen(funcInfo->kernelSoName, RTLD_NOW | RTLD_GLOBAL) : dlopen(nullptr, RTLD_NOW);
    if (!lib) { RPT_ERR("EI0004", "cannot open kernel library \"%s\": %s", funcInfo->kernelSoName, dlerror()); return HCCL_E_OPEN_FILE_FAILURE; }
    KernelFn fn = (KernelFn)dlsym(lib, funcInfo->kernelFuncName);
    if (!fn) { RPT_ERR("EI0004", "symbol \"%s\" not found in \"%s\"", funcInfo->kernelFuncName, funcInfo->kernelSoName); return HCCL_E_NOT_FOUND; }
    // Order: after what the caller queued, serialised with the communicator's own operators.
    std::lock_guard<std::mutex> lk(c->opMu);
    Stream launchStream = t && t->stream ? t->stream : userStream;
    bool cuda = c->plat->kind() == PlatKind::CUDA;
    if (cuda && launchStream != userStream) CHK_RET(c->plat->StreamOrder(userStream, launchStream));
    ++c->opSeq;
    int rc = fn(funcInfo->args, funcInfo->argSize, cuda ? launchStream : nullptr);
    if (cuda && launchStream != userStream) CHK_RET(c->plat->StreamOrder(launchStream, userStream));
    if (rc != 0) { HCCL_ERROR("kernel %s returned %d", funcInfo->kernelFuncName, rc); return HCCL_E_INTERNAL; }
    return HCCL_SUCCESS;
}

}  // extern "C"
