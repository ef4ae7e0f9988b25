// base_res_api.cc - the communicator-free resource layer of include/hcomm_res.h and hcomm_channel.h:
// endpoints, registered / exported / imported memory and endpoint-to-endpoint channels.  It is what
// another communication library would build on (reference: src/base_comm/primitives/api_c_adpt/
// hcomm_endpoint_c_adpt.cc, hcomm_mem_c_adpt.cc, hcomm_channel_c_adpt.cc).
//
// Memory descriptors.  HcommMemExport produces 96 bytes {magic, platform kind, pid, fd, allocation size,
// offset, size, IPC token}.  The importer duplicates the exporter's file descriptor with
// pidfd_open/pidfd_getfd (same host, same user) - or dup() inside one process - and maps the block;
// memory that is not VMM-backed travels as a CUDA IPC token.
//
// Channels.  HcommChannelCreate connects to (role CLIENT) or accepts from (role SERVER) the remote
// endpoint on `port`, swaps {notify block descriptor, memory descriptors}, imports them and becomes
// READY; HcommChannelGetStatus reports the state machine INIT -> SOCKET_OK -> READY / SOCKET_TIMEOUT /
// FAILED.  The data-plane verbs of hcomm_primitives.h work on these channels unchanged.
#include <sys/syscall.h>
#include <unistd.h>

#include <cstring>
#include <map>
#include <mutex>

#include "../comm/comm.h"
#include "../core/env.h"
#include "../core/log.h"
#include "../topo/nvml_topo.h"
#include "hcomm_channel.h"
#include "hcomm_res.h"

using namespace hc;

namespace hc {
ChannelRes *AsChannel(ChannelHandle h);
}

namespace {

constexpr uint32_t kDescMagic = 0x484d454d;   // "HMEM"

struct MemDesc {
    uint32_t magic, platKind, pid;
    int32_t fd;
    uint64_t allocBytes, offset, size;
    uint32_t ipcLen;
    uint8_t ipc[72];
};

struct RegEntry {
    std::string tag;
    CommMem mem;
    MemDesc desc;
    bool exported = false;
    PhysMem phys;
};

struct Endpoint {
    uint32_t magic = 0x454e4450;   // "ENDP"
    EndpointDesc desc;
    Platform *plat;
    std::mutex mu;
    std::vector<std::unique_ptr<RegEntry>> mems;
    int listenFd = -1, listenPort = 0;
    struct Import { PhysMem phys; void *va; size_t bytes; void *ipcBase; };
    std::map<std::string, Import> imports;   // keyed by the raw descriptor bytes
};

Endpoint *AsEndpoint(EndpointHandle h)
{
    Endpoint *e = (Endpoint *)h;
    return (e && e->magic == 0x454e4450) ? e : nullptr;
}

int DupFromProcess(uint32_t pid, int fd)
{
    if (pid == (uint32_t)getpid()) return dup(fd);
#ifdef SYS_pidfd_open
    int pfd = (int)syscall(SYS_pidfd_open, (pid_t)pid, 0);
    if (pfd < 0) return -1;
    int got = (int)syscall(SYS_pidfd_getfd, pfd, fd, 0);
    close(pfd);
    return got;
#else
    return -1;
#endif
}

HcclResult ImportDesc(Endpoint *ep, const MemDesc &d, CommMem *out, Endpoint::Import *imp)
{
    Platform *P = ep->plat;
    imp->phys = PhysMem(); imp->va = nullptr; imp->bytes = 0; imp->ipcBase = nullptr;
    if (d.magic != kDescMagic || d.platKind != (uint32_t)P->kind()) {
        RPT_ERR("EI0003", "memory descriptor is malformed or comes from another platform kind");
        return HCCL_E_PARA;
    }
    if (d.ipcLen) {
        std::vector<uint8_t> tok(d.ipc, d.ipc + d.ipcLen);
        CHK_RET(P->IpcImport(tok, &imp->ipcBase));
        out->addr = (char *)imp->ipcBase + d.offset;
    } else {
        int fd = DupFromProcess(d.pid, d.fd);
        if (fd < 0) {
            RPT_ERR("EI0003", "cannot duplicate descriptor %d of process %u (same host and user are required)", d.fd, d.pid);
            return HCCL_E_SYSCALL;
        }
        HcclResult r = P->PhysImportFd(fd, d.allocBytes, &imp->phys);
        close(fd);
        CHK_RET(r);
        CHK_RET(P->VaReserve(d.allocBytes, &imp->va));
        CHK_RET(P->Map(imp->va, imp->phys, d.allocBytes));
        imp->bytes = d.allocBytes;
        out->addr = (char *)imp->va + d.offset;
    }
    out->type = COMM_MEM_TYPE_DEVICE;
    out->size = d.size;
    return HCCL_SUCCESS;
}

std::mutex g_chanMu;
std::vector<std::unique_ptr<ChannelRes>> g_baseChannels;
struct NotifyBlock { void *va; PhysMem phys; size_t bytes; int fd; };
std::map<ChannelRes *, NotifyBlock> g_notifyBlocks;

}  // namespace

extern "C" {

HcommResult HcommEndpointGetDescNum(int32_t deviceLogicId, uint32_t *descNum)
{
    if (!descNum) return HCCL_E_PTR;
    (void)deviceLogicId;
    *descNum = 1;   // one NVLink port group per GPU
    return HCCL_SUCCESS;
}

HcommResult HcommEndpointGetDescs(int32_t deviceLogicId, uint32_t *descNum, EndpointDesc *descs)
{
    if (!descNum || !descs) return HCCL_E_PTR;
    if (*descNum < 1) return HCCL_E_PARA;
    Platform *P = DefaultPlatform();
    if (!P) return HCCL_E_NOT_SUPPORT;
    EndpointDescInit(descs, 1);
    memset(descs->commAddr.raws, 0, sizeof(descs->commAddr.raws));
    memset(descs->loc.raws, 0, sizeof(descs->loc.raws));
    descs->protocol = P->kind() == PlatKind::CUDA ? COMM_PROTOCOL_NVLINK : COMM_PROTOCOL_SHM;
    descs->commAddr.type = COMM_ADDR_TYPE_IP_V4;
    inet_pton(AF_INET, net::PickLocalIp().c_str(), &descs->commAddr.addr);
    descs->loc.locType = ENDPOINT_LOC_TYPE_DEVICE;
    descs->loc.device.devPhyId = (uint32_t)deviceLogicId;
    *descNum = 1;
    return HCCL_SUCCESS;
}

HcommResult HcommEndpointCreate(const EndpointDesc *endpoint, EndpointHandle *handle)
{
    if (!endpoint || !handle) return HCCL_E_PTR;
    Platform *P = DefaultPlatform();
    if (!P) return HCCL_E_NOT_SUPPORT;
    if (endpoint->protocol != COMM_PROTOCOL_NVLINK && endpoint->protocol != COMM_PROTOCOL_SHM && endpoint->protocol != COMM_PROTOCOL_HCCS) {
        RPT_ERR("EI0003", "endpoint protocol %d has no implementation on one NVSwitch node", (int)endpoint->protocol);
        return HCCL_E_NOT_SUPPORT;
    }
    Endpoint *e = new Endpoint();
    e->desc = *endpoint;
    e->plat = P;
    *handle = e;
    return HCCL_SUCCESS;
}

HcommResult HcommEndpointDestroy(EndpointHandle handle)
{
    Endpoint *e = AsEndpoint(handle);
    if (!e) return HCCL_E_PTR;
    for (auto &kv : e->imports) {
        if (kv.second.ipcBase) e->plat->IpcClose(kv.second.ipcBase);
        if (kv.second.va) { e->plat->Unmap(kv.second.va, kv.second.bytes); e->plat->VaFree(kv.second.va, kv.second.bytes); e->plat->PhysRelease(&kv.second.phys); }
    }
    for (auto &m : e->mems) {
        if (m->exported && m->desc.fd >= 0) close(m->desc.fd);
        if (m->phys.bytes) e->plat->PhysRelease(&m->phys);
    }
    net::Close(e->listenFd);
    e->magic = 0;
    delete e;
    return HCCL_SUCCESS;
}

HcommResult HcommEndpointGetListenPort(EndpointHandle handle, uint32_t *port)
{
    Endpoint *e = AsEndpoint(handle);
    if (!e || !port) return HCCL_E_PTR;
    std::lock_guard<std::mutex> lk(e->mu);
    if (e->listenFd < 0) CHK_RET(net::TcpListen("0.0.0.0", 0, 0, &e->listenFd, &e->listenPort));
    *port = (uint32_t)e->listenPort;
    return HCCL_SUCCESS;
}

HcommResult HcommEndpointCheckFeature(HcommEndpointFeatureType feature, const EndpointDesc *desc, bool *value)
{
    if (!desc || !value) return HCCL_E_PTR;
    Platform *P = DefaultPlatform();
    switch (feature) {
        case HCOMM_ENDPOINT_FEATURE_NDA: *value = desc->protocol == COMM_PROTOCOL_NVLINK; return HCCL_SUCCESS;   // device-initiated transfers
        case HCOMM_ENDPOINT_FEATURE_MULTICAST: *value = P && P->kind() == PlatKind::CUDA && P->MulticastSupported(); return HCCL_SUCCESS;
        default: return HCCL_E_PARA;
    }
}

HcommResult HcommMemReg(EndpointHandle handle, const char *memTag, const CommMem *mem, HcommMemHandle *memHandle)
{
    Endpoint *e = AsEndpoint(handle);
    if (!e || !memTag || !mem || !memHandle) return HCCL_E_PTR;
    if (!mem->addr || !mem->size) return HCCL_E_PARA;
    std::lock_guard<std::mutex> lk(e->mu);
    std::unique_ptr<RegEntry> r(new RegEntry());
    r->tag = memTag;
    r->mem = *mem;
    *memHandle = r.get();
    e->mems.push_back(std::move(r));
    return HCCL_SUCCESS;
}

HcommResult HcommMemUnreg(EndpointHandle handle, HcommMemHandle memHandle)
{
    Endpoint *e = AsEndpoint(handle);
    if (!e || !memHandle) return HCCL_E_PTR;
    std::lock_guard<std::mutex> lk(e->mu);
    for (auto it = e->mems.begin(); it != e->mems.end(); ++it) {
        if (it->get() == memHandle) {
            if ((*it)->exported && (*it)->desc.fd >= 0) close((*it)->desc.fd);
            if ((*it)->phys.bytes) e->plat->PhysRelease(&(*it)->phys);
            e->mems.erase(it);
            return HCCL_SUCCESS;
        }
    }
    return HCCL_E_NOT_FOUND;
}

HcommResult HcommMemExport(EndpointHandle handle, HcommMemHandle memHandle, void **memDesc, uint32_t *memDescLen)
{
    Endpoint *e = AsEndpoint(handle);
    if (!e || !memHandle || !memDesc || !memDescLen) return HCCL_E_PTR;
    std::lock_guard<std::mutex> lk(e->mu);
    RegEntry *r = nullptr;
    for (auto &m : e->mems)
        if (m.get() == memHandle) r = m.get();
    if (!r) return HCCL_E_NOT_FOUND;
    if (!r->exported) {
        MemDesc &d = r->desc;
        memset(&d, 0, sizeof(d));
        d.magic = kDescMagic;
        d.platKind = (uint32_t)e->plat->kind();
        d.pid = (uint32_t)getpid();
        d.fd = -1;
        d.size = r->mem.size;
        void *base = nullptr;
        size_t allocBytes = 0;
        if (e->plat->RetainPhys(r->mem.addr, &r->phys, &base, &allocBytes) == HCCL_SUCCESS) {
            int fd = -1;
            CHK_RET(e->plat->PhysExportFd(r->phys, &fd));
            d.fd = fd;   // stays open in this process until unregistration so that importers can duplicate it
            d.allocBytes = allocBytes;
            d.offset = (uint64_t)((char *)r->mem.addr - (char *)base);
        } else {
            std::vector<uint8_t> tok;
            size_t off = 0;
            HcclResult rr = e->plat->IpcExport(r->mem.addr, &tok, &off);
            if (rr != HCCL_SUCCESS || tok.size() > sizeof(d.ipc)) {
                RPT_ERR("EI0003", "memory \"%s\" cannot be exported: allocate it with HcommMemAlloc or cudaMalloc", r->tag.c_str());
                return HCCL_E_NOT_SUPPORT;
            }
            d.ipcLen = (uint32_t)tok.size();
            memcpy(d.ipc, tok.data(), tok.size());
            d.offset = off;
        }
        r->exported = true;
    }
    *memDesc = &r->desc;
    *memDescLen = sizeof(MemDesc);
    return HCCL_SUCCESS;
}

HcommResult HcommMemImport(EndpointHandle handle, const void *memDesc, uint32_t descLen, CommMem *outMem)
{
    Endpoint *e = AsEndpoint(handle);
    if (!e || !memDesc || !outMem) return HCCL_E_PTR;
    if (descLen < sizeof(MemDesc)) return HCCL_E_PARA;
    MemDesc d;
    memcpy(&d, memDesc, sizeof(d));
    std::string key((const char *)memDesc, sizeof(MemDesc));
    std::lock_guard<std::mutex> lk(e->mu);
    if (e->imports.count(key)) { RPT_ERR("EI0003", "this memory descriptor is already imported on the endpoint"); return HCCL_E_PARA; }
    Endpoint::Import imp;
    CHK_RET(ImportDesc(e, d, outMem, &imp));
    e->imports[key] = imp;
    return HCCL_SUCCESS;
}

HcommResult HcommMemUnimport(EndpointHandle handle, const void *memDesc, uint32_t descLen)
{
    Endpoint *e = AsEndpoint(handle);
    if (!e || !memDesc) return HCCL_E_PTR;
    if (descLen < sizeof(MemDesc)) return HCCL_E_PARA;
    std::string key((const char *)memDesc, sizeof(MemDesc));
    std::lock_guard<std::mutex> lk(e->mu);
    auto it = e->imports.find(key);
    if (it == e->imports.end()) return HCCL_E_NOT_FOUND;
    if (it->second.ipcBase) e->plat->IpcClose(it->second.ipcBase);
    if (it->second.va) { e->plat->Unmap(it->second.va, it->second.bytes); e->plat->VaFree(it->second.va, it->second.bytes); e->plat->PhysRelease(&it->second.phys); }
    e->imports.erase(it);
    return HCCL_SUCCESS;
}

// ------------------------------------------------------------------------------ base channels

HcommResult HcommChannelConfigCreate(HcommChannelConfig *config)
{
    if (!config) return HCCL_E_PTR;
    *config = new uint32_t(0);
    return HCCL_SUCCESS;
}
HcommResult HcommChannelConfigDestroy(HcommChannelConfig config)
{
    if (!config) return HCCL_E_PTR;
    delete (uint32_t *)config;
    return HCCL_SUCCESS;
}
HcommResult HcommChannelConfigSetInt(HcommChannelConfig config, HcommChannelConfigType type, uint32_t value)
{
    if (!config) return HCCL_E_PTR;
    if (type != HCOMM_CHANNEL_CONFIG_TYPE_IS_SHARED_QUEUE) return HCCL_E_PARA;
    *(uint32_t *)config = value;
    return HCCL_SUCCESS;
}

static HcclResult CreateOne(Endpoint *ep, CommEngine engine, HcommChannelDesc &d, ChannelHandle *out)
{
    if (d.header.magicWord != HCOMM_CHANNEL_MAGIC_WORD) { RPT_ERR("EI0003", "HcommChannelDesc was not initialised with HcommChannelDescInit"); return HCCL_E_PARA; }
    if (d.notifyNum > HCOMM_CHANNEL_MAX_NOTIFY || d.memHandleNum > HCOMM_CHANNEL_MAX_MEM_HANDLES) return HCCL_E_PARA;
    if (d.role != HCOMM_SOCKET_ROLE_CLIENT && d.role != HCOMM_SOCKET_ROLE_SERVER) { RPT_ERR("EI0003", "channel role must be CLIENT or SERVER"); return HCCL_E_PARA; }
    Platform *P = ep->plat;
    std::unique_ptr<ChannelRes> ch(new ChannelRes());
    ch->engine = engine;
    ch->plat = P;
    ch->notifyNum = d.notifyNum;
    ch->waited.assign(d.notifyNum, 0);
    ch->protocol = ep->desc.protocol;
    ch->status.store(HCOMM_CHANNEL_STATUS_INIT);
    ChannelRes *raw = ch.get();
    *out = (ChannelHandle)(uintptr_t)raw;
    {
        std::lock_guard<std::mutex> lk(g_chanMu);
        g_baseChannels.push_back(std::move(ch));
    }
    // control connection
    int64_t deadline = net::NowMs() + (int64_t)EnvConfig::Get().connectTimeoutSec.value * 1000;
    int sock = -1;
    HcclResult r;
    if (d.socket) {
        sock = (int)(intptr_t)d.socket;
    } else if (d.role == HCOMM_SOCKET_ROLE_SERVER) {
        uint32_t port = 0;
        if (d.port) {
            std::lock_guard<std::mutex> lk(ep->mu);
            if (ep->listenFd < 0) { r = net::TcpListen("0.0.0.0", d.port, d.port, &ep->listenFd, &ep->listenPort); if (r != HCCL_SUCCESS) { raw->status.store(HCOMM_CHANNEL_STATUS_FAILED); return r; } }
        } else {
            HcommEndpointGetListenPort(ep, &port);
        }
        r = net::TcpAccept(ep->listenFd, deadline, &sock, nullptr);
        if (r != HCCL_SUCCESS) { raw->status.store(HCOMM_CHANNEL_STATUS_SOCKET_TIMEOUT); RPT_ERR("EI0006", "no peer connected to port %d within the connect timeout", ep->listenPort); return HCCL_E_TIMEOUT; }
    } else {
        char ip[INET_ADDRSTRLEN] = "127.0.0.1";
        if (d.remoteEndpoint.commAddr.type == COMM_ADDR_TYPE_IP_V4) inet_ntop(AF_INET, &d.remoteEndpoint.commAddr.addr, ip, sizeof(ip));
        r = net::TcpConnect(ip, d.port, deadline, &sock);
        if (r != HCCL_SUCCESS) { raw->status.store(HCOMM_CHANNEL_STATUS_SOCKET_TIMEOUT); RPT_ERR("EI0006", "cannot connect to %s:%u within the connect timeout", ip, d.port); return HCCL_E_TIMEOUT; }
    }
    raw->sock = sock;
    raw->status.store(HCOMM_CHANNEL_STATUS_SOCKET_OK);

    // my notify block: exportable memory holding notifyNum words
    NotifyBlock nb{};
    size_t gran = P->Granularity();
    nb.bytes = gran;
    r = P->PhysAlloc(nb.bytes, &nb.phys);
    if (r == HCCL_SUCCESS) r = P->VaReserve(nb.bytes, &nb.va);
    if (r == HCCL_SUCCESS) r = P->Map(nb.va, nb.phys, nb.bytes);
    if (r == HCCL_SUCCESS) r = P->MemsetSync(nb.va, 0, 4096);
    if (r == HCCL_SUCCESS) r = P->PhysExportFd(nb.phys, &nb.fd);
    if (r != HCCL_SUCCESS) { raw->status.store(HCOMM_CHANNEL_STATUS_RES_UNAVAIL); return HCCL_E_UNAVAIL; }
    raw->localNotify = (uint64_t *)nb.va;
    {
        std::lock_guard<std::mutex> lk(g_chanMu);
        g_notifyBlocks[raw] = nb;
    }
    // frame: name, notify count, notify block descriptor, memory descriptors with tags
    std::string name = d.channelName ? d.channelName : "";
    std::vector<uint8_t> msg;
    auto put = [&](const void *p, size_t n) { msg.insert(msg.end(), (const uint8_t *)p, (const uint8_t *)p + n); };
    uint32_t hdr[4] = {0x48434843, d.notifyNum, (uint32_t)name.size(), 0};
    MemDesc nd{};
    nd.magic = kDescMagic; nd.platKind = (uint32_t)P->kind(); nd.pid = (uint32_t)getpid(); nd.fd = nb.fd; nd.allocBytes = nb.bytes; nd.size = nb.bytes;
    std::vector<std::pair<MemDesc, std::string>> mine;
    {
        for (auto &m : ep->mems) {
            bool wanted = d.exchangeAllMems;
            for (uint32_t i = 0; i < d.memHandleNum && d.memHandles; ++i) wanted |= (d.memHandles[i] == m.get());
            if (!wanted) continue;
            void *p;
            uint32_t l;
            if (HcommMemExport(ep, m.get(), &p, &l) != HCCL_SUCCESS) continue;
            mine.push_back({m->desc, m->tag});
        }
    }
    hdr[3] = (uint32_t)mine.size();
    put(hdr, sizeof(hdr)); put(name.data(), name.size()); put(&nd, sizeof(nd));
    for (auto &kv : mine) { uint32_t tl = (uint32_t)kv.second.size(); put(&kv.first, sizeof(MemDesc)); put(&tl, 4); put(kv.second.data(), tl); }
    uint64_t len = msg.size();
    if (net::SendAll(sock, &len, 8) != HCCL_SUCCESS || net::SendAll(sock, msg.data(), msg.size()) != HCCL_SUCCESS) { raw->status.store(HCOMM_CHANNEL_STATUS_FAILED); return HCCL_E_TCP_TRANSFER; }
    uint64_t plen = 0;
    if (net::RecvAll(sock, &plen, 8, deadline) != HCCL_SUCCESS || plen > (64u << 20)) { raw->status.store(HCOMM_CHANNEL_STATUS_SOCKET_TIMEOUT); return HCCL_E_TIMEOUT; }
    std::vector<uint8_t> peer(plen);
    if (net::RecvAll(sock, peer.data(), plen, deadline) != HCCL_SUCCESS) { raw->status.store(HCOMM_CHANNEL_STATUS_FAILED); return HCCL_E_TCP_TRANSFER; }
    const uint8_t *p = peer.data();
    uint32_t ph[4];
    memcpy(ph, p, 16); p += 16;
    std::string pname((const char *)p, ph[2]); p += ph[2];
    if (ph[0] != hdr[0] || ph[1] != d.notifyNum || pname != name) {
        raw->status.store(HCOMM_CHANNEL_STATUS_FAILED);
        RPT_ERR("EI0006", "channel ends disagree: name \"%s\"/\"%s\", notifies %u/%u", name.c_str(), pname.c_str(), d.notifyNum, ph[1]);
        return HCCL_E_PARA;
    }
    MemDesc pnd;
    memcpy(&pnd, p, sizeof(pnd)); p += sizeof(pnd);
    CommMem nm;
    Endpoint::Import imp;
    r = ImportDesc(ep, pnd, &nm, &imp);
    if (r != HCCL_SUCCESS) { raw->status.store(HCOMM_CHANNEL_STATUS_FAILED); return r; }
    raw->remoteNotify = (uint64_t *)nm.addr;
    raw->importedBases.push_back(imp.va);
    {
        std::lock_guard<std::mutex> lk(ep->mu);
        ep->imports[std::string((const char *)&pnd, sizeof(pnd)) + "#notify" + std::to_string((uintptr_t)raw)] = imp;
    }
    for (uint32_t i = 0; i < ph[3]; ++i) {
        MemDesc md;
        uint32_t tl;
        memcpy(&md, p, sizeof(md)); p += sizeof(md);
        memcpy(&tl, p, 4); p += 4;
        std::string tag((const char *)p, tl); p += tl;
        CommMem cm;
        Endpoint::Import mi;
        if (ImportDesc(ep, md, &cm, &mi) != HCCL_SUCCESS) continue;
        std::lock_guard<std::mutex> lk(ep->mu);
        ep->imports[std::string((const char *)&md, sizeof(md)) + "#chan" + std::to_string((uintptr_t)raw)] = mi;
        raw->remoteMems.push_back(cm);
        raw->remoteTags.push_back(tag);
    }
    for (auto &s : raw->remoteTags) raw->tagPtrs.push_back(const_cast<char *>(s.c_str()));
    raw->status.store(HCOMM_CHANNEL_STATUS_READY);
    return HCCL_SUCCESS;
}

HcommResult HcommChannelCreate(EndpointHandle endpoint, CommEngine engine, HcommChannelDesc *descs, uint32_t channelNum, ChannelHandle *channels)
{
    Endpoint *ep = AsEndpoint(endpoint);
    if (!ep || !descs || !channels) return HCCL_E_PTR;
    if (engine == COMM_ENGINE_CPU && ep->plat->kind() == PlatKind::CUDA) return HCCL_E_NOT_SUPPORT;
    for (uint32_t i = 0; i < channelNum; ++i) {
        HcclResult r = CreateOne(ep, engine, descs[i], &channels[i]);
        if (r != HCCL_SUCCESS) return r;
    }
    return HCCL_SUCCESS;
}

HcommResult HcommChannelCreateWithConfig(EndpointHandle endpoint, CommEngine engine, HcommChannelDesc *descs, uint32_t channelNum,
                                         HcommChannelConfig config, ChannelHandle *channels)
{
    (void)config;
    return HcommChannelCreate(endpoint, engine, descs, channelNum, channels);
}

HcommResult HcommChannelGetStatus(const ChannelHandle *channels, uint32_t num, int32_t *statusList)
{
    if (!channels || !statusList) return HCCL_E_PTR;
    for (uint32_t i = 0; i < num; ++i) {
        ChannelRes *ch = AsChannel(channels[i]);
        if (!ch) return HCCL_E_PARA;
        statusList[i] = ch->status.load();
    }
    return HCCL_SUCCESS;
}

HcommResult HcommChannelDestroy(const ChannelHandle *channels, uint32_t num)
{
    if (!channels) return HCCL_E_PTR;
    std::lock_guard<std::mutex> lk(g_chanMu);
    for (uint32_t i = 0; i < num; ++i) {
        ChannelRes *ch = AsChannel(channels[i]);
        if (!ch) return HCCL_E_PARA;
        if (ch->comm) continue;   // communicator channels go through HcclChannelDestroy
        auto nb = g_notifyBlocks.find(ch);
        if (nb != g_notifyBlocks.end()) {
            ch->plat->Unmap(nb->second.va, nb->second.bytes);
            ch->plat->VaFree(nb->second.va, nb->second.bytes);
            ch->plat->PhysRelease(&nb->second.phys);
            if (nb->second.fd >= 0) close(nb->second.fd);
            g_notifyBlocks.erase(nb);
        }
        if (ch->sock >= 0) net::Close(ch->sock);
        for (auto it = g_baseChannels.begin(); it != g_baseChannels.end(); ++it)
            if (it->get() == ch) { ch->magic = 0; g_baseChannels.erase(it); break; }
    }
    return HCCL_SUCCESS;
}

}  // extern "C"
