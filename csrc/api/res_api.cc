// res_api.cc - per-communicator resources: CCL buffer, threads, channels, engine contexts, registered
// memory, symmetric windows (include/hccl/hccl_res.h, hccl_channel.h, hccl_sym_win.h and the
// base-level include/hcomm_res.h, hcomm_channel.h).
//
// Channel creation follows the shape of the reference pipeline (my_rank.cc:1181-1258): validate the
// descriptor (ABI header, limits), reuse an identical channel, otherwise allocate notify slots, swap a
// consistency frame {rank-table CRC, library version, notify count, engine} with the peer over the
// control plane (timeout -> HCCL_E_TIMEOUT + EI0006 with a dump of both ends), record the peer's
// registered memories and mark the channel READY.
#include <unistd.h>

#include <cstring>

#include "../comm/comm.h"
#include "../core/env.h"
#include "../core/log.h"
#include "hccl/hccl_channel.h"
#include "hccl/hccl_res.h"
#include "hccl/hccl_sym_win.h"
#include "hcomm_res.h"

using namespace hc;

namespace hc {
ThreadRes *AsThread(ThreadHandle h);
ChannelRes *AsChannel(ChannelHandle h);
}  // namespace hc

namespace {

constexpr uint32_t kLibVersion = 0x00010000;
constexpr uint32_t kMaxChannelsPerCall = 1u << 20;

bool EngineUsable(Comm *c, CommEngine e)
{
    switch (e) {
        case COMM_ENGINE_CPU: return c->plat->kind() == PlatKind::SIM;   // a host thread cannot dereference device memory
        case COMM_ENGINE_CPU_TS: case COMM_ENGINE_AICPU: case COMM_ENGINE_AICPU_TS: return true;
        case COMM_ENGINE_AIV: return c->plat->kind() == PlatKind::CUDA;
        case COMM_ENGINE_CCU: return c->mcBase != nullptr;
        default: return false;
    }
}

// The expansion mode of the communicator restricts which engines may be asked for (reference:
// coll_comm_res_c_adpt.cc:574-580).
bool EngineMatchesMode(Comm *c, CommEngine e)
{
    switch (c->cfg.opExpansionMode) {
        case 1: case 2: return e == COMM_ENGINE_CPU || e == COMM_ENGINE_CPU_TS || e == COMM_ENGINE_AICPU || e == COMM_ENGINE_AICPU_TS;
        case 4: return e == COMM_ENGINE_AIV;
        case 5: case 6: return e == COMM_ENGINE_CCU || e == COMM_ENGINE_AIV;
        default: return true;
    }
}

HcclResult NewThread(Comm *c, Platform *plat, CommEngine engine, uint32_t notifyNum, Stream wrap, ThreadRes **out)
{
    std::unique_ptr<ThreadRes> t(new ThreadRes());
    t->comm = c;
    t->plat = plat;
    t->engine = engine;
    t->notifyNum = notifyNum;
    t->waited.assign(notifyNum, 0);
    if (wrap) {
        t->stream = wrap;
    } else if (plat->kind() == PlatKind::CUDA || engine != COMM_ENGINE_CPU) {
        CHK_RET(plat->StreamCreate(&t->stream));
        t->ownsStream = true;
    }
    if (notifyNum) {
        void *p = nullptr;
        CHK_RET(plat->HostAlloc(notifyNum * sizeof(uint64_t), &p));
        memset(p, 0, notifyNum * sizeof(uint64_t));
        t->notify = (uint64_t *)p;
        t->ownsNotify = true;
    }
    *out = t.get();
    if (c) {
        std::lock_guard<std::mutex> lk(c->resMu);
        c->threads.push_back(std::move(t));
    } else {
        t.release();   // freed by HcommThreadFree
    }
    return HCCL_SUCCESS;
}

struct CheckFrame {
    uint32_t magic, libVersion, tableCrc, notifyNum, engine, rank, memCount, reserved;
};

std::mutex g_cfgMu;
struct ChannelCfg { uint32_t sharedQueue = 0; std::string tag; };

}  // namespace

extern "C" {

// ------------------------------------------------------------------------------------ buffers

HcclResult HcclGetHcclBuffer(HcclComm comm, void **buffer, uint64_t *size)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(buffer); CHK_PTR_NULL(size);
    *buffer = c->CclBuffer();
    *size = 2 * c->halfBytes;
    return HCCL_SUCCESS;
}

HcclResult HcclGetHcclBufferCleared(HcclComm comm, void **buffer, uint64_t *size)
{
    CHK_RET(HcclGetHcclBuffer(comm, buffer, size));
    Comm *c = AsComm(comm);
    return c->plat->MemsetSync(*buffer, 0, *size);
}

// ------------------------------------------------------------------------------------ threads

HcclResult HcclThreadAcquire(HcclComm comm, CommEngine engine, uint32_t threadNum, uint32_t notifyNumPerThread, ThreadHandle *threads)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(threads);
    if (threadNum == 0 || threadNum > 1024 || notifyNumPerThread > 1024) return HCCL_E_PARA;
    if (!EngineUsable(c, engine)) { RPT_ERR("EI0003", "engine %d is not available on platform %s", (int)engine, c->plat->name()); return HCCL_E_NOT_SUPPORT; }
    if (!EngineMatchesMode(c, engine)) { RPT_ERR("EI0003", "engine %d contradicts op expansion mode %u", (int)engine, c->cfg.opExpansionMode); return HCCL_E_PARA; }
    for (uint32_t i = 0; i < threadNum; ++i) {
        ThreadRes *t = nullptr;
        CHK_RET(NewThread(c, c->plat, engine, notifyNumPerThread, nullptr, &t));
        threads[i] = (ThreadHandle)(uintptr_t)t;
    }
    return HCCL_SUCCESS;
}

HcclResult HcclThreadAcquireWithConfig(HcclComm comm, CommEngine engine, uint32_t threadNum, ThreadType type, const ThreadConfig *config,
                                       ThreadHandle *threads)
{
    CHK_PTR_NULL(config);
    if (type != THREAD_TYPE_TS) return HCCL_E_NOT_SUPPORT;
    if (config->header.magicWord != HCOMM_THREAD_CONFIG_MAGIC_WORD) { RPT_ERR("EI0003", "ThreadConfig was not initialised with ThreadConfigInit"); return HCCL_E_PARA; }
    return HcclThreadAcquire(comm, engine, threadNum, config->notifyNumPerThread, threads);
}

HcclResult HcclThreadAcquireWithStream(HcclComm comm, CommEngine engine, aclrtStream stream, uint32_t notifyNum, ThreadHandle *thread)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(thread);
    if (!EngineUsable(c, engine)) return HCCL_E_NOT_SUPPORT;
    ThreadRes *t = nullptr;
    if (c->plat->kind() == PlatKind::SIM) stream = nullptr;
    CHK_RET(NewThread(c, c->plat, engine, notifyNum, stream, &t));
    if (!stream && t->ownsStream && c->plat->kind() == PlatKind::CUDA) {
        // wrapping the default stream: keep the handle null so work lands on stream 0
        c->plat->StreamDestroy(t->stream);
        t->stream = nullptr;
        t->ownsStream = false;
    }
    *thread = (ThreadHandle)(uintptr_t)t;
    return HCCL_SUCCESS;
}

HcclResult HcclDedicatedThreadAcquire(HcclComm comm, HcclDedicatedThreadType useType, uint32_t notifyNumPerThread, ThreadHandle *thread)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(thread);
    if (useType < HCCL_DED_THREAD_TYPE_AICPU_LAUNCH || useType > HCCL_DED_THREAD_TYPE_AICPU_ORDER_LAUNCH_DEVICE) return HCCL_E_PARA;
    {
        std::lock_guard<std::mutex> lk(c->resMu);
        auto it = c->dedicatedThreads.find((int)useType);
        if (it != c->dedicatedThreads.end()) {
            if (it->second->notifyNum < notifyNumPerThread) {
                RPT_ERR("EI0003", "dedicated thread %d exists with %u notifies, %u requested", (int)useType, it->second->notifyNum, notifyNumPerThread);
                return HCCL_E_PARA;
            }
            *thread = (ThreadHandle)(uintptr_t)it->second;
            return HCCL_SUCCESS;
        }
    }
    ThreadRes *t = nullptr;
    CHK_RET(NewThread(c, c->plat, COMM_ENGINE_CPU_TS, notifyNumPerThread, nullptr, &t));
    std::lock_guard<std::mutex> lk(c->resMu);
    c->dedicatedThreads[(int)useType] = t;
    *thread = (ThreadHandle)(uintptr_t)t;
    return HCCL_SUCCESS;
}

HcclResult HcclThreadResGetInfo(HcclComm comm, ThreadHandle thread, ThreadResType resType, uint32_t infoLen, void **info)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    return (HcclResult)HcommThreadResGetInfo(thread, resType, infoLen, info);
}

HcommResult HcommThreadResGetInfo(ThreadHandle thread, ThreadResType resType, uint32_t infoLen, void **info)
{
    ThreadRes *t = AsThread(thread);
    if (!t || !info) return HCCL_E_PTR;
    if (resType != THREAD_RES_TYPE_STREAM) return HCCL_E_NOT_SUPPORT;
    if (infoLen < sizeof(void *)) return HCCL_E_PARA;
    *info = t->stream;
    return HCCL_SUCCESS;
}

HcommResult HcommThreadAlloc(CommEngine engine, uint32_t threadNum, const uint32_t *notifyNumPerThread, ThreadHandle *threads)
{
    if (!threads || !notifyNumPerThread) return HCCL_E_PTR;
    Platform *plat = DefaultPlatform();
    if (!plat) return HCCL_E_NOT_SUPPORT;
    if (engine == COMM_ENGINE_CPU && plat->kind() == PlatKind::CUDA) return HCCL_E_NOT_SUPPORT;
    for (uint32_t i = 0; i < threadNum; ++i) {
        ThreadRes *t = nullptr;
        HcclResult r = NewThread(nullptr, plat, engine, notifyNumPerThread[i], nullptr, &t);
        if (r != HCCL_SUCCESS) return r;
        threads[i] = (ThreadHandle)(uintptr_t)t;
    }
    return HCCL_SUCCESS;
}

HcommResult HcommThreadFree(const ThreadHandle *threads, uint32_t threadNum)
{
    if (!threads) return HCCL_E_PTR;
    for (uint32_t i = 0; i < threadNum; ++i) {
        ThreadRes *t = AsThread(threads[i]);
        if (!t) return HCCL_E_PARA;
        if (t->comm) continue;   // owned by a communicator, released with it
        if (t->ownsStream && t->stream) { t->plat->StreamSync(t->stream); t->plat->StreamDestroy(t->stream); }
        if (t->ownsNotify && t->notify) t->plat->HostFree(t->notify);
        t->magic = 0;
        delete t;
    }
    return HCCL_SUCCESS;
}

// ----------------------------------------------------------------------------- engine contexts

HcclResult HcclEngineCtxCreate(HcclComm comm, const char *ctxTag, CommEngine engine, uint64_t size, void **ctx)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(ctxTag); CHK_PTR_NULL(ctx);
    if (strnlen(ctxTag, HCCL_RES_TAG_MAX_LEN + 1) > HCCL_RES_TAG_MAX_LEN || size == 0) return HCCL_E_PARA;
    std::string key = std::string(ctxTag) + "#" + std::to_string((int)engine);
    std::lock_guard<std::mutex> lk(c->resMu);
    if (c->engineCtxs.count(key)) { RPT_ERR("EI0003", "engine context \"%s\" already exists", ctxTag); return HCCL_E_PARA; }
    void *p = nullptr;
    bool onDevice = (engine == COMM_ENGINE_AIV || engine == COMM_ENGINE_CCU);
    if (onDevice) CHK_RET(c->plat->DevAlloc(size, &p));
    else { p = calloc(1, size); if (!p) return HCCL_E_OOM; }
    c->engineCtxs[key] = {p, size, engine};
    *ctx = p;
    return HCCL_SUCCESS;
}

HcclResult HcclEngineCtxGet(HcclComm comm, const char *ctxTag, CommEngine engine, void **ctx, uint64_t *size)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(ctxTag); CHK_PTR_NULL(ctx);
    std::lock_guard<std::mutex> lk(c->resMu);
    auto it = c->engineCtxs.find(std::string(ctxTag) + "#" + std::to_string((int)engine));
    if (it == c->engineCtxs.end()) return HCCL_E_NOT_FOUND;
    *ctx = it->second.ptr;
    if (size) *size = it->second.size;
    return HCCL_SUCCESS;
}

HcclResult HcclEngineCtxCopy(HcclComm comm, CommEngine engine, const char *ctxTag, const void *srcCtx, uint64_t size, uint64_t dstCtxOffset)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(ctxTag); CHK_PTR_NULL(srcCtx);
    void *dst = nullptr;
    uint64_t cap = 0;
    CHK_RET(HcclEngineCtxGet(comm, ctxTag, engine, &dst, &cap));
    if (dstCtxOffset + size > cap) { RPT_ERR("EI0003", "copy of %llu bytes at offset %llu overruns engine context \"%s\" (%llu bytes)", (unsigned long long)size, (unsigned long long)dstCtxOffset, ctxTag, (unsigned long long)cap); return HCCL_E_PARA; }
    return c->plat->MemcpySync((char *)dst + dstCtxOffset, srcCtx, size);
}

HcclResult HcclEngineCtxDestroy(HcclComm comm, const char *ctxTag, CommEngine engine)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(ctxTag);
    std::lock_guard<std::mutex> lk(c->resMu);
    auto it = c->engineCtxs.find(std::string(ctxTag) + "#" + std::to_string((int)engine));
    if (it == c->engineCtxs.end()) return HCCL_E_NOT_FOUND;
    if (it->second.engine == COMM_ENGINE_AIV || it->second.engine == COMM_ENGINE_CCU) c->plat->DevFree(it->second.ptr);
    else free(it->second.ptr);
    c->engineCtxs.erase(it);
    return HCCL_SUCCESS;
}

// --------------------------------------------------------------------------- registered memory

HcclResult HcclCommMemReg(HcclComm comm, const char *memTag, const CommMem *mem, HcclMemHandle *memHandle)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(memTag); CHK_PTR_NULL(mem); CHK_PTR_NULL(memHandle);
    if (!mem->addr || mem->size == 0 || strnlen(memTag, HCCL_RES_TAG_MAX_LEN + 1) > HCCL_RES_TAG_MAX_LEN) return HCCL_E_PARA;
    std::lock_guard<std::mutex> lk(c->resMu);
    for (auto &m : c->regMems)
        if (m->tag == memTag) { RPT_ERR("EI0003", "memory tag \"%s\" is already registered", memTag); return HCCL_E_PARA; }
    std::unique_ptr<RegMem> r(new RegMem());
    r->tag = memTag;
    r->mem = *mem;
    char *a = (char *)mem->addr;
    if (a >= c->LocalHeap() && a + mem->size <= c->LocalHeap() + c->heapBytes) {
        r->symmetric = true;
        r->heapOffset = (uint64_t)(a - c->LocalHeap());
    }
    *memHandle = r.get();
    c->regMems.push_back(std::move(r));
    return HCCL_SUCCESS;
}

HcclResult HcclCommMemUnreg(HcclComm comm, HcclMemHandle memHandle)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(memHandle);
    std::lock_guard<std::mutex> lk(c->resMu);
    for (auto it = c->regMems.begin(); it != c->regMems.end(); ++it)
        if (it->get() == memHandle) { c->regMems.erase(it); return HCCL_SUCCESS; }
    return HCCL_E_NOT_FOUND;
}

// ----------------------------------------------------------------------------------- channels

namespace {
struct PendingChannel {
    std::unique_ptr<ChannelRes> ch;     // null when an existing channel was reused
    CheckFrame mine;
    ChannelHandle reused = 0;
};
uint32_t &NotifyCursor(Comm *c, uint32_t peer)
{
    if (c->nextChanNotify.size() != c->nRanks) c->nextChanNotify.assign(c->nRanks, 8u);
    return c->nextChanNotify[peer];
}
}  // namespace

// First half of a channel acquisition: checks, slot allocation and the handshake frame on its way to the peer.
// All frames of one HcclChannelAcquire call are sent before any answer is awaited, so ranks that acquire channels
// to different peers in different orders (a ring: right neighbour first everywhere) cannot wait on each other in a cycle.
static HcclResult AcquireBegin(Comm *c, CommEngine engine, const HcclChannelDesc &d, PendingChannel *pend)
{
    if (d.header.magicWord != HCCL_CHANNEL_MAGIC_WORD || d.header.version == 0 || d.header.size < offsetof(HcclChannelDesc, memHandles)) {
        RPT_ERR("EI0003", "HcclChannelDesc was not initialised with HcclChannelDescInit (magic 0x%x version %u)", d.header.magicWord, d.header.version);
        return HCCL_E_PARA;
    }
    if (d.remoteRank >= c->nRanks || d.remoteRank == c->rank) { RPT_ERR("EI0003", "channel to rank %u is not possible from rank %u of %u", d.remoteRank, c->rank, c->nRanks); return HCCL_E_PARA; }
    if (d.notifyNum > HCOMM_CHANNEL_MAX_NOTIFY) { RPT_ERR("EI0003", "a channel holds at most %u notifies (asked %u)", HCOMM_CHANNEL_MAX_NOTIFY, d.notifyNum); return HCCL_E_PARA; }
    if (d.memHandleNum > HCOMM_CHANNEL_MAX_MEM_HANDLES) return HCCL_E_PARA;
    std::vector<GraphLink> links;
    c->graph.Links(0, c->rank, d.remoteRank, &links);
    CommProtocol proto = links.empty() ? COMM_PROTOCOL_RESERVED : links[0].protocol;
    if (d.channelProtocol != COMM_PROTOCOL_RESERVED && d.channelProtocol != proto) {
        RPT_ERR("EI0003", "protocol %d does not connect rank %u and rank %u (the rank graph offers %d)", (int)d.channelProtocol, c->rank, d.remoteRank, (int)proto);
        return HCCL_E_NOT_SUPPORT;
    }
    {   // reuse
        std::lock_guard<std::mutex> lk(c->resMu);
        for (auto &ch : c->channels)
            if (ch->engine == engine && ch->remoteRank == d.remoteRank && ch->notifyNum == d.notifyNum && ch->status.load() == HCOMM_CHANNEL_STATUS_READY) {
                pend->reused = (ChannelHandle)(uintptr_t)ch.get();
                return HCCL_SUCCESS;
            }
        if (NotifyCursor(c, d.remoteRank) + d.notifyNum > HC_CHAN_NOTIFY) {
            // out of notify slots: the caller may fall back to fewer notifies or release channels
            return HCCL_E_UNAVAIL;
        }
    }
    std::unique_ptr<ChannelRes> ch(new ChannelRes());
    ch->comm = c;
    ch->engine = engine;
    ch->remoteRank = d.remoteRank;
    ch->protocol = proto;
    ch->notifyNum = d.notifyNum;
    ch->waited.assign(d.notifyNum, 0);
    ch->plat = c->plat;
    {
        std::lock_guard<std::mutex> lk(c->resMu);
        ch->notifyBase = NotifyCursor(c, d.remoteRank);
        NotifyCursor(c, d.remoteRank) += d.notifyNum;
    }
    ch->remoteNotify = (uint64_t *)(c->PeerHeap(d.remoteRank) + HC_OFF_CHAN_NOTIFY) + (uint64_t)c->rank * HC_CHAN_NOTIFY + ch->notifyBase;
    ch->localNotify = (uint64_t *)(c->LocalHeap() + HC_OFF_CHAN_NOTIFY) + (uint64_t)d.remoteRank * HC_CHAN_NOTIFY + ch->notifyBase;
    // Handshake: both ends must ask for the same thing.  The frame also carries my registered memories.
    CheckFrame mine{0x43484b46, kLibVersion, c->table.Crc(), d.notifyNum, (uint32_t)engine, c->rank, 0, ch->notifyBase};
    Blob msg;
    std::vector<RegMem *> exported;
    {
        std::lock_guard<std::mutex> lk(c->resMu);
        for (auto &m : c->regMems) {
            bool wanted = d.memHandleNum == 0;
            for (uint32_t i = 0; i < d.memHandleNum && d.memHandles; ++i) wanted |= (d.memHandles[i] == m.get());
            if (wanted && m->symmetric) exported.push_back(m.get());
        }
    }
    mine.memCount = (uint32_t)exported.size();
    msg.insert(msg.end(), (uint8_t *)&mine, (uint8_t *)&mine + sizeof(mine));
    for (RegMem *m : exported) {
        uint64_t v[2] = {m->heapOffset, m->mem.size};
        msg.insert(msg.end(), (uint8_t *)v, (uint8_t *)v + 16);
        uint32_t tl = (uint32_t)m->tag.size();
        msg.insert(msg.end(), (uint8_t *)&tl, (uint8_t *)&tl + 4);
        msg.insert(msg.end(), m->tag.begin(), m->tag.end());
    }
    const uint64_t tag = ((uint64_t)c->group.id << 32) | 0x43480000u | ((uint32_t)engine << 8);
    ch->status.store(HCOMM_CHANNEL_STATUS_INIT);
    CHK_RET(c->boot->Send(c->worldRanks[d.remoteRank], tag, msg));
    ch->status.store(HCOMM_CHANNEL_STATUS_SOCKET_OK);
    pend->mine = mine;
    pend->ch = std::move(ch);
    return HCCL_SUCCESS;
}

// Second half: the peer's frame is awaited and compared, the peer's memories are recorded.
static HcclResult AcquireFinish(Comm *c, CommEngine engine, const HcclChannelDesc &d, PendingChannel *pend, ChannelHandle *out)
{
    if (pend->reused) { *out = pend->reused; return HCCL_SUCCESS; }
    std::unique_ptr<ChannelRes> ch = std::move(pend->ch);
    const CheckFrame mine = pend->mine;
    const CommProtocol proto = ch->protocol;
    const uint64_t tag = ((uint64_t)c->group.id << 32) | 0x43480000u | ((uint32_t)engine << 8);
    Blob theirs;
    HcclResult r = c->boot->Recv(c->worldRanks[d.remoteRank], tag, &theirs, EnvConfig::Get().connectTimeoutSec.value * 1000);
    if (r != HCCL_SUCCESS) {
        ch->status.store(r == HCCL_E_TIMEOUT ? HCOMM_CHANNEL_STATUS_SOCKET_TIMEOUT : HCOMM_CHANNEL_STATUS_FAILED);
        RPT_ERR("EI0006", "channel rank %u -> rank %u (engine %d, protocol %d, %u notifies): the peer did not answer the handshake within %d s; "
                          "local: device %d pid %d; remote: device %d host %s",
                c->rank, d.remoteRank, (int)engine, (int)proto, d.notifyNum, EnvConfig::Get().connectTimeoutSec.value, c->device, (int)getpid(),
                c->table.ranks[d.remoteRank].deviceId, c->table.ranks[d.remoteRank].serverId.c_str());
        std::lock_guard<std::mutex> lk(c->resMu);
        c->channels.push_back(std::move(ch));   // keep the record so its status can be queried
        return r == HCCL_E_TIMEOUT ? HCCL_E_TIMEOUT : r;
    }
    CheckFrame peer;
    if (theirs.size() < sizeof(peer)) return HCCL_E_INTERNAL;
    memcpy(&peer, theirs.data(), sizeof(peer));
    if (peer.magic != mine.magic || peer.libVersion != mine.libVersion || peer.tableCrc != mine.tableCrc || peer.notifyNum != mine.notifyNum ||
        peer.engine != mine.engine || peer.rank != d.remoteRank) {
        ch->status.store(HCOMM_CHANNEL_STATUS_FAILED);
        RPT_ERR("EI0006", "channel rank %u <-> rank %u: the two ends disagree (version %x/%x, rank table crc %08x/%08x, notifies %u/%u, engine %u/%u)",
                c->rank, d.remoteRank, mine.libVersion, peer.libVersion, mine.tableCrc, peer.tableCrc, mine.notifyNum, peer.notifyNum, mine.engine, peer.engine);
        return HCCL_E_PARA;
    }
    if (peer.reserved != ch->notifyBase) {
        // both ends number slots in acquisition order; differing bases mean the two ranks acquired channels in different orders
        ch->status.store(HCOMM_CHANNEL_STATUS_FAILED);
        RPT_ERR("EI0006", "channel rank %u <-> rank %u: notify slots differ (%u vs %u); acquire channels in the same order on both ranks", c->rank,
                d.remoteRank, ch->notifyBase, peer.reserved);
        return HCCL_E_PARA;
    }
    // peer memories: the CCL buffer first, then what the peer registered
    CommMem buf{COMM_MEM_TYPE_DEVICE, c->PeerHeap(d.remoteRank) + HC_CTRL_BYTES, 2 * c->halfBytes};
    ch->remoteMems.push_back(buf);
    ch->remoteTags.push_back("HcclBuffer");
    const uint8_t *p = theirs.data() + sizeof(peer), *e = theirs.data() + theirs.size();
    for (uint32_t i = 0; i < peer.memCount && p + 20 <= e; ++i) {
        uint64_t v[2];
        uint32_t tl;
        memcpy(v, p, 16); memcpy(&tl, p + 16, 4); p += 20;
        if (p + tl > e) break;
        CommMem m{COMM_MEM_TYPE_DEVICE, c->PeerHeap(d.remoteRank) + v[0], v[1]};
        ch->remoteMems.push_back(m);
        ch->remoteTags.emplace_back((const char *)p, tl);
        p += tl;
    }
    for (auto &s : ch->remoteTags) ch->tagPtrs.push_back(const_cast<char *>(s.c_str()));
    ch->status.store(HCOMM_CHANNEL_STATUS_READY);
    *out = (ChannelHandle)(uintptr_t)ch.get();
    std::lock_guard<std::mutex> lk(c->resMu);
    c->channels.push_back(std::move(ch));
    return HCCL_SUCCESS;
}

HcclResult HcclChannelAcquire(HcclComm comm, CommEngine engine, const HcclChannelDesc *descs, uint32_t channelNum, ChannelHandle *channels)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(descs); CHK_PTR_NULL(channels);
    if (channelNum == 0 || channelNum > kMaxChannelsPerCall) return HCCL_E_PARA;
    if (!EngineUsable(c, engine)) return HCCL_E_NOT_SUPPORT;
    if (!EngineMatchesMode(c, engine)) { RPT_ERR("EI0003", "engine %d contradicts op expansion mode %u", (int)engine, c->cfg.opExpansionMode); return HCCL_E_PARA; }
    size_t before;
    std::vector<uint32_t> notifyBefore;
    {
        std::lock_guard<std::mutex> lk(c->resMu);
        before = c->channels.size();
        NotifyCursor(c, 0);
        notifyBefore = c->nextChanNotify;
    }
    std::vector<PendingChannel> pending(channelNum);
    for (uint32_t i = 0; i < channelNum; ++i) {
        HcclResult r = AcquireBegin(c, engine, descs[i], &pending[i]);
        if (r == HCCL_E_UNAVAIL) {
            // Out of notify slots before anything of this request reached the peer beyond the frames of the earlier
            // descriptors: finish those (the peers answer them), then roll the whole call back so the caller can
            // retry with a smaller request.
            for (uint32_t j = 0; j < i; ++j) { ChannelHandle h = 0; AcquireFinish(c, engine, descs[j], &pending[j], &h); }
            std::lock_guard<std::mutex> lk(c->resMu);
            c->channels.resize(before);
            c->nextChanNotify = notifyBefore;
            for (uint32_t j = 0; j < channelNum; ++j) channels[j] = 0;
            return r;
        }
        if (r != HCCL_SUCCESS) return r;
    }
    for (uint32_t i = 0; i < channelNum; ++i) CHK_RET(AcquireFinish(c, engine, descs[i], &pending[i], &channels[i]));
    return HCCL_SUCCESS;
}

HcclResult HcclChannelConfigCreate(HcclChannelConfig *config)
{
    CHK_PTR_NULL(config);
    *config = new ChannelCfg();
    return HCCL_SUCCESS;
}
HcclResult HcclChannelConfigDestroy(HcclChannelConfig config)
{
    CHK_PTR_NULL(config);
    delete (ChannelCfg *)config;
    return HCCL_SUCCESS;
}
HcclResult HcclChannelConfigSetInt(HcclChannelConfig config, HcclChannelConfigType type, uint32_t value)
{
    CHK_PTR_NULL(config);
    if (type != HCCL_CHANNEL_CONFIG_TYPE_IS_SHARED_QUEUE) return HCCL_E_PARA;
    ((ChannelCfg *)config)->sharedQueue = value;
    return HCCL_SUCCESS;
}
HcclResult HcclChannelConfigSetStr(HcclChannelConfig config, HcclChannelConfigType type, const char *value)
{
    CHK_PTR_NULL(config); CHK_PTR_NULL(value);
    if (type != HCCL_CHANNEL_CONFIG_TYPE_SHARED_QUEUE_TAG || strlen(value) > HCCL_CHANNEL_CONFIG_SHARED_QUEUE_TAG_MAX_LEN) return HCCL_E_PARA;
    ((ChannelCfg *)config)->tag = value;
    return HCCL_SUCCESS;
}
// NVLink channels have no hardware queue to share; the configuration is accepted so that callers
// written for queue-based fabrics run unchanged.
HcclResult HcclChannelAcquireWithConfig(HcclComm comm, CommEngine engine, const HcclChannelDesc *descs, uint32_t channelNum, HcclChannelConfig config,
                                        ChannelHandle *channels)
{
    (void)config;
    return HcclChannelAcquire(comm, engine, descs, channelNum, channels);
}

HcclResult HcclChannelQuery(HcclComm comm, CommEngine engine, const HcclChannelDesc *descs, uint32_t channelNum, ChannelHandle *channels)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(descs); CHK_PTR_NULL(channels);
    std::lock_guard<std::mutex> lk(c->resMu);
    for (uint32_t i = 0; i < channelNum; ++i) {
        channels[i] = 0;
        for (auto &ch : c->channels)
            if (ch->engine == engine && ch->remoteRank == descs[i].remoteRank && ch->notifyNum == descs[i].notifyNum && ch->status.load() == HCOMM_CHANNEL_STATUS_READY)
                channels[i] = (ChannelHandle)(uintptr_t)ch.get();
    }
    return HCCL_SUCCESS;
}

HcclResult HcclChannelDestroy(HcclComm comm, const ChannelHandle *channels, uint32_t channelNum)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(channels);
    std::lock_guard<std::mutex> lk(c->resMu);
    for (uint32_t i = 0; i < channelNum; ++i) {
        bool found = false;
        for (auto it = c->channels.begin(); it != c->channels.end(); ++it) {
            if ((ChannelHandle)(uintptr_t)it->get() == channels[i]) {
                if ((*it)->devView) c->plat->DevFree((*it)->devView);
                (*it)->magic = 0;
                c->channels.erase(it);
                found = true;
                break;
            }
        }
        if (!found) return HCCL_E_NOT_FOUND;
    }
    return HCCL_SUCCESS;
}

HcclResult HcclChannelGetHcclBuffer(HcclComm comm, ChannelHandle channel, void **buffer, uint64_t *size)
{
    Comm *c = AsComm(comm);
    ChannelRes *ch = AsChannel(channel);
    CHK_PTR_NULL(c); CHK_PTR_NULL(ch); CHK_PTR_NULL(buffer); CHK_PTR_NULL(size);
    *buffer = c->PeerHeap(ch->remoteRank) + HC_CTRL_BYTES;
    *size = 2 * c->halfBytes;
    return HCCL_SUCCESS;
}

HcclResult HcclChannelGetRemoteMems(HcclComm comm, ChannelHandle channel, uint32_t *memNum, CommMem **remoteMems, char ***memTags)
{
    Comm *c = AsComm(comm);
    ChannelRes *ch = AsChannel(channel);
    CHK_PTR_NULL(c); CHK_PTR_NULL(ch); CHK_PTR_NULL(memNum); CHK_PTR_NULL(remoteMems);
    *memNum = (uint32_t)ch->remoteMems.size();
    *remoteMems = ch->remoteMems.data();
    if (memTags) *memTags = ch->tagPtrs.data();
    return HCCL_SUCCESS;
}

// Device-side view for kernels of the SM engine: {peer heap base, local/remote notify words, slot count}.
struct DeviceChannelView {
    char *peerHeap;
    uint64_t *remoteNotify;   // where my records land (in the peer's memory)
    uint64_t *localNotify;    // where the peer's records land (in my memory)
    uint32_t notifyNum;
    uint32_t remoteRank;
    uint64_t cclOffset, cclBytes;
};

HcclResult HcclChannelGetDeviceView(HcclComm comm, ChannelHandle channel, void **deviceChannel)
{
    Comm *c = AsComm(comm);
    ChannelRes *ch = AsChannel(channel);
    CHK_PTR_NULL(c); CHK_PTR_NULL(ch); CHK_PTR_NULL(deviceChannel);
    if (!ch->devView) {
        DeviceChannelView v;
        v.peerHeap = c->PeerHeap(ch->remoteRank);
        v.remoteNotify = (uint64_t *)(c->PeerHeap(ch->remoteRank) + HC_OFF_CHAN_NOTIFY) + (uint64_t)c->rank * HC_CHAN_NOTIFY + ch->notifyBase;
        v.localNotify = (uint64_t *)(c->LocalHeap() + HC_OFF_CHAN_NOTIFY) + (uint64_t)ch->remoteRank * HC_CHAN_NOTIFY + ch->notifyBase;
        v.notifyNum = ch->notifyNum;
        v.remoteRank = ch->remoteRank;
        v.cclOffset = HC_CTRL_BYTES;
        v.cclBytes = 2 * c->halfBytes;
        CHK_RET(c->plat->DevAlloc(sizeof(v), &ch->devView));
        CHK_RET(c->plat->MemcpySync(ch->devView, &v, sizeof(v)));
    }
    *deviceChannel = ch->devView;
    return HCCL_SUCCESS;
}

// ----------------------------------------------------------------------------------- windows
//
// Registration is collective.  Three cases, tried in this order:
//   1. the range lies inside the communicator's symmetric heap  -> peer addresses are computed;
//   2. the range is backed by a VMM allocation (HcommMemAlloc, or the caller's own cuMemCreate with
//      a POSIX-fd handle type) -> each rank exports the backing block and maps every peer's block
//      into one reserved range, stride = largest block;
//   3. otherwise (cudaMalloc memory) -> legacy CUDA IPC handles.
// All ranks must take the same case; the exchange checks it.

namespace {
// Gives a window backed by a virtual-memory allocation a multicast alias (multimem loads reduce the ranks' copies in the
// switch, multimem stores replicate to all of them), the way the communicator's own heap has one.  Needs the same
// allocation size and the same window offset on every rank; every step is agreed on by all ranks so that they keep
// or drop the alias together.  Failure leaves the window without alias: operators then use peer loads and stores.
void WindowSetupMulticast(Comm *c, Window *w, const PhysMem &phys, uint64_t allocBytes, bool sameLayout)
{
    Platform *P = c->plat;
    const uint32_t n = c->nRanks;
    auto agree = [&](bool ok) {
        std::vector<Blob> all;
        Blob mine(1, ok ? 1 : 0);
        if (c->boot->AllGather(c->group, mine, &all) != HCCL_SUCCESS) return false;
        for (auto &b : all)
            if (b.empty() || !b[0]) return false;
        return true;
    };
    const uint64_t gran = P->Granularity();
    bool want = c->mcBase != nullptr && sameLayout && allocBytes % gran == 0 && P->MulticastSupported();
    if (!agree(want)) return;
    const uint64_t tag = ((uint64_t)c->group.id << 32) | 0x4d000000u | (uint32_t)(c->windows.size() & 0xffffff);
    bool ok = true;
    if (c->rank == 0) {
        ok = P->McCreate(allocBytes, (int)n, &w->mcPhys) == HCCL_SUCCESS;
        for (uint32_t q = 1; q < n && ok; ++q) {
            int fd = -1;
            ok = P->PhysExportFd(w->mcPhys, &fd) == HCCL_SUCCESS && c->boot->SendFd(c->worldRanks[q], tag, fd) == HCCL_SUCCESS;
            if (fd >= 0) ::close(fd);
        }
    }
    if (!agree(ok)) { if (w->mcPhys.bytes) P->PhysRelease(&w->mcPhys); w->mcPhys = PhysMem(); return; }
    if (c->rank != 0) {
        int fd = -1;
        ok = c->boot->RecvFd(c->worldRanks[0], tag, &fd) == HCCL_SUCCESS && P->PhysImportFd(fd, allocBytes, &w->mcPhys) == HCCL_SUCCESS;
        if (fd >= 0) ::close(fd);
    }
    ok = ok && P->McAddDevice(w->mcPhys) == HCCL_SUCCESS;
    if (!agree(ok)) { if (w->mcPhys.bytes) P->PhysRelease(&w->mcPhys); w->mcPhys = PhysMem(); return; }
    ok = P->McBind(w->mcPhys, 0, phys, allocBytes) == HCCL_SUCCESS;
    w->mcBound = ok;
    void *va = nullptr;
    ok = ok && P->VaReserve(allocBytes, &va) == HCCL_SUCCESS && P->Map(va, w->mcPhys, allocBytes) == HCCL_SUCCESS;
    if (!agree(ok)) {
        if (w->mcBound) { P->McUnbind(w->mcPhys, 0, allocBytes); w->mcBound = false; }
        if (w->mcPhys.bytes) P->PhysRelease(&w->mcPhys);
        w->mcPhys = PhysMem();
        return;
    }
    w->mcVa = va;
    w->mcBytes = allocBytes;
    w->mcPtr = (char *)va + w->allocOffset;
}
}  // namespace

HcclResult HcclCommSymWinRegister(HcclComm comm, void *addr, uint64_t size, HcclCommSymWindow *winHandle, uint32_t flag)
{
    (void)flag;
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(addr); CHK_PTR_NULL(winHandle);
    if (size == 0) return HCCL_E_PARA;
    Platform *P = c->plat;
    std::unique_ptr<Window> w(new Window());
    w->comm = c;
    w->localAddr = addr;
    w->size = size;
    w->peerPtr.assign(c->nRanks, nullptr);
    const uint32_t n = c->nRanks, me = c->rank;

    struct Desc { uint32_t kind; uint32_t pad; uint64_t size, allocBytes, offset; };
    Desc mine{0, 0, size, 0, 0};
    PhysMem phys;
    void *allocBase = nullptr;
    size_t allocBytes = 0;
    std::vector<uint8_t> ipcToken;
    char *a = (char *)addr;
    if (a >= c->LocalHeap() && a + size <= c->LocalHeap() + c->heapBytes) {
        mine.kind = Window::HEAP;
        mine.offset = (uint64_t)(a - c->LocalHeap());
    } else if (P->RetainPhys(addr, &phys, &allocBase, &allocBytes) == HCCL_SUCCESS) {
        mine.kind = Window::VMM;
        mine.allocBytes = allocBytes;
        mine.offset = (uint64_t)(a - (char *)allocBase);
    } else {
        size_t off = 0;
        HcclResult r = P->IpcExport(addr, &ipcToken, &off);
        if (r != HCCL_SUCCESS) {
            RPT_ERR("EI0003", "memory at %p can be shared neither through the virtual-memory API nor through CUDA IPC", addr);
            return HCCL_E_NOT_SUPPORT;
        }
        mine.kind = Window::IPC;
        mine.offset = off;
    }
    Blob blob((uint8_t *)&mine, (uint8_t *)&mine + sizeof(mine));
    blob.insert(blob.end(), ipcToken.begin(), ipcToken.end());
    std::vector<Blob> all;
    HcclResult r = c->boot->AllGather(c->group, blob, &all);
    if (r != HCCL_SUCCESS) { if (phys.bytes) P->PhysRelease(&phys); return r; }
    std::vector<Desc> descs(n);
    uint64_t maxAlloc = 0;
    for (uint32_t q = 0; q < n; ++q) {
        memcpy(&descs[q], all[q].data(), sizeof(Desc));
        if (descs[q].kind != mine.kind || descs[q].size != size) {
            RPT_ERR("EI0003", "window registration differs between ranks: rank %u registers %llu bytes (kind %u), rank %u %llu bytes (kind %u)", me,
                    (unsigned long long)size, mine.kind, q, (unsigned long long)descs[q].size, descs[q].kind);
            if (phys.bytes) P->PhysRelease(&phys);
            return HCCL_E_PARA;
        }
        maxAlloc = std::max(maxAlloc, descs[q].allocBytes);
    }
    w->kind = (Window::Kind)mine.kind;
    w->allocOffset = mine.offset;
    w->peerPtr[me] = addr;
    if (w->kind == Window::HEAP) {
        for (uint32_t q = 0; q < n; ++q) w->peerPtr[q] = c->PeerHeap(q) + descs[q].offset;
        if (c->mcBase) w->mcPtr = c->mcBase + mine.offset;
    } else if (w->kind == Window::VMM) {
        const uint64_t tag = ((uint64_t)c->group.id << 32) | 0x57000000u | (uint32_t)(c->windows.size() & 0xffffff);
        uint64_t gran = P->Granularity();
        w->mapStride = (maxAlloc + gran - 1) / gran * gran;
        w->vaBytes = w->mapStride * n;
        CHK_RET(P->VaReserve(w->vaBytes, &w->vaBase));
        w->imported.assign(n, PhysMem());
        for (uint32_t i = 1; i < n; ++i) {
            uint32_t q = (me + i) % n;
            int fd = -1;
            CHK_RET(P->PhysExportFd(phys, &fd));
            r = c->boot->SendFd(c->worldRanks[q], tag, fd);
            ::close(fd);
            CHK_RET(r);
        }
        for (uint32_t i = 1; i < n; ++i) {
            uint32_t q = (me + n - i) % n;
            int fd = -1;
            CHK_RET(c->boot->RecvFd(c->worldRanks[q], tag, &fd));
            r = P->PhysImportFd(fd, descs[q].allocBytes, &w->imported[q]);
            ::close(fd);
            CHK_RET(r);
            char *va = (char *)w->vaBase + (size_t)q * w->mapStride;
            CHK_RET(P->Map(va, w->imported[q], descs[q].allocBytes));
            w->peerPtr[q] = va + descs[q].offset;
        }
        bool sameLayout = true;
        for (uint32_t q = 0; q < n; ++q) sameLayout = sameLayout && descs[q].allocBytes == mine.allocBytes && descs[q].offset == mine.offset;
        WindowSetupMulticast(c, w.get(), phys, mine.allocBytes, sameLayout);
        P->PhysRelease(&phys);
    } else {
        w->ipcBases.assign(n, nullptr);
        for (uint32_t q = 0; q < n; ++q) {
            if (q == me) continue;
            std::vector<uint8_t> tok(all[q].begin() + sizeof(Desc), all[q].end());
            void *base = nullptr;
            CHK_RET(P->IpcImport(tok, &base));
            w->ipcBases[q] = base;
            w->peerPtr[q] = (char *)base + descs[q].offset;
        }
    }
    CHK_RET(c->boot->Barrier(c->group));
    *winHandle = w.get();
    std::lock_guard<std::mutex> lk(c->resMu);
    c->windows.push_back(std::move(w));
    return HCCL_SUCCESS;
}

HcclResult HcclCommSymWinDeregister(HcclCommSymWindow winHandle)
{
    Window *w = (Window *)winHandle;
    if (!w || w->magic != 0x57494e44) return HCCL_E_PTR;
    Comm *c = w->comm;
    Platform *P = c->plat;
    c->boot->Barrier(c->group);   // nobody may still be using the peer views
    if (w->kind == Window::VMM) {
        for (uint32_t q = 0; q < c->nRanks; ++q)
            if (q != c->rank && w->imported[q].bytes) { P->Unmap((char *)w->vaBase + (size_t)q * w->mapStride, w->imported[q].bytes); P->PhysRelease(&w->imported[q]); }
        if (w->vaBase) P->VaFree(w->vaBase, w->vaBytes);
        if (w->mcVa) { P->Unmap(w->mcVa, w->mcBytes); P->VaFree(w->mcVa, w->mcBytes); }
        if (w->mcBound) P->McUnbind(w->mcPhys, 0, w->mcBytes);
        if (w->mcPhys.bytes) P->PhysRelease(&w->mcPhys);
        w->mcVa = nullptr; w->mcBound = false; w->mcPhys = PhysMem(); w->mcPtr = nullptr;
    } else if (w->kind == Window::IPC) {
        for (void *b : w->ipcBases)
            if (b) P->IpcClose(b);
    }
    w->kind = Window::HEAP;   // nothing left for the communicator's destructor to release
    std::lock_guard<std::mutex> lk(c->resMu);
    for (auto it = c->windows.begin(); it != c->windows.end(); ++it)
        if (it->get() == w) { w->magic = 0; c->windows.erase(it); break; }
    return HCCL_SUCCESS;
}

HcclResult HcclCommSymWinGet(HcclComm comm, void *ptr, size_t size, HcclCommSymWindow *winHandle, size_t *offset)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(ptr); CHK_PTR_NULL(winHandle); CHK_PTR_NULL(offset);
    std::lock_guard<std::mutex> lk(c->resMu);
    for (auto &w : c->windows) {
        char *b = (char *)w->localAddr;
        if ((char *)ptr >= b && (char *)ptr + size <= b + w->size) {
            *winHandle = w.get();
            *offset = (size_t)((char *)ptr - b);
            return HCCL_SUCCESS;
        }
    }
    return HCCL_E_NOT_FOUND;
}

HcclResult HcclSymWinGetPeerPointer(HcclCommSymWindow winHandle, size_t offset, uint32_t peerRank, void **ptr)
{
    Window *w = (Window *)winHandle;
    if (!w || w->magic != 0x57494e44) return HCCL_E_PTR;
    CHK_PTR_NULL(ptr);
    if (peerRank >= w->peerPtr.size() || offset >= w->size) return HCCL_E_PARA;
    *ptr = (char *)w->peerPtr[peerRank] + offset;
    return HCCL_SUCCESS;
}

HcclResult HcclSymWinGetMulticastPointer(HcclCommSymWindow winHandle, size_t offset, void **ptr)
{
    Window *w = (Window *)winHandle;
    if (!w || w->magic != 0x57494e44) return HCCL_E_PTR;
    CHK_PTR_NULL(ptr);
    if (offset >= w->size) return HCCL_E_PARA;
    *ptr = w->mcPtr ? (char *)w->mcPtr + offset : nullptr;
    return w->mcPtr ? HCCL_SUCCESS : HCCL_E_NOT_SUPPORT;
}

// ------------------------------------------------------------------------ zero-copy user ranges

HcclResult HcclCommSetMemoryRange(HcclComm comm, void *baseVirPtr, size_t size, size_t alignment, uint64_t flags)
{
    (void)alignment; (void)flags;
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(baseVirPtr);
    if (size == 0) return HCCL_E_PARA;
    CommMem m{COMM_MEM_TYPE_DEVICE, baseVirPtr, size};
    HcclMemHandle h;
    char tag[64];
    snprintf(tag, sizeof(tag), "range:%p", baseVirPtr);
    return HcclCommMemReg(comm, tag, &m, &h);
}
HcclResult HcclCommUnsetMemoryRange(HcclComm comm, void *baseVirPtr)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(baseVirPtr);
    char tag[64];
    snprintf(tag, sizeof(tag), "range:%p", baseVirPtr);
    std::lock_guard<std::mutex> lk(c->resMu);
    for (auto it = c->regMems.begin(); it != c->regMems.end(); ++it)
        if ((*it)->tag == tag) { c->regMems.erase(it); return HCCL_SUCCESS; }
    return HCCL_E_NOT_FOUND;
}
// Collective: the freshly backed sub-range becomes a symmetric window.
HcclResult HcclCommActivateCommMemory(HcclComm comm, void *virPtr, size_t size, size_t offset, uint64_t handle, uint64_t flags)
{
    (void)offset; (void)handle; (void)flags;
    HcclCommSymWindow w;
    return HcclCommSymWinRegister(comm, virPtr, size, &w, 0);
}
HcclResult HcclCommDeactivateCommMemory(HcclComm comm, void *virPtr)
{
    HcclCommSymWindow w;
    size_t off;
    HcclResult r = HcclCommSymWinGet(comm, virPtr, 1, &w, &off);
    if (r != HCCL_SUCCESS) return r;
    return HcclCommSymWinDeregister(w);
}

// ----------------------------------------------------------------- base-level memory allocator

namespace {
struct Alloc { PhysMem phys; void *va; size_t bytes; Platform *plat; };
std::mutex g_allocMu;
std::map<void *, Alloc> g_allocs;
}  // namespace

HcommResult HcommMemAlloc(void **ptr, size_t size)
{
    if (!ptr) return HCCL_E_PTR;
    if (size == 0) return HCCL_E_PARA;
    Platform *P = DefaultPlatform();
    if (!P) return HCCL_E_NOT_SUPPORT;
    size_t gran = P->Granularity(), bytes = (size + gran - 1) / gran * gran;
    Alloc a;
    a.plat = P;
    a.bytes = bytes;
    HcclResult r = P->PhysAlloc(bytes, &a.phys);
    if (r != HCCL_SUCCESS) return r;
    r = P->VaReserve(bytes, &a.va);
    if (r == HCCL_SUCCESS) r = P->Map(a.va, a.phys, bytes);
    if (r != HCCL_SUCCESS) { P->PhysRelease(&a.phys); return r; }
    *ptr = a.va;
    std::lock_guard<std::mutex> lk(g_allocMu);
    g_allocs[a.va] = a;
    return HCCL_SUCCESS;
}

HcommResult HcommMemFree(void *ptr)
{
    if (!ptr) return HCCL_E_PTR;
    Alloc a;
    {
        std::lock_guard<std::mutex> lk(g_allocMu);
        auto it = g_allocs.find(ptr);
        if (it == g_allocs.end()) return HCCL_E_NOT_FOUND;
        a = it->second;
        g_allocs.erase(it);
    }
    a.plat->Unmap(a.va, a.bytes);
    a.plat->VaFree(a.va, a.bytes);
    a.plat->PhysRelease(&a.phys);
    return HCCL_SUCCESS;
}

}  // extern "C"
