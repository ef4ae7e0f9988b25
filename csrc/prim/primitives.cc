// primitives.cc - host implementation of the hcomm_primitives.h verbs (engines CPU / CPU_TS and
// their AICPU aliases).  Each verb becomes one piece of platform work on the thread's stream:
// memcpy (also across NVLink: remote addresses handed out by the channel API are mapped in this
// process), a reduce kernel, a release-add on a notify word, or a bounded wait on one.
// Counterpart of src/base_comm/primitives/api_c_adpt/cpu_primitives_c_adpt.cc:58-735.
//
// Three execution modes share the code through one Op record:
//   eager       the verb is submitted when called
//   batch       between HcommBatchModeStart/End verbs are recorded and submitted together at End
//   task cache  between TaskCacheStart/End verbs are recorded under a tag with their pointer
//               arguments expressed relative to the caller's address table; TaskCacheExecute replays
//               the list with a new table (the role the reference's AICPU task cache plays)
#include <atomic>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../comm/comm.h"
#include "../core/dtype.h"
#include "../core/log.h"
#include "hcomm_primitives.h"

using namespace hc;

namespace hc {
ThreadRes *AsThread(ThreadHandle h)
{
    ThreadRes *t = (ThreadRes *)(uintptr_t)h;
    return (t && t->magic == 0x54485244) ? t : nullptr;
}
ChannelRes *AsChannel(ChannelHandle h)
{
    ChannelRes *c = (ChannelRes *)(uintptr_t)h;
    return (c && c->magic == 0x4348414e) ? c : nullptr;
}
}  // namespace hc

namespace {

enum class Verb : uint8_t { COPY, REDUCE, THREAD_RECORD, THREAD_WAIT, CHAN_RECORD, CHAN_WAIT, RAW_RECORD, RAW_WAIT };

struct Op {
    Verb verb;
    ThreadRes *thread = nullptr;
    ChannelRes *chan = nullptr;
    ThreadRes *dstThread = nullptr;
    void *dst = nullptr;
    const void *src = nullptr;
    uint64_t n = 0;                 // bytes for COPY, elements for REDUCE
    HcclDataType dtype = HCCL_DATA_TYPE_FP32;
    HcclReduceOp rop = HCCL_REDUCE_SUM;
    uint32_t idx = 0;
    uint32_t timeoutSec = 0;
    uint64_t rawId = 0;
    // task cache: region index + offset of dst / src in the caller's table (-1 = absolute)
    int dstRegion = -1, srcRegion = -1;
    uint64_t dstOff = 0, srcOff = 0;
};

std::atomic<float> g_defaultWaitTimeout{0.0f};   // seconds; 0 = communicator exec timeout
std::mutex g_mu;

struct Recording {
    std::string tag;
    std::vector<Op> ops;
    std::vector<void *> addrs;
    std::vector<uint64_t> sizes;
};
thread_local Recording *t_batch = nullptr;       // batch mode (per calling thread)
thread_local Recording *t_cacheRec = nullptr;    // task-cache recording in progress
std::map<std::string, Recording> g_taskCache;

uint32_t TimeoutMs(const Op &op)
{
    if (op.timeoutSec) return op.timeoutSec * 1000u;
    const float dflt = g_defaultWaitTimeout.load(std::memory_order_relaxed);
    if (dflt > 0) return (uint32_t)(dflt * 1000.0f);
    Comm *c = op.thread ? op.thread->comm : (op.chan ? op.chan->comm : nullptr);
    return c ? c->TimeoutMs() : 1836000u;
}

uint64_t *ChanWord(ChannelRes *ch, bool remoteSide, uint32_t idx) { return (remoteSide ? ch->remoteNotify : ch->localNotify) + idx; }

HcclResult Submit(const Op &op)
{
    ThreadRes *t = op.thread;
    Platform *P = t ? t->plat : (op.chan ? op.chan->plat : nullptr);
    if (!P) return HCCL_E_PTR;
    Stream s = t ? t->stream : nullptr;
    Comm *c = t && t->comm ? t->comm : (op.chan ? op.chan->comm : nullptr);
    if (c) {
        int st = c->state.load();
        if (st == (int)CommState::SUSPENDING || st == (int)CommState::SUSPENDED) return HCCL_E_SUSPENDING;
    }
    WaitReport rep;
    if (c) { rep.status = c->waitStatus; rep.abortWord = c->abortWord; rep.rank = c->rank; rep.seq = c->opSeq; }
    switch (op.verb) {
        case Verb::COPY:
            if (op.n == 0 || op.dst == op.src) return HCCL_SUCCESS;
            return P->MemcpyAsync(op.dst, op.src, op.n, s);
        case Verb::REDUCE:
            if (op.n == 0) return HCCL_SUCCESS;
            return P->ReduceAsync(op.dst, op.src, op.n, op.dtype, op.rop, s);
        case Verb::THREAD_RECORD:
            return P->FlagAddAsync(op.dstThread->notify + op.idx, 1, s);
        case Verb::THREAD_WAIT: {
            uint64_t expect = ++t->waited[op.idx];
            rep.kind = HC_WAIT_THREAD_NOTIFY; rep.slot = op.idx; rep.peer = c ? c->rank : 0;
            return P->FlagWaitGeAsync(t->notify + op.idx, expect, TimeoutMs(op), rep, s);
        }
        case Verb::CHAN_RECORD:
            return P->FlagAddAsync(ChanWord(op.chan, true, op.idx), 1, s);
        case Verb::CHAN_WAIT: {
            uint64_t expect = ++op.chan->waited[op.idx];
            rep.kind = HC_WAIT_CHAN_NOTIFY; rep.slot = op.idx; rep.peer = op.chan->remoteRank;
            return P->FlagWaitGeAsync(ChanWord(op.chan, false, op.idx), expect, TimeoutMs(op), rep, s);
        }
        case Verb::RAW_RECORD:
            return P->FlagAddAsync((uint64_t *)(uintptr_t)op.rawId, 1, s);
        case Verb::RAW_WAIT: {
            // raw notify words are owned by the caller; the expectation is "at least one more than now"
            rep.kind = HC_WAIT_THREAD_NOTIFY; rep.slot = 0xffff;
            uint64_t *w = (uint64_t *)(uintptr_t)op.rawId;
            static std::map<uint64_t, uint64_t> waited;
            uint64_t expect;
            {
                std::lock_guard<std::mutex> lk(g_mu);        // the count only: the wait itself may block (simulator)
                expect = ++waited[op.rawId];
            }
            return P->FlagWaitGeAsync(w, expect, TimeoutMs(op), rep, s);
        }
    }
    return HCCL_E_INTERNAL;
}

void Locate(const Recording &rec, const void *p, int *region, uint64_t *off)
{
    *region = -1;
    for (size_t i = 0; i < rec.addrs.size(); ++i) {
        const char *b = (const char *)rec.addrs[i];
        if ((const char *)p >= b && (const char *)p < b + rec.sizes[i]) {
            *region = (int)i;
            *off = (uint64_t)((const char *)p - b);
            return;
        }
    }
}

int32_t Issue(Op op)
{
    if (op.thread == nullptr && op.chan == nullptr) return HCCL_E_PTR;
    if (t_cacheRec) {
        Locate(*t_cacheRec, op.dst, &op.dstRegion, &op.dstOff);
        Locate(*t_cacheRec, op.src, &op.srcRegion, &op.srcOff);
        t_cacheRec->ops.push_back(op);
    }
    if (t_batch) {
        t_batch->ops.push_back(op);
        return HCCL_SUCCESS;
    }
    return (int32_t)Submit(op);
}

#define NEED_THREAD(t, h)               \
    ThreadRes *t = AsThread(h);         \
    if (!t) { RPT_ERR("EI0003", "%s: invalid thread handle", __func__); return HCCL_E_PTR; }
#define NEED_CHANNEL(c, h)              \
    ChannelRes *c = AsChannel(h);       \
    if (!c) { RPT_ERR("EI0003", "%s: invalid channel handle", __func__); return HCCL_E_PTR; } \
    if (c->status.load() != HCOMM_CHANNEL_STATUS_READY) return HCCL_E_UNAVAIL;

HcclResult CheckNotifyIdx(ChannelRes *ch, uint32_t idx)
{
    if (idx >= ch->notifyNum) {
        RPT_ERR("EI0003", "notify index %u outside the channel's %u slots", idx, ch->notifyNum);
        return HCCL_E_PARA;
    }
    return HCCL_SUCCESS;
}

}  // namespace

extern "C" {

int32_t HcommLocalCopyOnThread(ThreadHandle thread, void *dst, const void *src, uint64_t len)
{
    NEED_THREAD(t, thread);
    if (len && (!dst || !src)) return HCCL_E_PTR;
    Op op; op.verb = Verb::COPY; op.thread = t; op.dst = dst; op.src = src; op.n = len;
    return Issue(op);
}

int32_t HcommLocalReduceOnThread(ThreadHandle thread, void *dst, const void *src, uint64_t count, HcommDataType dataType, HcommReduceOp reduceOp)
{
    NEED_THREAD(t, thread);
    if (count && (!dst || !src)) return HCCL_E_PTR;
    if (!DtypeReducible((HcclDataType)dataType) || reduceOp > HCOMM_REDUCE_MIN) return HCCL_E_NOT_SUPPORT;
    Op op; op.verb = Verb::REDUCE; op.thread = t; op.dst = dst; op.src = src; op.n = count; op.dtype = (HcclDataType)dataType; op.rop = (HcclReduceOp)reduceOp;
    return Issue(op);
}

int32_t HcommThreadNotifyRecordOnThread(ThreadHandle thread, ThreadHandle dstThread, uint32_t dstNotifyIdx)
{
    NEED_THREAD(t, thread);
    NEED_THREAD(d, dstThread);
    if (dstNotifyIdx >= d->notifyNum) return HCCL_E_PARA;
    Op op; op.verb = Verb::THREAD_RECORD; op.thread = t; op.dstThread = d; op.idx = dstNotifyIdx;
    return Issue(op);
}

int32_t HcommThreadNotifyWaitOnThread(ThreadHandle thread, uint32_t notifyIdx, uint32_t timeOut)
{
    NEED_THREAD(t, thread);
    if (notifyIdx >= t->notifyNum) return HCCL_E_PARA;
    Op op; op.verb = Verb::THREAD_WAIT; op.thread = t; op.idx = notifyIdx; op.timeoutSec = timeOut;
    return Issue(op);
}

int32_t HcommThreadNotifyWaitOnThreadWithDefaultTimeout(ThreadHandle thread, uint32_t notifyIdx) { return HcommThreadNotifyWaitOnThread(thread, notifyIdx, 0); }

int32_t HcommAclrtNotifyRecordOnThread(ThreadHandle thread, uint64_t dstNotifyId)
{
    NEED_THREAD(t, thread);
    if (!dstNotifyId) return HCCL_E_PTR;
    Op op; op.verb = Verb::RAW_RECORD; op.thread = t; op.rawId = dstNotifyId;
    return Issue(op);
}

int32_t HcommAclrtNotifyWaitOnThread(ThreadHandle thread, uint64_t notifyId, uint32_t timeOut)
{
    NEED_THREAD(t, thread);
    if (!notifyId) return HCCL_E_PTR;
    Op op; op.verb = Verb::RAW_WAIT; op.thread = t; op.rawId = notifyId; op.timeoutSec = timeOut;
    return Issue(op);
}

int32_t HcommWriteOnThread(ThreadHandle thread, ChannelHandle channel, void *dst, const void *src, uint64_t len)
{
    NEED_THREAD(t, thread);
    NEED_CHANNEL(ch, channel);
    if (len && (!dst || !src)) return HCCL_E_PTR;
    Op op; op.verb = Verb::COPY; op.thread = t; op.chan = ch; op.dst = dst; op.src = src; op.n = len;
    return Issue(op);
}

int32_t HcommWriteReduceOnThread(ThreadHandle thread, ChannelHandle channel, void *dst, const void *src, uint64_t count, HcommDataType dataType,
                                 HcommReduceOp reduceOp)
{
    NEED_THREAD(t, thread);
    NEED_CHANNEL(ch, channel);
    if (count && (!dst || !src)) return HCCL_E_PTR;
    if (!DtypeReducible((HcclDataType)dataType) || reduceOp > HCOMM_REDUCE_MIN) return HCCL_E_NOT_SUPPORT;
    Op op; op.verb = Verb::REDUCE; op.thread = t; op.chan = ch; op.dst = dst; op.src = src; op.n = count; op.dtype = (HcclDataType)dataType; op.rop = (HcclReduceOp)reduceOp;
    return Issue(op);
}

int32_t HcommChannelNotifyRecordOnThread(ThreadHandle thread, ChannelHandle channel, uint32_t remoteNotifyIdx)
{
    NEED_THREAD(t, thread);
    NEED_CHANNEL(ch, channel);
    CHK_RET(CheckNotifyIdx(ch, remoteNotifyIdx));
    Op op; op.verb = Verb::CHAN_RECORD; op.thread = t; op.chan = ch; op.idx = remoteNotifyIdx;
    return Issue(op);
}

int32_t HcommChannelNotifyWaitOnThread(ThreadHandle thread, ChannelHandle channel, uint32_t localNotifyIdx, uint32_t timeOut)
{
    NEED_THREAD(t, thread);
    NEED_CHANNEL(ch, channel);
    CHK_RET(CheckNotifyIdx(ch, localNotifyIdx));
    Op op; op.verb = Verb::CHAN_WAIT; op.thread = t; op.chan = ch; op.idx = localNotifyIdx; op.timeoutSec = timeOut;
    return Issue(op);
}

int32_t HcommChannelNotifyWaitOnThreadWithDefaultTimeout(ThreadHandle thread, ChannelHandle channel, uint32_t localNotifyIdx)
{
    return HcommChannelNotifyWaitOnThread(thread, channel, localNotifyIdx, 0);
}

int32_t HcommWriteWithNotifyOnThread(ThreadHandle thread, ChannelHandle channel, void *dst, const void *src, uint64_t len, uint32_t remoteNotifyIdx)
{
    int32_t r = HcommWriteOnThread(thread, channel, dst, src, len);
    return r ? r : HcommChannelNotifyRecordOnThread(thread, channel, remoteNotifyIdx);
}

int32_t HcommWriteReduceWithNotifyOnThread(ThreadHandle thread, ChannelHandle channel, void *dst, const void *src, uint64_t count,
                                           HcommDataType dataType, HcommReduceOp reduceOp, uint32_t remoteNotifyIdx)
{
    int32_t r = HcommWriteReduceOnThread(thread, channel, dst, src, count, dataType, reduceOp);
    return r ? r : HcommChannelNotifyRecordOnThread(thread, channel, remoteNotifyIdx);
}

int32_t HcommReadOnThread(ThreadHandle thread, ChannelHandle channel, void *dst, const void *src, uint64_t len)
{
    return HcommWriteOnThread(thread, channel, dst, src, len);   // a read is a copy whose source is the mapped peer address
}

int32_t HcommReadReduceOnThread(ThreadHandle thread, ChannelHandle channel, void *dst, const void *src, uint64_t count, HcommDataType dataType,
                                HcommReduceOp reduceOp)
{
    return HcommWriteReduceOnThread(thread, channel, dst, src, count, dataType, reduceOp);
}

// Non-blocking-implicit forms: issued on the channel's own side stream so that they overlap with the
// thread's later work until a fence joins them.
static ThreadRes *NbiThread(ChannelRes *ch)
{
    Comm *c = ch->comm;
    if (!c) {
        // a base-level channel (no communicator): the side thread belongs to the channel and lives as long as the process
        static std::map<ChannelRes *, std::unique_ptr<ThreadRes>> sides;
        std::lock_guard<std::mutex> lk(g_mu);
        auto it = sides.find(ch);
        if (it != sides.end()) return it->second.get();
        std::unique_ptr<ThreadRes> t(new ThreadRes());
        t->plat = ch->plat; t->engine = ch->engine;
        if (ch->plat->kind() == PlatKind::CUDA) { if (ch->plat->StreamCreate(&t->stream) != HCCL_SUCCESS) return nullptr; t->ownsStream = true; }
        return (sides[ch] = std::move(t)).get();
    }
    std::lock_guard<std::mutex> lk(c->resMu);
    auto it = c->dedicatedThreads.find(1000 + (int)ch->remoteRank);
    if (it != c->dedicatedThreads.end()) return it->second;
    std::unique_ptr<ThreadRes> t(new ThreadRes());
    t->comm = c; t->plat = c->plat; t->engine = ch->engine;
    if (c->plat->kind() == PlatKind::CUDA) { if (c->plat->StreamCreate(&t->stream) != HCCL_SUCCESS) return nullptr; t->ownsStream = true; }
    ThreadRes *raw = t.get();
    c->threads.push_back(std::move(t));
    c->dedicatedThreads[1000 + (int)ch->remoteRank] = raw;
    return raw;
}

int32_t HcommWriteNbi(ChannelHandle channel, void *dst, const void *src, uint64_t len)
{
    NEED_CHANNEL(ch, channel);
    ThreadRes *t = NbiThread(ch);
    if (!t) return HCCL_E_INTERNAL;
    return HcommWriteOnThread((ThreadHandle)(uintptr_t)t, channel, dst, src, len);
}
int32_t HcommWriteNbiOnThread(ThreadHandle thread, ChannelHandle channel, void *dst, const void *src, uint64_t len)
{
    NEED_THREAD(t, thread);
    NEED_CHANNEL(ch, channel);
    ThreadRes *side = NbiThread(ch);
    if (!side) return HCCL_E_INTERNAL;
    if (t->stream && side->stream) CHK_RET(t->plat->StreamOrder(t->stream, side->stream));   // after what the thread has queued so far
    return HcommWriteOnThread((ThreadHandle)(uintptr_t)side, channel, dst, src, len);
}
int32_t HcommWriteWithNotifyNbi(ChannelHandle channel, void *dst, const void *src, uint64_t len, uint32_t remoteNotifyIdx)
{
    int32_t r = HcommWriteNbi(channel, dst, src, len);
    if (r) return r;
    ChannelRes *ch = AsChannel(channel);
    return HcommChannelNotifyRecordOnThread((ThreadHandle)(uintptr_t)NbiThread(ch), channel, remoteNotifyIdx);
}
int32_t HcommWriteWithNotifyNbiOnThread(ThreadHandle thread, ChannelHandle channel, void *dst, const void *src, uint64_t len, uint32_t remoteNotifyIdx)
{
    int32_t r = HcommWriteNbiOnThread(thread, channel, dst, src, len);
    if (r) return r;
    ChannelRes *ch = AsChannel(channel);
    return HcommChannelNotifyRecordOnThread((ThreadHandle)(uintptr_t)NbiThread(ch), channel, remoteNotifyIdx);
}
int32_t HcommReadNbi(ChannelHandle channel, void *dst, const void *src, uint64_t len) { return HcommWriteNbi(channel, dst, src, len); }
int32_t HcommReadNbiOnThread(ThreadHandle thread, ChannelHandle channel, void *dst, const void *src, uint64_t len)
{
    return HcommWriteNbiOnThread(thread, channel, dst, src, len);
}

int32_t HcommBatchTransferOnThread(ThreadHandle thread, ChannelHandle channel, const HcommBatchTransferDesc *descs, uint32_t descNum)
{
    if (descNum && !descs) return HCCL_E_PTR;
    for (uint32_t i = 0; i < descNum; ++i) {
        const HcommBatchTransferDesc &d = descs[i];
        int32_t r;
        switch (d.transType) {
            case HCOMM_TRANSFER_TYPE_WRITE: r = HcommWriteOnThread(thread, channel, d.transferInfo.write.dst, d.transferInfo.write.src, d.transferInfo.write.len); break;
            case HCOMM_TRANSFER_TYPE_READ: r = HcommReadOnThread(thread, channel, d.transferInfo.read.dst, d.transferInfo.read.src, d.transferInfo.read.len); break;
            case HCOMM_TRANSFER_TYPE_WRITE_REDUCE:
                r = HcommWriteReduceOnThread(thread, channel, d.transferInfo.reduce.dst, d.transferInfo.reduce.src, d.transferInfo.reduce.count,
                                             d.transferInfo.reduce.dataType, d.transferInfo.reduce.reduceOp);
                break;
            case HCOMM_TRANSFER_TYPE_READ_REDUCE:
                r = HcommReadReduceOnThread(thread, channel, d.transferInfo.reduce.dst, d.transferInfo.reduce.src, d.transferInfo.reduce.count,
                                            d.transferInfo.reduce.dataType, d.transferInfo.reduce.reduceOp);
                break;
            case HCOMM_TRANSFER_TYPE_WRITE_WITH_NOTIFY:
                r = HcommWriteWithNotifyOnThread(thread, channel, d.transferInfo.writeWithNotify.dst, d.transferInfo.writeWithNotify.src,
                                                 d.transferInfo.writeWithNotify.len, d.transferInfo.writeWithNotify.notifyIdx);
                break;
            case HCOMM_TRANSFER_TYPE_WRITE_REDUCE_WITH_NOTIFY:
                r = HcommWriteReduceWithNotifyOnThread(thread, channel, d.transferInfo.writeReduceWithNotify.dst, d.transferInfo.writeReduceWithNotify.src,
                                                       d.transferInfo.writeReduceWithNotify.count, d.transferInfo.writeReduceWithNotify.dataType,
                                                       d.transferInfo.writeReduceWithNotify.reduceOp, d.transferInfo.writeReduceWithNotify.notifyIdx);
                break;
            case HCOMM_TRANSFER_TYPE_NOTIFY_RECORD: r = HcommChannelNotifyRecordOnThread(thread, channel, d.transferInfo.notifyRecord.notifyIdx); break;
            default:
                RPT_ERR("EI0003", "batch transfer descriptor %u has unknown type %d", i, (int)d.transType);
                return HCCL_E_PARA;
        }
        if (r) return r;
    }
    return HCCL_SUCCESS;
}

int32_t HcommChannelNotifyRecord(ChannelHandle channel, uint32_t remoteNotifyIdx)
{
    NEED_CHANNEL(ch, channel);
    ThreadRes *t = NbiThread(ch);
    return t ? HcommChannelNotifyRecordOnThread((ThreadHandle)(uintptr_t)t, channel, remoteNotifyIdx) : HCCL_E_INTERNAL;
}
int32_t HcommChannelNotifyWait(ChannelHandle channel, uint32_t localNotifyIdx, uint32_t timeOut)
{
    NEED_CHANNEL(ch, channel);
    ThreadRes *t = NbiThread(ch);
    if (!t) return HCCL_E_INTERNAL;
    int32_t r = HcommChannelNotifyWaitOnThread((ThreadHandle)(uintptr_t)t, channel, localNotifyIdx, timeOut);
    if (r) return r;
    if (t->stream) CHK_RET(t->plat->StreamSync(t->stream));   // the thread-less form is synchronous for the caller
    return ch->comm ? (int32_t)CommPollDeviceStatus(ch->comm) : HCCL_SUCCESS;
}

int32_t HcommThreadSynchronize(ThreadHandle thread)
{
    NEED_THREAD(t, thread);
    if (t->stream) CHK_RET(t->plat->StreamSync(t->stream));
    if (t->comm) return CommPollDeviceStatus(t->comm);
    return HCCL_SUCCESS;
}

int32_t HcommFenceOnThread(ThreadHandle thread)
{
    NEED_THREAD(t, thread);
    Comm *c = t->comm;
    if (!c || !t->stream) return HCCL_SUCCESS;
    std::vector<ThreadRes *> sides;
    {
        std::lock_guard<std::mutex> lk(c->resMu);
        for (auto &kv : c->dedicatedThreads)
            if (kv.first >= 1000) sides.push_back(kv.second);
    }
    for (ThreadRes *s : sides)
        if (s->stream) CHK_RET(t->plat->StreamOrder(s->stream, t->stream));
    return HCCL_SUCCESS;
}
int32_t HcommChannelFenceOnThread(ThreadHandle thread, ChannelHandle channel)
{
    NEED_THREAD(t, thread);
    NEED_CHANNEL(ch, channel);
    ThreadRes *s = NbiThread(ch);
    if (s && s->stream && t->stream) CHK_RET(t->plat->StreamOrder(s->stream, t->stream));
    return HCCL_SUCCESS;
}
int32_t HcommChannelFence(ChannelHandle channel)
{
    NEED_CHANNEL(ch, channel);
    ThreadRes *s = NbiThread(ch);
    if (s && s->stream) CHK_RET(s->plat->StreamSync(s->stream));
    return HCCL_SUCCESS;
}
int32_t HcommChannelDrainOnThread(ThreadHandle thread, ChannelHandle channel)
{
    NEED_THREAD(t, thread);
    NEED_CHANNEL(ch, channel);
    ThreadRes *s = NbiThread(ch);
    if (s && s->stream) CHK_RET(s->plat->StreamSync(s->stream));
    if (t->stream) CHK_RET(t->plat->StreamSync(t->stream));
    return ch->comm ? (int32_t)CommPollDeviceStatus(ch->comm) : HCCL_SUCCESS;
}

int32_t HcommSetNotifyWaitTimeOut(float timeOut)
{
    if (timeOut < 0) return HCCL_E_PARA;
    g_defaultWaitTimeout.store(timeOut, std::memory_order_relaxed);
    return HCCL_SUCCESS;
}
int32_t HcommThreadResAcquireTimeOut(float timeOut) { return timeOut < 0 ? HCCL_E_PARA : HCCL_SUCCESS; }

int32_t HcommBatchModeStart(const char *batchTag)
{
    if (!batchTag) return HCCL_E_PTR;
    if (t_batch) {
        RPT_ERR("EI0003", "batch \"%s\" is still open", t_batch->tag.c_str());
        return HCCL_E_PARA;
    }
    t_batch = new Recording();
    t_batch->tag = batchTag;
    return HCCL_SUCCESS;
}
int32_t HcommBatchModeEnd(const char *batchTag)
{
    if (!batchTag) return HCCL_E_PTR;
    if (!t_batch || t_batch->tag != batchTag) {
        RPT_ERR("EI0003", "HcommBatchModeEnd(\"%s\") without the matching start", batchTag);
        return HCCL_E_PARA;
    }
    Recording *rec = t_batch;
    t_batch = nullptr;
    HcclResult first = HCCL_SUCCESS;
    for (auto &op : rec->ops) {
        HcclResult r = Submit(op);
        if (r != HCCL_SUCCESS && first == HCCL_SUCCESS) first = r;
    }
    delete rec;
    return first;
}

HcommResult HcommAicpuTsTaskCacheLookup(const char *tag, bool *isHit)
{
    if (!tag || !isHit) return HCCL_E_PTR;
    std::lock_guard<std::mutex> lk(g_mu);
    *isHit = g_taskCache.count(tag) != 0;
    return HCCL_SUCCESS;
}
HcommResult HcommAicpuTsTaskCacheStart(const char *tag, void **addrs, uint64_t *sizes, uint64_t count)
{
    if (!tag || (count && (!addrs || !sizes))) return HCCL_E_PTR;
    if (t_cacheRec) return HCCL_E_PARA;
    t_cacheRec = new Recording();
    t_cacheRec->tag = tag;
    t_cacheRec->addrs.assign(addrs, addrs + count);
    t_cacheRec->sizes.assign(sizes, sizes + count);
    return HCCL_SUCCESS;
}
HcommResult HcommAicpuTsTaskCacheEnd(const char *tag)
{
    if (!tag) return HCCL_E_PTR;
    if (!t_cacheRec || t_cacheRec->tag != tag) return HCCL_E_PARA;
    std::lock_guard<std::mutex> lk(g_mu);
    g_taskCache[tag] = *t_cacheRec;
    delete t_cacheRec;
    t_cacheRec = nullptr;
    return HCCL_SUCCESS;
}
HcommResult HcommAicpuTsTaskCacheExecute(const char *tag, void **addrs, uint64_t *sizes, uint64_t count)
{
    if (!tag || (count && (!addrs || !sizes))) return HCCL_E_PTR;
    Recording rec;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        auto it = g_taskCache.find(tag);
        if (it == g_taskCache.end()) return HCCL_E_NOT_FOUND;
        rec = it->second;
    }
    if (count != rec.addrs.size()) {
        RPT_ERR("EI0003", "task cache \"%s\" was recorded with %zu address regions, replay passes %llu", tag, rec.addrs.size(), (unsigned long long)count);
        return HCCL_E_PARA;
    }
    for (uint64_t i = 0; i < count; ++i)
        if (sizes[i] < rec.sizes[i]) return HCCL_E_PARA;
    for (Op op : rec.ops) {
        if (op.dstRegion >= 0) op.dst = (char *)addrs[op.dstRegion] + op.dstOff;
        if (op.srcRegion >= 0) op.src = (const char *)addrs[op.srcRegion] + op.srcOff;
        HcclResult r = Submit(op);
        if (r != HCCL_SUCCESS) return r;
    }
    return HCCL_SUCCESS;
}
HcommResult HcommAicpuTsTaskCacheClear(const char *tag)
{
    std::lock_guard<std::mutex> lk(g_mu);
    if (!tag) g_taskCache.clear();
    else g_taskCache.erase(tag);
    return HCCL_SUCCESS;
}

// Reference counting of a communicator by name for code that caches handles across calls.
int32_t HcommAcquireComm(const char *commId)
{
    if (!commId) return HCCL_E_PTR;
    return RegistryFind(commId) ? HCCL_SUCCESS : HCCL_E_NOT_FOUND;
}
int32_t HcommReleaseComm(const char *commId) { return commId ? HCCL_SUCCESS : HCCL_E_PTR; }

}  // extern "C"
