// ops.cc - operator front end.
//
// Flow of one operator (compare HcclAllReduceInner -> ExecOp in the reference,
// framework/op_base/src/op_base_host.cc:62-184, hccl_communicator_host.cc:4574-4810):
//   validate arguments -> (group mode: queue) -> lock communicator -> check state -> select
//   strategy + engine -> run on the engine (splitting into passes that fit the CCL buffer)
//   -> record the operator in the diagnostics ring.
#include "ops.h"

#include <time.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "../core/dtype.h"
#include "../core/env.h"
#include "../core/log.h"
#include "../core/nvtx_range.h"
#include "../device/coll_kernels.h"
#include "../device/emu_launch.h"
#include "exec.h"

namespace hc {

namespace {

uint64_t NowNs()
{
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}

std::mutex g_algoMu;
std::map<std::string, AlgoConfig> g_algoCfg;

struct GroupJob {
    std::function<HcclResult()> fn;
    uint64_t volume;
    bool p2p;
    bool variable;
    Comm *comm;
    OpDesc desc;
    size_t order;
};
thread_local int t_groupDepth = 0;
thread_local std::vector<GroupJob> t_groupJobs;

void Record(Comm *c, const OpDesc &d, const Selection &sel, uint64_t t0)
{
    std::lock_guard<std::mutex> lk(c->diagMu);
    HcclOpRecord &r = c->opRing[c->opRingNext % c->opRing.size()];
    memset(&r, 0, sizeof(r));
    r.seq = c->opSeq;
    r.cmdType = d.cmd; r.dataType = d.dtype; r.count = d.count; r.reduceOp = d.op; r.root = d.root;
    snprintf(r.algName, sizeof(r.algName), "%s", sel.name.c_str());
    r.hostStartNs = t0;
    r.hostEndNs = NowNs();
    ++c->opRingNext;
    if (c->profiling) DfxReportOp(c, r.algName, r.hostStartNs, r.hostEndNs);
}

// CTAs per rank.  Small transfers are latency bound (few CTAs keep the barrier cheap); large ones need many CTAs
// to keep enough 16-byte accesses in flight for NVLink: measured on B200, a 256 MB all-reduce runs at 275 GB/s bus
// bandwidth with 32 CTAs, 413 with 64 and 520 with 128.
int PickCtas(Comm *c, const Selection &sel, uint64_t bytesPerRank)
{
    const int cap = EnvConfig::Get().maxCtas.value, forced = EnvConfig::Get().forceCtas.value;
    int ctas;
    if (sel.ctas) ctas = (int)sel.ctas;
    else if (bytesPerRank >= (32ull << 20)) ctas = 144;
    else if (bytesPerRank >= (8ull << 20)) ctas = 96;
    else if (bytesPerRank >= (2ull << 20)) ctas = 48;
    else ctas = (int)std::min<uint64_t>(32, std::max<uint64_t>(1, (bytesPerRank + (16 << 10) - 1) / (16 << 10)));
    if (cap > 0) ctas = std::min(ctas, cap);
    const uint32_t own = __atomic_load_n(&c->ctaLimit, __ATOMIC_RELAXED);     // this communicator's share of the SMs
    if (own > 0) ctas = std::min(ctas, (int)own);
    if (forced > 0) ctas = forced;
    if (c->emuSameDevice) ctas = std::min(ctas, 4);
    return std::max(1, std::min(ctas, HC_MAX_CTAS));
}

void FillBase(Comm *c, const OpDesc &d, CollArgs &a)
{
    memset(&a, 0, sizeof(a));
    a.dev = c->devStruct;
    a.dtype = d.dtype;
    a.op = d.op;
    a.root = (int32_t)d.root;
    a.scale = d.scale;
    a.useScale = d.useScale ? 1 : 0;
    a.elemSize = DtypeSize(d.dtype);
    a.p2pOffset = c->p2pOffset;
    a.p2pSlotBytes = c->p2pSlotBytes;
}

HcclResult Launch(Comm *c, int kind, CollArgs &a, int ctas, Stream stream)
{
    FastLaunch l;
    memset(&l, 0, sizeof(l));
    l.kind = kind;
    a.preBarrier = (c->lastOpOnHost && kind != FK_SEND && kind != FK_RECV) ? 1 : 0;
    l.args = a;
    l.ctas = ctas;
    l.threads = 512;
    l.stream = stream;
    HcclResult r = LaunchForRank(c, l);
    if (r == HCCL_SUCCESS && kind != FK_SEND && kind != FK_RECV) c->lastOpOnHost = false;
    return r;
}

uint64_t AlignDownElems(uint64_t elems, uint32_t esz)
{
    uint64_t q = esz >= 16 ? 1 : 16 / esz;
    return elems / q * q;
}

// Small all-reduce / all-gather / all-to-all / reduce-scatter: one flag-in-data kernel without any barrier.
// Returns true (and the launch result in *res) when the operator was served here.
bool TrySmallLL(Comm *c, const OpDesc &d, const Selection &sel, HcclResult *res)
{
    const int32_t limit = EnvConfig::Get().llMaxBytes.value;
    if (limit <= 0 || c->nRanks < 2 || c->nRanks > HC_KERNEL_MAX_RANKS || c->lastOpOnHost) return false;
    if (sel.reason == "forced by configuration" || (sel.engine != Engine::SM_FAST && sel.engine != Engine::NVLS)) return false;
    if (!d.sendCounts.empty() || !d.recvCounts.empty()) return false;
    int mode;
    switch (d.cmd) {
        case HCCL_CMD_ALLREDUCE: mode = LL_ALLREDUCE; break;
        case HCCL_CMD_ALLGATHER: mode = LL_ALLGATHER; break;
        case HCCL_CMD_ALLTOALL: mode = LL_ALLTOALL; break;
        case HCCL_CMD_REDUCE_SCATTER: mode = LL_REDUCE_SCATTER; break;
        default: return false;
    }
    const uint32_t n = c->nRanks, esz = DtypeSize(d.dtype);
    const uint64_t blockBytes = d.count * esz;
    if (blockBytes == 0 || blockBytes > (uint64_t)limit || blockBytes > HC_LL_MAX_PAYLOAD) return false;
    if ((uint64_t)(n - 1) * blockBytes > (uint64_t)EnvConfig::Get().llMaxRecvBytes.value) return false;      // what one rank receives: beyond this the two-phase kernels win
    const bool reducing = mode == LL_ALLREDUCE || mode == LL_REDUCE_SCATTER;
    if (reducing && !DtypeReducible(d.dtype)) return false;
    const uint64_t inBytes = (mode == LL_ALLTOALL || mode == LL_REDUCE_SCATTER) ? blockBytes * n : blockBytes;
    const uint64_t outBytes = (mode == LL_ALLGATHER || mode == LL_ALLTOALL) ? blockBytes * n : blockBytes;
    const uintptr_t in = (uintptr_t)d.in, out = (uintptr_t)d.out;
    // whole aligned vectors, or a tiny block of any shape that the kernel moves byte by byte
    const bool bytewise = blockBytes % 16 != 0 || ((in | out) & 15) != 0;
    if (bytewise && blockBytes > 256) return false;
    const bool overlap = in < out + outBytes && out < in + inBytes;
    if (overlap && !(mode == LL_ALLREDUCE && in == out)) return false;     // in-place all-reduce reads and writes the same vector per thread
    CollArgs a;
    FillBase(c, d, a);
    a.in = d.in; a.out = d.out; a.count = d.count; a.peer = mode; a.root = bytewise ? 1 : 0;
    OpDesc typed = d;
    if (!reducing) typed.dtype = HCCL_DATA_TYPE_FP32;                        // byte movers share the fp32 instantiation
    a.dtype = typed.dtype;
    const int ctas = (int)std::min<uint64_t>(32, std::max<uint64_t>(1, blockBytes / 8192));
    *res = Launch(c, FK_SMALL_LL, a, c->emuSameDevice ? std::min(ctas, 4) : ctas, d.stream);
    return true;
}

// -------------------------------------------------------------------------- fast-kernel drivers

// Zero-copy on registered memory: when a buffer lies inside a window registered with HcclCommSymWinRegister (or an
// activated HcclCommSetMemoryRange), kernels read the peers' copies of it in place instead of staging through the CCL
// buffer - what the reference's zero-copy address manager and graph-mode kernels are for
// (communicator/impl/zero_copy/zero_copy_address_mgr.cc, aiv_all_reduce_910b_bigdata_graph.h).  HCCL_ZERO_COPY=0 turns it off.
// HCCL_WINDOWS_IN_KERNEL=0: operands beyond the staging are cut into one launch per window by the host instead of
// being walked inside one launch (kept for comparison).
bool WindowsInKernel()
{
    static const bool on = [] { const char *e = getenv("HCCL_WINDOWS_IN_KERNEL"); return !(e && e[0] == '0'); }();
    return on;
}

bool ZeroCopyEnabled()
{
    static const bool on = [] { const char *e = getenv("HCCL_ZERO_COPY"); return !(e && e[0] == '0'); }();
    return on;
}
// Fills a.inPeer / a.inMc when [in, in + bytes) is registered (and 16-byte aligned); returns whether it is.
bool RegisteredInput(Comm *c, const void *in, uint64_t bytes, CollArgs &a, bool needMc)
{
    if (!ZeroCopyEnabled() || c->emuSameDevice || ((uintptr_t)in & 15) != 0) return false;
    uint64_t off = 0;
    Window *w = FindWindow(c, in, bytes, &off);
    if (!w || (needMc && !w->mcPtr)) return false;
    for (uint32_t r = 0; r < c->nRanks; ++r) a.inPeer[r] = (const char *)w->peerPtr[r] + off;
    a.inMc = w->mcPtr ? (const char *)w->mcPtr + off : nullptr;
    return true;
}
void *RegisteredOutputMc(Comm *c, void *out, uint64_t bytes)
{
    if (!ZeroCopyEnabled() || c->emuSameDevice || ((uintptr_t)out & 15) != 0) return nullptr;
    uint64_t off = 0;
    Window *w = FindWindow(c, out, bytes, &off);
    return (w && w->mcPtr) ? (char *)w->mcPtr + off : nullptr;
}
void ClearRegistered(CollArgs &a)
{
    memset(a.inPeer, 0, sizeof(a.inPeer));
    a.inMc = nullptr;
    a.outMc = nullptr;
}

static bool NvlsPipelineEnabled()
{
    static const bool on = [] { const char *e = getenv("HCCL_NVLS_PIPELINE"); return !(e && e[0] == '0'); }();
    return on;
}
// Smallest operand that takes the pipelined kernel (HCCL_NVLS_PIPELINE_MIN_MB, default 96 MB): below it the extra
// barriers cost more than the overlapped copies save.
static uint64_t NvlsPipelineMinBytes()
{
    static const uint64_t v = [] { const char *e = getenv("HCCL_NVLS_PIPELINE_MIN_MB"); return (uint64_t)(e ? std::max(1, atoi(e)) : 96) << 20; }();
    return v;
}

HcclResult FastAllReduce(Comm *c, const OpDesc &d, const Selection &sel)
{
    const uint32_t n = c->nRanks, esz = DtypeSize(d.dtype);
    CollArgs a;
    FillBase(c, d, a);
    int kind = sel.engine == Engine::NVLS ? FK_ALLREDUCE_NVLS : (sel.algo == Algo::MESH_ONESHOT ? FK_ALLREDUCE_ONESHOT : FK_ALLREDUCE_TWOSHOT);
    const uint64_t oneShotCap = AlignDownElems(c->halfBytes / n / esz, esz);
    if (kind == FK_ALLREDUCE_ONESHOT && d.count > oneShotCap) kind = FK_ALLREDUCE_TWOSHOT;
    a.in = d.in; a.out = d.out; a.count = d.count;
    // in-switch reduction straight from the registered input into the registered output: no staging, any size
    const bool nvlsTypes = d.op == HCCL_REDUCE_SUM && (d.dtype == HCCL_DATA_TYPE_FP32 || d.dtype == HCCL_DATA_TYPE_FP16 || d.dtype == HCCL_DATA_TYPE_BFP16);
    // (up to 4 GPUs the mesh kernels measured faster than in-switch reduction, registered or not)
    if (c->mcBase && n > 4 && nvlsTypes && __atomic_load_n(&c->cfg.deterministic, __ATOMIC_RELAXED) == 0 && sel.reason != "forced by configuration" && d.count * esz >= 64 * 1024 &&
        RegisteredInput(c, d.in, d.count * esz, a, true)) {
        a.outMc = RegisteredOutputMc(c, d.out, d.count * esz);
        if (a.outMc) return Launch(c, FK_ALLREDUCE_NVLS, a, PickCtas(c, sel, d.count * esz), d.stream);
        ClearRegistered(a);
    }
    // One launch whatever the size: operands beyond the staging are walked in windows inside the kernel.
    if (kind == FK_ALLREDUCE_ONESHOT) { a.sliceElems = oneShotCap; a.winElems = 0; }
    else if (kind == FK_ALLREDUCE_TWOSHOT) { a.winElems = AlignDownElems(c->halfBytes / (2 * n) / esz, esz) * n; a.sliceElems = d.count <= a.winElems ? AlignedSliceCount(d.count, n, esz) : 0; }
    else {
        a.winElems = AlignDownElems(c->halfBytes / esz, esz);
        a.sliceElems = 0;
        // Large operands: eight or more windows, with copy-in, in-switch reduction and copy-out of neighbouring windows
        // overlapped inside the kernel (HCCL_NVLS_PIPELINE=0 keeps the phase-by-phase kernel).
        const uint64_t bytes = d.count * esz;
        if (NvlsPipelineEnabled() && WindowsInKernel() && bytes >= NvlsPipelineMinBytes() && bytes % 16 == 0 && (((uintptr_t)d.in | (uintptr_t)d.out) & 15) == 0) {
            const uint64_t winBytes = std::min<uint64_t>(c->halfBytes & ~(uint64_t)4095, std::max<uint64_t>(8ull << 20, ((bytes / 8 + 4095) & ~(uint64_t)4095)));
            a.winElems = winBytes / esz;
            return Launch(c, FK_ALLREDUCE_NVLS_PIPE, a, PickCtas(c, sel, bytes), d.stream);
        }
    }
    const uint64_t perWin = a.winElems ? std::min<uint64_t>(d.count, a.winElems) : d.count;
    const uint64_t perRank = kind == FK_ALLREDUCE_ONESHOT ? perWin * esz : (d.count > perWin ? perWin * esz : perWin * esz / n * 2);
    if (a.winElems && d.count > a.winElems && !WindowsInKernel()) {
        const uint64_t W = a.winElems;
        a.winElems = 0;
        for (uint64_t off = 0; off < d.count; off += W) {
            const uint64_t cnt = std::min(W, d.count - off);
            a.in = (const char *)d.in + off * esz; a.out = (char *)d.out + off * esz; a.count = cnt;
            a.sliceElems = kind == FK_ALLREDUCE_TWOSHOT ? AlignedSliceCount(cnt, n, esz) : 0;
            CHK_RET(Launch(c, kind, a, PickCtas(c, sel, perRank), d.stream));
        }
        return HCCL_SUCCESS;
    }
    if (kind == FK_ALLREDUCE_TWOSHOT && d.count > a.winElems) kind = FK_ALLREDUCE_TWOSHOT_WIN;
    return Launch(c, kind, a, PickCtas(c, sel, perRank), d.stream);
}

HcclResult FastReduce(Comm *c, const OpDesc &d, const Selection &sel)
{
    const uint32_t n = c->nRanks, esz = DtypeSize(d.dtype);
    CollArgs a;
    FillBase(c, d, a);
    uint64_t maxPerLaunch = AlignDownElems(c->halfBytes / (n + 1) / esz, esz) * n;
    for (uint64_t off = 0; off < d.count; off += maxPerLaunch) {
        uint64_t cnt = std::min(maxPerLaunch, d.count - off);
        a.in = (const char *)d.in + off * esz;
        a.out = d.out ? (char *)d.out + off * esz : nullptr;
        a.count = cnt;
        a.sliceElems = AlignedSliceCount(cnt, n, esz);
        CHK_RET(Launch(c, FK_REDUCE, a, PickCtas(c, sel, cnt * esz / n), d.stream));
    }
    return HCCL_SUCCESS;
}

// ReduceScatter and its V form: block q = sendCounts[q] elements at sendDispls[q].  One launch: blocks longer than a
// staging slot travel in column windows inside the kernel.
HcclResult FastReduceScatter(Comm *c, const OpDesc &d, const Selection &sel)
{
    const uint32_t n = c->nRanks, esz = DtypeSize(d.dtype);
    CollArgs a;
    FillBase(c, d, a);
    const bool uniform = d.sendCounts.empty();
    uint64_t maxCnt = 0;
    for (uint32_t q = 0; q < n; ++q) {
        a.sendCounts[q] = uniform ? d.count : d.sendCounts[q];
        a.sendDispls[q] = uniform ? (uint64_t)q * d.count : d.sendDispls[q];
        maxCnt = std::max(maxCnt, a.sendCounts[q]);
    }
    a.in = d.in; a.out = d.out; a.count = maxCnt;
    const uint64_t cap = AlignDownElems(c->halfBytes / n / esz, esz);
    a.sliceElems = cap;
    const uint64_t moved = std::min(cap, maxCnt) * esz * std::max(1u, n - 1);       // bytes this rank moves per window
    const bool vectors = uniform && (d.count * esz) % 16 == 0 && (((uintptr_t)d.in | (uintptr_t)d.out) & 15) == 0;
    const bool nvlsTypes = d.op == HCCL_REDUCE_SUM && (d.dtype == HCCL_DATA_TYPE_FP32 || d.dtype == HCCL_DATA_TYPE_FP16 || d.dtype == HCCL_DATA_TYPE_BFP16);
    const bool nvls = sel.engine == Engine::NVLS && c->mcBase && vectors && nvlsTypes && __atomic_load_n(&c->cfg.deterministic, __ATOMIC_RELAXED) == 0;
    if (uniform && sel.reason != "forced by configuration" && d.count * esz >= 16 * 1024 && RegisteredInput(c, d.in, (uint64_t)n * d.count * esz, a, false)) {
        // registered input: pull the peers' blocks in place (through the switch when the window has a multicast alias)
        if (a.inMc && nvls) return Launch(c, FK_REDUCE_SCATTER_NVLS, a, PickCtas(c, sel, moved), d.stream);
        a.inMc = nullptr;
        return Launch(c, FK_REDUCE_SCATTER_INPLACE, a, PickCtas(c, sel, moved), d.stream);
    }
    ClearRegistered(a);
    if (nvls) return Launch(c, FK_REDUCE_SCATTER_NVLS, a, PickCtas(c, sel, moved), d.stream);
    if (maxCnt > cap && !WindowsInKernel()) {
        std::vector<uint64_t> cnt(a.sendCounts, a.sendCounts + n), dsp(a.sendDispls, a.sendDispls + n);
        for (uint64_t c0 = 0; c0 < maxCnt; c0 += cap) {
            for (uint32_t q = 0; q < n; ++q) {
                const uint64_t hi = std::min(cnt[q], c0 + cap);
                a.sendCounts[q] = hi > c0 ? hi - c0 : 0;
                a.sendDispls[q] = dsp[q] + c0;
            }
            a.out = (char *)d.out + c0 * esz;
            a.count = std::min(cap, maxCnt - c0);
            CHK_RET(Launch(c, FK_REDUCE_SCATTER, a, PickCtas(c, sel, moved), d.stream));
        }
        return HCCL_SUCCESS;
    }
    return Launch(c, maxCnt > cap ? FK_REDUCE_SCATTER_WIN : FK_REDUCE_SCATTER, a, PickCtas(c, sel, moved), d.stream);
}

HcclResult FastAllGather(Comm *c, const OpDesc &d, const Selection &sel)
{
    const uint32_t n = c->nRanks, esz = DtypeSize(d.dtype);
    CollArgs a;
    FillBase(c, d, a);
    const bool uniform = d.recvCounts.empty();
    uint64_t maxCnt = 0;
    for (uint32_t q = 0; q < n; ++q) {
        a.recvCounts[q] = uniform ? d.count : d.recvCounts[q];
        a.recvDispls[q] = uniform ? (uint64_t)q * d.count : d.recvDispls[q];
        maxCnt = std::max(maxCnt, a.recvCounts[q]);
    }
    a.in = d.in; a.out = d.out; a.count = maxCnt;
    const bool vectors = uniform && (d.count * esz) % 16 == 0 && (((uintptr_t)d.in | (uintptr_t)d.out) & 15) == 0;
    const bool nvls = sel.engine == Engine::NVLS && c->mcBase && vectors;
    const bool mayZeroCopy = uniform && sel.reason != "forced by configuration" && d.count * esz >= 16 * 1024;
    if (nvls) {
        // every rank stores its block once, the switch replicates it: straight into a registered output, else via the staging
        a.outMc = mayZeroCopy ? RegisteredOutputMc(c, d.out, (uint64_t)n * d.count * esz) : nullptr;
        a.sliceElems = AlignDownElems(c->halfBytes / n / esz, esz);
        return Launch(c, FK_ALLGATHER_NVLS, a, PickCtas(c, sel, std::min(a.sliceElems, maxCnt) * esz * std::max(1u, n - 1)), d.stream);
    }
    a.sliceElems = AlignDownElems(c->halfBytes / esz, esz);
    const uint64_t moved = std::min(a.sliceElems, maxCnt) * esz * std::max(1u, n - 1);
    if (mayZeroCopy && RegisteredInput(c, d.in, d.count * esz, a, false)) { a.inMc = nullptr; return Launch(c, FK_ALLGATHER, a, PickCtas(c, sel, moved), d.stream); }
    ClearRegistered(a);
    return Launch(c, FK_ALLGATHER, a, PickCtas(c, sel, moved), d.stream);
}

HcclResult FastAlltoAll(Comm *c, const OpDesc &d, const Selection &sel)
{
    const uint32_t n = c->nRanks, esz = DtypeSize(d.dtype);
    CollArgs a;
    FillBase(c, d, a);
    uint64_t maxCnt = 0;
    for (uint32_t q = 0; q < n; ++q) {
        a.sendCounts[q] = d.sendCounts.empty() ? d.count : d.sendCounts[q];
        a.sendDispls[q] = d.sendCounts.empty() ? (uint64_t)q * d.count : d.sendDispls[q];
        a.recvCounts[q] = d.recvCounts.empty() ? d.count : d.recvCounts[q];
        a.recvDispls[q] = d.recvCounts.empty() ? (uint64_t)q * d.count : d.recvDispls[q];
        maxCnt = std::max(maxCnt, std::max(a.sendCounts[q], a.recvCounts[q]));
    }
    uint64_t cap = AlignDownElems(c->halfBytes / n / esz, esz);
    a.sliceElems = cap;
    a.in = d.in;
    a.out = d.out;
    a.count = maxCnt;                                  // this rank's longest block
    a.root = d.sendCounts.empty() ? 0 : 1;             // variable counts: agree on the job-wide maximum in the kernel
    return Launch(c, FK_ALLTOALL, a, PickCtas(c, sel, std::min(cap, maxCnt) * esz * (n - 1)), d.stream);
}

HcclResult FastBroadcast(Comm *c, const OpDesc &d, const Selection &sel)
{
    const uint32_t n = c->nRanks, esz = DtypeSize(d.dtype);
    CollArgs a;
    FillBase(c, d, a);
    int kind = sel.engine == Engine::NVLS ? FK_BROADCAST_NVLS : (sel.algo == Algo::MESH_ONESHOT ? FK_BROADCAST_PUSH : FK_BROADCAST_TWOSHOT);
    uint64_t cap = AlignDownElems(c->halfBytes / esz, esz);
    for (uint64_t off = 0; off < d.count; off += cap) {
        uint64_t cnt = std::min(cap, d.count - off);
        a.in = (const char *)d.in + off * esz;
        a.out = (char *)d.out + off * esz;
        a.count = cnt;
        a.sliceElems = AlignedSliceCount(cnt, n, esz);
        CHK_RET(Launch(c, kind, a, PickCtas(c, sel, cnt * esz), d.stream));
    }
    return HCCL_SUCCESS;
}

HcclResult FastScatterGather(Comm *c, const OpDesc &d, const Selection &sel, bool scatter)
{
    const uint32_t n = c->nRanks, esz = DtypeSize(d.dtype);
    CollArgs a;
    FillBase(c, d, a);
    uint64_t cap = AlignDownElems(c->halfBytes / (scatter ? 1 : n) / esz, esz);
    if (d.count > cap) {
        RPT_ERR("EI0003", "%s of %llu elements per rank exceeds what one CCL half holds (%llu); raise HCCL_BUFFSIZE", scatter ? "scatter" : "gather",
                (unsigned long long)d.count, (unsigned long long)cap);
        return HCCL_E_MEMORY;
    }
    a.in = d.in; a.out = d.out; a.count = d.count; a.sliceElems = cap;
    return Launch(c, scatter ? FK_SCATTER : FK_GATHER, a, PickCtas(c, sel, d.count * esz), d.stream);
}

HcclResult FastSendRecv(Comm *c, const OpDesc &d, bool send, Stream stream)
{
    if (c->emuSameDevice) {
        RPT_ERR("EI0003", "send/recv kernels of two ranks cannot share one GPU; use one GPU per rank or the simulator");
        return HCCL_E_NOT_SUPPORT;
    }
    const uint32_t esz = DtypeSize(d.dtype);
    CollArgs a;
    FillBase(c, d, a);
    a.peer = (int32_t)d.peer;
    a.count = d.count;
    uint64_t bytes = d.count * esz, sub = c->p2pSlotBytes / 2, chunks = (bytes + sub - 1) / sub;
    if (send) { a.in = d.in; a.p2pDataBase = c->p2pSent[d.peer]; c->p2pSent[d.peer] += chunks; }
    else { a.out = d.out; a.p2pDataBase = c->p2pRecvd[d.peer]; c->p2pRecvd[d.peer] += chunks; }
    int ctas = (int)std::min<uint64_t>(16, std::max<uint64_t>(1, bytes >> 18));
    return Launch(c, send ? FK_SEND : FK_RECV, a, ctas, stream);
}

// ------------------------------------------------------------------------------- host drivers

// Builds (or finds in the per-communicator cache) the schedule of an operator.
static HcclResult GetSchedule(Comm *c, const OpDesc &d, const Selection &sel, std::shared_ptr<Schedule> *out)
{
    CollShape sh;
    sh.cmd = d.cmd;
    sh.nRanks = c->nRanks;
    sh.root = d.root;
    sh.count = d.count;
    sh.elemSize = DtypeSize(d.dtype);
    sh.onlyRank = (int)c->rank;
    std::string key;
    bool cacheable = d.sendCounts.empty() && d.recvCounts.empty();
    switch (d.cmd) {
        case HCCL_CMD_REDUCE_SCATTER_V:
            sh.sendCounts = {d.sendCounts}; sh.sendDispls = {d.sendDispls};
            break;
        case HCCL_CMD_ALLGATHER_V:
            sh.recvCounts = {d.recvCounts}; sh.recvDispls = {d.recvDispls};
            break;
        case HCCL_CMD_ALLTOALLV: case HCCL_CMD_ALLTOALLVC:
            sh.sendCounts.assign(c->nRanks, {}); sh.sendDispls.assign(c->nRanks, {});
            sh.recvCounts.assign(c->nRanks, {}); sh.recvDispls.assign(c->nRanks, {});
            sh.sendCounts[c->rank] = d.sendCounts; sh.sendDispls[c->rank] = d.sendDispls;
            sh.recvCounts[c->rank] = d.recvCounts; sh.recvDispls[c->rank] = d.recvDispls;
            break;
        case HCCL_CMD_SEND: sh.p2pSrc = c->rank; sh.p2pDst = d.peer; break;
        case HCCL_CMD_RECEIVE: sh.p2pSrc = d.peer; sh.p2pDst = c->rank; break;
        default: break;
    }
    std::shared_ptr<Schedule> sched;
    if (cacheable) {
        key = std::string(CmdName(d.cmd)) + "/" + AlgoName(sel.algo) + "/" + std::to_string(d.count) + "/" + std::to_string(sh.elemSize) + "/" +
              std::to_string(d.root) + "/" + std::to_string(d.peer);
        auto it = c->schedCache.find(key);
        if (it != c->schedCache.end()) sched = it->second;
    }
    if (!sched) {
        sched = std::make_shared<Schedule>();
        std::string why;
        if (!BuildSchedule(sh, sel.algo, sched.get(), &why)) {
            RPT_ERR("EI0003", "cannot build %s with algorithm %s: %s", CmdName(d.cmd), AlgoName(sel.algo), why.c_str());
            return HCCL_E_NOT_SUPPORT;
        }
        HCCL_DEBUG_CAT(CAT_ALG, "built %s: %zu primitives for rank %u", sched->name.c_str(), sched->ranks[c->rank].prims.size(), c->rank);
        if (cacheable) {
            if (c->schedCache.size() > 512) c->schedCache.clear();
            c->schedCache[key] = sched;
        }
    }
    *out = sched;
    return HCCL_SUCCESS;
}

HcclResult HostCollective(Comm *c, const OpDesc &d, const Selection &sel)
{
    std::shared_ptr<Schedule> sched;
    CHK_RET(GetSchedule(c, d, sel, &sched));
    // All-to-all with per-rank counts: every rank must walk the same number of passes, so the ranks agree on
    // the longest block of the job over the control plane (the reference gathers the whole count matrix
    // for the same reason before it stages AlltoAllV).
    if (d.cmd == HCCL_CMD_ALLTOALLV || d.cmd == HCCL_CMD_ALLTOALLVC) {
        uint64_t localMax = 0;
        for (auto v : d.sendCounts) localMax = std::max(localMax, v);
        for (auto v : d.recvCounts) localMax = std::max(localMax, v);
        Blob mine((uint8_t *)&localMax, (uint8_t *)&localMax + 8);
        std::vector<Blob> all;
        CHK_RET(c->boot->AllGather(c->group, mine, &all));
        uint64_t gmax = 0;
        for (auto &b : all) { uint64_t v = 0; if (b.size() == 8) memcpy(&v, b.data(), 8); gmax = std::max(gmax, v); }
        for (auto &L : sched->input) L.sliceCount = std::max(L.sliceCount, gmax);
        for (auto &L : sched->output) L.sliceCount = std::max(L.sliceCount, gmax);
        sched->scratch.sliceCount = std::max(sched->scratch.sliceCount, gmax);
    }
    ExecArgs ea;
    ea.in = d.in; ea.out = d.out; ea.dtype = d.dtype; ea.op = d.op;
    ea.stream = c->plat->kind() == PlatKind::SIM ? nullptr : d.stream;
    CHK_RET(ExecuteOnHost(c, *sched, ea));
    c->lastOpOnHost = true;
    return HCCL_SUCCESS;
}

// Batch of sends and receives executed on the host engine in three phases so that no pairing of
// sends and receives can deadlock: announce all receives, perform all sends, complete all receives.
HcclResult HostBatchSendRecv(Comm *c, const OpDesc &d)
{
    Platform *P = c->plat;
    Stream st = P->kind() == PlatKind::SIM ? nullptr : d.stream;
    const uint32_t n = c->nRanks;
    const uint64_t slotBytes = (c->halfBytes / n) & ~255ull;
    auto notify = [&](uint32_t owner, uint32_t from, uint32_t idx) {
        return (uint64_t *)(c->PeerHeap(owner) + HC_OFF_CHAN_NOTIFY) + (uint64_t)from * HC_CHAN_NOTIFY + idx;
    };
    // landing slots in the CCL half that the next collective will use (idle now; see ExecuteOnHost)
    const uint64_t halfOff = (uint64_t)(c->hostLaunches & 1u) * c->halfBytes;
    auto slot = [&](uint32_t owner, uint32_t from) { return c->PeerHeap(owner) + HC_CTRL_BYTES + halfOff + (uint64_t)from * slotBytes; };
    auto wait = [&](uint32_t peer, uint32_t idx) -> HcclResult {
        uint64_t &w = c->chanWaited[(size_t)peer * HC_CHAN_NOTIFY + idx];
        ++w;
        WaitReport rep;
        rep.status = c->waitStatus; rep.abortWord = c->abortWord; rep.rank = c->rank; rep.peer = peer; rep.kind = HC_WAIT_CHAN_NOTIFY; rep.slot = idx; rep.seq = c->opSeq;
        return P->FlagWaitGeAsync(notify(c->rank, peer, idx), w, c->TimeoutMs(), rep, st);
    };
    // items between the same ordered pair are served in successive rounds
    std::vector<uint64_t> progress(d.batch.size(), 0);
    for (;;) {
        std::vector<bool> sendBusy(n, false), recvBusy(n, false);
        std::vector<size_t> round;
        for (size_t i = 0; i < d.batch.size(); ++i) {
            const HcclSendRecvItem &it = d.batch[i];
            uint64_t bytes = it.count * DtypeSize(it.dataType);
            if (progress[i] >= bytes && !(bytes == 0 && progress[i] == 0)) continue;
            std::vector<bool> &busy = it.sendRecvType == HCCL_SEND ? sendBusy : recvBusy;
            if (busy[it.remoteRank]) continue;
            busy[it.remoteRank] = true;
            round.push_back(i);
        }
        if (round.empty()) break;
        for (size_t i : round)
            if (d.batch[i].sendRecvType == HCCL_RECV) CHK_RET(P->FlagAddAsync(notify(d.batch[i].remoteRank, c->rank, N_READY), 1, st));
        for (size_t i : round) {
            const HcclSendRecvItem &it = d.batch[i];
            if (it.sendRecvType != HCCL_SEND) continue;
            uint64_t bytes = it.count * DtypeSize(it.dataType), len = std::min(slotBytes, bytes - progress[i]);
            CHK_RET(wait(it.remoteRank, N_READY));
            if (len) CHK_RET(P->MemcpyAsync(slot(it.remoteRank, c->rank), (char *)it.buf + progress[i], len, st));
            CHK_RET(P->FlagAddAsync(notify(it.remoteRank, c->rank, N_DATA), 1, st));
        }
        for (size_t i : round) {
            const HcclSendRecvItem &it = d.batch[i];
            uint64_t bytes = it.count * DtypeSize(it.dataType), len = std::min(slotBytes, bytes - progress[i]);
            if (it.sendRecvType == HCCL_RECV) {
                CHK_RET(wait(it.remoteRank, N_DATA));
                if (len) CHK_RET(P->MemcpyAsync((char *)it.buf + progress[i], slot(c->rank, it.remoteRank), len, st));
            }
            progress[i] += len;
            if (bytes == 0) progress[i] = 1;
        }
    }
    c->lastOpOnHost = true;
    return HCCL_SUCCESS;
}

HcclResult FastBatchSendRecv(Comm *c, const OpDesc &d)
{
    Platform *P = c->plat;
    while (c->auxStreams.size() < 2) {
        Stream s;
        CHK_RET(P->StreamCreate(&s));
        c->auxStreams.push_back(s);
    }
    Stream sendSt = c->auxStreams[0], recvSt = c->auxStreams[1];
    CHK_RET(P->StreamOrder(d.stream, sendSt));
    CHK_RET(P->StreamOrder(d.stream, recvSt));
    for (auto &it : d.batch) {
        OpDesc one;
        one.cmd = it.sendRecvType == HCCL_SEND ? HCCL_CMD_SEND : HCCL_CMD_RECEIVE;
        one.in = it.buf; one.out = it.buf; one.count = it.count; one.dtype = it.dataType; one.peer = it.remoteRank;
        CHK_RET(FastSendRecv(c, one, it.sendRecvType == HCCL_SEND, it.sendRecvType == HCCL_SEND ? sendSt : recvSt));
    }
    CHK_RET(P->StreamOrder(sendSt, d.stream));
    CHK_RET(P->StreamOrder(recvSt, d.stream));
    return HCCL_SUCCESS;
}

}  // namespace

// Engine "sm-ir": the schedule of a forced (non-mesh) algorithm runs in the interpreter kernel, one launch per column
// pass.  Operators with per-rank counts and programs longer than a ring slot stay on the stream engine.
constexpr uint32_t kIrSlotPrims = 2048;
HcclResult IrCollective(Comm *c, const OpDesc &d, const Selection &sel, bool *served)
{
    *served = false;
    if (!d.sendCounts.empty() || !d.recvCounts.empty() || c->nRanks > HC_KERNEL_MAX_RANKS || !IrKernelFor(d.dtype)) return HCCL_SUCCESS;
    switch (d.cmd) {
        case HCCL_CMD_ALLREDUCE: case HCCL_CMD_ALLGATHER: case HCCL_CMD_REDUCE_SCATTER: case HCCL_CMD_ALLTOALL: case HCCL_CMD_BROADCAST:
        case HCCL_CMD_REDUCE: case HCCL_CMD_SCATTER: case HCCL_CMD_GATHER: break;
        default: return HCCL_SUCCESS;
    }
    std::shared_ptr<Schedule> sched;
    CHK_RET(GetSchedule(c, d, sel, &sched));
    const Schedule &s = *sched;
    const SliceLayout &in = s.In(c->rank), &out = s.Out(c->rank);
    const RankProgram &prog = s.ranks[c->rank];
    if (!in.displ.empty() || !in.count.empty() || !out.displ.empty() || !out.count.empty() || prog.prims.size() > kIrSlotPrims || s.nNotify > HC_IR_NOTIFY) return HCCL_SUCCESS;
    const uint32_t esz = DtypeSize(d.dtype);
    const uint64_t cap = ScratchCapacityElems(c, s, esz);
    if (cap == 0) return HCCL_SUCCESS;
    if (!c->irPrimRing) CHK_RET(c->plat->DevAlloc(sizeof(DevPrim) * kIrSlotPrims * 8, &c->irPrimRing));
    std::vector<DevPrim> dev(prog.prims.size());
    for (size_t i = 0; i < prog.prims.size(); ++i) {
        const Prim &p = prog.prims[i];
        DevPrim &q = dev[i];
        memset(&q, 0, sizeof(q));
        q.op = (uint8_t)p.op; q.thread = p.thread; q.srcBuf = (uint8_t)p.srcBuf; q.dstBuf = (uint8_t)p.dstBuf; q.peer = p.peer; q.notify = p.notify;
        q.srcSlice = p.srcSlice; q.dstSlice = p.dstSlice; q.nSlices = p.nSlices; q.toThread = p.toThread; q.step = p.step; q.lenBuf = (uint8_t)p.lenBuf;
        q.lenSlice = p.lenSlice;
        if (p.op != PrimOp::POST && p.op != PrimOp::WAIT && p.op != PrimOp::NOP && (p.lenBuf == BufId::NONE || p.srcBuf == BufId::NONE || p.dstBuf == BufId::NONE)) return HCCL_SUCCESS;
    }
    DevPrim *slot = (DevPrim *)c->irPrimRing + (size_t)c->irPrimNext * kIrSlotPrims;
    c->irPrimNext = (c->irPrimNext + 1) % 8;
    // the source is pageable host memory: the runtime stages it before the call returns, so the vector may go away
    if (!dev.empty()) CHK_RET(c->plat->MemcpyAsync(slot, dev.data(), sizeof(DevPrim) * dev.size(), d.stream));
    uint64_t maxSlice = std::max(in.sliceCount, out.sliceCount);
    for (auto &L : s.input) maxSlice = std::max(maxSlice, L.sliceCount);
    for (auto &L : s.output) maxSlice = std::max(maxSlice, L.sliceCount);
    const uint64_t q16 = esz >= 16 ? 1 : 16 / esz, chunk = cap / q16 * q16;
    const uint64_t passes = maxSlice == 0 ? 1 : (maxSlice + chunk - 1) / chunk;
    IrArgs a;
    memset(&a, 0, sizeof(a));
    a.dev = c->devStruct; a.prims = slot; a.nPrims = (uint32_t)dev.size(); a.dtype = d.dtype; a.op = d.op; a.elemSize = esz; a.in = d.in; a.out = d.out;
    a.lay[0] = {in.sliceCount, in.total}; a.lay[1] = {out.sliceCount, out.total}; a.lay[2] = {s.scratch.sliceCount, s.scratch.total};
    a.cap = cap;
    int ctas = (int)std::min<uint64_t>(HC_IR_MAX_CTAS, std::max<uint64_t>(1, std::min(maxSlice, chunk) * esz / (64 << 10)));
    if (c->emuSameDevice) ctas = std::min(ctas, 4);
    for (uint64_t pass = 0; pass < passes; ++pass) {
        a.col0 = pass * chunk; a.col1 = (pass + 1) * chunk;
        a.preBarrier = c->lastOpOnHost ? 1 : 0;
        HcclResult r;
        if (c->emuSameDevice && c->nRanks > 1) {
            r = EmuLaunchGeneric(c->identifier + "#ir" + std::to_string(c->group.id), c->nRanks, c->rank, 9200 + (int)d.cmd, &a, sizeof(a), d.stream,
                                 [=](const void *devTable, uint32_t n, void *st) { return LaunchIrKernel(a, ctas, st, (const IrArgs *)devTable, (int)n); });
        } else {
            r = LaunchIrKernel(a, ctas, d.stream, nullptr, 0);
        }
        CHK_RET(r);
        c->lastOpOnHost = false;
    }
    *served = true;
    return HCCL_SUCCESS;
}

// A specialised kernel that follows a host-engine operator must not touch peer staging before every rank has
// left that operator; fused kernels (which have no barrier of their own) call this first.
HcclResult LaunchBarrierIfNeeded(Comm *c, void *stream)
{
    if (!c->lastOpOnHost || c->nRanks == 1) { c->lastOpOnHost = false; return HCCL_SUCCESS; }
    OpDesc d;
    CollArgs a;
    FillBase(c, d, a);
    return Launch(c, FK_BARRIER, a, 1, stream);
}

HcclResult DescribeSelection(Comm *c, HcclCMDType cmd, uint64_t count, HcclDataType dtype, HcclReduceOp op, bool variableCounts, Selection *sel, int *ctas)
{
    SelectInput si;
    si.cmd = cmd; si.nRanks = c->nRanks; si.dtype = dtype; si.op = op;
    si.bytes = count * DtypeSize(dtype);
    si.opExpansionMode = c->cfg.opExpansionMode;
    si.deterministic = __atomic_load_n(&c->cfg.deterministic, __ATOMIC_RELAXED);
    si.cuda = c->plat->kind() == PlatKind::CUDA;
    si.singleDomain = c->nRanks <= HC_KERNEL_MAX_RANKS && c->graph.SingleNvlinkDomain();
    si.nvlsAvailable = c->mcBase != nullptr;
    si.variableCounts = variableCounts;
    CHK_RET(SelectAlgorithm(si, AlgoConfigOf(c), sel));
    if (ctas) *ctas = (sel->engine == Engine::HOST) ? 0 : PickCtas(c, *sel, si.bytes);
    return HCCL_SUCCESS;
}

const AlgoConfig &AlgoConfigOf(Comm *c)
{
    std::lock_guard<std::mutex> lk(g_algoMu);
    auto it = g_algoCfg.find(c->cfg.algo);
    if (it != g_algoCfg.end()) return it->second;
    AlgoConfig cfg;
    std::string err;
    if (!cfg.Parse(c->cfg.algo, &err)) {
        HCCL_WARNING("algorithm configuration \"%s\" ignored: %s", c->cfg.algo.c_str(), err.c_str());
        cfg.perCmd.clear();
    }
    return g_algoCfg[c->cfg.algo] = cfg;
}

HcclResult LaunchForRank(Comm *c, FastLaunch &l)
{
    if (c->emuSameDevice && c->nRanks > 1) return EmuLaunch(c->identifier + "#" + std::to_string(c->group.id), c->nRanks, c->rank, l);
    return LaunchFastKernel(l);
}

uint64_t OpDataVolume(const Comm *c, const OpDesc &d)
{
    uint64_t esz = DtypeSize(d.dtype);
    switch (d.cmd) {
        case HCCL_CMD_ALLGATHER: case HCCL_CMD_REDUCE_SCATTER: case HCCL_CMD_ALLTOALL: case HCCL_CMD_SCATTER: case HCCL_CMD_GATHER:
            return d.count * esz * c->nRanks;
        default: return d.count * esz;
    }
}

bool GroupActive() { return t_groupDepth > 0; }

HcclResult RunOp(Comm *c, const OpDesc &d)
{
    HcclResult r;
    uint64_t seq;
    {
        std::lock_guard<std::mutex> lk(c->opMu);
        r = RunOpLocked(c, d);
        seq = c->opSeq;
    }
    // an expired wait that a host engine reports synchronously: the retry rounds run the operator again
    if (r == HCCL_E_TIMEOUT && c->retry) r = RetryAfterTimeout(c, seq);
    return r;
}

HcclResult RunOpLocked(Comm *c, const OpDesc &d)
{
    int st = c->state.load();
    if (st == (int)CommState::SUSPENDING || st == (int)CommState::SUSPENDED) return HCCL_E_SUSPENDING;
    if (st == (int)CommState::DESTROYED) return HCCL_E_PARA;
    if (c->asyncError.load() != 0) return (HcclResult)c->asyncError.load();
    uint64_t t0 = NowNs();
    ++c->opSeq;
    RetryNoteOp(c, d);
    const bool cuda = c->plat->kind() == PlatKind::CUDA;
    const uint32_t esz = DtypeSize(d.dtype);

    SelectInput si;
    si.cmd = d.cmd; si.nRanks = c->nRanks; si.dtype = d.dtype; si.op = d.op;
    si.bytes = d.count * esz;
    si.opExpansionMode = c->cfg.opExpansionMode;
    si.deterministic = __atomic_load_n(&c->cfg.deterministic, __ATOMIC_RELAXED);
    si.cuda = cuda;
    si.singleDomain = c->nRanks <= HC_KERNEL_MAX_RANKS && c->graph.SingleNvlinkDomain();
    si.nvlsAvailable = c->mcBase != nullptr;
    si.variableCounts = !d.sendCounts.empty() || !d.recvCounts.empty();
    Selection sel;
    if (d.cmd == HCCL_CMD_BATCH_SEND_RECV || d.cmd == HCCL_CMD_BARRIER) {
        bool hostOnly = !cuda || c->cfg.opExpansionMode == 1 || c->cfg.opExpansionMode == 2 || (c->emuSameDevice && d.cmd == HCCL_CMD_BATCH_SEND_RECV);
        sel.engine = hostOnly ? Engine::HOST : Engine::SM_FAST;
        sel.algo = d.cmd == HCCL_CMD_BARRIER ? Algo::MESH_ONESHOT : Algo::MESH;
        sel.name = std::string(CmdName(d.cmd)) + "@" + EngineName(sel.engine);
    } else {
        CHK_RET(SelectAlgorithm(si, AlgoConfigOf(c), &sel));
    }
    static thread_local std::string lastLogged;
    if (lastLogged != sel.name) {
        HCCL_DEBUG_CAT(CAT_ALG, "%s: %llu elements of %s -> %s (%s)", CmdName(d.cmd), (unsigned long long)d.count, DtypeName(d.dtype), sel.name.c_str(), sel.reason.c_str());
        lastLogged = sel.name;
    }

    char rangeName[128] = "";
    if (c->profiling) snprintf(rangeName, sizeof(rangeName), "hccl:%s %llu x %s [%s]", CmdName(d.cmd), (unsigned long long)d.count, DtypeName(d.dtype), sel.name.c_str());
    NvtxRange nvtxRange(c->profiling, rangeName);    // covers selection's outcome: every launch of this operator sits inside it

    HcclResult r = HCCL_SUCCESS;
    bool irServed = false;
    // The specialised kernels are written for 16-byte vector (and multimem) accesses to the user buffers and fall back to
    // element accesses otherwise.  The interpreter assigns elements to CTAs by their index inside the slice and picks the
    // access width block by block, so calls whose buffers do not start on a 16-byte boundary go there.
    if (cuda && (sel.engine == Engine::SM_FAST || sel.engine == Engine::NVLS) && ((((uintptr_t)d.in) | ((uintptr_t)d.out)) & 15) != 0 &&
        d.sendCounts.empty() && d.recvCounts.empty() && !d.useScale && c->nRanks > 1 && d.count * DtypeSize(d.dtype) > 256 &&
        (d.cmd == HCCL_CMD_ALLREDUCE || d.cmd == HCCL_CMD_ALLGATHER || d.cmd == HCCL_CMD_REDUCE_SCATTER || d.cmd == HCCL_CMD_ALLTOALL ||
         d.cmd == HCCL_CMD_BROADCAST || d.cmd == HCCL_CMD_REDUCE)) {
        sel.engine = Engine::SM_IR;
        if (sel.algo != Algo::MESH_ONESHOT) sel.algo = Algo::MESH;
        sel.reason = "buffers not 16-byte aligned";
    }
    if (sel.engine == Engine::SM_IR) {
        r = IrCollective(c, d, sel, &irServed);
        if (r != HCCL_SUCCESS) { Record(c, d, sel, t0); return r; }
        if (!irServed) sel.engine = Engine::HOST;   // the stream engine runs every template
    }
    if (irServed) {
        // done by the interpreter kernel
    } else if (sel.engine == Engine::HOST) {
        if (cuda && c->emuSameDevice && c->nRanks > 1) {
            RPT_ERR("EI0003", "the stream engine cannot run ranks that share one GPU; use the SM kernels or the simulator");
            return HCCL_E_NOT_SUPPORT;
        }
        if (d.cmd == HCCL_CMD_BATCH_SEND_RECV) r = HostBatchSendRecv(c, d);
        else if (d.cmd == HCCL_CMD_BARRIER) {
            OpDesc b = d;
            b.cmd = HCCL_CMD_ALLREDUCE; b.count = 1; b.dtype = HCCL_DATA_TYPE_FP32; b.op = HCCL_REDUCE_SUM;
            void *scratch = c->LocalHeap() + HC_OFF_ONESIDED;   // internal one-element buffer, as the reference uses
            b.in = scratch; b.out = (char *)scratch + 64;
            Selection s2 = sel;
            s2.algo = Algo::MESH_ONESHOT;
            r = HostCollective(c, b, s2);
        } else r = HostCollective(c, d, sel);
        // the stream engine has no fused scale: a second pass over the result applies it
        if (r == HCCL_SUCCESS && d.useScale) r = c->plat->ScaleAsync(d.out, d.count, d.dtype, d.scale, c->plat->kind() == PlatKind::SIM ? nullptr : d.stream);
        if (r == HCCL_SUCCESS && c->plat->kind() == PlatKind::SIM) r = CommPollDeviceStatus(c);
    } else if (TrySmallLL(c, d, sel, &r)) {
        // served by the flag-in-data kernel
    } else {
        switch (d.cmd) {
            case HCCL_CMD_ALLREDUCE: r = FastAllReduce(c, d, sel); break;
            case HCCL_CMD_REDUCE: r = FastReduce(c, d, sel); break;
            case HCCL_CMD_REDUCE_SCATTER: case HCCL_CMD_REDUCE_SCATTER_V: r = FastReduceScatter(c, d, sel); break;
            case HCCL_CMD_ALLGATHER: case HCCL_CMD_ALLGATHER_V: r = FastAllGather(c, d, sel); break;
            case HCCL_CMD_ALLTOALL: case HCCL_CMD_ALLTOALLV: case HCCL_CMD_ALLTOALLVC: r = FastAlltoAll(c, d, sel); break;
            case HCCL_CMD_BROADCAST: r = FastBroadcast(c, d, sel); break;
            case HCCL_CMD_SCATTER: r = FastScatterGather(c, d, sel, true); break;
            case HCCL_CMD_GATHER: r = FastScatterGather(c, d, sel, false); break;
            case HCCL_CMD_SEND: r = FastSendRecv(c, d, true, d.stream); break;
            case HCCL_CMD_RECEIVE: r = FastSendRecv(c, d, false, d.stream); break;
            case HCCL_CMD_BATCH_SEND_RECV: r = FastBatchSendRecv(c, d); break;
            case HCCL_CMD_BARRIER: {
                CollArgs a;
                FillBase(c, d, a);
                r = Launch(c, FK_BARRIER, a, 1, d.stream);
                break;
            }
            default: r = HCCL_E_NOT_SUPPORT;
        }
    }
    Record(c, d, sel, t0);
    return r;
}

void GroupQueue(std::function<HcclResult()> job, uint64_t volume, bool isP2p, Comm *c, const OpDesc *p2p)
{
    GroupJob j;
    j.fn = std::move(job);
    j.volume = volume;
    j.p2p = isP2p;
    j.variable = false;
    j.comm = c;
    if (p2p) j.desc = *p2p;
    j.order = t_groupJobs.size();
    t_groupJobs.push_back(std::move(j));
}

HcclResult SubmitOp(Comm *c, const OpDesc &d)
{
    if (GroupActive()) {
        bool p2p = d.cmd == HCCL_CMD_SEND || d.cmd == HCCL_CMD_RECEIVE;
        OpDesc copy = d;
        GroupQueue([c, copy] { return RunOp(c, copy); }, OpDataVolume(c, d), p2p, c, &copy);
        t_groupJobs.back().variable = !d.sendCounts.empty() || !d.recvCounts.empty();
        return HCCL_SUCCESS;
    }
    return RunOp(c, d);
}

}  // namespace hc

// -------------------------------------------------------------------------------- group C API

using namespace hc;

extern "C" HcclResult HcclGroupStart(void)
{
    ++t_groupDepth;
    return HCCL_SUCCESS;
}

extern "C" HcclResult HcclGroupStatusGet(bool *isGroupEnabled)
{
    CHK_PTR_NULL(isGroupEnabled);
    *isGroupEnabled = t_groupDepth > 0;
    return HCCL_SUCCESS;
}

// Launch order at the outermost End (reference: framework/group/hccl_group.cc:181-230): queued
// communicator initialisations first, then all sends/receives of a communicator fused into one batch,
// then fixed-count collectives by descending data volume, variable-count ones last in issue order.
extern "C" HcclResult HcclGroupEnd(void)
{
    if (t_groupDepth == 0) {
        RPT_ERR("EI0003", "HcclGroupEnd without a matching HcclGroupStart");
        return HCCL_E_PARA;
    }
    if (--t_groupDepth > 0) return HCCL_SUCCESS;
    std::vector<GroupJob> jobs;
    jobs.swap(t_groupJobs);
    HcclResult first = HCCL_SUCCESS;
    auto keep = [&](HcclResult r) { if (r != HCCL_SUCCESS && first == HCCL_SUCCESS) first = r; };
    for (auto &j : jobs)
        if (!j.comm) keep(j.fn());   // communicator bring-up jobs
    std::map<Comm *, OpDesc> batches;
    std::vector<Comm *> batchOrder;
    for (auto &j : jobs) {
        if (!j.comm || !j.p2p) continue;
        if (!batches.count(j.comm)) {
            batchOrder.push_back(j.comm);
            batches[j.comm].cmd = HCCL_CMD_BATCH_SEND_RECV;
            batches[j.comm].stream = j.desc.stream;
        }
        HcclSendRecvItem it;
        it.sendRecvType = j.desc.cmd == HCCL_CMD_SEND ? HCCL_SEND : HCCL_RECV;
        it.buf = j.desc.cmd == HCCL_CMD_SEND ? const_cast<void *>(j.desc.in) : j.desc.out;
        it.count = j.desc.count;
        it.dataType = j.desc.dtype;
        it.remoteRank = j.desc.peer;
        batches[j.comm].batch.push_back(it);
    }
    for (Comm *c : batchOrder) keep(RunOp(c, batches[c]));
    std::vector<GroupJob *> fixed, variable;
    for (auto &j : jobs) {
        if (!j.comm || j.p2p) continue;
        (j.variable ? variable : fixed).push_back(&j);
    }
    std::stable_sort(fixed.begin(), fixed.end(), [](const GroupJob *a, const GroupJob *b) { return a->volume > b->volume; });
    for (auto *j : fixed) keep(j->fn());
    for (auto *j : variable) keep(j->fn());
    return first;
}
