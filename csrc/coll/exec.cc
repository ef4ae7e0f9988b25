#include "exec.h"

#include <algorithm>

#include "../core/dtype.h"
#include "../core/log.h"

namespace hc {

uint64_t ScratchCapacityElems(const Comm *c, const Schedule &s, uint32_t elemSize)
{
    uint64_t perSliceBytes = c->halfBytes / std::max<uint32_t>(1, s.scratch.nSlices);
    perSliceBytes &= ~(uint64_t)255;   // keep every slot 256-byte aligned
    return perSliceBytes / elemSize;
}

namespace {

struct Walker {
    Comm *c;
    const Schedule &s;
    const ExecArgs &a;
    uint32_t esz;
    uint64_t cap;        // elements per scratch slot in this pass
    uint64_t col0, col1; // column window of this pass
    uint32_t half;       // which CCL half this operator uses

    char *Scratch(uint32_t rank, uint32_t slot) const
    {
        return c->PeerHeap(rank) + HC_CTRL_BYTES + (uint64_t)half * c->halfBytes + (uint64_t)slot * cap * esz;
    }
    uint64_t *NotifyWord(uint32_t owner, uint32_t from, uint32_t idx) const
    {
        return (uint64_t *)(c->PeerHeap(owner) + HC_OFF_CHAN_NOTIFY) + (uint64_t)from * HC_CHAN_NOTIFY + idx;
    }
    const SliceLayout &LayoutOf(BufId b) const
    {
        return b == BufId::INPUT ? s.In(c->rank) : (b == BufId::OUTPUT ? s.Out(c->rank) : s.scratch);
    }
    // Address of column col0 of `slice` in buffer b as seen for `rank` (rank matters only for scratch).
    char *Addr(BufId b, uint32_t slice, uint32_t rank) const
    {
        if (b == BufId::SCRATCH) return Scratch(rank, slice);
        char *base = b == BufId::INPUT ? (char *)a.in : (char *)a.out;
        return base + (LayoutOf(b).DisplOf(slice) + col0) * esz;
    }
    // Elements of moved slice i that fall into the column window.
    uint64_t Len(const Prim &p, uint32_t i) const
    {
        uint64_t cnt = LayoutOf(p.lenBuf).CountOf(p.lenSlice + i);
        if (cnt <= col0) return 0;
        return std::min(cnt, col1) - col0;
    }

    HcclResult Run()
    {
        Platform *P = c->plat;
        const RankProgram &prog = s.ranks[c->rank];
        for (const Prim &p : prog.prims) {
            switch (p.op) {
                case PrimOp::POST:
                    CHK_RET(P->FlagAddAsync(NotifyWord((uint32_t)p.peer, c->rank, p.notify), 1, a.stream));
                    break;
                case PrimOp::WAIT: {
                    uint64_t &waited = c->chanWaited[(size_t)p.peer * HC_CHAN_NOTIFY + p.notify];
                    ++waited;
                    WaitReport rep;
                    rep.status = c->waitStatus; rep.abortWord = c->abortWord; rep.rank = c->rank; rep.peer = (uint32_t)p.peer;
                    rep.kind = HC_WAIT_CHAN_NOTIFY; rep.slot = p.notify; rep.seq = c->opSeq;
                    CHK_RET(P->FlagWaitGeAsync(NotifyWord(c->rank, (uint32_t)p.peer, p.notify), waited, c->TimeoutMs(), rep, a.stream));
                    break;
                }
                case PrimOp::NOP: break;
                default: {
                    bool remoteDst = p.op == PrimOp::WRITE || p.op == PrimOp::WRITE_REDUCE;
                    bool remoteSrc = p.op == PrimOp::READ || p.op == PrimOp::READ_REDUCE;
                    bool reduce = p.op == PrimOp::REDUCE || p.op == PrimOp::WRITE_REDUCE || p.op == PrimOp::READ_REDUCE;
                    uint32_t srcRank = remoteSrc ? (uint32_t)p.peer : c->rank, dstRank = remoteDst ? (uint32_t)p.peer : c->rank;
                    for (uint32_t i = 0; i < p.nSlices; ++i) {
                        uint64_t n = Len(p, i);
                        if (n == 0) continue;
                        char *src = Addr(p.srcBuf, p.srcSlice + i, srcRank);
                        char *dst = Addr(p.dstBuf, p.dstSlice + i, dstRank);
                        if (reduce) CHK_RET(P->ReduceAsync(dst, src, n, a.dtype, a.op, a.stream));
                        else if (src != dst) CHK_RET(P->MemcpyAsync(dst, src, n * esz, a.stream));
                    }
                }
            }
        }
        return HCCL_SUCCESS;
    }
};

}  // namespace

HcclResult ExecuteOnHost(Comm *c, const Schedule &s, const ExecArgs &a)
{
    if (c->rank >= s.ranks.size()) return HCCL_E_INTERNAL;
    uint32_t esz = DtypeSize(a.dtype);
    uint64_t cap = ScratchCapacityElems(c, s, esz);
    if (cap == 0) {
        RPT_ERR("EI0003", "the CCL buffer (%u MB) is too small for %u scratch slots", c->cfg.bufferMB, s.scratch.nSlices);
        return HCCL_E_MEMORY;
    }
    uint64_t maxSlice = 0;
    maxSlice = std::max(maxSlice, s.In(c->rank).sliceCount);
    maxSlice = std::max(maxSlice, s.Out(c->rank).sliceCount);
    // Every rank must loop the same number of times: use the schedule-wide maximum.
    for (auto &L : s.input) maxSlice = std::max(maxSlice, L.sliceCount);
    for (auto &L : s.output) maxSlice = std::max(maxSlice, L.sliceCount);
    uint64_t q = esz >= 16 ? 1 : 16 / esz;
    uint64_t chunk = cap / q * q;
    uint64_t passes = maxSlice == 0 ? 1 : (maxSlice + chunk - 1) / chunk;
    // Collectives alternate between the two CCL halves, pass by pass: every rank runs the same collectives in the same
    // order, so the ranks agree on the half without talking.  A send or receive involves two ranks only and must not
    // advance that count (the ranks would disagree from then on, first of all the two partners when one of them has
    // sent or received more often than the other).  It lands in the half that the next collective will use, which
    // is idle: a rank that has finished collective k knows that every rank has entered k and so has finished k-1.  Its
    // passes need no alternation, each one starts with the receiver's READY.
    const bool pointToPoint = s.cmd == HCCL_CMD_SEND || s.cmd == HCCL_CMD_RECEIVE;
    for (uint64_t pass = 0; pass < passes; ++pass) {
        Walker w{c, s, a, esz, cap, pass * chunk, (pass + 1) * chunk, c->hostLaunches & 1u};
        CHK_RET(w.Run());
        if (!pointToPoint) ++c->hostLaunches;
    }
    return HCCL_SUCCESS;
}

}  // namespace hc
