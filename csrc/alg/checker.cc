#include "checker.h"

#include <algorithm>
#include <map>
#include <sstream>

namespace hc {
namespace {

// Multiset of contributions: key = rank * 65536 + inputSlice.
using Content = std::map<uint32_t, int>;
using Clock = std::vector<uint32_t>;

struct SliceState {
    Content content;
    bool written = false;
    Clock lastWrite;                 // clock of the last write
    int lastWriter = -1;
    std::vector<std::pair<int, Clock>> readsSinceWrite;
};

bool Leq(const Clock &a, const Clock &b)
{
    for (size_t i = 0; i < a.size(); ++i)
        if (a[i] > b[i]) return false;
    return true;
}
void Join(Clock &a, const Clock &b)
{
    for (size_t i = 0; i < a.size(); ++i) a[i] = std::max(a[i], b[i]);
}

struct Sim {
    const Schedule &s;
    const CheckOptions &opt;
    CheckReport rep;
    uint32_t p;
    // memory[rank][buf][slice]
    std::vector<std::vector<std::vector<SliceState>>> mem;
    std::vector<size_t> pc;
    std::vector<Clock> clock;
    // posts[dst][src][notify] = queue of sender clocks
    std::map<uint64_t, std::vector<Clock>> posts;
    std::map<uint64_t, size_t> consumed;

    Sim(const Schedule &sch, const CheckOptions &o) : s(sch), opt(o), p(sch.nRanks) {}

    void Err(const std::string &m)
    {
        rep.ok = false;
        if (rep.errors.size() < 20) rep.errors.push_back(m);
    }
    static uint64_t Key(uint32_t dst, uint32_t src, uint32_t n) { return ((uint64_t)dst << 40) | ((uint64_t)src << 16) | n; }

    SliceState *Loc(uint32_t rank, BufId b, uint32_t slice, const Prim &pr, uint32_t actor)
    {
        if (rank >= p) { Err("rank out of range"); return nullptr; }
        uint32_t bi = (uint32_t)b;
        if (opt.inPlace && b == BufId::INPUT && s.In(rank).nSlices == s.Out(rank).nSlices) bi = (uint32_t)BufId::OUTPUT;
        auto &v = mem[rank][bi];
        if (slice >= v.size()) {
            std::ostringstream os;
            os << s.name << ": rank " << actor << " step " << (int)pr.step << " " << PrimOpName(pr.op) << " addresses slice " << slice
               << " of buffer " << (int)b << " on rank " << rank << " which has " << v.size();
            Err(os.str());
            return nullptr;
        }
        return &v[slice];
    }

    uint64_t LenOf(uint32_t rank, const Prim &pr, uint32_t i) const
    {
        switch (pr.lenBuf) {
            case BufId::INPUT: return s.In(rank).CountOf(pr.lenSlice + i);
            case BufId::OUTPUT: return s.Out(rank).CountOf(pr.lenSlice + i);
            case BufId::SCRATCH: return s.scratch.CountOf(pr.lenSlice + i);
            default: return 0;
        }
    }
    uint64_t CapOf(uint32_t rank, BufId b, uint32_t slice) const
    {
        switch (b) {
            case BufId::INPUT: return s.In(rank).CountOf(slice);
            case BufId::OUTPUT: return s.Out(rank).CountOf(slice);
            case BufId::SCRATCH: return s.scratch.sliceCount;
            default: return 0;
        }
    }

    void Access(SliceState *st, bool isWrite, uint32_t actor, const Prim &pr, const char *what)
    {
        if (!opt.checkRaces || !st) return;
        const Clock &c = clock[actor];
        if (st->written && st->lastWriter != (int)actor && !Leq(st->lastWrite, c)) {
            std::ostringstream os;
            os << s.name << ": memory conflict: rank " << actor << " step " << (int)pr.step << " " << PrimOpName(pr.op) << " " << what
               << " a slice last written by rank " << st->lastWriter << " without an ordering notify";
            Err(os.str());
        }
        if (isWrite) {
            for (auto &rd : st->readsSinceWrite) {
                if (rd.first != (int)actor && !Leq(rd.second, c)) {
                    std::ostringstream os;
                    os << s.name << ": memory conflict: rank " << actor << " step " << (int)pr.step << " " << PrimOpName(pr.op)
                       << " overwrites a slice that rank " << rd.first << " may still be reading";
                    Err(os.str());
                    break;
                }
            }
            st->written = true;
            st->lastWrite = c;
            st->lastWriter = (int)actor;
            st->readsSinceWrite.clear();
        } else {
            st->readsSinceWrite.push_back({(int)actor, c});
        }
    }

    // Returns true when the primitive executed (false = blocked on a wait).
    bool Step(uint32_t r)
    {
        const Prim &pr = s.ranks[r].prims[pc[r]];
        clock[r][r]++;
        rep.maxStep = std::max<uint32_t>(rep.maxStep, pr.step);
        switch (pr.op) {
            case PrimOp::POST: {
                if (pr.peer < 0 || (uint32_t)pr.peer >= p) { Err(s.name + ": POST to a rank outside the communicator"); break; }
                posts[Key((uint32_t)pr.peer, r, pr.notify)].push_back(clock[r]);
                break;
            }
            case PrimOp::WAIT: {
                if (pr.peer < 0 || (uint32_t)pr.peer >= p) { Err(s.name + ": WAIT on a rank outside the communicator"); break; }
                uint64_t k = Key(r, (uint32_t)pr.peer, pr.notify);
                auto &q = posts[k];
                size_t &c = consumed[k];
                if (c >= q.size()) { clock[r][r]--; return false; }
                Join(clock[r], q[c]);
                ++c;
                break;
            }
            case PrimOp::NOP: break;
            default: {
                bool remoteDst = pr.op == PrimOp::WRITE || pr.op == PrimOp::WRITE_REDUCE;
                bool remoteSrc = pr.op == PrimOp::READ || pr.op == PrimOp::READ_REDUCE;
                bool reduce = pr.op == PrimOp::REDUCE || pr.op == PrimOp::WRITE_REDUCE || pr.op == PrimOp::READ_REDUCE;
                if ((remoteDst || remoteSrc) && (pr.peer < 0 || (uint32_t)pr.peer >= p)) { Err(s.name + ": transfer names a rank outside the communicator"); break; }
                uint32_t srcRank = remoteSrc ? (uint32_t)pr.peer : r, dstRank = remoteDst ? (uint32_t)pr.peer : r;
                if (remoteDst && pr.dstBuf != BufId::SCRATCH) Err(s.name + ": remote WRITE must target the peer's scratch");
                if (remoteSrc && pr.srcBuf != BufId::SCRATCH) Err(s.name + ": remote READ must source the peer's scratch");
                for (uint32_t i = 0; i < pr.nSlices; ++i) {
                    SliceState *src = Loc(srcRank, pr.srcBuf, pr.srcSlice + i, pr, r);
                    SliceState *dst = Loc(dstRank, pr.dstBuf, pr.dstSlice + i, pr, r);
                    if (!src || !dst) continue;
                    uint64_t len = LenOf(r, pr, i);
                    if (len > CapOf(srcRank, pr.srcBuf, pr.srcSlice + i) || len > CapOf(dstRank, pr.dstBuf, pr.dstSlice + i)) {
                        std::ostringstream os;
                        os << s.name << ": rank " << r << " step " << (int)pr.step << " moves " << len << " elements through a slice that holds fewer";
                        Err(os.str());
                    }
                    if (len == 0) continue;
                    Access(src, false, r, pr, "reads");
                    Access(dst, true, r, pr, "writes");
                    if (!src->written && pr.srcBuf != BufId::INPUT && !(opt.inPlace && pr.srcBuf == BufId::OUTPUT)) {
                        std::ostringstream os;
                        os << s.name << ": rank " << r << " step " << (int)pr.step << " " << PrimOpName(pr.op) << " reads a slice nobody has written";
                        Err(os.str());
                    }
                    if (reduce) {
                        for (auto &kv : src->content) dst->content[kv.first] += kv.second;
                    } else if (src != dst) {
                        dst->content = src->content;
                    }
                }
            }
        }
        ++pc[r];
        ++rep.primsExecuted;
        return true;
    }

    void Run()
    {
        mem.assign(p, std::vector<std::vector<SliceState>>(3));
        for (uint32_t r = 0; r < p; ++r) {
            mem[r][0].resize(s.In(r).nSlices);
            mem[r][1].resize(s.Out(r).nSlices);
            mem[r][2].resize(s.scratch.nSlices);
            for (uint32_t i = 0; i < s.In(r).nSlices; ++i) {
                mem[r][0][i].content[r * 65536u + i] = 1;
                mem[r][0][i].written = true;
                mem[r][0][i].lastWrite.assign(p, 0);
                mem[r][0][i].lastWriter = (int)r;
            }
            if (opt.inPlace && s.In(r).nSlices == s.Out(r).nSlices) mem[r][1] = mem[r][0];
        }
        pc.assign(p, 0);
        clock.assign(p, Clock(p, 0));
        for (;;) {
            bool progress = false, pending = false;
            for (uint32_t r = 0; r < p; ++r) {
                while (pc[r] < s.ranks[r].prims.size()) {
                    if (!Step(r)) break;
                    progress = true;
                }
                if (pc[r] < s.ranks[r].prims.size()) pending = true;
            }
            if (!pending) break;
            if (!progress) {
                std::ostringstream os;
                os << s.name << ": deadlock;";
                for (uint32_t r = 0; r < p; ++r)
                    if (pc[r] < s.ranks[r].prims.size()) {
                        const Prim &pr = s.ranks[r].prims[pc[r]];
                        os << " rank " << r << " waits for rank " << pr.peer << " notify " << pr.notify << " at step " << (int)pr.step << ";";
                    }
                Err(os.str());
                return;
            }
        }
        for (auto &kv : posts) {
            size_t c = consumed.count(kv.first) ? consumed[kv.first] : 0;
            if (c != kv.second.size()) {
                std::ostringstream os;
                os << s.name << ": notify imbalance: rank " << (kv.first >> 40) << " got " << kv.second.size() << " posts from rank "
                   << ((kv.first >> 16) & 0xffffff) << " on slot " << (kv.first & 0xffff) << " but waited " << c << " times";
                Err(os.str());
            }
        }
        Semantics();
    }

    bool Expect(uint32_t r, uint32_t outSlice, const Content &want, const char *what)
    {
        uint32_t bi = (uint32_t)BufId::OUTPUT;
        if (outSlice >= mem[r][bi].size()) { Err(s.name + ": output slice missing"); return false; }
        if (s.Out(r).CountOf(outSlice) == 0) return true;
        if (mem[r][bi][outSlice].content != want) {
            std::ostringstream os;
            os << s.name << ": semantics: rank " << r << " output slice " << outSlice << " does not hold " << what << " (holds";
            for (auto &kv : mem[r][bi][outSlice].content) os << " r" << (kv.first >> 16) << ".s" << (kv.first & 0xffff) << "x" << kv.second;
            os << ")";
            Err(os.str());
            return false;
        }
        return true;
    }

    void Semantics()
    {
        if (!rep.ok) return;
        switch (s.cmd) {
            case HCCL_CMD_ALLREDUCE:
                for (uint32_t r = 0; r < p; ++r)
                    for (uint32_t i = 0; i < s.Out(r).nSlices; ++i) {
                        Content w;
                        for (uint32_t q = 0; q < p; ++q) w[q * 65536u + i] = 1;
                        if (!Expect(r, i, w, "the sum over all ranks")) return;
                    }
                break;
            case HCCL_CMD_REDUCE_SCATTER: case HCCL_CMD_REDUCE_SCATTER_V:
                for (uint32_t r = 0; r < p; ++r) {
                    Content w;
                    for (uint32_t q = 0; q < p; ++q) w[q * 65536u + r] = 1;
                    if (!Expect(r, 0, w, "the sum of everyone's slice r")) return;
                }
                break;
            case HCCL_CMD_ALLGATHER: case HCCL_CMD_ALLGATHER_V:
                for (uint32_t r = 0; r < p; ++r)
                    for (uint32_t q = 0; q < p; ++q) {
                        Content w; w[q * 65536u + 0] = 1;
                        if (!Expect(r, q, w, "rank q's input")) return;
                    }
                break;
            case HCCL_CMD_ALLTOALL: case HCCL_CMD_ALLTOALLV: case HCCL_CMD_ALLTOALLVC:
                for (uint32_t r = 0; r < p; ++r)
                    for (uint32_t q = 0; q < p; ++q) {
                        Content w; w[q * 65536u + r] = 1;
                        if (!Expect(r, q, w, "slice r of rank q's input")) return;
                    }
                break;
            case HCCL_CMD_BROADCAST:
                for (uint32_t r = 0; r < p; ++r)
                    for (uint32_t i = 0; i < s.Out(r).nSlices; ++i) {
                        Content w; w[s.root * 65536u + i] = 1;
                        if (!Expect(r, i, w, "the root's data")) return;
                    }
                break;
            case HCCL_CMD_REDUCE:
                for (uint32_t i = 0; i < s.Out(s.root).nSlices; ++i) {
                    Content w;
                    for (uint32_t q = 0; q < p; ++q) w[q * 65536u + i] = 1;
                    if (!Expect(s.root, i, w, "the sum over all ranks")) return;
                }
                break;
            case HCCL_CMD_SCATTER:
                for (uint32_t r = 0; r < p; ++r) {
                    Content w; w[s.root * 65536u + r] = 1;
                    if (!Expect(r, 0, w, "slice r of the root's input")) return;
                }
                break;
            case HCCL_CMD_GATHER:
                for (uint32_t q = 0; q < p; ++q) {
                    Content w; w[q * 65536u + 0] = 1;
                    if (!Expect(s.root, q, w, "rank q's input")) return;
                }
                break;
            default: break;
        }
    }
};

}  // namespace

std::string CheckReport::Summary() const
{
    std::ostringstream os;
    os << (ok ? "OK" : "FAILED") << " prims=" << primsExecuted << " steps=" << maxStep;
    for (auto &e : errors) os << "\n  " << e;
    return os.str();
}

CheckReport CheckSchedule(const Schedule &s, const CheckOptions &opt)
{
    Sim sim(s, opt);
    if (s.ranks.size() != s.nRanks) {
        sim.rep.ok = false;
        sim.rep.errors.push_back("schedule lacks a program for every rank");
        return sim.rep;
    }
    sim.Run();
    return sim.rep;
}

}  // namespace hc
