#include "templates.h"

#include <algorithm>
#include <sstream>

namespace hc {

const char *PrimOpName(PrimOp op)
{
    static const char *n[] = {"COPY", "REDUCE", "WRITE", "WRITE_REDUCE", "READ", "READ_REDUCE", "POST", "WAIT", "NOP"};
    return n[(int)op];
}

const char *AlgoName(Algo a)
{
    switch (a) {
        case Algo::AUTO: return "auto"; case Algo::MESH: return "mesh"; case Algo::MESH_ONESHOT: return "mesh_oneshot";
        case Algo::RING: return "ring"; case Algo::HD: return "H-D_R"; case Algo::BRUCK: return "NB";
        case Algo::PAIRWISE: return "pairwise"; case Algo::TREE: return "tree"; case Algo::NVLS: return "nvls";
        case Algo::STAR: return "star";
        case Algo::NHR: return "NHR";
    }
    return "?";
}

bool ParseAlgoName(const std::string &raw, Algo *out)
{
    std::string s;
    for (char c : raw) s += (char)tolower((unsigned char)c);
    if (s == "ring") *out = Algo::RING;
    else if (s == "fullmesh" || s == "mesh" || s == "pipeline") *out = Algo::MESH;
    else if (s == "mesh_oneshot" || s == "oneshot") *out = Algo::MESH_ONESHOT;
    else if (s == "h-d_r" || s == "hd" || s == "rhd" || s == "ahc" || s == "ahc_broke") *out = Algo::HD;
    else if (s == "nhr" || s == "nhr_v1") *out = Algo::NHR;
    else if (s == "nb" || s == "bruck") *out = Algo::BRUCK;
    else if (s == "pairwise") *out = Algo::PAIRWISE;
    else if (s == "tree") *out = Algo::TREE;
    else if (s == "star") *out = Algo::STAR;
    else if (s == "nvls") *out = Algo::NVLS;
    else if (s == "null" || s == "na" || s == "auto" || s.empty()) *out = Algo::AUTO;
    else return false;
    return true;
}

uint64_t AlignedSliceCount(uint64_t total, uint32_t nSlices, uint32_t elemSize)
{
    if (nSlices == 0) return 0;
    uint64_t per = (total + nSlices - 1) / nSlices;
    uint64_t q = elemSize >= 16 ? 1 : 16 / elemSize;   // elements per 16 bytes
    return (per + q - 1) / q * q;
}

std::string Schedule::Dump(uint32_t rank) const
{
    std::ostringstream os;
    os << name << " rank " << rank << "/" << nRanks << "\n";
    if (rank >= ranks.size()) return os.str();
    static const char *bn[] = {"IN", "OUT", "SCR", "-"};
    for (auto &p : ranks[rank].prims) {
        os << "  s" << (int)p.step << " t" << (int)p.thread << " " << PrimOpName(p.op);
        if (p.op == PrimOp::POST || p.op == PrimOp::WAIT) os << " peer=" << p.peer << " n=" << p.notify;
        else {
            os << " " << bn[(int)p.srcBuf] << "[" << p.srcSlice << "]->" << bn[(int)p.dstBuf] << "[" << p.dstSlice << "] x" << p.nSlices;
            if (p.peer >= 0) os << " peer=" << p.peer;
        }
        os << "\n";
    }
    return os.str();
}

size_t Schedule::TotalPrims() const
{
    size_t n = 0;
    for (auto &r : ranks) n += r.prims.size();
    return n;
}

namespace {

// Emits the primitives of one rank.
struct Emit {
    RankProgram &prog;
    uint8_t step = 0;
    explicit Emit(RankProgram &p) : prog(p) {}
    void Data(PrimOp op, int peer, BufId sb, uint32_t ss, BufId db, uint32_t ds, uint32_t n, BufId lb, uint32_t ls)
    {
        if (n == 0) return;
        Prim p;
        p.op = op; p.peer = (int16_t)peer; p.srcBuf = sb; p.srcSlice = ss; p.dstBuf = db; p.dstSlice = ds; p.nSlices = n;
        p.lenBuf = lb; p.lenSlice = ls; p.step = step;
        prog.prims.push_back(p);
    }
    void Copy(BufId sb, uint32_t ss, BufId db, uint32_t ds, uint32_t n, BufId lb, uint32_t ls) { Data(PrimOp::COPY, -1, sb, ss, db, ds, n, lb, ls); }
    void Reduce(BufId sb, uint32_t ss, BufId db, uint32_t ds, uint32_t n, BufId lb, uint32_t ls) { Data(PrimOp::REDUCE, -1, sb, ss, db, ds, n, lb, ls); }
    void Write(int peer, BufId sb, uint32_t ss, uint32_t ds, uint32_t n, BufId lb, uint32_t ls) { Data(PrimOp::WRITE, peer, sb, ss, BufId::SCRATCH, ds, n, lb, ls); }
    void Read(int peer, uint32_t ss, BufId db, uint32_t ds, uint32_t n, BufId lb, uint32_t ls) { Data(PrimOp::READ, peer, BufId::SCRATCH, ss, db, ds, n, lb, ls); }
    void Sync(PrimOp op, int peer, uint16_t notify)
    {
        Prim p;
        p.op = op; p.peer = (int16_t)peer; p.notify = notify; p.step = step;
        prog.prims.push_back(p);
    }
    void Post(int peer, uint16_t n) { Sync(PrimOp::POST, peer, n); }
    void Wait(int peer, uint16_t n) { Sync(PrimOp::WAIT, peer, n); }
};

constexpr BufId IN = BufId::INPUT, OUT = BufId::OUTPUT, SCR = BufId::SCRATCH;

void Uniform(SliceLayout &L, uint32_t n, uint64_t total, uint32_t esz)
{
    L.nSlices = n; L.sliceCount = AlignedSliceCount(total, n, esz); L.total = total; L.displ.clear(); L.count.clear();
}
void Fixed(SliceLayout &L, uint32_t n, uint64_t per)
{
    L.nSlices = n; L.sliceCount = per; L.total = (uint64_t)n * per; L.displ.clear(); L.count.clear();
}
void Explicit(SliceLayout &L, const std::vector<uint64_t> &cnt, const std::vector<uint64_t> &dsp)
{
    L.nSlices = (uint32_t)cnt.size(); L.count = cnt; L.displ = dsp; L.sliceCount = 0; L.total = 0;
    for (size_t i = 0; i < cnt.size(); ++i) { L.sliceCount = std::max(L.sliceCount, cnt[i]); L.total = std::max(L.total, dsp[i] + cnt[i]); }
}
uint64_t MaxSlice(const Schedule &s)
{
    uint64_t m = 0;
    for (auto &L : s.input) m = std::max(m, L.sliceCount);
    for (auto &L : s.output) m = std::max(m, L.sliceCount);
    return m;
}
void FinishScratch(Schedule &s, uint32_t nSlices, uint32_t esz)
{
    uint64_t per = MaxSlice(s);
    uint64_t q = esz >= 16 ? 1 : 16 / esz;
    per = (per + q - 1) / q * q;
    s.scratch.nSlices = nSlices; s.scratch.sliceCount = per; s.scratch.total = per * nSlices;
}
uint32_t FloorPow2(uint32_t p) { uint32_t b = 1; while (b * 2 <= p) b *= 2; return b; }
uint32_t Log2(uint32_t b) { uint32_t l = 0; while ((1u << l) < b) ++l; return l; }
bool WantRank(const CollShape &sh, uint32_t r) { return sh.onlyRank < 0 || (uint32_t)sh.onlyRank == r; }

// ------------------------------------------------------------------------------------ AllReduce

void AllReduceOneShot(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks;
    s.name = "AllReduceMeshOneShot";
    s.input.resize(1); s.output.resize(1);
    Fixed(s.input[0], 1, sh.count); Fixed(s.output[0], 1, sh.count);
    FinishScratch(s, p, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        for (uint32_t i = 1; i < p; ++i) e.Post((r + i) % p, N_READY);
        e.Copy(IN, 0, SCR, r, 1, IN, 0);
        e.step = 1;
        for (uint32_t i = 1; i < p; ++i) {
            uint32_t q = (r + i) % p;
            e.Wait(q, N_READY); e.Write(q, IN, 0, r, 1, IN, 0); e.Post(q, N_DATA);
        }
        e.step = 2;
        for (uint32_t i = 1; i < p; ++i) e.Wait((r + i) % p, N_DATA);
        e.Copy(SCR, 0, OUT, 0, 1, OUT, 0);
        for (uint32_t i = 1; i < p; ++i) e.Reduce(SCR, i, OUT, 0, 1, OUT, 0);
    }
}

void AllReduceTwoShot(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks;
    s.name = "AllReduceMeshTwoShot";
    s.input.resize(1); s.output.resize(1);
    Uniform(s.input[0], p, sh.count, sh.elemSize); Uniform(s.output[0], p, sh.count, sh.elemSize);
    FinishScratch(s, p + 1, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        for (uint32_t i = 1; i < p; ++i) e.Post((r + i) % p, N_READY);
        e.Copy(IN, r, SCR, r, 1, IN, r);
        e.step = 1;   // scatter my contributions
        for (uint32_t i = 1; i < p; ++i) {
            uint32_t q = (r + i) % p;
            e.Wait(q, N_READY); e.Write(q, IN, q, r, 1, IN, q); e.Post(q, N_DATA);
        }
        e.step = 2;   // reduce my slice in rank order
        for (uint32_t i = 1; i < p; ++i) e.Wait((r + i) % p, N_DATA);
        e.Copy(SCR, 0, SCR, p, 1, OUT, r);
        for (uint32_t i = 1; i < p; ++i) e.Reduce(SCR, i, SCR, p, 1, OUT, r);
        e.Copy(SCR, p, OUT, r, 1, OUT, r);
        for (uint32_t i = 1; i < p; ++i) e.Post((r + i) % p, N_FIN);
        e.step = 3;   // gather the other slices by reading them where they were reduced
        for (uint32_t i = 1; i < p; ++i) {
            uint32_t q = (r + i) % p;
            e.Wait(q, N_FIN); e.Read(q, p, OUT, q, 1, OUT, q); e.Post(q, N_DONE);
        }
        for (uint32_t i = 1; i < p; ++i) e.Wait((r + i) % p, N_DONE);
    }
}

void AllReduceRing(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks;
    s.name = "AllReduceRing";
    s.input.resize(1); s.output.resize(1);
    Uniform(s.input[0], p, sh.count, sh.elemSize); Uniform(s.output[0], p, sh.count, sh.elemSize);
    FinishScratch(s, 2 * (p - 1) + 1, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        uint32_t R = (r + 1) % p, L = (r + p - 1) % p;
        e.Copy(IN, 0, OUT, 0, p, OUT, 0);
        if (p == 1) continue;
        e.Post(L, N_READY);
        e.Wait(R, N_READY);
        for (uint32_t st = 0; st + 1 < p; ++st) {   // reduce-scatter half
            e.step = (uint8_t)(1 + st);
            uint32_t sendIdx = (r + p - st) % p, recvIdx = (r + 2 * p - st - 1) % p;
            e.Write(R, OUT, sendIdx, st, 1, OUT, sendIdx); e.Post(R, N_DATA);
            e.Wait(L, N_DATA); e.Reduce(SCR, st, OUT, recvIdx, 1, OUT, recvIdx);
        }
        for (uint32_t st = 0; st + 1 < p; ++st) {   // all-gather half
            e.step = (uint8_t)(p + st);
            uint32_t sendIdx = (r + 1 + p - st) % p, recvIdx = (r + p - st) % p;
            e.Write(R, OUT, sendIdx, p - 1 + st, 1, OUT, sendIdx); e.Post(R, N_DATA);
            e.Wait(L, N_DATA); e.Copy(SCR, p - 1 + st, OUT, recvIdx, 1, OUT, recvIdx);
        }
    }
}

// Recursive halving then doubling over `block` = largest power of two <= p virtual ranks; the
// 2*(p-block) lowest ranks are folded in pairs: the odd member ships its whole vector to the even
// one before the exchange and receives the result afterwards.
void AllReduceHD(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks, block = FloorPow2(p), extra = p - block, lg = Log2(block), nS = block;
    s.name = "AllReduceRecursiveHD";
    s.input.resize(1); s.output.resize(1);
    Uniform(s.input[0], nS, sh.count, sh.elemSize); Uniform(s.output[0], nS, sh.count, sh.elemSize);
    FinishScratch(s, 3 * nS, sh.elemSize);
    auto real = [&](uint32_t v) { return v < extra ? 2 * v : v + extra; };
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        bool folded = r < 2 * extra;
        if (folded && (r & 1)) {   // passive member of a folded pair
            uint32_t buddy = r - 1;
            e.Post(buddy, N_READY);
            e.Wait(buddy, N_READY); e.Write(buddy, IN, 0, 0, nS, IN, 0); e.Post(buddy, N_DATA);
            e.step = (uint8_t)(2 * lg + 2);
            e.Wait(buddy, N_DATA); e.Copy(SCR, 0, OUT, 0, nS, OUT, 0);
            continue;
        }
        uint32_t v = folded ? r / 2 : r - extra;
        e.Copy(IN, 0, OUT, 0, nS, OUT, 0);
        for (uint32_t k = 0; k < lg; ++k) e.Post(real(v ^ (block >> (k + 1))), N_READY);
        if (folded) {
            uint32_t buddy = r + 1;
            e.Post(buddy, N_READY); e.Wait(buddy, N_DATA); e.Reduce(SCR, 0, OUT, 0, nS, OUT, 0);
        }
        uint32_t lo = 0, len = nS;
        for (uint32_t k = 0; k < lg; ++k) {
            e.step = (uint8_t)(1 + k);
            uint32_t d = block >> (k + 1), partner = real(v ^ d), half = len / 2;
            uint32_t keepLo = (v & d) ? lo + half : lo, sendLo = (v & d) ? lo : lo + half;
            uint32_t base = nS + (nS - (nS >> k));
            e.Wait(partner, N_READY);
            e.Write(partner, OUT, sendLo, base, half, OUT, sendLo); e.Post(partner, N_DATA);
            e.Wait(partner, N_DATA); e.Reduce(SCR, base, OUT, keepLo, half, OUT, keepLo);
            lo = keepLo; len = half;
        }
        for (int k = (int)lg - 1; k >= 0; --k) {
            e.step = (uint8_t)(1 + lg + (lg - 1 - k));
            uint32_t d = block >> (k + 1), partner = real(v ^ d);
            uint32_t other = lo ^ len, base = 2 * nS + (nS - (nS >> k));
            e.Write(partner, OUT, lo, base, len, OUT, lo); e.Post(partner, N_DATA);
            e.Wait(partner, N_DATA); e.Copy(SCR, base, OUT, other, len, OUT, other);
            lo = std::min(lo, other); len *= 2;
        }
        if (folded) {
            uint32_t buddy = r + 1;
            e.step = (uint8_t)(2 * lg + 1);
            e.Wait(buddy, N_READY); e.Write(buddy, OUT, 0, 0, nS, OUT, 0); e.Post(buddy, N_DATA);
        }
    }
}

// -------------------------------------------------------------------------------- ReduceScatter

void SetRsLayouts(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks;
    if (!sh.sendCounts.empty()) {   // ReduceScatterV: same counts on every rank
        s.input.resize(1); s.output.resize(p);
        Explicit(s.input[0], sh.sendCounts[0], sh.sendDispls[0]);
        for (uint32_t r = 0; r < p; ++r) Explicit(s.output[r], {sh.sendCounts[0][r]}, {0});
    } else {
        s.input.resize(1); s.output.resize(1);
        Fixed(s.input[0], p, sh.count); Fixed(s.output[0], 1, sh.count);
    }
}

void ReduceScatterMesh(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks;
    s.name = "ReduceScatterMesh";
    SetRsLayouts(sh, s);
    FinishScratch(s, p, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        for (uint32_t i = 1; i < p; ++i) e.Post((r + i) % p, N_READY);
        e.Copy(IN, r, SCR, r, 1, IN, r);
        e.step = 1;
        for (uint32_t i = 1; i < p; ++i) {
            uint32_t q = (r + i) % p;
            e.Wait(q, N_READY); e.Write(q, IN, q, r, 1, IN, q); e.Post(q, N_DATA);
        }
        e.step = 2;
        for (uint32_t i = 1; i < p; ++i) e.Wait((r + i) % p, N_DATA);
        e.Copy(SCR, 0, OUT, 0, 1, OUT, 0);
        for (uint32_t i = 1; i < p; ++i) e.Reduce(SCR, i, OUT, 0, 1, OUT, 0);
    }
}

void ReduceScatterRing(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks;
    s.name = "ReduceScatterRing";
    SetRsLayouts(sh, s);
    FinishScratch(s, p, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        if (p == 1) { e.Copy(IN, 0, OUT, 0, 1, OUT, 0); continue; }
        uint32_t R = (r + 1) % p, L = (r + p - 1) % p;
        e.Post(L, N_READY);
        e.Wait(R, N_READY);
        for (uint32_t st = 0; st + 1 < p; ++st) {
            e.step = (uint8_t)(1 + st);
            uint32_t sendIdx = (r + 2 * p - 1 - st) % p, recvIdx = (r + 2 * p - 2 - st) % p;
            if (st == 0) e.Write(R, IN, sendIdx, 0, 1, IN, sendIdx);
            else e.Write(R, SCR, st - 1, st, 1, IN, sendIdx);
            e.Post(R, N_DATA);
            e.Wait(L, N_DATA); e.Reduce(IN, recvIdx, SCR, st, 1, IN, recvIdx);
        }
        e.Copy(SCR, p - 2, OUT, 0, 1, OUT, 0);
    }
}

bool ReduceScatterHD(const CollShape &sh, Schedule &s, std::string *why)
{
    uint32_t p = sh.nRanks;
    if (FloorPow2(p) != p) { if (why) *why = "halving-doubling reduce-scatter needs a power-of-two rank count"; return false; }
    if (!sh.sendCounts.empty()) { if (why) *why = "halving-doubling does not serve variable counts"; return false; }
    uint32_t lg = Log2(p);
    s.name = "ReduceScatterRecursiveHD";
    SetRsLayouts(sh, s);
    FinishScratch(s, 2 * p, sh.elemSize);   // [0,p) working copy, [p,2p) receive regions
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        for (uint32_t k = 0; k < lg; ++k) e.Post(r ^ (p >> (k + 1)), N_READY);
        e.Copy(IN, 0, SCR, 0, p, IN, 0);
        uint32_t lo = 0, len = p;
        for (uint32_t k = 0; k < lg; ++k) {
            e.step = (uint8_t)(1 + k);
            uint32_t d = p >> (k + 1), partner = r ^ d, half = len / 2;
            uint32_t keepLo = (r & d) ? lo + half : lo, sendLo = (r & d) ? lo : lo + half;
            uint32_t base = p + (p - (p >> k));
            e.Wait(partner, N_READY);
            e.Write(partner, SCR, sendLo, base, half, IN, sendLo); e.Post(partner, N_DATA);
            e.Wait(partner, N_DATA); e.Reduce(SCR, base, SCR, keepLo, half, IN, keepLo);
            lo = keepLo; len = half;
        }
        e.Copy(SCR, r, OUT, 0, 1, OUT, 0);
    }
    return true;
}

// ------------------------------------------------------------------------------------ AllGather

void SetAgLayouts(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks;
    if (!sh.recvCounts.empty()) {   // AllGatherV
        s.input.resize(p); s.output.resize(1);
        Explicit(s.output[0], sh.recvCounts[0], sh.recvDispls[0]);
        for (uint32_t r = 0; r < p; ++r) Explicit(s.input[r], {sh.recvCounts[0][r]}, {0});
    } else {
        s.input.resize(1); s.output.resize(1);
        Fixed(s.input[0], 1, sh.count); Fixed(s.output[0], p, sh.count);
    }
}

void AllGatherMesh(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks;
    s.name = "AllGatherMesh";
    SetAgLayouts(sh, s);
    FinishScratch(s, p, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        for (uint32_t i = 1; i < p; ++i) e.Post((r + i) % p, N_READY);
        e.Copy(IN, 0, OUT, r, 1, OUT, r);
        e.step = 1;
        for (uint32_t i = 1; i < p; ++i) {
            uint32_t q = (r + i) % p;
            e.Wait(q, N_READY); e.Write(q, IN, 0, r, 1, OUT, r); e.Post(q, N_DATA);
        }
        e.step = 2;
        for (uint32_t i = 1; i < p; ++i) {
            uint32_t q = (r + p - i) % p;
            e.Wait(q, N_DATA); e.Copy(SCR, q, OUT, q, 1, OUT, q);
        }
    }
}

void AllGatherRing(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks;
    s.name = "AllGatherRing";
    SetAgLayouts(sh, s);
    FinishScratch(s, p, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        e.Copy(IN, 0, OUT, r, 1, OUT, r);
        if (p == 1) continue;
        uint32_t R = (r + 1) % p, L = (r + p - 1) % p;
        e.Post(L, N_READY);
        e.Wait(R, N_READY);
        for (uint32_t st = 0; st + 1 < p; ++st) {
            e.step = (uint8_t)(1 + st);
            uint32_t sendIdx = (r + p - st) % p, recvIdx = (r + 2 * p - st - 1) % p;
            e.Write(R, OUT, sendIdx, st, 1, OUT, sendIdx); e.Post(R, N_DATA);
            e.Wait(L, N_DATA); e.Copy(SCR, st, OUT, recvIdx, 1, OUT, recvIdx);
        }
    }
}

bool AllGatherHD(const CollShape &sh, Schedule &s, std::string *why)
{
    uint32_t p = sh.nRanks;
    if (FloorPow2(p) != p) { if (why) *why = "recursive-doubling all-gather needs a power-of-two rank count (use NB)"; return false; }
    uint32_t lg = Log2(p);
    s.name = "AllGatherRecursiveHD";
    SetAgLayouts(sh, s);
    FinishScratch(s, p, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        for (uint32_t k = 0; k < lg; ++k) e.Post(r ^ (1u << k), N_READY);
        e.Copy(IN, 0, OUT, r, 1, OUT, r);
        for (uint32_t k = 0; k < lg; ++k) {
            e.step = (uint8_t)(1 + k);
            uint32_t d = 1u << k, partner = r ^ d, lo = r & ~(d - 1), other = lo ^ d, base = d - 1;
            e.Wait(partner, N_READY);
            e.Write(partner, OUT, lo, base, d, OUT, lo); e.Post(partner, N_DATA);
            e.Wait(partner, N_DATA); e.Copy(SCR, base, OUT, other, d, OUT, other);
        }
    }
    return true;
}

// Bruck: scratch slot j of rank r holds the block of rank (r+j) mod p; step k ships the first
// min(2^k, p-2^k) slots to rank r-2^k, which stores them from slot 2^k on.
void AllGatherBruck(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks;
    s.name = "AllGatherBruck";
    SetAgLayouts(sh, s);
    FinishScratch(s, p, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        for (uint32_t d = 1; d < p; d *= 2) e.Post((r + d) % p, N_READY);
        e.Copy(IN, 0, SCR, 0, 1, OUT, r);
        uint8_t st = 1;
        for (uint32_t d = 1; d < p; d *= 2, ++st) {
            e.step = st;
            uint32_t cnt = std::min(d, p - d), dst = (r + p - d) % p, src = (r + d) % p;
            e.Wait(dst, N_READY);
            for (uint32_t j = 0; j < cnt; ++j) e.Write(dst, SCR, j, d + j, 1, OUT, (r + j) % p);
            e.Post(dst, N_DATA);
            e.Wait(src, N_DATA);
        }
        for (uint32_t j = 0; j < p; ++j) e.Copy(SCR, j, OUT, (r + j) % p, 1, OUT, (r + j) % p);
    }
}

// ------------------------------------------------------------------------------------------ NHR
//
// Non-uniform hierarchical ring (reference: alg_template/nonuniform_hierarchical_ring_base.cc:20-62 and the step tables
// of temp_reduce_scatter/reduce_scatter_nhr.cc:552-590, temp_all_gather/all_gather_nhr.cc:228-260): a ring walked in
// ceil(log2 p) steps of doubling distance that works for ANY rank count.  Reduce-scatter step k (distance d = 2^k):
// rank r sends to r - d the partial sums of the slices  r - d, r - d - 2d, r - d - 4d, ...  (floor((p - 1 + d) / 2d)
// of them) and receives from r + d the slices  r, r - 2d, r - 4d, ...  which it adds to its own partials; after the last
// step slice r is complete on rank r.  All-gather runs the same steps backwards with the roles of the two lists swapped.
uint32_t NhrSteps(uint32_t p) { uint32_t k = 0; while ((1u << k) < p) ++k; return k; }
void NhrSlices(uint32_t p, uint32_t r, uint32_t k, std::vector<uint32_t> *sent, std::vector<uint32_t> *received)
{
    const uint32_t d = 1u << k, n = (p - 1 + d) / (2 * d);
    sent->clear(); received->clear();
    for (uint32_t i = 0; i < n; ++i) {
        const uint64_t back = (uint64_t)i * 2 * d;
        sent->push_back((uint32_t)(((uint64_t)r + (uint64_t)p * (back / p + 2) - d - back) % p));
        received->push_back((uint32_t)(((uint64_t)r + (uint64_t)p * (back / p + 2) - back) % p));
    }
}

// Reduce-scatter on accumulators in scratch: slots [0, p) hold this rank's partial sum of every block, slots from p
// on receive (a fresh range per step, so nothing is reused inside one call).
void ReduceScatterNhr(const CollShape &sh, Schedule &s)
{
    const uint32_t p = sh.nRanks, steps = NhrSteps(p);
    s.name = "ReduceScatterNHR";
    SetRsLayouts(sh, s);
    FinishScratch(s, 2 * p, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        if (p == 1) { e.Copy(IN, 0, OUT, 0, 1, OUT, 0); continue; }
        for (uint32_t k = 0; k < steps; ++k) e.Post((r + (1u << k)) % p, N_READY);        // to the ranks that will write into my scratch
        e.Copy(IN, 0, SCR, 0, p, IN, 0);
        uint32_t slot = p;
        std::vector<uint32_t> tx, rx;
        for (uint32_t k = 0; k < steps; ++k) {
            e.step = (uint8_t)(1 + k);
            const uint32_t d = 1u << k, to = (r + p - d % p) % p, from = (r + d) % p;
            NhrSlices(p, r, k, &tx, &rx);
            e.Wait(to, N_READY);
            for (uint32_t i = 0; i < tx.size(); ++i) e.Write(to, SCR, tx[i], slot + i, 1, IN, tx[i]);
            e.Post(to, N_DATA);
            e.Wait(from, N_DATA);
            for (uint32_t i = 0; i < rx.size(); ++i) e.Reduce(SCR, slot + i, SCR, rx[i], 1, IN, rx[i]);
            slot += (uint32_t)tx.size();
        }
        e.Copy(SCR, r, OUT, 0, 1, OUT, 0);
    }
}

// All-gather in the caller's output: the steps of the reduce-scatter backwards, data flowing the other way.
void AllGatherNhr(const CollShape &sh, Schedule &s)
{
    const uint32_t p = sh.nRanks, steps = NhrSteps(p);
    s.name = "AllGatherNHR";
    SetAgLayouts(sh, s);
    FinishScratch(s, p, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        e.Copy(IN, 0, OUT, r, 1, OUT, r);
        if (p == 1) continue;
        for (uint32_t k = 0; k < steps; ++k) e.Post((r + p - (1u << k) % p) % p, N_READY);
        uint32_t slot = 0;
        std::vector<uint32_t> have, get;
        for (uint32_t k = steps; k-- > 0;) {
            e.step = (uint8_t)(steps - k);
            const uint32_t d = 1u << k, to = (r + d) % p, from = (r + p - d % p) % p;
            NhrSlices(p, r, k, &get, &have);                 // what I received in the reduce-scatter I now own and send
            e.Wait(to, N_READY);
            for (uint32_t i = 0; i < have.size(); ++i) e.Write(to, OUT, have[i], slot + i, 1, OUT, have[i]);
            e.Post(to, N_DATA);
            e.Wait(from, N_DATA);
            for (uint32_t i = 0; i < get.size(); ++i) e.Copy(SCR, slot + i, OUT, get[i], 1, OUT, get[i]);
            slot += (uint32_t)have.size();
        }
    }
}

// All-reduce = NHR reduce-scatter on the output's slices followed by NHR all-gather.
void AllReduceNhr(const CollShape &sh, Schedule &s)
{
    const uint32_t p = sh.nRanks, steps = NhrSteps(p);
    s.name = "AllReduceNHR";
    s.input.resize(1); s.output.resize(1);
    Uniform(s.input[0], p, sh.count, sh.elemSize); Uniform(s.output[0], p, sh.count, sh.elemSize);
    FinishScratch(s, 2 * p, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        e.Copy(IN, 0, OUT, 0, p, OUT, 0);
        if (p == 1) continue;
        for (uint32_t k = 0; k < steps; ++k) { e.Post((r + (1u << k)) % p, N_READY); e.Post((r + p - (1u << k) % p) % p, N_READY); }
        uint32_t slot = 0;
        std::vector<uint32_t> tx, rx;
        for (uint32_t k = 0; k < steps; ++k) {
            e.step = (uint8_t)(1 + k);
            const uint32_t d = 1u << k, to = (r + p - d % p) % p, from = (r + d) % p;
            NhrSlices(p, r, k, &tx, &rx);
            e.Wait(to, N_READY);
            for (uint32_t i = 0; i < tx.size(); ++i) e.Write(to, OUT, tx[i], slot + i, 1, OUT, tx[i]);
            e.Post(to, N_DATA);
            e.Wait(from, N_DATA);
            for (uint32_t i = 0; i < rx.size(); ++i) e.Reduce(SCR, slot + i, OUT, rx[i], 1, OUT, rx[i]);
            slot += (uint32_t)tx.size();
        }
        for (uint32_t k = steps; k-- > 0;) {
            e.step = (uint8_t)(2 * steps - k);
            const uint32_t d = 1u << k, to = (r + d) % p, from = (r + p - d % p) % p;
            NhrSlices(p, r, k, &rx, &tx);
            e.Wait(to, N_READY);
            for (uint32_t i = 0; i < tx.size(); ++i) e.Write(to, OUT, tx[i], slot + i, 1, OUT, tx[i]);
            e.Post(to, N_DATA);
            e.Wait(from, N_DATA);
            for (uint32_t i = 0; i < rx.size(); ++i) e.Copy(SCR, slot + i, OUT, rx[i], 1, OUT, rx[i]);
            slot += (uint32_t)tx.size();
        }
    }
}

// Reduce-scatter along the Bruck tree, the all-gather's dissemination run backwards: accumulator slot j of rank r holds
// the partial sum of block (r + j) mod p; for d = largest power of two below p down to 1, slots [d, d + min(d, p - d))
// go to rank r + d, which adds them to its slots [0, min(d, p - d)).  Slot 0 ends as the complete block r.
void ReduceScatterBruck(const CollShape &sh, Schedule &s)
{
    const uint32_t p = sh.nRanks;
    s.name = "ReduceScatterBruck";
    SetRsLayouts(sh, s);
    FinishScratch(s, 2 * p, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        if (p == 1) { e.Copy(IN, 0, OUT, 0, 1, OUT, 0); continue; }
        for (uint32_t d = 1; d < p; d *= 2) e.Post((r + p - d) % p, N_READY);
        for (uint32_t j = 0; j < p; ++j) e.Copy(IN, (r + j) % p, SCR, j, 1, IN, (r + j) % p);
        uint32_t top = 1;
        while (top * 2 < p) top *= 2;
        uint32_t slot = p;
        uint8_t st = 1;
        for (uint32_t d = top; d >= 1; d /= 2, ++st) {
            e.step = st;
            const uint32_t cnt = std::min(d, p - d), to = (r + d) % p, from = (r + p - d) % p;
            e.Wait(to, N_READY);
            for (uint32_t j = 0; j < cnt; ++j) e.Write(to, SCR, d + j, slot + j, 1, IN, (r + d + j) % p);
            e.Post(to, N_DATA);
            e.Wait(from, N_DATA);
            for (uint32_t j = 0; j < cnt; ++j) e.Reduce(SCR, slot + j, SCR, j, 1, IN, (r + j) % p);
            slot += cnt;
            if (d == 1) break;
        }
        e.Copy(SCR, 0, OUT, 0, 1, OUT, 0);
    }
}

// ------------------------------------------------------------------------------------- AlltoAll

void SetA2aLayouts(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks;
    if (!sh.sendCounts.empty()) {
        s.input.resize(p); s.output.resize(p);
        for (uint32_t r = 0; r < p; ++r) {
            if (sh.sendCounts.size() > r && !sh.sendCounts[r].empty()) Explicit(s.input[r], sh.sendCounts[r], sh.sendDispls[r]);
            if (sh.recvCounts.size() > r && !sh.recvCounts[r].empty()) Explicit(s.output[r], sh.recvCounts[r], sh.recvDispls[r]);
        }
    } else {
        s.input.resize(1); s.output.resize(1);
        Fixed(s.input[0], p, sh.count); Fixed(s.output[0], p, sh.count);
    }
}

void AlltoAll(const CollShape &sh, Schedule &s, bool pairwise)
{
    uint32_t p = sh.nRanks;
    s.name = pairwise ? "AlltoAllPairwise" : "AlltoAllMesh";
    SetA2aLayouts(sh, s);
    FinishScratch(s, p, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        for (uint32_t i = 1; i < p; ++i) e.Post((r + i) % p, N_READY);
        e.Copy(IN, r, OUT, r, 1, OUT, r);
        for (uint32_t i = 1; i < p; ++i) {
            e.step = pairwise ? (uint8_t)i : 1;
            uint32_t dst = (r + i) % p, src = (r + p - i) % p;
            e.Wait(dst, N_READY); e.Write(dst, IN, dst, r, 1, IN, dst); e.Post(dst, N_DATA);
            if (pairwise) { e.Wait(src, N_DATA); e.Copy(SCR, src, OUT, src, 1, OUT, src); }
        }
        if (!pairwise) {
            e.step = 2;
            for (uint32_t i = 1; i < p; ++i) {
                uint32_t src = (r + p - i) % p;
                e.Wait(src, N_DATA); e.Copy(SCR, src, OUT, src, 1, OUT, src);
            }
        }
    }
}

// ------------------------------------------------------------------------------------ Broadcast

void BcastLayouts(const CollShape &sh, Schedule &s, uint32_t nSlices)
{
    s.input.resize(1); s.output.resize(1);
    Uniform(s.input[0], nSlices, sh.count, sh.elemSize); Uniform(s.output[0], nSlices, sh.count, sh.elemSize);
}

void BroadcastOneShot(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks, root = sh.root;
    s.name = "BroadcastMeshOneShot";
    BcastLayouts(sh, s, 1);
    FinishScratch(s, 1, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        if (r == root) {
            e.Copy(IN, 0, OUT, 0, 1, OUT, 0);
            for (uint32_t i = 1; i < p; ++i) {
                uint32_t q = (r + i) % p;
                e.Wait(q, N_READY); e.Write(q, IN, 0, 0, 1, IN, 0); e.Post(q, N_DATA);
            }
        } else {
            e.Post(root, N_READY); e.Wait(root, N_DATA); e.Copy(SCR, 0, OUT, 0, 1, OUT, 0);
        }
    }
}

// Scatter from the root, then every rank forwards its slice to everyone else.
void BroadcastTwoShot(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks, root = sh.root;
    s.name = "BroadcastMeshTwoShot";
    BcastLayouts(sh, s, p);
    FinishScratch(s, p, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        for (uint32_t i = 1; i < p; ++i) e.Post((r + i) % p, N_READY);
        if (r == root) {
            e.Copy(IN, 0, OUT, 0, p, OUT, 0);
            e.step = 1;
            for (uint32_t i = 1; i < p; ++i) {
                uint32_t q = (r + i) % p;
                e.Wait(q, N_READY);
                e.Write(q, IN, q, q, 1, IN, q);
                e.Write(q, IN, root, root, 1, IN, root);
                e.Post(q, N_DATA);
            }
            // consume the READY/DATA traffic of the forwarding phase so counters stay balanced
        } else {
            e.step = 1;
            e.Wait(root, N_DATA);
            e.step = 2;
            for (uint32_t i = 1; i < p; ++i) {
                uint32_t q = (r + i) % p;
                if (q == root) continue;
                e.Wait(q, N_READY); e.Write(q, SCR, r, r, 1, OUT, r); e.Post(q, N_DATA);
            }
            for (uint32_t i = 1; i < p; ++i) {
                uint32_t q = (r + i) % p;
                if (q == root) continue;
                e.Wait(q, N_DATA);
            }
            e.Copy(SCR, 0, OUT, 0, p, OUT, 0);
            e.Wait(root, N_READY);   // the root's READY is not needed for data; consume it
        }
    }
}

void BroadcastRing(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks, root = sh.root;
    s.name = "BroadcastRing";
    BcastLayouts(sh, s, p);
    FinishScratch(s, p, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        uint32_t pos = (r + p - root) % p, R = (r + 1) % p, L = (r + p - 1) % p;
        if (pos == 0) e.Copy(IN, 0, OUT, 0, p, OUT, 0);
        if (p == 1) continue;
        if (pos > 0) e.Post(L, N_READY);
        if (pos + 1 < p) e.Wait(R, N_READY);
        for (uint32_t i = 0; i < p; ++i) {   // pipeline slice by slice down the chain
            e.step = (uint8_t)(1 + i);
            if (pos > 0) { e.Wait(L, N_DATA); e.Copy(SCR, i, OUT, i, 1, OUT, i); }
            if (pos + 1 < p) { e.Write(R, pos == 0 ? IN : SCR, i, i, 1, OUT, i); e.Post(R, N_DATA); }
        }
    }
}

void BroadcastTree(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks, root = sh.root;
    s.name = "BroadcastTree";
    BcastLayouts(sh, s, 1);
    FinishScratch(s, 1, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        uint32_t vr = (r + p - root) % p;
        auto real = [&](uint32_t v) { return (v + root) % p; };
        if (vr == 0) e.Copy(IN, 0, OUT, 0, 1, OUT, 0);
        else {
            uint32_t hb = FloorPow2(vr);      // parent = vr without its highest bit
            uint32_t parent = real(vr - hb);
            e.Post(parent, N_READY); e.Wait(parent, N_DATA); e.Copy(SCR, 0, OUT, 0, 1, OUT, 0);
        }
        uint32_t first = vr == 0 ? 1 : FloorPow2(vr) * 2;
        uint8_t st = 1;
        for (uint32_t d = first; vr + d < p; d *= 2, ++st) {
            e.step = st;
            uint32_t child = real(vr + d);
            e.Wait(child, N_READY); e.Write(child, OUT, 0, 0, 1, OUT, 0); e.Post(child, N_DATA);
        }
    }
}

// --------------------------------------------------------------------------------------- Reduce

void ReduceMesh(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks, root = sh.root;
    s.name = "ReduceMesh";
    s.input.resize(1); s.output.resize(1);
    Uniform(s.input[0], p, sh.count, sh.elemSize); Uniform(s.output[0], p, sh.count, sh.elemSize);
    FinishScratch(s, 2 * p + 1, sh.elemSize);   // [0,p) contributions, p reduced slice, [p+1,2p+1) gathered at root
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        for (uint32_t i = 1; i < p; ++i) e.Post((r + i) % p, N_READY);
        e.Copy(IN, r, SCR, r, 1, IN, r);
        e.step = 1;
        for (uint32_t i = 1; i < p; ++i) {
            uint32_t q = (r + i) % p;
            e.Wait(q, N_READY); e.Write(q, IN, q, r, 1, IN, q); e.Post(q, N_DATA);
        }
        e.step = 2;
        for (uint32_t i = 1; i < p; ++i) e.Wait((r + i) % p, N_DATA);
        e.Copy(SCR, 0, SCR, p, 1, IN, r);
        for (uint32_t i = 1; i < p; ++i) e.Reduce(SCR, i, SCR, p, 1, IN, r);
        e.step = 3;
        if (r == root) {
            e.Copy(SCR, p, OUT, r, 1, OUT, r);
            for (uint32_t i = 1; i < p; ++i) {
                uint32_t q = (r + i) % p;
                e.Wait(q, N_DATA); e.Copy(SCR, p + 1 + q, OUT, q, 1, OUT, q);
            }
        } else {
            e.Write(root, SCR, p, p + 1 + r, 1, IN, r); e.Post(root, N_DATA);
        }
    }
}

void ReduceRing(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks, root = sh.root;
    s.name = "ReduceRing";
    s.input.resize(1); s.output.resize(1);
    Uniform(s.input[0], p, sh.count, sh.elemSize); Uniform(s.output[0], p, sh.count, sh.elemSize);
    FinishScratch(s, p, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        if (p == 1) { e.Copy(IN, 0, OUT, 0, p, OUT, 0); continue; }
        uint32_t k = (r + 2 * p - root - 1) % p;   // position in the chain; the root is last
        uint32_t R = (r + 1) % p, L = (r + p - 1) % p;
        if (k > 0) e.Post(L, N_READY);
        if (k + 1 < p) e.Wait(R, N_READY);
        for (uint32_t i = 0; i < p; ++i) {
            e.step = (uint8_t)(1 + i);
            if (k > 0) { e.Wait(L, N_DATA); e.Reduce(IN, i, SCR, i, 1, IN, i); }
            if (k + 1 < p) { e.Write(R, k == 0 ? IN : SCR, i, i, 1, IN, i); e.Post(R, N_DATA); }
            else e.Copy(SCR, i, OUT, i, 1, OUT, i);
        }
    }
}

void ReduceTree(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks, root = sh.root;
    s.name = "ReduceTree";
    s.input.resize(1); s.output.resize(1);
    Fixed(s.input[0], 1, sh.count); Fixed(s.output[0], 1, sh.count);
    uint32_t rounds = Log2(FloorPow2(p) == p ? p : FloorPow2(p) * 2);
    FinishScratch(s, rounds + 1, sh.elemSize);   // slot `rounds` is the accumulator, slot k receives round k
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        uint32_t vr = (r + p - root) % p;
        auto real = [&](uint32_t v) { return (v + root) % p; };
        uint32_t acc = rounds;
        // children: vr + d for d = 1,2,4.. while (vr & d)==0 ; parent at the first set bit
        for (uint32_t k = 0, d = 1; k < rounds; ++k, d *= 2) {
            if (vr & d) break;
            if (vr + d < p) e.Post(real(vr + d), N_READY);
        }
        e.Copy(IN, 0, SCR, acc, 1, IN, 0);
        uint32_t k = 0, d = 1;
        for (; k < rounds; ++k, d *= 2) {
            e.step = (uint8_t)(1 + k);
            if (vr & d) {
                uint32_t parent = real(vr - d);
                e.Wait(parent, N_READY); e.Write(parent, SCR, acc, k, 1, IN, 0); e.Post(parent, N_DATA);
                break;
            }
            if (vr + d < p) { e.Wait(real(vr + d), N_DATA); e.Reduce(SCR, k, SCR, acc, 1, IN, 0); }
        }
        if (vr == 0) e.Copy(SCR, acc, OUT, 0, 1, OUT, 0);
    }
}

// ----------------------------------------------------------------------------- Scatter / Gather

void ScatterMesh(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks, root = sh.root;
    s.name = "ScatterMesh";
    s.input.resize(1); s.output.resize(1);
    Fixed(s.input[0], p, sh.count); Fixed(s.output[0], 1, sh.count);
    FinishScratch(s, 1, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        if (r == root) {
            e.Copy(IN, r, OUT, 0, 1, OUT, 0);
            for (uint32_t i = 1; i < p; ++i) {
                uint32_t q = (r + i) % p;
                e.Wait(q, N_READY); e.Write(q, IN, q, 0, 1, IN, q); e.Post(q, N_DATA);
            }
        } else {
            e.Post(root, N_READY); e.Wait(root, N_DATA); e.Copy(SCR, 0, OUT, 0, 1, OUT, 0);
        }
    }
}

// Chain: the root hands its neighbour every slice that lives further down; each hop keeps its own.
void ScatterRing(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks, root = sh.root;
    s.name = "ScatterRing";
    s.input.resize(1); s.output.resize(1);
    Fixed(s.input[0], p, sh.count); Fixed(s.output[0], 1, sh.count);
    FinishScratch(s, p, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        uint32_t pos = (r + p - root) % p, R = (r + 1) % p, L = (r + p - 1) % p;
        if (pos == 0) e.Copy(IN, r, OUT, 0, 1, OUT, 0);
        if (p == 1) continue;
        if (pos > 0) e.Post(L, N_READY);
        if (pos + 1 < p) e.Wait(R, N_READY);
        // slices travel farthest-first so that every hop forwards as soon as a slice lands
        for (uint32_t t = p - 1; t > pos; --t) {
            uint32_t owner = (root + t) % p;
            e.step = (uint8_t)(p - t);
            if (pos > 0) e.Wait(L, N_DATA);
            e.Write(R, pos == 0 ? IN : SCR, owner, owner, 1, pos == 0 ? IN : OUT, pos == 0 ? owner : 0);
            e.Post(R, N_DATA);
        }
        if (pos > 0) { e.Wait(L, N_DATA); e.Copy(SCR, r, OUT, 0, 1, OUT, 0); }
    }
}

void GatherMesh(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks, root = sh.root;
    s.name = "GatherMesh";
    s.input.resize(1); s.output.resize(1);
    Fixed(s.input[0], 1, sh.count); Fixed(s.output[0], p, sh.count);
    FinishScratch(s, p, sh.elemSize);
    for (uint32_t r = 0; r < p; ++r) {
        if (!WantRank(sh, r)) continue;
        Emit e(s.ranks[r]);
        if (r == root) {
            for (uint32_t i = 1; i < p; ++i) e.Post((r + i) % p, N_READY);
            e.Copy(IN, 0, OUT, r, 1, OUT, r);
            for (uint32_t i = 1; i < p; ++i) {
                uint32_t q = (r + i) % p;
                e.Wait(q, N_DATA); e.Copy(SCR, q, OUT, q, 1, OUT, q);
            }
        } else {
            e.Wait(root, N_READY); e.Write(root, IN, 0, r, 1, IN, 0); e.Post(root, N_DATA);
        }
    }
}

// ---------------------------------------------------------------------------------- Send / Recv

void SendRecv(const CollShape &sh, Schedule &s)
{
    uint32_t p = sh.nRanks, src = sh.p2pSrc, dst = sh.p2pDst;
    s.name = "SendRecv";
    s.input.resize(1); s.output.resize(1);
    Fixed(s.input[0], 1, sh.count); Fixed(s.output[0], 1, sh.count);
    FinishScratch(s, p, sh.elemSize);   // one landing slot per possible sender
    if (WantRank(sh, src)) {
        Emit e(s.ranks[src]);
        e.Wait(dst, N_READY); e.Write(dst, IN, 0, src, 1, IN, 0); e.Post(dst, N_DATA);
    }
    if (WantRank(sh, dst)) {
        Emit e(s.ranks[dst]);
        e.Post(src, N_READY); e.Wait(src, N_DATA); e.Copy(SCR, src, OUT, 0, 1, OUT, 0);
    }
}

}  // namespace

std::vector<Algo> AlgosFor(HcclCMDType cmd, uint32_t nRanks)
{
    bool pow2 = nRanks != 0 && (nRanks & (nRanks - 1)) == 0;
    switch (cmd) {
        case HCCL_CMD_ALLREDUCE: return {Algo::MESH, Algo::MESH_ONESHOT, Algo::RING, Algo::HD, Algo::NHR};
        case HCCL_CMD_REDUCE_SCATTER:
            return pow2 ? std::vector<Algo>{Algo::MESH, Algo::RING, Algo::HD, Algo::NHR, Algo::BRUCK} : std::vector<Algo>{Algo::MESH, Algo::RING, Algo::NHR, Algo::BRUCK};
        case HCCL_CMD_REDUCE_SCATTER_V: return {Algo::MESH, Algo::RING, Algo::NHR, Algo::BRUCK};
        case HCCL_CMD_ALLGATHER: case HCCL_CMD_ALLGATHER_V:
            return pow2 ? std::vector<Algo>{Algo::MESH, Algo::RING, Algo::HD, Algo::BRUCK, Algo::NHR} : std::vector<Algo>{Algo::MESH, Algo::RING, Algo::BRUCK, Algo::NHR};
        case HCCL_CMD_ALLTOALL: case HCCL_CMD_ALLTOALLV: case HCCL_CMD_ALLTOALLVC: return {Algo::MESH, Algo::PAIRWISE};
        case HCCL_CMD_BROADCAST: return {Algo::MESH, Algo::MESH_ONESHOT, Algo::RING, Algo::TREE};
        case HCCL_CMD_REDUCE: return {Algo::MESH, Algo::RING, Algo::TREE};
        case HCCL_CMD_SCATTER: return {Algo::MESH, Algo::RING};
        case HCCL_CMD_GATHER: return {Algo::MESH};
        case HCCL_CMD_SEND: case HCCL_CMD_RECEIVE: return {Algo::MESH};
        default: return {};
    }
}

bool BuildSchedule(const CollShape &sh, Algo algo, Schedule *out, std::string *why)
{
    Schedule s;
    s.cmd = sh.cmd; s.nRanks = sh.nRanks; s.root = sh.root; s.nNotify = N_COUNT;
    s.ranks.assign(sh.nRanks, RankProgram());
    if (sh.nRanks == 0) { if (why) *why = "no ranks"; return false; }
    if ((sh.cmd == HCCL_CMD_BROADCAST || sh.cmd == HCCL_CMD_REDUCE || sh.cmd == HCCL_CMD_SCATTER || sh.cmd == HCCL_CMD_GATHER) && sh.root >= sh.nRanks) {
        if (why) *why = "root outside the communicator";
        return false;
    }
    bool ok = true;
    auto unsupported = [&]() { if (why) *why = std::string("strategy ") + AlgoName(algo) + " does not exist for this collective"; ok = false; };
    switch (sh.cmd) {
        case HCCL_CMD_ALLREDUCE:
            if (algo == Algo::MESH_ONESHOT) AllReduceOneShot(sh, s);
            else if (algo == Algo::MESH || algo == Algo::AUTO) AllReduceTwoShot(sh, s);
            else if (algo == Algo::RING) AllReduceRing(sh, s);
            else if (algo == Algo::HD) AllReduceHD(sh, s);
            else if (algo == Algo::NHR) AllReduceNhr(sh, s);
            else unsupported();
            break;
        case HCCL_CMD_REDUCE_SCATTER: case HCCL_CMD_REDUCE_SCATTER_V:
            if (algo == Algo::MESH || algo == Algo::AUTO) ReduceScatterMesh(sh, s);
            else if (algo == Algo::RING) ReduceScatterRing(sh, s);
            else if (algo == Algo::HD) ok = ReduceScatterHD(sh, s, why);
            else if (algo == Algo::NHR) ReduceScatterNhr(sh, s);
            else if (algo == Algo::BRUCK) ReduceScatterBruck(sh, s);
            else unsupported();
            break;
        case HCCL_CMD_ALLGATHER: case HCCL_CMD_ALLGATHER_V:
            if (algo == Algo::MESH || algo == Algo::AUTO) AllGatherMesh(sh, s);
            else if (algo == Algo::RING) AllGatherRing(sh, s);
            else if (algo == Algo::HD) ok = AllGatherHD(sh, s, why);
            else if (algo == Algo::BRUCK) AllGatherBruck(sh, s);
            else if (algo == Algo::NHR) AllGatherNhr(sh, s);
            else unsupported();
            break;
        case HCCL_CMD_ALLTOALL: case HCCL_CMD_ALLTOALLV: case HCCL_CMD_ALLTOALLVC:
            if (algo == Algo::MESH || algo == Algo::AUTO) AlltoAll(sh, s, false);
            else if (algo == Algo::PAIRWISE) AlltoAll(sh, s, true);
            else unsupported();
            break;
        case HCCL_CMD_BROADCAST:
            if (algo == Algo::MESH_ONESHOT || algo == Algo::STAR) BroadcastOneShot(sh, s);
            else if (algo == Algo::MESH || algo == Algo::AUTO) BroadcastTwoShot(sh, s);
            else if (algo == Algo::RING) BroadcastRing(sh, s);
            else if (algo == Algo::TREE || algo == Algo::HD || algo == Algo::BRUCK || algo == Algo::NHR) BroadcastTree(sh, s);
            else unsupported();
            break;
        case HCCL_CMD_REDUCE:
            if (algo == Algo::MESH || algo == Algo::AUTO) ReduceMesh(sh, s);
            else if (algo == Algo::RING) ReduceRing(sh, s);
            else if (algo == Algo::TREE || algo == Algo::HD || algo == Algo::NHR) ReduceTree(sh, s);
            else unsupported();
            break;
        case HCCL_CMD_SCATTER:
            if (algo == Algo::MESH || algo == Algo::AUTO || algo == Algo::STAR) ScatterMesh(sh, s);
            else if (algo == Algo::RING) ScatterRing(sh, s);
            else unsupported();
            break;
        case HCCL_CMD_GATHER:
            if (algo == Algo::MESH || algo == Algo::AUTO || algo == Algo::STAR) GatherMesh(sh, s);
            else unsupported();
            break;
        case HCCL_CMD_SEND: case HCCL_CMD_RECEIVE:
            SendRecv(sh, s);
            break;
        default:
            if (why) *why = "no template for this command";
            ok = false;
    }
    if (!ok) return false;
    *out = std::move(s);
    return true;
}

}  // namespace hc
