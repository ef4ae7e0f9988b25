#include "selector.h"

#include <algorithm>
#include <fstream>
#include <mutex>
#include <sstream>

#include "../core/dtype.h"
#include "../core/env.h"
#include "../core/log.h"

namespace hc {

const char *EngineName(Engine e)
{
    switch (e) {
        case Engine::HOST: return "host"; case Engine::SM_FAST: return "sm"; case Engine::SM_IR: return "sm-ir"; case Engine::NVLS: return "nvls";
    }
    return "?";
}

const char *CmdName(HcclCMDType cmd)
{
    switch (cmd) {
        case HCCL_CMD_BROADCAST: return "broadcast"; case HCCL_CMD_ALLREDUCE: return "allreduce"; case HCCL_CMD_REDUCE: return "reduce";
        case HCCL_CMD_SEND: return "send"; case HCCL_CMD_RECEIVE: return "receive"; case HCCL_CMD_ALLGATHER: return "allgather";
        case HCCL_CMD_REDUCE_SCATTER: return "reducescatter"; case HCCL_CMD_ALLTOALLV: return "alltoallv"; case HCCL_CMD_ALLTOALLVC: return "alltoallvc";
        case HCCL_CMD_ALLTOALL: return "alltoall"; case HCCL_CMD_GATHER: return "gather"; case HCCL_CMD_SCATTER: return "scatter";
        case HCCL_CMD_BATCH_SEND_RECV: return "batchsendrecv"; case HCCL_CMD_ALLGATHER_V: return "allgatherv";
        case HCCL_CMD_REDUCE_SCATTER_V: return "reducescatterv"; case HCCL_CMD_BARRIER: return "barrier"; default: return "unknown";
    }
}

static int CmdFromName(std::string s)
{
    for (auto &c : s) c = (char)tolower((unsigned char)c);
    static const HcclCMDType all[] = {HCCL_CMD_BROADCAST, HCCL_CMD_ALLREDUCE, HCCL_CMD_REDUCE, HCCL_CMD_SEND, HCCL_CMD_RECEIVE, HCCL_CMD_ALLGATHER,
                                      HCCL_CMD_REDUCE_SCATTER, HCCL_CMD_ALLTOALLV, HCCL_CMD_ALLTOALLVC, HCCL_CMD_ALLTOALL, HCCL_CMD_GATHER,
                                      HCCL_CMD_SCATTER, HCCL_CMD_BATCH_SEND_RECV, HCCL_CMD_ALLGATHER_V, HCCL_CMD_REDUCE_SCATTER_V};
    if (s == "others" || s == "all") return -1;
    if (s == "alltoall") return HCCL_CMD_ALLTOALL;
    for (auto c : all)
        if (s == CmdName(c)) return c;
    return -2;
}

static bool ParseLevels(const std::string &text, std::vector<Algo> *levels, std::string *err)
{
    levels->assign(4, Algo::AUTO);
    std::stringstream ss(text);
    std::string item;
    while (std::getline(ss, item, ';')) {
        if (item.empty()) continue;
        auto colon = item.find(':');
        if (colon == std::string::npos || item.compare(0, 5, "level") != 0 || colon != 6 || item[5] < '0' || item[5] > '3') {
            if (err) *err = "\"" + item + "\" is not of the form levelN:algorithm";
            return false;
        }
        Algo a;
        if (!ParseAlgoName(item.substr(colon + 1), &a)) {
            if (err) *err = "unknown algorithm \"" + item.substr(colon + 1) + "\"";
            return false;
        }
        (*levels)[item[5] - '0'] = a;
    }
    return true;
}

bool AlgoConfig::Parse(const std::string &text, std::string *err)
{
    perCmd.clear();
    if (text.empty()) return true;
    if (text.find('=') == std::string::npos) {
        std::vector<Algo> lv;
        if (!ParseLevels(text, &lv, err)) return false;
        perCmd[-1] = lv;
        return true;
    }
    std::stringstream ss(text);
    std::string part;
    while (std::getline(ss, part, '/')) {
        if (part.empty()) continue;
        auto eq = part.find('=');
        if (eq == std::string::npos) {
            if (err) *err = "\"" + part + "\" lacks operator=";
            return false;
        }
        int cmd = CmdFromName(part.substr(0, eq));
        if (cmd == -2) {
            if (err) *err = "unknown operator \"" + part.substr(0, eq) + "\"";
            return false;
        }
        std::vector<Algo> lv;
        if (!ParseLevels(part.substr(eq + 1), &lv, err)) return false;
        if (perCmd.count(cmd)) {
            if (err) *err = "operator \"" + part.substr(0, eq) + "\" configured twice";
            return false;
        }
        perCmd[cmd] = lv;
    }
    return true;
}

Algo AlgoConfig::Forced(HcclCMDType cmd, uint32_t level) const
{
    // The V-variants share their base collective's setting.
    int key = cmd;
    if (cmd == HCCL_CMD_ALLGATHER_V) key = HCCL_CMD_ALLGATHER;
    if (cmd == HCCL_CMD_REDUCE_SCATTER_V) key = HCCL_CMD_REDUCE_SCATTER;
    if (cmd == HCCL_CMD_ALLTOALLV || cmd == HCCL_CMD_ALLTOALLVC) key = HCCL_CMD_ALLTOALL;
    auto it = perCmd.find(key);
    if (it == perCmd.end()) it = perCmd.find(-1);
    if (it == perCmd.end() || level >= it->second.size()) return Algo::AUTO;
    return it->second[level];
}

std::string AlgoConfig::Describe() const
{
    std::ostringstream os;
    for (auto &kv : perCmd) {
        os << (kv.first < 0 ? "others" : CmdName((HcclCMDType)kv.first)) << "=";
        for (size_t l = 0; l < kv.second.size(); ++l)
            if (kv.second[l] != Algo::AUTO) os << "level" << l << ":" << AlgoName(kv.second[l]) << ";";
        os << "/";
    }
    return os.str();
}

// ------------------------------------------------------------------------------------- tuning

namespace {
std::mutex g_tuneMu;
TuneTable *g_tune = nullptr;

Engine EngineFromName(const std::string &s)
{
    if (s == "host") return Engine::HOST;
    if (s == "sm-ir") return Engine::SM_IR;
    if (s == "nvls") return Engine::NVLS;
    return Engine::SM_FAST;
}

// Built-in buckets.  One-shot below the size where pushing p copies costs less than a second
// barrier; two-shot mesh up to where in-switch reduction wins; NVLS above (when available).
void Builtin(TuneTable &t)
{
    const uint64_t KB = 1024, MB = 1024 * 1024;
    for (uint32_t p = 2; p <= 16u; ++p) {
        std::string n = std::to_string(p);
        t.buckets["allreduce/" + n] = {{(p <= 4 ? 512 : 256) * KB, Algo::MESH_ONESHOT, Engine::SM_FAST, 0},
                                       {p <= 4 ? UINT64_MAX : 4 * MB, Algo::MESH, Engine::SM_FAST, 0},   // up to 4 GPUs the mesh kernel measured faster than in-switch reduction
                                       {UINT64_MAX, Algo::NVLS, Engine::NVLS, 0}};
        t.buckets["broadcast/" + n] = {{1 * MB, Algo::MESH_ONESHOT, Engine::SM_FAST, 0}, {UINT64_MAX, Algo::NVLS, Engine::NVLS, 0}};
        // all-gather (bytes per rank): multicast stores win in the middle range on 8 GPUs (4 MB in total: 39 us against 54,
        // 16 MB: 57 against 72), lose below (32 - 35 us against 22 - 25) and at 64 MB in total (152 us against 143);
        // on 2 and 4 GPUs the mesh kernel is faster at every size.  The buckets are what `python -m hcomm_b200.utils.tune
        // --from-sweeps` makes of the 8-GPU sweeps of the two families (hcomm_b200/utils/tune_tables/).
        if (p >= 6) t.buckets["allgather/" + n] = {{128 * KB, Algo::MESH, Engine::SM_FAST, 0}, {2 * MB, Algo::NVLS, Engine::NVLS, 0}, {UINT64_MAX, Algo::MESH, Engine::SM_FAST, 0}};
        else t.buckets["allgather/" + n] = {{UINT64_MAX, Algo::MESH, Engine::SM_FAST, 0}};
        t.buckets["reducescatter/" + n] = {{UINT64_MAX, Algo::MESH, Engine::SM_FAST, 0}};
        t.buckets["alltoall/" + n] = {{UINT64_MAX, Algo::MESH, Engine::SM_FAST, 0}};
        t.buckets["reduce/" + n] = {{UINT64_MAX, Algo::MESH, Engine::SM_FAST, 0}};
    }
}
}  // namespace

bool TuneTable::LoadJson(const Json &j, std::string *err)
{
    if (!j.isObject()) { if (err) *err = "tuning table must be a JSON object"; return false; }
    for (auto &cmdName : j.keys()) {
        const Json &perRanks = j[cmdName];
        if (!perRanks.isObject()) continue;
        for (auto &ranks : perRanks.keys()) {
            const Json &arr = perRanks[ranks];
            std::vector<TuneBucket> v;
            for (size_t i = 0; i < arr.size(); ++i) {
                TuneBucket b;
                int64_t mb = arr[i]["max_bytes"].intOr(-1);
                b.maxBytes = mb < 0 ? UINT64_MAX : (uint64_t)mb;
                if (!ParseAlgoName(arr[i]["algo"].strOr("mesh"), &b.algo)) { if (err) *err = "unknown algo in tuning table"; return false; }
                b.engine = EngineFromName(arr[i]["engine"].strOr("sm"));
                b.ctas = (uint32_t)arr[i]["ctas"].intOr(0);
                v.push_back(b);
            }
            std::sort(v.begin(), v.end(), [](const TuneBucket &a, const TuneBucket &b) { return a.maxBytes < b.maxBytes; });
            if (!v.empty()) buckets[cmdName + "/" + ranks] = v;
        }
    }
    return true;
}

const TuneTable &TuneTable::Get()
{
    std::lock_guard<std::mutex> lk(g_tuneMu);
    if (!g_tune) {
        g_tune = new TuneTable();
        Builtin(*g_tune);
        const std::string &path = EnvConfig::Get().tuneFile.value;
        if (!path.empty()) {
            std::ifstream f(path);
            std::stringstream ss;
            ss << f.rdbuf();
            Json j;
            std::string err;
            if (!f || !Json::Parse(ss.str(), j, &err) || !g_tune->LoadJson(j, &err)) HCCL_WARNING("tuning file %s ignored: %s", path.c_str(), err.c_str());
            else HCCL_INFO("tuning table loaded from %s", path.c_str());
        }
    }
    return *g_tune;
}

void TuneTable::Reset()
{
    std::lock_guard<std::mutex> lk(g_tuneMu);
    delete g_tune;
    g_tune = nullptr;
}

const TuneBucket *TuneTable::Lookup(HcclCMDType cmd, uint32_t nRanks, uint64_t bytes) const
{
    HcclCMDType base = cmd;
    if (cmd == HCCL_CMD_ALLGATHER_V) base = HCCL_CMD_ALLGATHER;
    if (cmd == HCCL_CMD_REDUCE_SCATTER_V) base = HCCL_CMD_REDUCE_SCATTER;
    if (cmd == HCCL_CMD_ALLTOALLV || cmd == HCCL_CMD_ALLTOALLVC) base = HCCL_CMD_ALLTOALL;
    auto it = buckets.find(std::string(CmdName(base)) + "/" + std::to_string(nRanks));
    if (it == buckets.end()) return nullptr;
    for (auto &b : it->second)
        if (bytes <= b.maxBytes) return &b;
    return it->second.empty() ? nullptr : &it->second.back();
}

// ------------------------------------------------------------------------------------ selection

static bool FastKernelServes(const SelectInput &in, Algo a)
{
    if (!in.cuda || !in.singleDomain || in.nRanks > 16) return false;
    switch (in.cmd) {
        case HCCL_CMD_ALLREDUCE: case HCCL_CMD_REDUCE_SCATTER: case HCCL_CMD_REDUCE: case HCCL_CMD_REDUCE_SCATTER_V:
            if (!DtypeReducible(in.dtype)) return false;
            return a == Algo::MESH || a == Algo::MESH_ONESHOT || a == Algo::AUTO;
        case HCCL_CMD_ALLGATHER: case HCCL_CMD_ALLGATHER_V: case HCCL_CMD_ALLTOALL: case HCCL_CMD_ALLTOALLV: case HCCL_CMD_ALLTOALLVC:
        case HCCL_CMD_BROADCAST: case HCCL_CMD_SCATTER: case HCCL_CMD_GATHER: case HCCL_CMD_SEND: case HCCL_CMD_RECEIVE:
            return a == Algo::MESH || a == Algo::MESH_ONESHOT || a == Algo::AUTO || a == Algo::PAIRWISE || a == Algo::STAR;
        default: return false;
    }
}

static bool NvlsServes(const SelectInput &in)
{
    if (!in.cuda || !in.nvlsAvailable) return false;
    if (in.cmd == HCCL_CMD_BROADCAST) return true;
    if (in.cmd == HCCL_CMD_ALLGATHER) return !in.variableCounts;       // multicast stores move bytes of any type
    if (in.cmd != HCCL_CMD_ALLREDUCE && in.cmd != HCCL_CMD_REDUCE_SCATTER) return false;
    if (in.variableCounts) return false;
    // multimem.ld_reduce exists for f32/f16/bf16 add and integer min/max/add; keep to what is exercised
    bool typeOk = in.dtype == HCCL_DATA_TYPE_FP32 || in.dtype == HCCL_DATA_TYPE_FP16 || in.dtype == HCCL_DATA_TYPE_BFP16;
    return typeOk && in.op == HCCL_REDUCE_SUM && in.deterministic == 0;
}

HcclResult SelectAlgorithm(const SelectInput &in, const AlgoConfig &forced, Selection *out)
{
    Selection s;
    Algo want = forced.Forced(in.cmd, 0);
    std::vector<Algo> known = AlgosFor(in.cmd, in.nRanks);
    auto knows = [&](Algo a) { return std::find(known.begin(), known.end(), a) != known.end(); };

    // engine family from the expansion mode
    bool hostOnly = !in.cuda || in.opExpansionMode == 1 || in.opExpansionMode == 2;
    bool smOnly = in.opExpansionMode == 4;
    bool nvlsOnly = in.opExpansionMode == 5 || in.opExpansionMode == 6;

    if (in.nRanks == 1) {
        s.algo = Algo::MESH; s.engine = in.cuda ? Engine::SM_FAST : Engine::HOST; s.reason = "single rank";
        if (hostOnly) s.engine = Engine::HOST;
    } else if (want != Algo::AUTO) {
        if (want == Algo::NVLS) {
            if (!NvlsServes(in)) { RPT_ERR("EI0003", "HCCL_ALGO asks for nvls but it cannot serve %s here", CmdName(in.cmd)); return HCCL_E_NOT_SUPPORT; }
            s.algo = Algo::NVLS; s.engine = Engine::NVLS;
        } else {
            if (!knows(want)) {
                // same behaviour as the reference: an algorithm that does not exist for the operator falls back with a warning
                HCCL_WARNING("algorithm %s is not available for %s on %u ranks, using the default", AlgoName(want), CmdName(in.cmd), in.nRanks);
                want = known.empty() ? Algo::MESH : known[0];
            }
            s.algo = want;
            if (hostOnly) s.engine = Engine::HOST;
            else if (FastKernelServes(in, want)) s.engine = Engine::SM_FAST;
            else s.engine = (in.singleDomain && in.nRanks <= 16 && DtypeReducible(in.dtype)) ? Engine::SM_IR : Engine::HOST;
        }
        s.reason = "forced by configuration";
    } else {
        const TuneBucket *b = in.cuda ? TuneTable::Get().Lookup(in.cmd, in.nRanks, in.bytes) : nullptr;
        if (b && !hostOnly) {
            s.algo = b->algo; s.engine = b->engine; s.ctas = b->ctas; s.reason = "bandwidth table";
            if (s.engine == Engine::NVLS && (!NvlsServes(in) || smOnly)) { s.engine = Engine::SM_FAST; s.algo = Algo::MESH; s.reason = "bandwidth table (nvls unavailable)"; }
            if (s.engine == Engine::SM_FAST && !FastKernelServes(in, s.algo)) { s.engine = Engine::HOST; s.algo = known.empty() ? Algo::MESH : known[0]; s.reason = "kernel ineligible, host fallback"; }
            if (in.deterministic && s.algo == Algo::NVLS) { s.algo = Algo::MESH; s.engine = Engine::SM_FAST; }
        } else {
            s.algo = known.empty() ? Algo::MESH : known[0];
            // small all-reduce on the host engines: one-shot saves a round of notifies
            if (in.cmd == HCCL_CMD_ALLREDUCE && in.bytes <= 64 * 1024) s.algo = Algo::MESH_ONESHOT;
            if (in.cmd == HCCL_CMD_BROADCAST && in.bytes <= 64 * 1024) s.algo = Algo::MESH_ONESHOT;
            s.engine = (!hostOnly && FastKernelServes(in, s.algo)) ? Engine::SM_FAST : Engine::HOST;
            s.reason = "default";
        }
    }
    if (nvlsOnly && in.nRanks > 1) {
        if (!NvlsServes(in)) { RPT_ERR("EI0003", "op expansion mode %u (NVLS) cannot serve %s %s", in.opExpansionMode, CmdName(in.cmd), DtypeName(in.dtype)); return HCCL_E_NOT_SUPPORT; }
        s.algo = Algo::NVLS; s.engine = Engine::NVLS;
    }
    if (smOnly && s.engine == Engine::HOST) {
        RPT_ERR("EI0003", "op expansion mode 4 (SM kernels only) cannot serve %s with algorithm %s", CmdName(in.cmd), AlgoName(s.algo));
        return HCCL_E_NOT_SUPPORT;
    }
    if (!in.cuda) s.engine = Engine::HOST;
    s.name = std::string(CmdName(in.cmd)) + "/" + AlgoName(s.algo) + "@" + EngineName(s.engine);
    *out = s;
    return HCCL_SUCCESS;
}

}  // namespace hc
