// selector.h - which strategy and which engine run an operator.
//
// Order of precedence, as in the reference (coll_alg_operator.cc:128-291, env_func.cc:287-479):
//   1. per-communicator HcclCommConfig.hcclAlgo, else the HCCL_ALGO environment variable, in the
//      reference grammar:   "level0:ring;level1:H-D_R"   or per operator
//      "allreduce=level0:fullmesh;level1:ring/allgather=level0:ring/others=level0:NA"
//      Level 0 is the NVLink domain, higher levels are accepted and recorded but one NVSwitch node
//      has nothing to run on them.
//   2. automatic choice from a bandwidth table.  Where the reference evaluates a closed-form
//      alpha-beta model with constants per chip, this build looks the operator up in a table of
//      size buckets that is measured on the machine (HCCL_TUNE_FILE, written by
//      hcomm_b200.utils.tune) and falls back to built-in thresholds derived from B200 runs.
// The op-expansion mode decides the engine family: host streams, SM kernels, or NVLS.
#pragma once
#include <map>
#include <string>
#include <vector>

#include "../core/json.h"
#include "hccl/hccl_types.h"
#include "templates.h"

namespace hc {

enum class Engine : uint8_t { HOST = 0, SM_FAST = 1, SM_IR = 2, NVLS = 3 };
const char *EngineName(Engine e);

struct AlgoConfig {
    // forced strategy per command for level 0..3; AUTO = not forced
    std::map<int, std::vector<Algo>> perCmd;     // key: HcclCMDType, or -1 for "all / others"
    bool Parse(const std::string &text, std::string *err);
    Algo Forced(HcclCMDType cmd, uint32_t level = 0) const;
    std::string Describe() const;
};

struct TuneBucket {
    uint64_t maxBytes;      // bucket covers message sizes <= maxBytes
    Algo algo;
    Engine engine;
    uint32_t ctas;          // 0 = engine default
};

struct TuneTable {
    // key: cmd name + "/" + nRanks
    std::map<std::string, std::vector<TuneBucket>> buckets;
    bool LoadJson(const Json &j, std::string *err);
    static const TuneTable &Get();       // HCCL_TUNE_FILE or built-in
    static void Reset();
    const TuneBucket *Lookup(HcclCMDType cmd, uint32_t nRanks, uint64_t bytes) const;
};

struct SelectInput {
    HcclCMDType cmd;
    uint32_t nRanks;
    uint64_t bytes;            // payload per rank that crosses the fabric, used for bucket lookup
    HcclDataType dtype;
    HcclReduceOp op;
    uint32_t opExpansionMode;  // resolved communicator setting
    uint32_t deterministic;
    bool cuda;                 // false on the simulator
    bool singleDomain;         // all ranks under one NVSwitch domain
    bool nvlsAvailable;
    bool variableCounts;
};

struct Selection {
    Algo algo = Algo::MESH;
    Engine engine = Engine::HOST;
    uint32_t ctas = 0;
    std::string name;          // e.g. "AllReduce/mesh_oneshot@sm"
    std::string reason;
};

const char *CmdName(HcclCMDType cmd);
// HCCL_E_NOT_SUPPORT when the configuration demands an engine that cannot serve the operator.
HcclResult SelectAlgorithm(const SelectInput &in, const AlgoConfig &forced, Selection *out);

}  // namespace hc
