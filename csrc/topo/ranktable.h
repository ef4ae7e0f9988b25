// ranktable.h - the job description: which rank runs on which device of which host, and how the
// hosts are grouped into network layers.
//
// Two on-disk dialects are accepted (reference: rank_table_info.cc:150-172, new_rank_info.cc:46-108,
// topoinfo_ranktable*.cc):
//   1.0  {"version":"1.0","server_count":..,"server_list":[{"server_id","host_nic_ip",
//         "device":[{"device_id","device_ip","rank_id"}]}],"super_pod_list":[...]}
//   2.0  {"version":"2.0","rank_count":N,"rank_list":[{"rank_id","device_id","local_id",
//         "level_list":[{"net_layer","net_instance_id","net_type","net_attr",
//                        "rank_addr_list":[{"addr_type","addr","ports","plane_id"}]}]}]}
// The same model is also what the rendezvous produces from the per-rank records, and what is
// serialised (with a CRC32 trailer) into snapshots and consistency checks.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "../core/json.h"
#include "hccl/hccl_types.h"

namespace hc {

constexpr uint32_t kMaxRanks = 65536;       // rank_table_info.h:23 of the reference
constexpr uint32_t kMaxNetLayers = 8;

struct RankAddr {
    std::string addrType = "IPV4";
    std::string addr;
    std::vector<std::string> ports;
    int planeId = 0;
};

struct RankLevel {
    uint32_t netLayer = 0;
    std::string netInstanceId;
    std::string netType;       // "TOPO_FILE_DESC", "CLOS", "NVSWITCH" ...
    std::string netAttr;
    std::vector<RankAddr> addrs;
};

struct RankEntry {
    uint32_t rankId = 0;
    int32_t deviceId = 0;      // device ordinal on its host
    int32_t localId = 0;       // index among the ranks of the same host
    std::string serverId;      // host identity (layer-0 instance)
    std::string hostIp;
    std::string deviceIp;
    std::string superPodId;
    uint32_t pid = 0;
    uint32_t platKind = 0;
    std::string busId;
    uint32_t nvlinkCount = 0;  // active NVLink links reported by NVML
    uint64_t fabricClique = 0; // NVLink domain id, 0 when unknown
    std::vector<RankLevel> levels;
};

struct RankTable {
    std::string version = "2.0";
    std::vector<RankEntry> ranks;     // sorted by rankId, dense 0..n-1

    uint32_t size() const { return (uint32_t)ranks.size(); }
    // Parses either dialect.  Errors name the offending key (EI0004 / EI0014 style).
    HcclResult ParseJson(const std::string &text, std::string *err);
    HcclResult LoadFile(const std::string &path, std::string *err);
    Json ToJson() const;              // always dialect 2.0
    // Flat byte stream + CRC32; stable across processes, used for cross-rank consistency checks.
    std::vector<uint8_t> Serialize() const;
    HcclResult Deserialize(const std::vector<uint8_t> &bytes);
    uint32_t Crc() const;
    // Checks density / duplicates / limits and fills serverId, localId and layer-0 levels when absent.
    HcclResult Normalize(std::string *err);
    // Table restricted to `rankIds` (renumbered 0..k-1 in the given order).
    RankTable Sub(const std::vector<uint32_t> &rankIds) const;
    uint32_t ServerCount() const;
    uint32_t ServerIndexOf(uint32_t rank) const;
};

uint32_t Crc32(const void *data, size_t len, uint32_t seed = 0);

}  // namespace hc
