#include "ranktable.h"

#include <algorithm>
#include <cstring>
#include <fstream>
#include <map>
#include <sstream>

#include "../core/log.h"

namespace hc {

uint32_t Crc32(const void *data, size_t len, uint32_t seed)
{
    struct Table {
        uint32_t v[256];
        Table()
        {
            for (uint32_t i = 0; i < 256; ++i) {
                uint32_t c = i;
                for (int k = 0; k < 8; ++k) c = (c & 1) ? (0xEDB88320u ^ (c >> 1)) : (c >> 1);
                v[i] = c;
            }
        }
    };
    static const Table built;                 // built once, also when several ranks of a process get here together
    const uint32_t *table = built.v;
    uint32_t c = ~seed;
    const uint8_t *p = (const uint8_t *)data;
    for (size_t i = 0; i < len; ++i) c = table[(c ^ p[i]) & 0xff] ^ (c >> 8);
    return ~c;
}

static bool NeedInt(const Json &obj, const char *key, int64_t &out, std::string *err, const std::string &where)
{
    if (!obj.has(key) || !obj[key].asInt(out)) {
        if (err) *err = where + ": key \"" + key + "\" is missing or not an integer";
        return false;
    }
    return true;
}

static HcclResult ParseV1(const Json &root, RankTable &t, std::string *err)
{
    const Json &servers = root["server_list"];
    if (!servers.isArray() || servers.size() == 0) {
        if (err) *err = "\"server_list\" is missing or empty";
        return HCCL_E_PARA;
    }
    int64_t declared = -1;
    if (root.has("server_count") && root["server_count"].asInt(declared) && (size_t)declared != servers.size()) {
        if (err) *err = "\"server_count\" (" + std::to_string(declared) + ") does not match the length of \"server_list\" (" + std::to_string(servers.size()) + ")";
        return HCCL_E_PARA;
    }
    // optional super-pod membership: super_pod_list[{super_pod_id, server_list[{server_id}]}]
    std::map<std::string, std::string> podOf;
    const Json &pods = root["super_pod_list"];
    for (size_t i = 0; i < pods.size(); ++i) {
        std::string pid = pods[i]["super_pod_id"].isString() ? pods[i]["super_pod_id"].str() : std::to_string(pods[i]["super_pod_id"].intOr((int64_t)i));
        const Json &sl = pods[i]["server_list"];
        for (size_t k = 0; k < sl.size(); ++k) podOf[sl[k]["server_id"].strOr("")] = pid;
    }
    for (size_t s = 0; s < servers.size(); ++s) {
        const Json &sv = servers[s];
        std::string where = "server_list[" + std::to_string(s) + "]";
        std::string serverId = sv["server_id"].strOr("");
        if (serverId.empty()) {
            if (err) *err = where + ": key \"server_id\" is missing";
            return HCCL_E_PARA;
        }
        const Json &devs = sv["device"];
        if (!devs.isArray() || devs.size() == 0) {
            if (err) *err = where + ": key \"device\" is missing or empty";
            return HCCL_E_PARA;
        }
        for (size_t d = 0; d < devs.size(); ++d) {
            RankEntry e;
            int64_t v;
            std::string w = where + ".device[" + std::to_string(d) + "]";
            if (!NeedInt(devs[d], "rank_id", v, err, w)) return HCCL_E_PARA;
            e.rankId = (uint32_t)v;
            if (!NeedInt(devs[d], "device_id", v, err, w)) return HCCL_E_PARA;
            e.deviceId = (int32_t)v;
            e.deviceIp = devs[d]["device_ip"].strOr("");
            e.serverId = serverId;
            e.hostIp = sv["host_nic_ip"].strOr(sv["host_ip"].strOr(""));
            e.localId = (int32_t)d;
            auto it = podOf.find(serverId);
            if (it != podOf.end()) e.superPodId = it->second;
            t.ranks.push_back(e);
        }
    }
    t.version = "1.0";
    return HCCL_SUCCESS;
}

static HcclResult ParseV2(const Json &root, RankTable &t, std::string *err)
{
    const Json &list = root["rank_list"];
    if (!list.isArray() || list.size() == 0) {
        if (err) *err = "\"rank_list\" is missing or empty";
        return HCCL_E_PARA;
    }
    int64_t declared;
    if (!NeedInt(root, "rank_count", declared, err, "root")) return HCCL_E_PARA;
    if ((size_t)declared != list.size()) {
        if (err) *err = "\"rank_count\" (" + std::to_string(declared) + ") does not match the length of \"rank_list\" (" + std::to_string(list.size()) + ")";
        return HCCL_E_PARA;
    }
    for (size_t i = 0; i < list.size(); ++i) {
        const Json &r = list[i];
        std::string where = "rank_list[" + std::to_string(i) + "]";
        RankEntry e;
        int64_t v;
        if (!NeedInt(r, "rank_id", v, err, where)) return HCCL_E_PARA;
        e.rankId = (uint32_t)v;
        if (!NeedInt(r, "device_id", v, err, where)) return HCCL_E_PARA;
        e.deviceId = (int32_t)v;
        e.localId = (int32_t)r["local_id"].intOr(e.deviceId);
        const Json &lv = r["level_list"];
        if (lv.size() > kMaxNetLayers) {
            if (err) *err = where + ": more than " + std::to_string(kMaxNetLayers) + " entries in \"level_list\"";
            return HCCL_E_PARA;
        }
        for (size_t k = 0; k < lv.size(); ++k) {
            RankLevel L;
            std::string w2 = where + ".level_list[" + std::to_string(k) + "]";
            if (!NeedInt(lv[k], "net_layer", v, err, w2)) return HCCL_E_PARA;
            L.netLayer = (uint32_t)v;
            L.netInstanceId = lv[k]["net_instance_id"].strOr("");
            if (L.netInstanceId.empty()) {
                if (err) *err = w2 + ": key \"net_instance_id\" is missing";
                return HCCL_E_PARA;
            }
            L.netType = lv[k]["net_type"].strOr("");
            L.netAttr = lv[k]["net_attr"].strOr("");
            const Json &al = lv[k]["rank_addr_list"];
            for (size_t a = 0; a < al.size(); ++a) {
                RankAddr A;
                A.addrType = al[a]["addr_type"].strOr("IPV4");
                A.addr = al[a]["addr"].strOr("");
                A.planeId = (int)al[a]["plane_id"].intOr(0);
                const Json &ps = al[a]["ports"];
                for (size_t p = 0; p < ps.size(); ++p) A.ports.push_back(ps[p].isString() ? ps[p].str() : std::to_string(ps[p].intOr(0)));
                L.addrs.push_back(A);
            }
            e.levels.push_back(L);
        }
        if (!e.levels.empty()) {
            e.serverId = e.levels[0].netInstanceId;
            if (!e.levels[0].addrs.empty()) e.deviceIp = e.levels[0].addrs[0].addr;
        }
        if (r.has("host_ip")) e.hostIp = r["host_ip"].strOr("");
        t.ranks.push_back(e);
    }
    t.version = "2.0";
    return HCCL_SUCCESS;
}

HcclResult RankTable::ParseJson(const std::string &text, std::string *err)
{
    ranks.clear();
    Json root;
    std::string perr;
    if (!Json::Parse(text, root, &perr)) {
        if (err) *err = "not valid JSON (" + perr + ")";
        return HCCL_E_PARA;
    }
    if (root.has("status") && root["status"].strOr("completed") != "completed") {
        if (err) *err = "\"status\" is \"" + root["status"].strOr("") + "\", expected \"completed\"";
        return HCCL_E_PARA;
    }
    std::string ver = root["version"].isString() ? root["version"].str() : "";
    HcclResult r;
    if (root.has("rank_list")) r = ParseV2(root, *this, err);
    else if (root.has("server_list")) r = ParseV1(root, *this, err);
    else {
        if (err) *err = "neither \"rank_list\" (2.0) nor \"server_list\" (1.0) is present (version=\"" + ver + "\")";
        return HCCL_E_PARA;
    }
    if (r != HCCL_SUCCESS) return r;
    return Normalize(err);
}

HcclResult RankTable::LoadFile(const std::string &path, std::string *err)
{
    std::ifstream f(path);
    if (!f) {
        if (err) *err = "cannot open " + path;
        return HCCL_E_OPEN_FILE_FAILURE;
    }
    std::stringstream ss;
    ss << f.rdbuf();
    return ParseJson(ss.str(), err);
}

HcclResult RankTable::Normalize(std::string *err)
{
    if (ranks.empty() || ranks.size() > kMaxRanks) {
        if (err) *err = "rank count " + std::to_string(ranks.size()) + " outside [1," + std::to_string(kMaxRanks) + "]";
        return HCCL_E_PARA;
    }
    std::sort(ranks.begin(), ranks.end(), [](const RankEntry &a, const RankEntry &b) { return a.rankId < b.rankId; });
    for (size_t i = 0; i < ranks.size(); ++i) {
        if (ranks[i].rankId != i) {
            if (err) *err = (i > 0 && ranks[i].rankId == ranks[i - 1].rankId) ? "rank_id " + std::to_string(ranks[i].rankId) + " appears twice"
                                                                            : "rank ids are not dense: expected " + std::to_string(i) + ", found " + std::to_string(ranks[i].rankId);
            return HCCL_E_PARA;
        }
    }
    std::map<std::string, int> perServer;
    std::map<std::string, std::map<int, uint32_t>> devSeen;
    for (auto &e : ranks) {
        if (e.serverId.empty()) e.serverId = e.hostIp.empty() ? "server0" : e.hostIp;
        auto &seen = devSeen[e.serverId];
        if (e.platKind != 0 /*not sim*/ && seen.count(e.deviceId) && version != "boot") {
            if (err) *err = "device_id " + std::to_string(e.deviceId) + " of server " + e.serverId + " is used by ranks " + std::to_string(seen[e.deviceId]) + " and " + std::to_string(e.rankId);
            return HCCL_E_PARA;
        }
        seen[e.deviceId] = e.rankId;
        int idx = perServer[e.serverId]++;
        if (e.localId < 0) e.localId = idx;
        if (e.levels.empty()) {
            RankLevel L;
            L.netLayer = 0;
            L.netInstanceId = e.serverId;
            L.netType = "NVSWITCH";
            RankAddr A;
            A.addr = e.deviceIp.empty() ? e.hostIp : e.deviceIp;
            if (!A.addr.empty()) L.addrs.push_back(A);
            e.levels.push_back(L);
        }
    }
    // More than one host: every rank also belongs to one layer-1 instance that spans the hosts.
    if (perServer.size() > 1) {
        for (auto &e : ranks) {
            bool has1 = false;
            for (auto &L : e.levels) has1 |= (L.netLayer == 1);
            if (!has1) {
                RankLevel L;
                L.netLayer = 1;
                L.netInstanceId = e.superPodId.empty() ? "cluster" : e.superPodId;
                L.netType = "CLOS";
                e.levels.push_back(L);
            }
        }
    }
    return HCCL_SUCCESS;
}

Json RankTable::ToJson() const
{
    Json root = Json::Object();
    root.set("version", Json(std::string("2.0")));
    root.set("rank_count", Json((int64_t)ranks.size()));
    root.set("status", Json(std::string("completed")));
    Json list = Json::Array();
    for (auto &e : ranks) {
        Json r = Json::Object();
        r.set("rank_id", Json((int64_t)e.rankId));
        r.set("device_id", Json((int64_t)e.deviceId));
        r.set("local_id", Json((int64_t)e.localId));
        if (!e.hostIp.empty()) r.set("host_ip", Json(e.hostIp));
        Json lv = Json::Array();
        for (auto &L : e.levels) {
            Json l = Json::Object();
            l.set("net_layer", Json((int64_t)L.netLayer));
            l.set("net_instance_id", Json(L.netInstanceId));
            l.set("net_type", Json(L.netType));
            l.set("net_attr", Json(L.netAttr));
            Json al = Json::Array();
            for (auto &A : L.addrs) {
                Json a = Json::Object();
                a.set("addr_type", Json(A.addrType));
                a.set("addr", Json(A.addr));
                Json ps = Json::Array();
                for (auto &p : A.ports) ps.push(Json(p));
                a.set("ports", ps);
                a.set("plane_id", Json((int64_t)A.planeId));
                al.push(a);
            }
            l.set("rank_addr_list", al);
            lv.push(l);
        }
        r.set("level_list", lv);
        list.push(r);
    }
    root.set("rank_list", list);
    return root;
}

namespace {
void W32(std::vector<uint8_t> &b, uint32_t v) { b.insert(b.end(), (uint8_t *)&v, (uint8_t *)&v + 4); }
void W64(std::vector<uint8_t> &b, uint64_t v) { b.insert(b.end(), (uint8_t *)&v, (uint8_t *)&v + 8); }
void WS(std::vector<uint8_t> &b, const std::string &s) { W32(b, (uint32_t)s.size()); b.insert(b.end(), s.begin(), s.end()); }
struct R {
    const uint8_t *p, *e;
    bool ok = true;
    uint32_t u32() { uint32_t v = 0; if (e - p < 4) { ok = false; return 0; } memcpy(&v, p, 4); p += 4; return v; }
    uint64_t u64() { uint64_t v = 0; if (e - p < 8) { ok = false; return 0; } memcpy(&v, p, 8); p += 8; return v; }
    std::string s() { uint32_t n = u32(); if (!ok || (uint32_t)(e - p) < n) { ok = false; return ""; } std::string r((const char *)p, n); p += n; return r; }
};
}  // namespace

std::vector<uint8_t> RankTable::Serialize() const
{
    std::vector<uint8_t> b;
    W32(b, 0x48435254);  // "HCRT"
    WS(b, version);
    W32(b, (uint32_t)ranks.size());
    for (auto &e : ranks) {
        W32(b, e.rankId); W32(b, (uint32_t)e.deviceId); W32(b, (uint32_t)e.localId);
        WS(b, e.serverId); WS(b, e.hostIp); WS(b, e.deviceIp); WS(b, e.superPodId);
        W32(b, e.pid); W32(b, e.platKind); WS(b, e.busId); W32(b, e.nvlinkCount); W64(b, e.fabricClique);
        W32(b, (uint32_t)e.levels.size());
        for (auto &L : e.levels) {
            W32(b, L.netLayer); WS(b, L.netInstanceId); WS(b, L.netType); WS(b, L.netAttr);
            W32(b, (uint32_t)L.addrs.size());
            for (auto &A : L.addrs) {
                WS(b, A.addrType); WS(b, A.addr); W32(b, (uint32_t)A.planeId);
                W32(b, (uint32_t)A.ports.size());
                for (auto &p : A.ports) WS(b, p);
            }
        }
    }
    W32(b, Crc32(b.data(), b.size()));
    return b;
}

HcclResult RankTable::Deserialize(const std::vector<uint8_t> &bytes)
{
    if (bytes.size() < 12) return HCCL_E_PARA;
    uint32_t crc;
    memcpy(&crc, bytes.data() + bytes.size() - 4, 4);
    if (crc != Crc32(bytes.data(), bytes.size() - 4)) {
        HCCL_ERROR("rank table stream fails its CRC check");
        return HCCL_E_PARA;
    }
    R r{bytes.data(), bytes.data() + bytes.size() - 4};
    if (r.u32() != 0x48435254) return HCCL_E_PARA;
    version = r.s();
    uint32_t n = r.u32();
    if (!r.ok || n > kMaxRanks) return HCCL_E_PARA;
    ranks.assign(n, RankEntry());
    for (auto &e : ranks) {
        e.rankId = r.u32(); e.deviceId = (int32_t)r.u32(); e.localId = (int32_t)r.u32();
        e.serverId = r.s(); e.hostIp = r.s(); e.deviceIp = r.s(); e.superPodId = r.s();
        e.pid = r.u32(); e.platKind = r.u32(); e.busId = r.s(); e.nvlinkCount = r.u32(); e.fabricClique = r.u64();
        uint32_t nl = r.u32();
        if (!r.ok || nl > kMaxNetLayers) return HCCL_E_PARA;
        e.levels.assign(nl, RankLevel());
        for (auto &L : e.levels) {
            L.netLayer = r.u32(); L.netInstanceId = r.s(); L.netType = r.s(); L.netAttr = r.s();
            uint32_t na = r.u32();
            if (!r.ok || na > 64) return HCCL_E_PARA;
            L.addrs.assign(na, RankAddr());
            for (auto &A : L.addrs) {
                A.addrType = r.s(); A.addr = r.s(); A.planeId = (int)r.u32();
                uint32_t np = r.u32();
                if (!r.ok || np > 64) return HCCL_E_PARA;
                for (uint32_t i = 0; i < np; ++i) A.ports.push_back(r.s());
            }
        }
    }
    return r.ok ? HCCL_SUCCESS : HCCL_E_PARA;
}

uint32_t RankTable::Crc() const
{
    // The CRC used for cross-rank consistency ignores per-process fields (pid).
    RankTable c = *this;
    for (auto &e : c.ranks) e.pid = 0;
    auto b = c.Serialize();
    uint32_t crc;
    memcpy(&crc, b.data() + b.size() - 4, 4);
    return crc;
}

RankTable RankTable::Sub(const std::vector<uint32_t> &rankIds) const
{
    RankTable t;
    t.version = version;
    for (size_t i = 0; i < rankIds.size(); ++i) {
        if (rankIds[i] >= ranks.size()) continue;
        RankEntry e = ranks[rankIds[i]];
        e.rankId = (uint32_t)i;
        t.ranks.push_back(e);
    }
    return t;
}

uint32_t RankTable::ServerCount() const
{
    std::vector<std::string> ids;
    for (auto &e : ranks)
        if (std::find(ids.begin(), ids.end(), e.serverId) == ids.end()) ids.push_back(e.serverId);
    return (uint32_t)ids.size();
}

uint32_t RankTable::ServerIndexOf(uint32_t rank) const
{
    std::vector<std::string> ids;
    for (auto &e : ranks) {
        if (std::find(ids.begin(), ids.end(), e.serverId) == ids.end()) ids.push_back(e.serverId);
        if (e.rankId == rank) return (uint32_t)(std::find(ids.begin(), ids.end(), e.serverId) - ids.begin());
    }
    return 0;
}

}  // namespace hc
