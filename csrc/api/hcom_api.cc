// hcom_api.cc - named-group API (include/hccl/hcom.h): the world group, sub groups by name, rank
// translation, gradient-fusion split strategies and operators addressed by group name.
// Reference: framework/hcom/hcom.cc, hcom_common.cc, gradient_segment/gradient_segment.cc.
#include <arpa/inet.h>
#include <unistd.h>
#include <algorithm>
#include <cstring>
#include <vector>
#include <string>
#include <atomic>
#include <map>
#include <mutex>

#include "../comm/comm.h"
#include "../core/env.h"
#include "../core/log.h"
#include "../core/net.h"
#include "../plat/platform.h"
#include "hccl/hccl.h"
#include "hccl/hccl_res.h"
#include "../coll/ops.h"
#include "hccl/hccl_diag.h"
#include "hccl/hccl_mc2.h"
#include "hccl/hccl_msg.h"
#include "hccl/hcom.h"

using namespace hc;

namespace {

struct GroupRec {
    Comm *comm = nullptr;
    bool owned = false;                      // created here (HcomCreateGroup / HcomInitByRankTable)
    std::vector<uint32_t> worldRanks;        // world rank of each group rank
    // gradient split strategy
    std::vector<uint32_t> idxList;           // segment end indices
    std::vector<float> sizeList;             // segment size percentages
};
std::mutex g_mu;
std::map<std::string, GroupRec> g_groups;
uint64_t g_subId = 1000;

bool ValidName(const char *g) { return g && *g && strlen(g) <= 127; }

GroupRec *Find(const char *group)
{
    auto it = g_groups.find(group ? group : HCCL_WORLD_GROUP);
    return it == g_groups.end() ? nullptr : &it->second;
}

HcclResult CommOf(const char *group, Comm **c)
{
    std::lock_guard<std::mutex> lk(g_mu);
    GroupRec *g = Find(group);
    if (!g) { RPT_ERR("EI0003", "group \"%s\" does not exist", group ? group : HCCL_WORLD_GROUP); return HCCL_E_NOT_FOUND; }
    *c = g->comm;
    return HCCL_SUCCESS;
}

}  // namespace

extern "C" {

HcclResult HcomInitByComm(HcclComm comm)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c);
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_groups.count(HCCL_WORLD_GROUP)) { RPT_ERR("EI0003", "the world group is already initialised"); return HCCL_E_PARA; }
    GroupRec g;
    g.comm = c;
    for (uint32_t i = 0; i < c->nRanks; ++i) g.worldRanks.push_back(i);
    g_groups[HCCL_WORLD_GROUP] = g;
    return HCCL_SUCCESS;
}

HcclResult HcomInitByRankTable(const char *rankTable, uint32_t rankId)
{
    CHK_PTR_NULL(rankTable);
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (g_groups.count(HCCL_WORLD_GROUP)) return HCCL_E_PARA;
    }
    HcclComm comm = nullptr;
    HcclCommConfig cfg;
    HcclCommConfigInit(&cfg);
    snprintf(cfg.hcclCommName, sizeof(cfg.hcclCommName), "%s", HCCL_WORLD_GROUP);
    CHK_RET(HcclCommInitClusterInfoConfig(rankTable, rankId, &cfg, &comm));
    CHK_RET(HcomInitByComm(comm));
    std::lock_guard<std::mutex> lk(g_mu);
    g_groups[HCCL_WORLD_GROUP].owned = true;
    return HCCL_SUCCESS;
}

HcclResult HcomDestroy(void)
{
    std::map<std::string, GroupRec> groups;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        groups.swap(g_groups);
    }
    for (auto &kv : groups)
        if (kv.second.owned && kv.first != HCCL_WORLD_GROUP) HcclCommDestroy((HcclComm)kv.second.comm);
    auto it = groups.find(HCCL_WORLD_GROUP);
    if (it != groups.end() && it->second.owned) HcclCommDestroy((HcclComm)it->second.comm);
    return HCCL_SUCCESS;
}

HcclResult HcomGetInitStatus(bool *initiated)
{
    CHK_PTR_NULL(initiated);
    std::lock_guard<std::mutex> lk(g_mu);
    *initiated = g_groups.count(HCCL_WORLD_GROUP) != 0;
    return HCCL_SUCCESS;
}

// Collective over the ranks of the world group that are listed; ranks outside the list must not call.
HcclResult HcomCreateGroup(const char *group, uint32_t rankNum, uint32_t *rankIds)
{
    if (!ValidName(group)) { RPT_ERR("EI0003", "group name is empty or longer than 127 characters"); return HCCL_E_PARA; }
    CHK_PTR_NULL(rankIds);
    if (rankNum == 0) return HCCL_E_PARA;
    Comm *world = nullptr;
    uint64_t subId;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        GroupRec *w = Find(HCCL_WORLD_GROUP);
        if (!w) { RPT_ERR("EI0003", "create the world group first (HcomInitByRankTable / HcomInitByComm)"); return HCCL_E_NOT_FOUND; }
        if (g_groups.count(group)) { RPT_ERR("EI0003", "group \"%s\" already exists", group); return HCCL_E_PARA; }
        world = w->comm;
        subId = g_subId++;
    }
    uint32_t myIdx = ~0u;
    for (uint32_t i = 0; i < rankNum; ++i)
        if (rankIds[i] == world->rank) myIdx = i;
    if (myIdx == ~0u) { RPT_ERR("EI0003", "rank %u creates group \"%s\" without being a member", world->rank, group); return HCCL_E_PARA; }
    HcclCommConfig cfg;
    HcclCommConfigInit(&cfg);
    snprintf(cfg.hcclCommName, sizeof(cfg.hcclCommName), "%s", group);
    cfg.hcclBufferSize = world->cfg.bufferMB;
    HcclComm parent = (HcclComm)world, sub = nullptr;
    // the sub id must agree on all members: derive it from the name, not from a local counter
    subId = Crc32(group, strlen(group), 0x6772);
    CHK_RET(HcclCreateSubCommConfig(&parent, rankNum, rankIds, subId, myIdx, &cfg, &sub));
    GroupRec g;
    g.comm = AsComm(sub);
    g.owned = true;
    g.worldRanks.assign(rankIds, rankIds + rankNum);
    std::lock_guard<std::mutex> lk(g_mu);
    g_groups[group] = g;
    return HCCL_SUCCESS;
}

HcclResult HcomDestroyGroup(const char *group)
{
    if (!ValidName(group)) return HCCL_E_PARA;
    if (strcmp(group, HCCL_WORLD_GROUP) == 0) { RPT_ERR("EI0003", "the world group is destroyed with HcomDestroy"); return HCCL_E_PARA; }
    GroupRec g;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        auto it = g_groups.find(group);
        if (it == g_groups.end()) return HCCL_E_NOT_FOUND;
        g = it->second;
        g_groups.erase(it);
    }
    return g.owned ? HcclCommDestroy((HcclComm)g.comm) : HCCL_SUCCESS;
}

HcclResult HcomGetCommHandleByGroup(const char *group, HcclComm *commHandle)
{
    CHK_PTR_NULL(commHandle);
    Comm *c;
    CHK_RET(CommOf(group, &c));
    *commHandle = (HcclComm)c;
    return HCCL_SUCCESS;
}

HcclResult HcomGetRankSize(const char *group, uint32_t *rankSize)
{
    CHK_PTR_NULL(rankSize);
    Comm *c;
    CHK_RET(CommOf(group, &c));
    *rankSize = c->nRanks;
    return HCCL_SUCCESS;
}

HcclResult HcomGetRankId(const char *group, uint32_t *rankId)
{
    CHK_PTR_NULL(rankId);
    Comm *c;
    CHK_RET(CommOf(group, &c));
    *rankId = c->rank;
    return HCCL_SUCCESS;
}

HcclResult HcomGetLocalRankSize(const char *group, uint32_t *localRankSize)
{
    CHK_PTR_NULL(localRankSize);
    Comm *c;
    CHK_RET(CommOf(group, &c));
    const NetInstance *ni = c->graph.InstanceOf(0, c->rank);
    *localRankSize = ni ? (uint32_t)ni->ranks.size() : 1;
    return HCCL_SUCCESS;
}

HcclResult HcomGetLocalRankId(const char *group, uint32_t *localRankId)
{
    CHK_PTR_NULL(localRankId);
    Comm *c;
    CHK_RET(CommOf(group, &c));
    const NetInstance *ni = c->graph.InstanceOf(0, c->rank);
    *localRankId = 0;
    if (ni) *localRankId = (uint32_t)(std::lower_bound(ni->ranks.begin(), ni->ranks.end(), c->rank) - ni->ranks.begin());
    return HCCL_SUCCESS;
}

HcclResult HcomGetWorldRankFromGroupRank(const char *group, uint32_t groupRank, uint32_t *worldRank)
{
    CHK_PTR_NULL(worldRank);
    std::lock_guard<std::mutex> lk(g_mu);
    GroupRec *g = Find(group);
    if (!g) return HCCL_E_NOT_FOUND;
    if (groupRank >= g->worldRanks.size()) return HCCL_E_PARA;
    *worldRank = g->worldRanks[groupRank];
    return HCCL_SUCCESS;
}

HcclResult HcomGetGroupRankFromWorldRank(uint32_t worldRank, const char *group, uint32_t *groupRank)
{
    CHK_PTR_NULL(groupRank);
    std::lock_guard<std::mutex> lk(g_mu);
    GroupRec *g = Find(group);
    if (!g) return HCCL_E_NOT_FOUND;
    for (uint32_t i = 0; i < g->worldRanks.size(); ++i)
        if (g->worldRanks[i] == worldRank) { *groupRank = i; return HCCL_SUCCESS; }
    return HCCL_E_PARA;
}

// ------------------------------------------------------------------- gradient fusion strategy
// By index: idxList are the (ascending) indices of the last gradient of each segment.
// By size:  sizeList are percentages of the total gradient bytes per segment, summing to 100.

HcclResult HcomSetGradFusionByIndex(const char *group, uint32_t segmentNum, const uint32_t *idxList)
{
    CHK_PTR_NULL(idxList);
    if (segmentNum == 0 || segmentNum > 8) { RPT_ERR("EI0003", "1 to 8 segments are supported, got %u", segmentNum); return HCCL_E_PARA; }
    for (uint32_t i = 1; i < segmentNum; ++i)
        if (idxList[i] <= idxList[i - 1]) { RPT_ERR("EI0003", "segment indices must be strictly ascending"); return HCCL_E_PARA; }
    std::lock_guard<std::mutex> lk(g_mu);
    GroupRec *g = Find(group);
    if (!g) return HCCL_E_NOT_FOUND;
    g->idxList.assign(idxList, idxList + segmentNum);
    g->sizeList.clear();
    return HCCL_SUCCESS;
}

HcclResult HcomSetGradFusionBySize(const char *group, uint32_t segmentNum, const float *sizeList)
{
    CHK_PTR_NULL(sizeList);
    if (segmentNum == 0 || segmentNum > 8) return HCCL_E_PARA;
    float sum = 0;
    for (uint32_t i = 0; i < segmentNum; ++i) {
        if (sizeList[i] < 0) return HCCL_E_PARA;
        sum += sizeList[i];
    }
    if (sum < 99.999f || sum > 100.001f) { RPT_ERR("EI0003", "segment sizes must sum to 100 percent, got %f", sum); return HCCL_E_PARA; }
    std::lock_guard<std::mutex> lk(g_mu);
    GroupRec *g = Find(group);
    if (!g) return HCCL_E_NOT_FOUND;
    g->sizeList.assign(sizeList, sizeList + segmentNum);
    g->idxList.clear();
    return HCCL_SUCCESS;
}

HcclResult HcomGetSplitStrategy(const char *group, uint32_t gradNum, const uint64_t *gradBytes, uint32_t *segIdx, uint32_t *segNum)
{
    CHK_PTR_NULL(segIdx); CHK_PTR_NULL(segNum);
    if (gradNum == 0) return HCCL_E_PARA;
    std::lock_guard<std::mutex> lk(g_mu);
    GroupRec *g = Find(group);
    if (!g) return HCCL_E_NOT_FOUND;
    std::vector<uint32_t> out;
    if (!g->idxList.empty()) {
        for (uint32_t v : g->idxList)
            if (v < gradNum - 1) out.push_back(v);
        out.push_back(gradNum - 1);
    } else if (!g->sizeList.empty() && gradBytes) {
        long double total = 0, acc = 0, target = 0;
        for (uint32_t i = 0; i < gradNum; ++i) total += gradBytes[i];
        size_t seg = 0;
        target = total * g->sizeList[0] / 100.0L;
        for (uint32_t i = 0; i < gradNum && seg + 1 < g->sizeList.size(); ++i) {
            acc += gradBytes[i];
            if (acc >= target) {
                if (i < gradNum - 1 && (out.empty() || out.back() != i)) out.push_back(i);
                ++seg;
                target += total * g->sizeList[seg] / 100.0L;
            }
        }
        out.push_back(gradNum - 1);
    } else {
        // default of the reference: two segments, the first holding ~96.54 % of the bytes
        if (gradBytes && gradNum > 1) {
            long double total = 0, acc = 0;
            for (uint32_t i = 0; i < gradNum; ++i) total += gradBytes[i];
            for (uint32_t i = 0; i < gradNum - 1; ++i) {
                acc += gradBytes[i];
                if (acc >= total * 0.9654L) { out.push_back(i); break; }
            }
        }
        out.push_back(gradNum - 1);
    }
    for (size_t i = 0; i < out.size(); ++i) segIdx[i] = out[i];
    *segNum = (uint32_t)out.size();
    return HCCL_SUCCESS;
}

// ---------------------------------------------------------------------------------- queries

HcclResult HcomGetInCCLbuffer(const char *group, void **buffer, uint64_t *size)
{
    Comm *c;
    CHK_RET(CommOf(group, &c));
    CHK_PTR_NULL(buffer); CHK_PTR_NULL(size);
    *buffer = c->CclBuffer();
    *size = c->halfBytes;
    return HCCL_SUCCESS;
}
HcclResult HcomGetOutCCLbuffer(const char *group, void **buffer, uint64_t *size)
{
    Comm *c;
    CHK_RET(CommOf(group, &c));
    CHK_PTR_NULL(buffer); CHK_PTR_NULL(size);
    *buffer = c->CclBuffer() + c->halfBytes;
    *size = c->halfBytes;
    return HCCL_SUCCESS;
}
HcclResult HcomGetCommCCLBufferSize(const char *group, uint64_t *size)
{
    Comm *c;
    CHK_RET(CommOf(group, &c));
    CHK_PTR_NULL(size);
    *size = c->halfBytes;
    return HCCL_SUCCESS;
}
// Per-direction bandwidth one GPU has at a network level, GB/s.
HcclResult HcomGetBandWidthPerNPU(uint32_t level, float *bandWidthGBs)
{
    CHK_PTR_NULL(bandWidthGBs);
    if (level > 2) return HCCL_E_PARA;
    *bandWidthGBs = level == 0 ? 900.0f : 50.0f;
    return HCCL_SUCCESS;
}
HcclResult HcomGetServerNumAndDeviceNumPerServer(uint32_t *serverNum, uint32_t *deviceNumPerServer, uint32_t *deviceNumPerAggregation)
{
    Comm *c;
    CHK_RET(CommOf(HCCL_WORLD_GROUP, &c));
    uint32_t servers = c->table.ServerCount();
    if (serverNum) *serverNum = servers;
    if (deviceNumPerServer) *deviceNumPerServer = servers ? c->nRanks / servers : c->nRanks;
    if (deviceNumPerAggregation) *deviceNumPerAggregation = servers ? c->nRanks / servers : c->nRanks;
    return HCCL_SUCCESS;
}
HcclResult HcomGetAlgorithm(uint32_t level, char **algo)
{
    CHK_PTR_NULL(algo);
    static thread_local char buf[64];
    Comm *c;
    CHK_RET(CommOf(HCCL_WORLD_GROUP, &c));
    snprintf(buf, sizeof(buf), "%s", level == 0 ? (c->cfg.algo.empty() ? "fullmesh" : c->cfg.algo.c_str()) : "NA");
    *algo = buf;
    return HCCL_SUCCESS;
}
HcclResult HcomGetL0TopoTypeEx(const char *group, CommTopo *topoType, uint32_t flag)
{
    (void)flag;
    Comm *c;
    CHK_RET(CommOf(group, &c));
    CHK_PTR_NULL(topoType);
    const NetInstance *ni = c->graph.InstanceOf(0, c->rank);
    *topoType = ni ? ni->topo : COMM_TOPO_1DMESH;
    return HCCL_SUCCESS;
}
HcclResult HcomSupportDeterministicOptim(const char *group, bool *isDeterministicOptim)
{
    Comm *c;
    CHK_RET(CommOf(group, &c));
    CHK_PTR_NULL(isDeterministicOptim);
    *isDeterministicOptim = true;   // the mesh kernels always reduce in rank order
    return HCCL_SUCCESS;
}

// ---------------------------------------------------------------------- operators by group name

#define HCOM_COMM(group) Comm *c; CHK_RET(CommOf(group, &c)); (void)tag

HcclResult HcomAllReduce(const char *tag, void *in, void *out, uint64_t count, HcclDataType dataType, HcclReduceOp op, const char *group, aclrtStream stream)
{ HCOM_COMM(group); return HcclAllReduce(in, out, count, dataType, op, (HcclComm)c, stream); }
HcclResult HcomAllGather(const char *tag, void *in, void *out, uint64_t inCount, HcclDataType dataType, const char *group, aclrtStream stream)
{ HCOM_COMM(group); return HcclAllGather(in, out, inCount, dataType, (HcclComm)c, stream); }
HcclResult HcomReduceScatter(const char *tag, void *in, void *out, uint64_t outCount, HcclDataType dataType, HcclReduceOp op, const char *group, aclrtStream stream)
{ HCOM_COMM(group); return HcclReduceScatter(in, out, outCount, dataType, op, (HcclComm)c, stream); }
HcclResult HcomBroadcast(const char *tag, void *ptr, uint64_t count, HcclDataType dataType, uint32_t root, const char *group, aclrtStream stream)
{ HCOM_COMM(group); return HcclBroadcast(ptr, count, dataType, root, (HcclComm)c, stream); }
HcclResult HcomReduce(const char *tag, void *in, void *out, uint64_t count, HcclDataType dataType, HcclReduceOp op, uint32_t root, const char *group, aclrtStream stream)
{ HCOM_COMM(group); return HcclReduce(in, out, count, dataType, op, root, (HcclComm)c, stream); }
HcclResult HcomSend(const char *tag, void *in, uint64_t count, HcclDataType dataType, uint32_t destRank, uint32_t srTag, const char *group, aclrtStream stream)
{ (void)srTag; HCOM_COMM(group); return HcclSend(in, count, dataType, destRank, (HcclComm)c, stream); }
HcclResult HcomReceive(const char *tag, void *out, uint64_t count, HcclDataType dataType, uint32_t srcRank, uint32_t srTag, const char *group, aclrtStream stream)
{ (void)srTag; HCOM_COMM(group); return HcclRecv(out, count, dataType, srcRank, (HcclComm)c, stream); }
HcclResult HcomAllToAll(const void *in, uint64_t sendCount, HcclDataType sendType, const void *out, uint64_t recvCount, HcclDataType recvType, const char *group,
                        aclrtStream stream, const char *tag)
{ HCOM_COMM(group); return HcclAlltoAll(in, sendCount, sendType, out, recvCount, recvType, (HcclComm)c, stream); }
HcclResult HcomAlltoAllV(const void *in, const void *sendCounts, const void *sdispls, HcclDataType sendType, const void *out, const void *recvCounts,
                         const void *rdispls, HcclDataType recvType, const char *group, aclrtStream stream, const char *tag)
{ HCOM_COMM(group); return HcclAlltoAllV(in, sendCounts, sdispls, sendType, out, recvCounts, rdispls, recvType, (HcclComm)c, stream); }
HcclResult HcomAllGatherV(const char *tag, const void *sendBuf, uint64_t sendCount, const void *recvBuf, const void *recvCounts, const void *rdispls,
                          HcclDataType dataType, const char *group, aclrtStream stream)
{ HCOM_COMM(group); return HcclAllGatherV((void *)sendBuf, sendCount, (void *)recvBuf, recvCounts, rdispls, dataType, (HcclComm)c, stream); }
HcclResult HcomReduceScatterV(const char *tag, void *sendBuf, const void *sendCounts, const void *sdispls, void *recvBuf, uint64_t recvCount, HcclDataType dataType,
                              HcclReduceOp op, const char *group, aclrtStream stream)
{ HCOM_COMM(group); return HcclReduceScatterV(sendBuf, sendCounts, sdispls, recvBuf, recvCount, dataType, op, (HcclComm)c, stream); }
HcclResult HcomAlltoAllVC(const void *sendBuf, const void *sendCountMatrix, HcclDataType sendType, const void *recvBuf, HcclDataType recvType, const char *group,
                          aclrtStream stream, const char *tag)
{ HCOM_COMM(group); return HcclAlltoAllVC(sendBuf, sendCountMatrix, sendType, recvBuf, recvType, (HcclComm)c, stream); }

// ------------------------------------------------------------------ further calls with a meaning here

HcclResult HcomInitByString(const char *rankTableM, const char *identify)
{
    CHK_PTR_NULL(rankTableM); CHK_PTR_NULL(identify);
    char *end = nullptr;
    unsigned long rank = strtoul(identify, &end, 10);
    if (end == identify || *end != 0) { RPT_ERR("EI0003", "HcomInitByString: \"%s\" is not a rank id", identify); return HCCL_E_PARA; }
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (g_groups.count(HCCL_WORLD_GROUP)) return HCCL_E_PARA;
    }
    HcclComm comm = nullptr;
    CHK_RET(HcclInitComm(rankTableM, (uint32_t)rank, nullptr, &comm));
    CHK_RET(HcomInitByComm(comm));
    std::lock_guard<std::mutex> lk(g_mu);
    g_groups[HCCL_WORLD_GROUP].owned = true;
    return HCCL_SUCCESS;
}

namespace {
struct MasterJoin { uint32_t magic; uint32_t ip; int32_t device; uint32_t pid; };
struct MasterAnswer { uint32_t magic; uint32_t rank; HcclRootInfo info; };
constexpr uint32_t kJoinMagic = 0x4e494f4a, kAnswerMagic = 0x57534e41;   // "JOIN", "ANSW"

bool ParseNumber(const char *s, long lo, long hi, long *out)
{
    if (!s || !*s) return false;
    char *end = nullptr;
    long v = strtol(s, &end, 10);
    if (*end != 0 || v < lo || v > hi) return false;
    *out = v;
    return true;
}
}  // namespace

HcclResult HcomInitByMasterInfo(const char *masterIp, const char *masterPort, const char *masterDeviceId, const char *rankSize, const char *rankIp)
{
    CHK_PTR_NULL(masterIp); CHK_PTR_NULL(masterPort); CHK_PTR_NULL(masterDeviceId); CHK_PTR_NULL(rankSize); CHK_PTR_NULL(rankIp);
    long port = 0, masterDev = 0, n = 0;
    struct in_addr mine4, master4;
    if (!ParseNumber(masterPort, 1, 65535, &port) || !ParseNumber(masterDeviceId, 0, 1 << 20, &masterDev) || !ParseNumber(rankSize, 1, 1 << 20, &n) ||
        inet_pton(AF_INET, masterIp, &master4) != 1 || inet_pton(AF_INET, rankIp, &mine4) != 1) {
        RPT_ERR("EI0003", "HcomInitByMasterInfo: master %s:%s device %s, %s ranks, own address %s - not all of these are numbers and IPv4 addresses", masterIp,
                masterPort, masterDeviceId, rankSize, rankIp);
        return HCCL_E_PARA;
    }
    {
        std::lock_guard<std::mutex> lk(g_mu);
        if (g_groups.count(HCCL_WORLD_GROUP)) { RPT_ERR("EI0003", "the world group is already initialised"); return HCCL_E_PARA; }
    }
    Platform *P = DefaultPlatform();
    MasterJoin me{kJoinMagic, mine4.s_addr, P ? P->CurrentDevice() : 0, (uint32_t)getpid()};
    const int64_t deadline = net::NowMs() + (int64_t)EnvConfig::Get().connectTimeoutSec.value * 1000;
    MasterAnswer answer;
    memset(&answer, 0, sizeof(answer));

    int listenFd = -1, listenPort = 0;
    // Whoever sits at the master's address on the master's device serves; if the port is taken there, somebody else does.
    if (mine4.s_addr == master4.s_addr && me.device == (int32_t)masterDev) {
        if (net::TcpListen(masterIp, (int)port, (int)port, &listenFd, &listenPort) != HCCL_SUCCESS) listenFd = -1;
    }
    if (listenFd >= 0) {
        struct Entry { MasterJoin join; int fd; uint32_t arrival; };
        std::vector<Entry> entries{{me, -1, 0}};
        HcclResult r = HCCL_SUCCESS;
        while (entries.size() < (size_t)n && r == HCCL_SUCCESS) {
            int fd = -1;
            r = net::TcpAccept(listenFd, deadline, &fd, nullptr);
            if (r != HCCL_SUCCESS) break;
            MasterJoin j;
            if (net::RecvAll(fd, &j, sizeof(j), net::NowMs() + 3000) != HCCL_SUCCESS || j.magic != kJoinMagic) { net::Close(fd); continue; }   // not one of ours
            entries.push_back({j, fd, (uint32_t)entries.size()});
        }
        if (r == HCCL_SUCCESS) r = HcclGetRootInfo(&answer.info);
        if (r == HCCL_SUCCESS) {
            std::stable_sort(entries.begin(), entries.end(), [](const Entry &a, const Entry &b) {
                if (a.join.ip != b.join.ip) return ntohl(a.join.ip) < ntohl(b.join.ip);
                if (a.join.device != b.join.device) return a.join.device < b.join.device;
                return a.arrival < b.arrival;
            });
            answer.magic = kAnswerMagic;
            uint32_t myRank = 0;
            for (uint32_t i = 0; i < entries.size(); ++i) {
                if (entries[i].fd < 0) { myRank = i; continue; }
                answer.rank = i;
                if (net::SendAll(entries[i].fd, &answer, sizeof(answer)) != HCCL_SUCCESS) r = HCCL_E_TCP_TRANSFER;
            }
            answer.rank = myRank;
        } else {
            RPT_ERR("EI0015", "HcomInitByMasterInfo: %zu of %ld processes reached the master at %s:%ld in time", entries.size(), n, masterIp, port);
        }
        for (auto &e : entries) net::Close(e.fd);
        net::Close(listenFd);
        if (r != HCCL_SUCCESS) return r;
    } else {
        int fd = -1;
        HcclResult r = net::TcpConnect(masterIp, (int)port, deadline, &fd);
        if (r != HCCL_SUCCESS) { RPT_ERR("EI0006", "HcomInitByMasterInfo: nobody answers at %s:%ld", masterIp, port); return HCCL_E_TIMEOUT; }
        r = net::SendAll(fd, &me, sizeof(me));
        if (r == HCCL_SUCCESS) r = net::RecvAll(fd, &answer, sizeof(answer), deadline);
        net::Close(fd);
        if (r != HCCL_SUCCESS || answer.magic != kAnswerMagic) {
            RPT_ERR("EI0015", "HcomInitByMasterInfo: the master at %s:%ld did not hand out a rank", masterIp, port);
            return r != HCCL_SUCCESS ? r : HCCL_E_INTERNAL;
        }
    }
    HcclComm comm = nullptr;
    HcclCommConfig cfg;
    HcclCommConfigInit(&cfg);
    snprintf(cfg.hcclCommName, sizeof(cfg.hcclCommName), "%s", HCCL_WORLD_GROUP);
    CHK_RET(HcclCommInitRootInfoConfig((uint32_t)n, &answer.info, answer.rank, &cfg, &comm));
    CHK_RET(HcomInitByComm(comm));
    std::lock_guard<std::mutex> lk(g_mu);
    g_groups[HCCL_WORLD_GROUP].owned = true;
    return HCCL_SUCCESS;
}

bool HcomFindGroup(const char *group)
{
    if (!group) return false;
    std::lock_guard<std::mutex> lk(g_mu);
    return g_groups.count(group) != 0;
}

HcclResult HcomGetRankSizeEx(const char *group, uint32_t *rankSize, uint32_t flag)
{
    (void)flag;
    return HcomGetRankSize(group, rankSize);
}

HcclResult HcomReleaseSubComms(void)
{
    std::vector<GroupRec> gone;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        for (auto it = g_groups.begin(); it != g_groups.end();) {
            if (it->first == HCCL_WORLD_GROUP) { ++it; continue; }
            gone.push_back(it->second);
            it = g_groups.erase(it);
        }
    }
    HcclResult first = HCCL_SUCCESS;
    for (auto &g : gone)
        if (g.owned) { HcclResult r = HcclCommDestroy((HcclComm)g.comm); if (r != HCCL_SUCCESS && first == HCCL_SUCCESS) first = r; }
    return first;
}

HcclResult HcomCreateCommCCLbuffer(const char *group)
{
    Comm *c;
    CHK_RET(CommOf(group, &c));
    return c->CclBuffer() ? HCCL_SUCCESS : HCCL_E_MEMORY;
}

static std::atomic<int> g_workflowMode{(int)HCCL_WORKFLOW_MODE_OP_BASE};
HcclWorkflowMode HcomGetWorkflowMode(void) { return (HcclWorkflowMode)g_workflowMode.load(); }
HcclResult HcomSetWorkflowMode(HcclWorkflowMode mode)
{
    if (mode != HCCL_WORKFLOW_MODE_OPS_KERNEL_INFO_LIB && mode != HCCL_WORKFLOW_MODE_OP_BASE) return HCCL_E_PARA;
    g_workflowMode.store((int)mode);
    return HCCL_SUCCESS;
}

HcclResult HcomSetProfilingMode(HcomProfilingMode profilingMode, const char *profilingOption)
{
    (void)profilingOption;
    if (profilingMode != PROFILING_CLOSE && profilingMode != PROFILING_OPEN) return HCCL_E_PARA;
    std::vector<Comm *> comms;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        for (auto &kv : g_groups) comms.push_back(kv.second.comm);
    }
    for (Comm *c : comms) CHK_RET(HcclDiagSetProfiling((HcclComm)c, profilingMode == PROFILING_OPEN));
    return HCCL_SUCCESS;
}

static HcclResult Describe(int64_t comm, const char *group, uint64_t count, void *counts, HcclDataType dataType, HcclReduceOp op, HcclCMDType opType,
                           int32_t aivCoreLimit, Selection *sel, int *ctas)
{
    Comm *c = comm ? AsComm((HcclComm)(intptr_t)comm) : nullptr;
    if (!c) CHK_RET(CommOf(group, &c));
    CHK_RET(DescribeSelection(c, opType, count, dataType, op, counts != nullptr, sel, ctas));
    if (ctas && aivCoreLimit > 0 && *ctas > aivCoreLimit) *ctas = aivCoreLimit;
    return HCCL_SUCCESS;
}

HcclResult HcomSelectAlg(int64_t comm, const char *group, uint64_t count, void *counts, HcclDataType dataType, HcclReduceOp op, HcclCMDType opType,
                         int32_t aivCoreLimit, bool *ifAiv, char *algName)
{
    CHK_PTR_NULL(ifAiv); CHK_PTR_NULL(algName);
    Selection sel;
    CHK_RET(Describe(comm, group, count, counts, dataType, op, opType, aivCoreLimit, &sel, nullptr));
    *ifAiv = sel.engine != Engine::HOST;
    snprintf(algName, 128, "%s", sel.name.c_str());
    return HCCL_SUCCESS;
}

HcclResult HcomCalcAivCoreNum(const char *group, HcclCMDType opType, uint64_t count, void *counts, HcclDataType dataType, int32_t aivCoreLimit, char *algName,
                              uint32_t *numBlocks)
{
    CHK_PTR_NULL(numBlocks);
    Selection sel;
    int ctas = 0;
    CHK_RET(Describe(0, group, count, counts, dataType, HCCL_REDUCE_SUM, opType, aivCoreLimit, &sel, &ctas));
    if (algName) snprintf(algName, 128, "%s", sel.name.c_str());
    *numBlocks = (uint32_t)ctas;
    return HCCL_SUCCESS;
}

HcclResult HcomSetAivCoreLimit(const char *group, uint32_t aivCoreLimit)
{
    Comm *c;
    CHK_RET(CommOf(group, &c));
    __atomic_store_n(&c->ctaLimit, aivCoreLimit, __ATOMIC_RELAXED);
    return HCCL_SUCCESS;
}

HcclResult HcomGenerateCclOpTag(const char *opType, int64_t hcomComm, const char *group, char *sTag)
{
    CHK_PTR_NULL(opType); CHK_PTR_NULL(sTag);
    (void)hcomComm;
    static std::mutex mu;
    static std::map<std::string, uint64_t> next;        // every rank issues its operators in the same order: the counters agree
    const std::string key = std::string(opType) + "_" + (group ? group : HCCL_WORLD_GROUP);
    uint64_t n;
    {
        std::lock_guard<std::mutex> lk(mu);
        n = next[key]++;
    }
    snprintf(sTag, 256, "%s_%llu", key.c_str(), (unsigned long long)n);
    return HCCL_SUCCESS;
}

HcclResult HcomCreateComResourceByComm(HcclComm comm, uint32_t streamMode, bool isOpbaseMode, void **commContext)
{
    (void)isOpbaseMode;
    return HcclAllocComResource(comm, streamMode, commContext);
}
HcclResult HcomGetAicpuOpStreamNotify(const char *group, aclrtStream *opStream, uint8_t aicpuNotifyNum, void **aicpuNotify)
{
    Comm *c;
    CHK_RET(CommOf(group, &c));
    return HcclGetAicpuOpStreamAndNotify((HcclComm)c, opStream, aicpuNotifyNum, aicpuNotify);
}
HcclResult HcomMc2AiCpuStreamAllocAndGet(const char *group, uint32_t streamMode, aclrtStream *aiCpuStream)
{
    (void)streamMode;
    Comm *c;
    CHK_RET(CommOf(group, &c));
    return HcclGetAicpuOpStreamAndNotify((HcclComm)c, aiCpuStream, 0, nullptr);
}

}  // extern "C"
