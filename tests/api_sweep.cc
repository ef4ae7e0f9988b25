// Calls the exported entry points that the scenario tests do not reach, with ranks as threads of this process on the host
// simulator, and checks what they return.  Built and run by tests/test_api_sweep.py; usage: api_sweep <ranks>.
// (The reference reaches its API the same way: ranks as threads over a stub runtime, test/ut/inter/hcom/*.cc.)
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cmath>
#include <cstring>
#include <fstream>
#include <numeric>
#include <sstream>
#include <string>

#include "../examples/common.h"
#include "hccl/hccl_channel.h"
#include "hccl/hccl_dfx.h"
#include "hccl/hccl_diag.h"
#include "hccl/hccl_launch.h"
#include "hccl/hccl_mc2.h"
#include "hccl/hccl_msg.h"
#include "hccl/hccl_one_sided.h"
#include "hccl/hccl_rank_graph.h"
#include "hccl/hccl_res.h"
#include "hccl/hccl_sym_win.h"
#include "hccl/hccl_team.h"
#include "hccl/hcom.h"
#include "hcomm_primitives.h"
#include "hcomm_res.h"

#define EXPECT_RC(call, want) EX_EXPECT((int)(call) == (int)(want))

// ------------------------------------------------------------------------------------------------ topology queries

static void RankGraph(uint32_t rank, uint32_t n, HcclComm comm)
{
    uint32_t *layers = nullptr, layerNum = 0;
    EX_CHECK(HcclRankGraphGetLayers(comm, &layers, &layerNum));
    EX_EXPECT(layerNum == 1 && layers[0] == 0);
    uint32_t *ranks = nullptr, rankNum = 0;
    EX_CHECK(HcclRankGraphGetRanksByLayer(comm, 0, &ranks, &rankNum));
    EX_EXPECT(rankNum == n);
    for (uint32_t i = 0; i < n; ++i) EX_EXPECT(ranks[i] == i);
    EXPECT_RC(HcclRankGraphGetRanksByLayer(comm, 7, &ranks, &rankNum), HCCL_E_PARA);
    EX_CHECK(HcclRankGraphGetRankSizeByLayer(comm, 0, &rankNum));
    EX_EXPECT(rankNum == n);
    EXPECT_RC(HcclRankGraphGetRankSizeByLayer(comm, 3, &rankNum), HCCL_E_PARA);
    CommTopo topo = COMM_TOPO_RESERVED;
    EX_CHECK(HcclRankGraphGetTopoTypeByLayer(comm, 0, &topo));
    EX_EXPECT(topo == COMM_TOPO_1DMESH);
    uint32_t *sizes = nullptr, sizeNum = 0;
    EX_CHECK(HcclRankGraphGetInstSizeListByLayer(comm, 0, &sizes, &sizeNum));
    EX_EXPECT(sizeNum == 1 && sizes[0] == n);
    EXPECT_RC(HcclRankGraphGetInstSizeListByLayer(comm, 2, &sizes, &sizeNum), HCCL_E_PARA);
    uint32_t *insts = nullptr, instNum = 0;
    EX_CHECK(HcclRankGraphGetTopoInstsByLayer(comm, 0, &insts, &instNum));
    EX_EXPECT(instNum == 1);
    const uint32_t inst = insts[0];
    topo = COMM_TOPO_RESERVED;
    EX_CHECK(HcclRankGraphGetTopoType(comm, 0, inst, &topo));
    EX_EXPECT(topo == COMM_TOPO_1DMESH);
    EXPECT_RC(HcclRankGraphGetTopoType(comm, 0, inst + 99, &topo), HCCL_E_PARA);
    EX_CHECK(HcclRankGraphGetRanksByTopoInst(comm, 0, inst, &ranks, &rankNum));
    EX_EXPECT(rankNum == n && ranks[n - 1] == n - 1);
    HcclHeterogMode mode = HCCL_HETEROG_MODE_INVALID;
    EX_CHECK(HcclGetHeterogMode(comm, &mode));
    EX_EXPECT(mode == HCCL_HETEROG_MODE_HOMOGENEOUS);
    uint32_t epNum = 0;
    EX_CHECK(HcclRankGraphGetEndpointNum(comm, 0, inst, &epNum));
    EX_EXPECT(epNum == 1);
    EndpointDesc ep;
    EX_CHECK(EndpointDescInit(&ep, 1));
    uint32_t descNum = 0;
    EXPECT_RC(HcclRankGraphGetEndpointDesc(comm, 0, inst, &descNum, &ep), HCCL_E_PARA);       // room for none
    descNum = 1;
    EX_CHECK(HcclRankGraphGetEndpointDesc(comm, 0, inst, &descNum, &ep));
    EX_EXPECT(descNum == 1);
    uint32_t v = 0;
    EX_CHECK(HcclRankGraphGetEndpointInfo(comm, rank, &ep, ENDPOINT_ATTR_BW_COEFF, sizeof(v), &v));
    EX_EXPECT(v >= 1);
    EX_CHECK(HcclRankGraphGetEndpointInfo(comm, rank, &ep, ENDPOINT_ATTR_LOCATION, sizeof(v), &v));
    EX_EXPECT(v == (uint32_t)ENDPOINT_LOC_TYPE_DEVICE);
    EXPECT_RC(HcclRankGraphGetEndpointInfo(comm, n, &ep, ENDPOINT_ATTR_DIE_ID, sizeof(v), &v), HCCL_E_PARA);
    EXPECT_RC(HcclRankGraphGetEndpointInfo(comm, rank, &ep, ENDPOINT_ATTR_DIE_ID, 2, &v), HCCL_E_PARA);
    if (n > 1) {
        CommLink *links = nullptr;
        uint32_t linkNum = 0;
        EX_CHECK(HcclRankGraphGetLinks(comm, 0, rank, (rank + 1) % n, &links, &linkNum));
        EX_EXPECT(linkNum >= 1 && links[0].linkAttr.hop >= 1);
    }
}

// ------------------------------------------------------------------------- communicator queries, process configuration

static std::atomic<int> g_stateCalls{0};
static HcclResult OnState(HcclComm, HcclCommStatePhase phase, void *args)
{
    if (args == (void *)&g_stateCalls && (phase == HCCL_COMM_STATE_PHASE_RESUME_PRE || phase == HCCL_COMM_STATE_PHASE_RESUME_POST)) ++g_stateCalls;
    return HCCL_SUCCESS;
}

static void CommQueries(uint32_t rank, uint32_t n, HcclComm comm)
{
    char name[COMM_NAME_MAX_LENGTH] = "";
    EX_CHECK(HcclGetCommName(comm, name));
    HcclComm found = nullptr;
    EX_CHECK(HcclCommGetHandleWithName(name, &found));
    EX_EXPECT(found != nullptr);                           // ranks of one process share the name; any of them is a hit
    EXPECT_RC(HcclCommGetHandleWithName("no such communicator", &found), HCCL_E_NOT_FOUND);
    HcclCommStatus status = HCCL_COMM_STATUS_RESERVED;
    EX_CHECK(HcclCommGetStatus(name, &status));
    EX_EXPECT(status == HCCL_COMM_STATUS_READY);
    EXPECT_RC(HcclCommGetStatus("no such communicator", &status), HCCL_E_NOT_FOUND);
    EX_EXPECT(status == HCCL_COMM_STATUS_INVALID);
    EX_EXPECT(std::string(HcclGetErrorString(HCCL_E_TIMEOUT)) == "timeout");
    EX_EXPECT(std::string(HcclGetErrorString((HcclResult)9999)) == "unknown error");

    std::vector<uint32_t> ranks(n);
    std::iota(ranks.begin(), ranks.end(), 0u);
    std::vector<char> backup(n, 0);
    EX_CHECK(HcclCommWorkingDevNicSet(comm, ranks.data(), (bool *)backup.data(), n));
    backup[0] = 1;                                         // one switch, one path: there is no backup port to move to
    EXPECT_RC(HcclCommWorkingDevNicSet(comm, ranks.data(), (bool *)backup.data(), n), HCCL_E_NOT_SUPPORT);
    ranks[0] = n;
    backup[0] = 0;
    EXPECT_RC(HcclCommWorkingDevNicSet(comm, ranks.data(), (bool *)backup.data(), n), HCCL_E_PARA);

    HcclOpExpansionMode mode = HCCL_OP_EXPANSION_MODE_INVALID;
    EX_CHECK(HcclConfigGetInfo(comm, HCCL_CONFIG_TYPE_OP_EXPANSION_MODE, sizeof(mode), &mode));
    EX_EXPECT(mode == HCCL_OP_EXPANSION_MODE_HOST);        // the simulator runs everything on the host engine
    char algo[64] = "";
    EX_CHECK(HcclConfigGetInfo(comm, HCCL_CONFIG_TYPE_HCCL_ALGO, sizeof(algo), algo));
    EX_EXPECT(std::string(algo) == "auto");
    EXPECT_RC(HcclConfigGetInfo(comm, HCCL_CONFIG_TYPE_HCCL_ALGO, 2, algo), HCCL_E_PARA);
    EXPECT_RC(HcclConfigGetInfo(comm, (HcclConfigType)7, sizeof(algo), algo), HCCL_E_NOT_SUPPORT);

    // the process-wide deterministic switch: set by one rank between two barriers, seen by all
    EX_CHECK(HcclBarrier(comm, nullptr));
    union HcclConfigValue value;
    if (rank == 0) {
        value.value = 1;
        EX_CHECK(HcclSetConfig(HCCL_DETERMINISTIC, value));
        EXPECT_RC(HcclSetConfig(HCCL_CONFIG_RESERVED, value), HCCL_E_NOT_SUPPORT);
    }
    EX_CHECK(HcclBarrier(comm, nullptr));
    value.value = -1;
    EX_CHECK(HcclGetConfig(HCCL_DETERMINISTIC, &value));
    EX_EXPECT(value.value == 1);
    EXPECT_RC(HcclGetConfig(HCCL_CONFIG_RESERVED, &value), HCCL_E_NOT_SUPPORT);
    EX_CHECK(HcclBarrier(comm, nullptr));
    if (rank == 0) {
        value.value = 0;
        EX_CHECK(HcclSetConfig(HCCL_DETERMINISTIC, value));
    }
    EX_CHECK(HcclBarrier(comm, nullptr));

    // state callbacks fire around a resume
    if (rank == 0) EX_CHECK(HcclCommRegCommStateCallback("sweep", OnState, &g_stateCalls));
    EX_CHECK(HcclBarrier(comm, nullptr));
    EX_CHECK(HcclCommSuspend(comm));
    EX_CHECK(HcclCommGetStatus(name, &status));
    EX_EXPECT(status == HCCL_COMM_STATUS_SUSPENDING || status == HCCL_COMM_STATUS_READY);      // another rank of this name may be looked at
    float one = 1.0f, sum = 0.0f;
    EXPECT_RC(HcclAllReduce(&one, &sum, 1, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, comm, nullptr), HCCL_E_SUSPENDING);
    EX_CHECK(HcclCommResume(comm));
    EX_CHECK(HcclAllReduce(&one, &sum, 1, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, comm, nullptr));
    EX_EXPECT(sum == (float)n);
    EX_EXPECT(g_stateCalls.load() >= 2);
    EX_CHECK(HcclBarrier(comm, nullptr));
    if (rank == 0) EX_CHECK(HcclCommRegCommStateCallback("sweep", nullptr, nullptr));
}

// ------------------------------------------------------ the operators under their second names, grouped calls, fused scale

static void InnerOperators(uint32_t rank, uint32_t n, HcclComm comm)
{
    const uint64_t cnt = 96;
    std::vector<float> x(n * cnt), y(n * cnt, 0.f);
    for (uint64_t i = 0; i < n * cnt; ++i) x[i] = (float)(i % 13) + (float)rank;
    const float rankSum = (float)(n * (n - 1) / 2);

    EX_CHECK(HcclAllReduceInner(x.data(), y.data(), n * cnt, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, comm, nullptr));
    for (uint64_t i = 0; i < n * cnt; ++i) EX_EXPECT(y[i] == (float)n * (float)(i % 13) + rankSum);

    std::vector<float> b(cnt, rank == 1 % n ? 5.f : 0.f);
    EX_CHECK(HcclBroadcastInner(b.data(), cnt, HCCL_DATA_TYPE_FP32, 1 % n, comm, nullptr));
    EX_EXPECT(b[0] == 5.f && b[cnt - 1] == 5.f);

    std::vector<float> rs(cnt, 0.f);
    EX_CHECK(HcclReduceScatterInner(x.data(), rs.data(), cnt, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, comm, nullptr));
    for (uint64_t i = 0; i < cnt; ++i) EX_EXPECT(rs[i] == (float)n * (float)((rank * cnt + i) % 13) + rankSum);

    std::vector<float> ag(n * cnt, 0.f);
    EX_CHECK(HcclAllGatherInner(x.data(), ag.data(), cnt, HCCL_DATA_TYPE_FP32, comm, nullptr));
    for (uint32_t q = 0; q < n; ++q) EX_EXPECT(ag[q * cnt + 5] == 5.f + (float)q);

    // variable counts: rank q owns q + 1 elements
    std::vector<uint64_t> counts(n), displs(n);
    uint64_t total = 0;
    for (uint32_t q = 0; q < n; ++q) { counts[q] = q + 1; displs[q] = total; total += q + 1; }
    std::vector<float> mine(rank + 1, (float)rank), agv(total, -1.f);
    EX_CHECK(HcclAllGatherVInner(mine.data(), rank + 1, agv.data(), counts.data(), displs.data(), HCCL_DATA_TYPE_FP32, comm, nullptr));
    for (uint32_t q = 0; q < n; ++q) EX_EXPECT(agv[displs[q]] == (float)q && agv[displs[q] + q] == (float)q);
    std::vector<float> full(total), rsv(rank + 1, 0.f);
    for (uint64_t i = 0; i < total; ++i) full[i] = (float)i + (float)rank;
    EX_CHECK(HcclReduceScatterVInner(full.data(), counts.data(), displs.data(), rsv.data(), rank + 1, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, comm, nullptr));
    for (uint32_t i = 0; i <= rank; ++i) EX_EXPECT(rsv[i] == (float)n * (float)(displs[rank] + i) + rankSum);

    std::vector<float> sc(cnt, 0.f);
    EX_CHECK(HcclScatterInner(x.data(), sc.data(), cnt, HCCL_DATA_TYPE_FP32, 0, comm, nullptr));
    for (uint64_t i = 0; i < cnt; ++i) EX_EXPECT(sc[i] == (float)((rank * cnt + i) % 13));      // rank 0's values

    std::vector<float> red(n * cnt, 0.f);
    EX_CHECK(HcclReduceInner(x.data(), red.data(), n * cnt, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_MAX, n - 1, comm, nullptr));
    if (rank == n - 1)
        for (uint64_t i = 0; i < n * cnt; ++i) EX_EXPECT(red[i] == (float)(i % 13) + (float)(n - 1));

    std::vector<int32_t> a2a(n * 4), a2aOut(n * 4, -1);
    for (uint32_t q = 0; q < n; ++q)
        for (int k = 0; k < 4; ++k) a2a[q * 4 + k] = (int32_t)(rank * 100 + q);
    EX_CHECK(HcclAlltoAllInner(a2a.data(), 4, HCCL_DATA_TYPE_INT32, a2aOut.data(), 4, HCCL_DATA_TYPE_INT32, comm, nullptr));
    for (uint32_t q = 0; q < n; ++q) EX_EXPECT(a2aOut[q * 4 + 3] == (int32_t)(q * 100 + rank));

    // rank i sends i + 1 elements to everybody
    std::vector<uint64_t> sendCounts(n, rank + 1), sendDispls(n);
    for (uint32_t q = 0; q < n; ++q) sendDispls[q] = (uint64_t)q * (rank + 1);
    std::vector<int32_t> v((size_t)n * (rank + 1), (int32_t)rank), vOut(total, -1);
    EX_CHECK(HcclAlltoAllVInner(v.data(), sendCounts.data(), sendDispls.data(), HCCL_DATA_TYPE_INT32, vOut.data(), counts.data(), displs.data(),
                                HCCL_DATA_TYPE_INT32, comm, nullptr));
    for (uint32_t q = 0; q < n; ++q) EX_EXPECT(vOut[displs[q]] == (int32_t)q && vOut[displs[q] + q] == (int32_t)q);
    std::vector<uint64_t> matrix((size_t)n * n);
    for (uint32_t i = 0; i < n; ++i)
        for (uint32_t j = 0; j < n; ++j) matrix[(size_t)i * n + j] = i + 1;
    std::fill(vOut.begin(), vOut.end(), -1);
    EX_CHECK(HcclAlltoAllVCInner(v.data(), matrix.data(), HCCL_DATA_TYPE_INT32, vOut.data(), HCCL_DATA_TYPE_INT32, comm, nullptr));
    for (uint32_t q = 0; q < n; ++q) EX_EXPECT(vOut[displs[q]] == (int32_t)q && vOut[displs[q] + q] == (int32_t)q);

    if (n > 1) {
        const uint32_t right = (rank + 1) % n, left = (rank + n - 1) % n;
        std::vector<int32_t> msg(33, (int32_t)rank), got(33, -1);
        if (rank % 2 == 0) {
            EX_CHECK(HcclSendInner(msg.data(), 33, HCCL_DATA_TYPE_INT32, right, comm, nullptr));
            EX_CHECK(HcclRecvInner(got.data(), 33, HCCL_DATA_TYPE_INT32, left, comm, nullptr));
        } else {
            EX_CHECK(HcclRecvInner(got.data(), 33, HCCL_DATA_TYPE_INT32, left, comm, nullptr));
            EX_CHECK(HcclSendInner(msg.data(), 33, HCCL_DATA_TYPE_INT32, right, comm, nullptr));
        }
        EX_EXPECT(got[0] == (int32_t)left && got[32] == (int32_t)left);
        std::fill(got.begin(), got.end(), -1);
        HcclSendRecvItem items[2];
        items[0].sendRecvType = HCCL_SEND; items[0].buf = msg.data(); items[0].count = 33; items[0].dataType = HCCL_DATA_TYPE_INT32; items[0].remoteRank = left;
        items[1].sendRecvType = HCCL_RECV; items[1].buf = got.data(); items[1].count = 33; items[1].dataType = HCCL_DATA_TYPE_INT32; items[1].remoteRank = right;
        EX_CHECK(HcclBatchSendRecvInner(items, 2, comm, nullptr));
        EX_EXPECT(got[0] == (int32_t)right);
    }

    // grouped calls: queued until the outermost End, nesting allowed
    bool grouped = true;
    EX_CHECK(HcclGroupStatusGet(&grouped));
    EX_EXPECT(!grouped);
    EXPECT_RC(HcclGroupEnd(), HCCL_E_PARA);
    EX_CHECK(HcclGroupStart());
    EX_CHECK(HcclGroupStart());
    EX_CHECK(HcclGroupStatusGet(&grouped));
    EX_EXPECT(grouped);
    std::fill(y.begin(), y.end(), 0.f);
    std::vector<float> small(8, 1.f), smallOut(8, 0.f);
    EX_CHECK(HcclAllReduce(small.data(), smallOut.data(), 8, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, comm, nullptr));
    EX_CHECK(HcclAllReduce(x.data(), y.data(), n * cnt, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, comm, nullptr));
    EX_CHECK(HcclGroupEnd());
    EX_EXPECT(smallOut[0] == 0.f && y[0] == 0.f);          // nothing has run yet
    EX_CHECK(HcclGroupEnd());
    EX_EXPECT(smallOut[7] == (float)n && y[1] == (float)n * 1.f + rankSum);
    EX_CHECK(HcclGroupStatusGet(&grouped));
    EX_EXPECT(!grouped);

    // all-reduce with the scale and the cast fused: the mean, in fp32 and written as bf16
    std::vector<float> g(64), mean(64, 0.f);
    for (int i = 0; i < 64; ++i) g[i] = (float)(i + 1) * (float)(rank + 1);
    EX_CHECK(HcclAllReduceScaled(g.data(), mean.data(), 64, HCCL_DATA_TYPE_FP32, HCCL_DATA_TYPE_FP32, 1.0f / (float)n, comm, nullptr));
    for (int i = 0; i < 64; ++i) EX_EXPECT(std::fabs(mean[i] - (float)(i + 1) * (float)(n + 1) / 2.f) < 1e-4f);
    // bf16 in, bf16 out, fp32 in between; a cast on the way is not offered
    std::vector<uint16_t> hin(64), hout(64, 0);
    for (int i = 0; i < 64; ++i) {
        float f = (float)(i + 1) * (float)(rank + 1);
        uint32_t bits;
        std::memcpy(&bits, &f, 4);
        hin[i] = (uint16_t)(bits >> 16);                  // small integers are exact in bf16
    }
    EX_CHECK(HcclAllReduceScaled(hin.data(), hout.data(), 64, HCCL_DATA_TYPE_BFP16, HCCL_DATA_TYPE_BFP16, 1.0f / (float)n, comm, nullptr));
    for (int i = 0; i < 64; ++i) {
        uint32_t bits = (uint32_t)hout[i] << 16;
        float f;
        std::memcpy(&f, &bits, 4);
        const float want = (float)(i + 1) * (float)(n + 1) / 2.f;
        EX_EXPECT(std::fabs(f - want) <= want / 128.f);
    }
    EXPECT_RC(HcclAllReduceScaled(g.data(), hout.data(), 64, HCCL_DATA_TYPE_FP32, HCCL_DATA_TYPE_BFP16, 1.0f, comm, nullptr), HCCL_E_NOT_SUPPORT);
    int32_t ints[4] = {1, 2, 3, 4};
    EXPECT_RC(HcclAllReduceScaled(ints, ints, 4, HCCL_DATA_TYPE_INT32, HCCL_DATA_TYPE_INT32, 0.5f, comm, nullptr), HCCL_E_NOT_SUPPORT);
}

// ------------------------------------------------------------ threads, channels, windows and the data-plane primitives

static void Resources(uint32_t rank, uint32_t n, HcclComm comm)
{
    void *ccl = nullptr;
    uint64_t cclSize = 0;
    EX_CHECK(HcclBarrier(comm, nullptr));                  // nobody is still staging through the buffer
    EX_CHECK(HcclGetHcclBufferCleared(comm, &ccl, &cclSize));
    EX_EXPECT(cclSize == 4u << 20 && ((char *)ccl)[12345] == 0);
    char *mine = (char *)ccl;
    const uint64_t base = 300u << 10;                      // away from the slot starts that built-in operators use

    // ---- threads in every flavour
    ThreadHandle t1 = 0, t2 = 0, t3 = 0, d1 = 0, d2 = 0;
    EX_CHECK(HcclThreadAcquire(comm, COMM_ENGINE_CPU_TS, 1, 4, &t1));
    ThreadConfig tc;
    EX_CHECK(ThreadConfigInit(&tc, 1));
    tc.notifyNumPerThread = 3;
    EX_CHECK(HcclThreadAcquireWithConfig(comm, COMM_ENGINE_CPU_TS, 1, THREAD_TYPE_TS, &tc, &t2));
    EXPECT_RC(HcclThreadAcquireWithConfig(comm, COMM_ENGINE_CPU_TS, 1, THREAD_TYPE_INVALID, &tc, &t3), HCCL_E_NOT_SUPPORT);
    tc.header.magicWord = 0;
    EXPECT_RC(HcclThreadAcquireWithConfig(comm, COMM_ENGINE_CPU_TS, 1, THREAD_TYPE_TS, &tc, &t3), HCCL_E_PARA);
    EX_CHECK(HcclThreadAcquireWithStream(comm, COMM_ENGINE_CPU_TS, nullptr, 2, &t3));
    EXPECT_RC(HcclThreadAcquire(comm, COMM_ENGINE_CPU_TS, 0, 1, &t3), HCCL_E_PARA);
    EX_CHECK(HcclDedicatedThreadAcquire(comm, HCCL_DED_THREAD_TYPE_AICPU_LAUNCH, 2, &d1));
    EX_CHECK(HcclDedicatedThreadAcquire(comm, HCCL_DED_THREAD_TYPE_AICPU_LAUNCH, 1, &d2));
    EX_EXPECT(d1 == d2 && d1 != 0);                        // one per use type
    EXPECT_RC(HcclDedicatedThreadAcquire(comm, HCCL_DED_THREAD_TYPE_AICPU_LAUNCH, 9, &d2), HCCL_E_PARA);
    EXPECT_RC(HcclDedicatedThreadAcquire(comm, HCCL_DED_THREAD_TYPE_INVALID, 1, &d2), HCCL_E_PARA);
    void *stream = (void *)1;
    EX_CHECK(HcclThreadResGetInfo(comm, t1, THREAD_RES_TYPE_STREAM, sizeof(void *), &stream));
    void *streamAgain = nullptr;
    EX_CHECK(HcommThreadResGetInfo(t1, THREAD_RES_TYPE_STREAM, sizeof(void *), &streamAgain));
    EX_EXPECT(streamAgain == stream);
    EXPECT_RC(HcclThreadResGetInfo(comm, t1, THREAD_RES_TYPE_INVALID, sizeof(void *), &stream), HCCL_E_NOT_SUPPORT);
    EXPECT_RC(HcommThreadResGetInfo(t1, THREAD_RES_TYPE_STREAM, 2, &stream), HCCL_E_PARA);
    ThreadHandle exported = 0;
    EX_CHECK(HcclThreadExportToCommEngine(comm, 1, &t1, COMM_ENGINE_AICPU_TS, &exported));
    EX_EXPECT(exported == t1);
    EXPECT_RC(HcclThreadExportToCommEngine(comm, 1, &t1, COMM_ENGINE_CCU, &exported), HCCL_E_NOT_SUPPORT);
    EX_CHECK(HcommThreadJoin(t1, 1));
    EXPECT_RC(HcommThreadJoin(0, 1), HCCL_E_PTR);

    // thread-to-thread and raw notifies
    EX_CHECK(HcommThreadNotifyRecordOnThread(t1, t2, 0));
    EX_CHECK(HcommThreadNotifyWaitOnThread(t2, 0, 5));
    EX_CHECK(HcommThreadNotifyRecordOnThread(t1, t2, 2));
    EX_CHECK(HcommThreadNotifyWaitOnThreadWithDefaultTimeout(t2, 2));
    EX_CHECK(HcommThreadSynchronize(t2));
    EXPECT_RC(HcommThreadNotifyRecordOnThread(t1, t2, 3), HCCL_E_PARA);      // t2 has three slots
    EXPECT_RC(HcommThreadNotifyWaitOnThread(t2, 7, 1), HCCL_E_PARA);
    uint64_t *word = new uint64_t(0);                      // never freed: its address stays unique for the process
    EX_CHECK(HcommAclrtNotifyRecordOnThread(t1, (uint64_t)(uintptr_t)word));
    EX_CHECK(HcommAclrtNotifyWaitOnThread(t1, (uint64_t)(uintptr_t)word, 5));
    EX_CHECK(HcommThreadSynchronize(t1));
    EX_EXPECT(*word == 1);
    EXPECT_RC(HcommAclrtNotifyRecordOnThread(t1, 0), HCCL_E_PTR);
    EXPECT_RC(HcommSetNotifyWaitTimeOut(-1.f), HCCL_E_PARA);
    EX_CHECK(HcommSetNotifyWaitTimeOut(30.f));
    EX_CHECK(HcommSetNotifyWaitTimeOut(0.f));
    EXPECT_RC(HcommThreadResAcquireTimeOut(-1.f), HCCL_E_PARA);
    EX_CHECK(HcommThreadResAcquireTimeOut(1.f));
    char name[COMM_NAME_MAX_LENGTH] = "";
    EX_CHECK(HcclGetCommName(comm, name));
    EX_CHECK(HcommAcquireComm(name));
    EXPECT_RC(HcommAcquireComm("no such communicator"), HCCL_E_NOT_FOUND);
    EX_CHECK(HcommReleaseComm(name));
    EXPECT_RC(HcommReleaseComm(nullptr), HCCL_E_PTR);

    // threads and memory without a communicator
    uint32_t notifies[2] = {2, 1};
    ThreadHandle bare[2] = {0, 0};
    EX_CHECK(HcommThreadAlloc(COMM_ENGINE_CPU_TS, 2, notifies, bare));
    EX_CHECK(HcommThreadNotifyRecordOnThread(bare[0], bare[1], 0));
    EX_CHECK(HcommThreadNotifyWaitOnThread(bare[1], 0, 5));
    EX_CHECK(HcommThreadSynchronize(bare[1]));
    EX_CHECK(HcommThreadFree(bare, 2));
    void *block = nullptr;
    EX_CHECK(HcommMemAlloc(&block, 100000));
    std::memset(block, 0x5a, 100000);
    EXPECT_RC(HcommMemAlloc(&block, 0), HCCL_E_PARA);
    EXPECT_RC(HcommMemFree((char *)block + 64), HCCL_E_NOT_FOUND);
    EX_CHECK(HcommMemFree(block));

    // ---- tagged device memory, task callbacks, exchange info, extra queries
    uint64_t devSize = 4096;
    void *dev = nullptr, *devAgain = nullptr;
    bool created = false;
    EX_CHECK(HcclDevMemAcquire(comm, "sweep", &devSize, &dev, &created));
    EX_EXPECT(created && dev != nullptr);
    devSize = 0;
    EX_CHECK(HcclDevMemAcquire(comm, "sweep", &devSize, &devAgain, &created));
    EX_EXPECT(!created && devAgain == dev && devSize == 4096);
    devSize = 0;
    EXPECT_RC(HcclDevMemAcquire(comm, "other", &devSize, &devAgain, &created), HCCL_E_PARA);
    static std::atomic<uint64_t> taskSum{0};
    EX_CHECK(HcclTaskRegister(comm, "add", [](uint64_t a, int32_t b) -> int32_t { taskSum += a + (uint64_t)b; return 0; }));
    EX_CHECK(HcclTaskNotify(comm, "add", 40, 2, nullptr));
    EXPECT_RC(HcclTaskNotify(comm, "missing", 1, 1, nullptr), HCCL_E_NOT_FOUND);
    EX_CHECK(HcclTaskUnRegister(comm, "add"));
    EXPECT_RC(HcclTaskUnRegister(comm, "add"), HCCL_E_NOT_FOUND);
    EX_CHECK(HcclBarrier(comm, nullptr));
    EX_EXPECT(taskSum.load() == 42ull * n);
    uint32_t blob[2] = {0xabcd0000u + rank, rank * 3};
    EX_CHECK(HcclCommAddExchangeInfo(comm, blob, sizeof(blob)));
    EXPECT_RC(HcclCommAddExchangeInfo(comm, blob, 0), HCCL_E_PARA);
    for (uint32_t q = 0; q < n; ++q) {
        uint32_t got[2] = {0, 0}, len = 0;
        EX_CHECK(HcclCommGetExchangeInfo(comm, q, got, sizeof(got), &len));
        EX_EXPECT(len == sizeof(got) && got[0] == 0xabcd0000u + q && got[1] == q * 3);
    }
    uint32_t len = 0;
    EXPECT_RC(HcclCommGetExchangeInfo(comm, 0, blob, 2, &len), HCCL_E_MEMORY);
    EXPECT_RC(HcclCommGetExchangeInfo(comm, n, blob, 8, &len), HCCL_E_PARA);
    EX_CHECK(HcclBarrier(comm, nullptr));
    EX_CHECK(HcclCommResetExchangeInfo(comm));
    HcclTopoDescs topo[2];
    EX_CHECK(HcclGetTopoDesc(comm, topo, 2));
    EX_EXPECT(topo[0].rankSize == n && (topo[0].algSets & 0x2d) == 0x2d && topo[1].rankSize == 1);
    EXPECT_RC(HcclGetTopoDesc(comm, topo, 0), HCCL_E_PARA);
    void *peerBuf = nullptr;
    uint64_t peerSize = 0;
    EX_CHECK(HcclGetRemoteIpcHcclBuf(comm, (rank + 1) % n, &peerBuf, &peerSize));
    EX_EXPECT(peerBuf != nullptr && peerSize == cclSize);
    EXPECT_RC(HcclGetRemoteIpcHcclBuf(comm, n, &peerBuf, &peerSize), HCCL_E_PARA);

    // ---- profiling reports reach the sink
    static std::atomic<int> reports{0};
    if (rank == 0) EX_CHECK(HcclProfilingSetSink([](int, const char *, const char *, uint64_t, uint64_t, void *) { ++reports; }, nullptr));
    EX_CHECK(HcclBarrier(comm, nullptr));
    const int before = reports.load();
    const uint64_t t0 = HcommGetProfilingSysCycleTime();
    EX_EXPECT(t0 != 0 && HcommGetProfilingSysCycleTime() >= t0);
    HcclDfxOpInfo info;
    std::memset(&info, 0, sizeof(info));
    std::snprintf(info.algTag, sizeof(info.algTag), "sweep_op_%u", rank);
    EX_CHECK(HcclDfxRegOpInfoByCommId(name, &info));
    EX_CHECK(HcclProfilingReportOp(comm, t0));
    char kernelName[] = "sweep_kernel";
    EX_CHECK(HcclReportAicpuKernel(comm, t0, kernelName));
    EX_CHECK(HcclReportAivKernel(comm, t0));
    EX_CHECK(HcommProfilingReportDeviceOp(name));
    EX_CHECK(HcommProfilingReportKernelStartTask(t1, name));
    EX_CHECK(HcommProfilingReportKernelEndTask(t1, name));
    EX_EXPECT(reports.load() >= before + 6);
    EX_CHECK(HcclBarrier(comm, nullptr));
    if (rank == 0) EX_CHECK(HcclProfilingSetSink(nullptr, nullptr));

    // ---- windows over a part of the communication buffer
    HcclCommSymWindow win = nullptr, found = nullptr;
    char *winBase = mine + (1u << 20) + (64u << 10);
    EX_CHECK(HcclCommSymWinRegister(comm, winBase, 64u << 10, &win, 0));
    size_t off = 99;
    EX_CHECK(HcclCommSymWinGet(comm, winBase + 4096, 128, &found, &off));
    EX_EXPECT(found == win && off == 4096);
    EXPECT_RC(HcclCommSymWinGet(comm, &off, 8, &found, &off), HCCL_E_NOT_FOUND);
    void *peerPtr = nullptr, *mcPtr = nullptr;
    EX_CHECK(HcclSymWinGetPeerPointer(win, 4096, rank, &peerPtr));
    EX_EXPECT(peerPtr == winBase + 4096);
    EXPECT_RC(HcclSymWinGetPeerPointer(win, 4096, n, &peerPtr), HCCL_E_PARA);
    EXPECT_RC(HcclSymWinGetMulticastPointer(win, 0, &mcPtr), HCCL_E_NOT_SUPPORT);          // no switch multicast on the host
    std::vector<uint32_t> everyone(n);
    std::iota(everyone.begin(), everyone.end(), 0u);
    EX_CHECK(HcclCommExchangeMem(comm, win, everyone.data(), n));
    everyone[0] = n;
    EXPECT_RC(HcclCommExchangeMem(comm, win, everyone.data(), n), HCCL_E_PARA);
    EX_CHECK(HcclCommSymWinDeregister(win));
    void *regHandle = nullptr;
    EX_CHECK(HcclCommRegister(comm, winBase, 64u << 10, &regHandle, 0));
    EX_CHECK(HcclCommDeregister(comm, regHandle));
    EX_CHECK(HcclCommSetMemoryRange(comm, winBase, 64u << 10, 4096, 0));
    EX_CHECK(HcclCommActivateCommMemory(comm, winBase, 32u << 10, 0, 0, 0));
    EX_CHECK(HcclCommSymWinGet(comm, winBase + 100, 8, &found, &off));
    EX_EXPECT(off == 100);
    EX_CHECK(HcclCommDeactivateCommMemory(comm, winBase));
    EXPECT_RC(HcclCommDeactivateCommMemory(comm, winBase), HCCL_E_NOT_FOUND);
    EX_CHECK(HcclCommUnsetMemoryRange(comm, winBase));
    EXPECT_RC(HcclCommUnsetMemoryRange(comm, winBase), HCCL_E_NOT_FOUND);
    EXPECT_RC(HcclCommSetMemoryRange(comm, winBase, 0, 4096, 0), HCCL_E_PARA);

    // ---- memory bound to the communicator through the process-wide registry, connections prepared
    static int globalBlock[64];
    CommMem gm{COMM_MEM_TYPE_HOST, globalBlock, sizeof(globalBlock)};
    // Written by rank 0 before a barrier, read by all after it.  An atomic, because the barrier's flags live in memory that
    // every rank maps at an address of its own, which a race detector cannot follow.
    static std::atomic<void *> sharedHandle{nullptr};
    if (rank == 0) {
        void *h = nullptr, *again = nullptr;
        EX_CHECK(HcclRegisterGlobalMem(&gm, &h));
        EXPECT_RC(HcclRegisterGlobalMem(&gm, &again), HCCL_E_PARA);
        sharedHandle.store(h);
    }
    EX_CHECK(HcclBarrier(comm, nullptr));
    void *globalHandle = sharedHandle.load();
    EX_CHECK(HcclCommBindMem(comm, globalHandle));
    EXPECT_RC(HcclCommBindMem(comm, &gm), HCCL_E_NOT_FOUND);
    EX_CHECK(HcclCommUnbindMem(comm, globalHandle));
    EXPECT_RC(HcclCommUnbindMem(comm, globalHandle), HCCL_E_NOT_FOUND);
    HcclPrepareConfig prep;
    std::memset(&prep, 0, sizeof(prep));
    prep.topoType = HCCL_TOPO_FULLMESH;
    EX_CHECK(HcclCommPrepare(comm, &prep, 20));
    prep.topoType = HCCL_TOPO_NUM;
    EXPECT_RC(HcclCommPrepare(comm, &prep, 20), HCCL_E_NOT_SUPPORT);
    EX_CHECK(HcclBarrier(comm, nullptr));
    if (rank == 0) {
        EX_CHECK(HcclDeregisterGlobalMem(globalHandle));
        EXPECT_RC(HcclDeregisterGlobalMem(globalHandle), HCCL_E_NOT_FOUND);
    }

    if (n < 2) return;
    // ---- channels to the ring neighbours (one channel when both are the same rank)
    const uint32_t right = (rank + 1) % n, left = (rank + n - 1) % n;
    std::vector<uint32_t> peers = right == left ? std::vector<uint32_t>{right} : std::vector<uint32_t>{std::min(right, left), std::max(right, left)};
    std::vector<HcclChannelDesc> descs(peers.size());
    EX_CHECK(HcclChannelDescInit(descs.data(), (uint32_t)descs.size()));
    for (size_t i = 0; i < peers.size(); ++i) { descs[i].remoteRank = peers[i]; descs[i].notifyNum = 8; }
    std::vector<ChannelHandle> ch(peers.size(), 0), seen(peers.size(), 1);
    EX_CHECK(HcclChannelQuery(comm, COMM_ENGINE_CPU_TS, descs.data(), (uint32_t)descs.size(), seen.data()));
    EX_EXPECT(seen[0] == 0);                               // nothing acquired yet
    HcclChannelConfig cfg = nullptr;
    EX_CHECK(HcclChannelConfigCreate(&cfg));
    EX_CHECK(HcclChannelConfigSetInt(cfg, HCCL_CHANNEL_CONFIG_TYPE_IS_SHARED_QUEUE, 1));
    EXPECT_RC(HcclChannelConfigSetInt(cfg, HCCL_CHANNEL_CONFIG_TYPE_SHARED_QUEUE_TAG, 1), HCCL_E_PARA);
    EX_CHECK(HcclChannelConfigSetStr(cfg, HCCL_CHANNEL_CONFIG_TYPE_SHARED_QUEUE_TAG, "sweep"));
    EXPECT_RC(HcclChannelConfigSetStr(cfg, HCCL_CHANNEL_CONFIG_TYPE_IS_SHARED_QUEUE, "sweep"), HCCL_E_PARA);
    EX_CHECK(HcclChannelAcquireWithConfig(comm, COMM_ENGINE_CPU_TS, descs.data(), (uint32_t)descs.size(), cfg, ch.data()));
    EX_CHECK(HcclChannelConfigDestroy(cfg));
    EX_CHECK(HcclChannelQuery(comm, COMM_ENGINE_CPU_TS, descs.data(), (uint32_t)descs.size(), seen.data()));
    for (size_t i = 0; i < peers.size(); ++i) EX_EXPECT(seen[i] == ch[i] && ch[i] != 0);
    const ChannelHandle chR = ch[peers[0] == right ? 0 : 1], chL = ch[peers[0] == left ? 0 : 1];
    void *view = nullptr;
    EX_CHECK(HcclChannelGetDeviceView(comm, chR, &view));
    EX_EXPECT(view != nullptr);
    void *rbuf = nullptr;
    uint64_t rsize = 0;
    EX_CHECK(HcclChannelGetHcclBuffer(comm, chR, &rbuf, &rsize));
    EX_EXPECT(rsize == cclSize);
    char *theirs = (char *)rbuf;
    const uint64_t len4k = 4096;
    std::vector<uint8_t> src(len4k);
    auto fill = [&](uint8_t salt, uint32_t r) { std::vector<uint8_t> v(len4k); for (uint64_t i = 0; i < len4k; ++i) v[i] = (uint8_t)(i * 7 + salt + r * 31); return v; };
    auto same = [&](const char *p, const std::vector<uint8_t> &v) { return std::memcmp(p, v.data(), v.size()) == 0; };

    // A: thread-less write with notify, thread-less wait
    src = fill(1, rank);
    EX_CHECK(HcommWriteWithNotifyNbi(chR, theirs + base, src.data(), len4k, 0));
    EX_CHECK(HcommChannelNotifyWait(chL, 0, 10));
    EX_EXPECT(same(mine + base, fill(1, left)));
    // B: write on the channel's side stream after the thread's work, fence, record, wait with the default limit
    src = fill(2, rank);
    EX_CHECK(HcommWriteNbiOnThread(t1, chR, theirs + base + len4k, src.data(), len4k));
    EX_CHECK(HcommChannelFenceOnThread(t1, chR));
    EX_CHECK(HcommChannelNotifyRecordOnThread(t1, chR, 1));
    EX_CHECK(HcommChannelNotifyWaitOnThreadWithDefaultTimeout(t1, chL, 1));
    EX_CHECK(HcommThreadSynchronize(t1));
    EX_EXPECT(same(mine + base + len4k, fill(2, left)));
    // C: the same with the notify attached to the write, joined by a fence over all side streams
    src = fill(3, rank);
    EX_CHECK(HcommWriteWithNotifyNbiOnThread(t1, chR, theirs + base + 2 * len4k, src.data(), len4k, 2));
    EX_CHECK(HcommFenceOnThread(t1));
    EX_CHECK(HcommChannelNotifyWaitOnThread(t1, chL, 2, 10));
    EX_CHECK(HcommThreadSynchronize(t1));
    EX_EXPECT(same(mine + base + 2 * len4k, fill(3, left)));
    EX_CHECK(HcommWriteNbi(chR, theirs + base + 3 * len4k, src.data(), 64));
    EX_CHECK(HcommChannelFence(chR));
    // D: a reducing write with notify into values the owner has put there
    float *acc = (float *)(mine + base + 4 * len4k);
    for (int i = 0; i < 256; ++i) acc[i] = 100.f;
    EX_CHECK(HcommChannelNotifyRecord(chL, 4));            // tell the writer (my left neighbour) that the target is ready
    EX_CHECK(HcommChannelNotifyWait(chR, 4, 10));
    std::vector<float> add(256);
    for (int i = 0; i < 256; ++i) add[i] = (float)(rank + 1) * (float)i;
    EX_CHECK(HcommWriteReduceWithNotifyOnThread(t1, chR, theirs + base + 4 * len4k, add.data(), 256, HCOMM_DATA_TYPE_FP32, HCOMM_REDUCE_SUM, 3));
    EX_CHECK(HcommChannelNotifyWaitOnThread(t1, chL, 3, 10));
    EX_CHECK(HcommThreadSynchronize(t1));
    for (int i = 0; i < 256; ++i) EX_EXPECT(acc[i] == 100.f + (float)(left + 1) * (float)i);
    EXPECT_RC(HcommChannelNotifyRecordOnThread(t1, chR, 8), HCCL_E_PARA);                    // eight slots: 0..7
    // E: reads of what I wrote into the right neighbour in step A
    std::vector<uint8_t> back(len4k, 0), back2(len4k, 0);
    EX_CHECK(HcommReadNbi(chR, back.data(), theirs + base, len4k));
    EX_CHECK(HcommChannelFence(chR));
    EX_EXPECT(back == fill(1, rank));
    EX_CHECK(HcommReadNbiOnThread(t1, chR, back2.data(), theirs + base, len4k));
    EX_CHECK(HcommChannelDrainOnThread(t1, chR));
    EX_EXPECT(back2 == fill(1, rank));
    // nobody leaves while a neighbour may still read from it
    EX_CHECK(HcommChannelNotifyRecord(chR, 5));
    EX_CHECK(HcommChannelNotifyRecord(chL, 5));
    EX_CHECK(HcommChannelNotifyWait(chR, 5, 10));
    EX_CHECK(HcommChannelNotifyWait(chL, 5, 10));
    EX_CHECK(HcclChannelDestroy(comm, ch.data(), (uint32_t)ch.size()));
    EX_CHECK(HcclChannelQuery(comm, COMM_ENGINE_CPU_TS, descs.data(), (uint32_t)descs.size(), seen.data()));
    EX_EXPECT(seen[0] == 0);
}

// ----------------------------------------- endpoints and a channel below the communicator level (ranks 0 and 1 only)

static std::atomic<uint32_t> g_serverPort{0};

static void BaseLevel(uint32_t rank, uint32_t n, HcclComm comm)
{
    uint32_t descNum = 0;
    EX_CHECK(HcommEndpointGetDescNum((int32_t)rank, &descNum));
    EX_EXPECT(descNum == 1);
    EndpointDesc desc;
    EX_CHECK(HcommEndpointGetDescs((int32_t)rank, &descNum, &desc));
    EX_EXPECT(desc.protocol == COMM_PROTOCOL_SHM);         // the host simulator's transport
    bool feature = true;
    EX_CHECK(HcommEndpointCheckFeature(HCOMM_ENDPOINT_FEATURE_NDA, &desc, &feature));
    EX_EXPECT(!feature);
    EX_CHECK(HcommEndpointCheckFeature(HCOMM_ENDPOINT_FEATURE_MULTICAST, &desc, &feature));
    EX_EXPECT(!feature);
    EXPECT_RC(HcommEndpointCheckFeature(HCOMM_ENDPOINT_FEATURE_INVALID, &desc, &feature), HCCL_E_PARA);
    HcommChannelConfig cfg = nullptr;
    EX_CHECK(HcommChannelConfigCreate(&cfg));
    EX_CHECK(HcommChannelConfigSetInt(cfg, HCOMM_CHANNEL_CONFIG_TYPE_IS_SHARED_QUEUE, 1));
    EXPECT_RC(HcommChannelConfigSetInt(cfg, HCOMM_CHANNEL_CONFIG_TYPE_INVALID, 1), HCCL_E_PARA);
    if (n >= 2 && rank < 2) {
        EndpointHandle ep = nullptr;
        EX_CHECK(HcommEndpointCreate(&desc, &ep));
        void *block = nullptr;
        EX_CHECK(HcommMemAlloc(&block, 1u << 16));
        std::memset(block, 0, 1u << 16);
        CommMem mem{COMM_MEM_TYPE_DEVICE, block, 1u << 16};
        HcommMemHandle mh = nullptr;
        EX_CHECK(HcommMemReg(ep, "base_block", &mem, &mh));
        HcommChannelDesc cd;
        EX_CHECK(HcommChannelDescInit(&cd, 1));
        cd.notifyNum = 2;
        cd.exchangeAllMems = true;
        cd.channelName = "sweep_base";
        cd.remoteEndpoint = desc;                          // same host: the peer is reached on the loopback address below
        ChannelHandle chan = 0;
        if (rank == 0) {
            uint32_t port = 0;
            EX_CHECK(HcommEndpointGetListenPort(ep, &port));
            EX_EXPECT(port != 0);
            g_serverPort.store(port);
            cd.role = HCOMM_SOCKET_ROLE_SERVER;
        } else {
            while (g_serverPort.load() == 0) usleep(1000);
            cd.role = HCOMM_SOCKET_ROLE_CLIENT;
            cd.port = (uint16_t)g_serverPort.load();
            cd.remoteEndpoint.commAddr.type = COMM_ADDR_TYPE_RESERVED;     // 127.0.0.1
        }
        EX_CHECK(HcommChannelCreateWithConfig(ep, COMM_ENGINE_CPU_TS, &cd, 1, cfg, &chan));
        int32_t status = -1;
        EX_CHECK(HcommChannelGetStatus(&chan, 1, &status));
        EX_EXPECT(status == HCOMM_CHANNEL_STATUS_READY);
        uint32_t memNum = 0;
        CommMem *remote = nullptr;
        char **tags = nullptr;
        EX_CHECK(HcclChannelGetRemoteMems(comm, chan, &memNum, &remote, &tags));
        EX_EXPECT(memNum == 1 && std::string(tags[0]) == "base_block" && remote[0].size == (1u << 16));
        // each side writes a line into the other's block and says so; thread-less forms work without a communicator
        char line[32];
        std::snprintf(line, sizeof(line), "hello from %u", rank);
        EX_CHECK(HcommWriteWithNotifyNbi(chan, (char *)remote[0].addr + 128, line, sizeof(line), 1));
        EX_CHECK(HcommChannelNotifyWait(chan, 1, 10));
        char want[32];
        std::snprintf(want, sizeof(want), "hello from %u", 1 - rank);
        EX_EXPECT(std::strcmp((char *)block + 128, want) == 0);
        EX_CHECK(HcommChannelNotifyRecord(chan, 0));       // both have read: the blocks may go
        EX_CHECK(HcommChannelNotifyWait(chan, 0, 10));
        EX_CHECK(HcommChannelDestroy(&chan, 1));
        EX_CHECK(HcommMemUnreg(ep, mh));
        EX_CHECK(HcommEndpointDestroy(ep));
        EX_CHECK(HcommMemFree(block));
    }
    EX_CHECK(HcommChannelConfigDestroy(cfg));
    EX_CHECK(HcclBarrier(comm, nullptr));
}

// ------------------------------------------------------------------------- teams below the world team, team channels

static void Teams(uint32_t rank, uint32_t n, HcclComm comm)
{
    HcclTeamCreateDesc td;
    EX_CHECK(HcclTeamCreateDescInit(&td));
    td.selfRankId = rank;
    td.requirement.signalCount = 1;
    td.requirement.barrierCount = 1;
    HcommTeamHandle world = nullptr;
    EX_CHECK(HcclWorldTeamCreate(comm, &td, &world));
    // the even ranks form a team of their own; an odd rank cannot create it
    std::vector<uint32_t> evens;
    for (uint32_t r = 0; r < n; r += 2) evens.push_back(r);
    HcclTeamCreateDesc sd = td;
    sd.rankIds = evens.data();
    sd.rankNum = (uint32_t)evens.size();
    HcommTeamHandle sub = nullptr;
    if (rank % 2 == 0) {
        EX_CHECK(HcclSubTeamCreate(world, &sd, &sub));
        uint32_t members = 0, myIdx = 99;
        EX_CHECK(HcclTeamGetInfo(sub, &members, &myIdx));
        EX_EXPECT(members == evens.size() && myIdx == rank / 2);
        for (int round = 1; round <= 3; ++round) EX_CHECK(HcclTeamBarrier(sub, 0, nullptr));
        const uint32_t next = (myIdx + 1) % members, prev = (myIdx + members - 1) % members;
        EX_CHECK(HcclTeamSignal(sub, next, 0, 5, nullptr));
        EX_CHECK(HcclTeamSignalWait(sub, prev, 0, 5, nullptr));
        EX_CHECK(HcclTeamDestroy(sub));
    } else {
        EXPECT_RC(HcclSubTeamCreate(world, &sd, &sub), HCCL_E_PARA);
    }
    uint32_t outside = n;
    HcclTeamCreateDesc bad = td;
    bad.rankIds = &outside;
    bad.rankNum = 1;
    EXPECT_RC(HcclSubTeamCreate(world, &bad, &sub), HCCL_E_PARA);
    bad.rankIds = nullptr;
    bad.rankNum = 0;
    EXPECT_RC(HcclSubTeamCreate(world, &bad, &sub), HCCL_E_PARA);      // a sub team names its members
    // channels between all members of the world team, found again by a query
    HcclTeamCreateChannelsDesc cd;
    EX_CHECK(HcclTeamCreateChannelsDescInit(&cd));
    cd.notifyNum = 3;
    EX_CHECK(HcclTeamChannelsCreate(comm, world, &cd));
    cd.header.magicWord = 0;
    EXPECT_RC(HcclTeamChannelsCreate(comm, world, &cd), HCCL_E_PARA);
    for (uint32_t q = 0; q < n; ++q) {
        if (q == rank) continue;
        HcclChannelDesc d;
        EX_CHECK(HcclChannelDescInit(&d, 1));
        d.remoteRank = q;
        d.notifyNum = 3;
        ChannelHandle h = 0;
        EX_CHECK(HcclChannelQuery(comm, COMM_ENGINE_CPU_TS, &d, 1, &h));
        EX_EXPECT(h != 0);
    }
    EX_CHECK(HcclTeamBarrier(world, 0, nullptr));
    EX_CHECK(HcclTeamDestroy(world));
    EXPECT_RC(HcclTeamDestroy(world), HCCL_E_PTR);
}

// ------------------------------------------------------------------- operator records, wait status, heartbeat switch

static void Diagnostics(uint32_t rank, uint32_t n, HcclComm comm)
{
    EX_CHECK(HcclDiagSetProfiling(comm, 1));
    std::vector<int32_t> v(777, (int32_t)rank), out(777, 0);
    EX_CHECK(HcclAllReduce(v.data(), out.data(), 777, HCCL_DATA_TYPE_INT32, HCCL_REDUCE_MAX, comm, nullptr));
    EX_EXPECT(out[776] == (int32_t)(n - 1));
    HcclOpRecord recs[8];
    uint32_t written = 0;
    EX_CHECK(HcclDiagGetOpRecords(comm, recs, 8, &written));
    EX_EXPECT(written >= 1);
    const HcclOpRecord &last = recs[written - 1];
    EX_EXPECT(last.cmdType == (uint32_t)HCCL_CMD_ALLREDUCE && last.count == 777 && last.dataType == (uint32_t)HCCL_DATA_TYPE_INT32 &&
              last.reduceOp == (uint32_t)HCCL_REDUCE_MAX && last.hostEndNs >= last.hostStartNs && last.algName[0] != 0);
    uint64_t launched = 0;
    EX_CHECK(HcclDiagGetOpCounters(comm, &launched, nullptr, nullptr));
    EX_EXPECT(launched == last.seq);
    uint64_t starts[4], ends[4];
    written = 99;
    EX_CHECK(HcclDiagGetKernelTimes(comm, starts, ends, 4, &written));
    EX_EXPECT(written == 0);                               // the simulator runs no kernels
    HcclDeviceWaitStatus ws;
    std::memset(&ws, 0xff, sizeof(ws));
    EX_CHECK(HcclDiagGetWaitStatus(comm, &ws));
    EX_EXPECT(ws.valid == 0);
    EX_CHECK(HcclDiagClearWaitStatus(comm));
    uint64_t lost = 99;
    std::vector<uint64_t> ages(n);
    EX_CHECK(HcclDiagGetHeartbeat(comm, ages.data(), n, &lost));
    EX_EXPECT(lost == 0);
    EX_CHECK(HcclDiagPauseHeartbeat(comm));                // heartbeats are off here: nothing to stop, nothing breaks
    char text[4096];
    EX_CHECK(HcclDiagDump(comm, text, sizeof(text)));
    EX_EXPECT(std::strstr(text, "AllReduce") != nullptr || std::strstr(text, "allreduce") != nullptr);
    HcclOpRetryStats stats;
    EX_CHECK(HcclCommGetOpRetryStats(comm, &stats));
    EX_EXPECT(stats.enabled == 0 && stats.requests == 0);
    EX_CHECK(HcclDiagSetProfiling(comm, 0));

    // the hooks around a snapshot of the process: Pre suspends every communicator of the process, each rank resumes its own
    EX_CHECK(HcclBarrier(comm, nullptr));
    if (rank == 0) EX_CHECK(HcclSnapshotPre());
    static std::atomic<int> suspendedSeen{0};
    if (rank == 0) suspendedSeen.store(1);
    while (suspendedSeen.load() == 0) usleep(1000);
    EXPECT_RC(HcclAllReduce(v.data(), out.data(), 777, HCCL_DATA_TYPE_INT32, HCCL_REDUCE_MAX, comm, nullptr), HCCL_E_SUSPENDING);
    EX_CHECK(HcclCommResume(comm));
    EX_CHECK(HcclAllReduce(v.data(), out.data(), 777, HCCL_DATA_TYPE_INT32, HCCL_REDUCE_SUM, comm, nullptr));
    EX_EXPECT(out[0] == (int32_t)(n * (n - 1) / 2));
    EX_CHECK(HcclBarrier(comm, nullptr));
    if (rank == 0) EX_CHECK(HcclSnapshotPost());           // nothing is suspended any more: a no-op
    EX_CHECK(HcclBarrier(comm, nullptr));
}

// ---------------------------------------------------------------- a host function launched in the communicator's order

struct SweepKernelArgs { std::atomic<int> *calls; int add; };
extern "C" int SweepKernel(void *args, uint32_t argSize, void *stream)
{
    if (argSize != sizeof(SweepKernelArgs) || stream != nullptr) return 7;
    SweepKernelArgs *a = (SweepKernelArgs *)args;
    a->calls->fetch_add(a->add);
    return 0;
}
extern "C" int SweepKernelFails(void *, uint32_t, void *) { return 3; }

static void Launch(uint32_t rank, uint32_t n, HcclComm comm)
{
    static std::atomic<int> calls{0};
    HcclOpDesc op;
    EX_CHECK(HcclOpDescInit(&op));
    std::snprintf(op.opName, sizeof(op.opName), "sweep");
    HcclKernelFuncInfo fi;
    std::memset(&fi, 0, sizeof(fi));
    std::snprintf(fi.kernelFuncName, sizeof(fi.kernelFuncName), "SweepKernel");       // in this program: no library name
    SweepKernelArgs args{&calls, (int)rank + 1};
    fi.args = &args;
    fi.argSize = sizeof(args);
    HcclKernelLaunchCfg cfg;
    EX_CHECK(HcclKernelLaunchCfgInit(&cfg));
    ThreadHandle t = 0;
    EX_CHECK(HcclThreadAcquire(comm, COMM_ENGINE_CPU_TS, 1, 1, &t));
    EX_CHECK(HcclAicpuKernelLaunch(comm, &op, &fi, 0, nullptr, &cfg));
    EX_CHECK(HcclAicpuKernelLaunch(comm, &op, &fi, 0, nullptr, nullptr));
    std::snprintf(fi.kernelFuncName, sizeof(fi.kernelFuncName), "SweepKernelFails");
    EXPECT_RC(HcclAicpuKernelLaunch(comm, &op, &fi, 0, nullptr, &cfg), HCCL_E_INTERNAL);
    std::snprintf(fi.kernelFuncName, sizeof(fi.kernelFuncName), "NoSuchKernel");
    EXPECT_RC(HcclAicpuKernelLaunch(comm, &op, &fi, 0, nullptr, &cfg), HCCL_E_NOT_FOUND);
    std::snprintf(fi.kernelSoName, sizeof(fi.kernelSoName), "/nonexistent/libsweep.so");
    EXPECT_RC(HcclAicpuKernelLaunch(comm, &op, &fi, 0, nullptr, &cfg), HCCL_E_OPEN_FILE_FAILURE);
    op.header.magicWord = 0;
    EXPECT_RC(HcclAicpuKernelLaunch(comm, &op, &fi, 0, nullptr, &cfg), HCCL_E_PARA);
    // what a fused compute + communication kernel is given: the communicator's device block, the launch stream, notifies
    void *ctx = nullptr, *ctx2 = nullptr, *ctx3 = nullptr;
    EX_CHECK(HcclAllocComResource(comm, 0, &ctx));
    EX_CHECK(HcclAllocComResourceByTiling(comm, nullptr, nullptr, &ctx2));
    char commName[COMM_NAME_MAX_LENGTH] = "";
    EX_CHECK(HcclGetCommName(comm, commName));
    EX_CHECK(HcclCreateComResource(commName, 0, &ctx3));
    EX_EXPECT(ctx != nullptr && ctx == ctx2 && ctx3 != nullptr);
    EXPECT_RC(HcclCreateComResource("no such communicator", 0, &ctx3), HCCL_E_NOT_FOUND);
    aclrtStream opStream = (aclrtStream)1;
    void *notifies[2] = {nullptr, nullptr};
    EX_CHECK(HcclGetAicpuOpStreamAndNotify(comm, &opStream, 2, notifies));
    EX_EXPECT(notifies[0] != nullptr && (char *)notifies[1] == (char *)notifies[0] + 8);
    void *one = nullptr;
    EX_CHECK(HcclGetAicpuOpStreamNotify(commName, &opStream, &one));
    EXPECT_RC(HcclGetAicpuOpStreamNotify("no such communicator", &opStream, &one), HCCL_E_NOT_FOUND);
    EX_CHECK(HcclBarrier(comm, nullptr));
    EX_EXPECT(calls.load() == (int)(n * (n + 1)));         // every rank launched twice with rank + 1
    EX_CHECK(HcclBarrier(comm, nullptr));
    if (rank == 0) calls.store(0);
}

// ------------------------------------------------------------------------- the other ways to create a communicator

static std::string MakeRankTable(uint32_t n, const char *instance)
{
    std::ostringstream os;
    os << "{\"version\": \"2.0\", \"rank_count\": " << n << ", \"status\": \"completed\", \"rank_list\": [";
    for (uint32_t r = 0; r < n; ++r) {
        os << (r ? ", " : "") << "{\"rank_id\": " << r << ", \"device_id\": " << r << ", \"local_id\": " << r
           << ", \"level_list\": [{\"net_layer\": 0, \"net_instance_id\": \"" << instance << "\", \"net_type\": \"TOPO_FILE_DESC\", \"net_attr\": \"\", "
           << "\"rank_addr_list\": [{\"addr_type\": \"IPV4\", \"addr\": \"127.0.0.1\", \"ports\": [\"0/" << r << "\"]}]}]}";
    }
    os << "]}";
    return os.str();
}

static void SumOverRanks(uint32_t n, const std::vector<HcclComm> &comms)
{
    std::vector<std::thread> ts;
    for (uint32_t r = 0; r < n; ++r)
        ts.emplace_back([&, r] {
            double x = (double)(r + 1), sum = 0;
            EX_CHECK(HcclAllReduce(&x, &sum, 1, HCCL_DATA_TYPE_FP64, HCCL_REDUCE_SUM, comms[r], nullptr));
            EX_EXPECT(sum == (double)n * (n + 1) / 2);
        });
    for (auto &t : ts) t.join();
}

static void OtherWaysToStart(uint32_t n)
{
    // all ranks from one call
    std::vector<int32_t> devices(n);
    std::iota(devices.begin(), devices.end(), 0);
    std::vector<HcclComm> comms(n, nullptr);
    EX_CHECK(HcclCommInitAll(n, devices.data(), comms.data()));
    EXPECT_RC(HcclCommInitAll(0, devices.data(), comms.data()), HCCL_E_PARA);
    SumOverRanks(n, comms);
    // one thread destroys them one after the other: no call may wait for ranks that only this thread can bring along
    const auto before = std::chrono::steady_clock::now();
    for (HcclComm c : comms) EX_CHECK(HcclCommDestroy(c));
    EX_EXPECT(std::chrono::steady_clock::now() - before < std::chrono::seconds(3));

    // root info with a configuration: a name of the caller's choice, a buffer size, a deterministic setting
    HcclRootInfo info;
    EX_CHECK(HcclGetRootInfo(&info));
    std::vector<std::thread> ts;
    for (uint32_t r = 0; r < n; ++r)
        ts.emplace_back([&, r] {
            HcclCommConfig cfg;
            HcclCommConfigInit(&cfg);
            std::snprintf(cfg.hcclCommName, sizeof(cfg.hcclCommName), "sweep_named");
            cfg.hcclBufferSize = 1;
            cfg.hcclDeterministic = 1;
            EX_CHECK(HcclCommInitRootInfoConfig(n, &info, r, &cfg, &comms[r]));
            char name[COMM_NAME_MAX_LENGTH] = "";
            EX_CHECK(HcclGetCommName(comms[r], name));
            EX_EXPECT(std::string(name) == "sweep_named");
            void *buf = nullptr;
            uint64_t size = 0;
            EX_CHECK(HcclGetHcclBuffer(comms[r], &buf, &size));
            EX_EXPECT(size == 2u << 20);
        });
    for (auto &t : ts) t.join();
    ts.clear();
    SumOverRanks(n, comms);
    for (HcclComm c : comms) EX_CHECK(HcclCommDestroy(c));

    // a rank table: every rank reads the same file, nothing else is exchanged beforehand
    const std::string path = "/tmp/hccl_sweep_table_" + std::to_string((long)getpid()) + ".json";
    {
        std::ofstream f(path);
        f << MakeRankTable(n, "sweep_node");
    }
    for (uint32_t r = 0; r < n; ++r)
        ts.emplace_back([&, r] {
            if (r % 2 == 0) {
                EX_CHECK(HcclCommInitClusterInfo(path.c_str(), r, &comms[r]));
            } else {
                HcclCommConfig cfg;
                HcclCommConfigInit(&cfg);
                EX_CHECK(HcclCommInitClusterInfoConfig(path.c_str(), r, &cfg, &comms[r]));
            }
        });
    for (auto &t : ts) t.join();
    ts.clear();
    SumOverRanks(n, comms);
    HcclComm none = nullptr;
    EXPECT_RC(HcclCommInitClusterInfo(path.c_str(), n, &none), HCCL_E_PARA);              // not in the table
    EX_EXPECT(HcclCommInitClusterInfo("/nonexistent/table.json", 0, &none) != HCCL_SUCCESS);
    for (HcclComm c : comms) EX_CHECK(HcclCommDestroy(c));
    unlink(path.c_str());

    // the same table handed over as text in memory
    {
        const std::string text = MakeRankTable(n, "sweep_text");
        for (uint32_t r = 0; r < n; ++r)
            ts.emplace_back([&, r] {
                CommAttr attr{HCCL_MODE_ANY, r};
                EX_CHECK(HcclInitComm(text.c_str(), r, &attr, &comms[r]));
            });
        for (auto &t : ts) t.join();
        ts.clear();
        SumOverRanks(n, comms);
        for (uint32_t r = 0; r < n; ++r) ts.emplace_back([&, r] { EX_CHECK(HcclFinalizeComm(comms[r])); });
        for (auto &t : ts) t.join();
        ts.clear();
    }

    // the world group from a rank table (one rank: the group is process-wide)
    const std::string solo = "/tmp/hccl_sweep_solo_" + std::to_string((long)getpid()) + ".json";
    {
        std::ofstream f(solo);
        f << MakeRankTable(1, "sweep_solo");
    }
    EX_CHECK(HcomInitByRankTable(solo.c_str(), 0));
    EXPECT_RC(HcomInitByRankTable(solo.c_str(), 0), HCCL_E_PARA);                          // already there
    uint32_t size = 0, id = 9;
    EX_CHECK(HcomGetRankSize(HCCL_WORLD_GROUP, &size));
    EX_CHECK(HcomGetRankId(HCCL_WORLD_GROUP, &id));
    EX_EXPECT(size == 1 && id == 0);
    float one = 3.f, res = 0.f;
    EX_CHECK(HcomAllReduce("t", &one, &res, 1, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, HCCL_WORLD_GROUP, nullptr));
    EX_EXPECT(res == 3.f);
    EX_CHECK(HcomDestroy());
    unlink(solo.c_str());
    // and from the table as text, with the rank as a string
    const std::string soloText = MakeRankTable(1, "sweep_solo_text");
    EXPECT_RC(HcomInitByString(soloText.c_str(), "zero"), HCCL_E_PARA);
    EX_CHECK(HcomInitByString(soloText.c_str(), "0"));
    EX_EXPECT(HcomFindGroup(HCCL_WORLD_GROUP));
    EX_CHECK(HcomDestroy());
    EX_EXPECT(!HcomFindGroup(HCCL_WORLD_GROUP));

    // a restored process image: what is left of its communicators is invalid
    HcclComm last = nullptr;
    EX_CHECK(HcclGetRootInfo(&info));
    EX_CHECK(HcclCommInitRootInfo(1, &info, 0, &last));
    char name[COMM_NAME_MAX_LENGTH] = "";
    EX_CHECK(HcclGetCommName(last, name));
    EX_CHECK(HcclSnapshotRestore());
    EXPECT_RC(HcclAllReduce(&one, &res, 1, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, last, nullptr), HCCL_E_PARA);
    HcclCommStatus status = HCCL_COMM_STATUS_READY;
    EX_CHECK(HcclCommGetStatus(name, &status));
    EX_EXPECT(status == HCCL_COMM_STATUS_INVALID);
}

// ------------------------------------------------- bring-up inside a group, channel requests that cannot be served

extern "C" void HcommToolReloadEnv(void);       // re-reads the environment variables (exported for tests)
static void SumOverRanks(uint32_t n, const std::vector<HcclComm> &comms);

static void EdgeCases(uint32_t n)
{
    // communicators whose creation is queued by a group: nothing exists before the group ends
    HcclRootInfo info;
    EX_CHECK(HcclGetRootInfo(&info));
    std::vector<HcclComm> comms(n, nullptr);
    std::vector<std::thread> ts;
    for (uint32_t r = 0; r < n; ++r)
        ts.emplace_back([&, r] {
            EX_CHECK(HcclGroupStart());
            EX_CHECK(HcclCommInitRootInfo(n, &info, r, &comms[r]));
            EX_EXPECT(comms[r] == nullptr);
            EX_CHECK(HcclGroupEnd());
            EX_EXPECT(comms[r] != nullptr);
        });
    for (auto &t : ts) t.join();
    ts.clear();
    SumOverRanks(n, comms);
    {
        // nobody is lost: the "survivors" are all ranks, and the new communicator is a second one of the same size
        std::vector<HcclComm> fresh(n, nullptr);
        for (uint32_t r = 0; r < n; ++r)
            ts.emplace_back([&, r] {
                uint32_t size = 0;
                std::vector<uint32_t> old(n, 99);
                EX_CHECK(HcclCommRecover(comms[r], 20, &fresh[r], &size, old.data()));
                EX_EXPECT(size == n && old[r] == r);
                uint32_t id = 99;
                EX_CHECK(HcclGetRankId(fresh[r], &id));
                EX_EXPECT(id == r);
            });
        for (auto &t : ts) t.join();
        ts.clear();
        SumOverRanks(n, fresh);
        for (uint32_t r = 0; r < n; ++r) ts.emplace_back([&, r] { EX_CHECK(HcclCommDestroy(fresh[r])); });
        for (auto &t : ts) t.join();
        ts.clear();
    }
    if (n >= 2) {
        // more notify slots than a pair of ranks has: the whole request is rolled back, a smaller one is served
        for (uint32_t r = 0; r < 2; ++r)
            ts.emplace_back([&, r] {
                HcclChannelDesc d[2];
                EX_CHECK(HcclChannelDescInit(d, 2));
                d[0].remoteRank = d[1].remoteRank = 1 - r;
                d[0].notifyNum = 40;
                d[1].notifyNum = 30;
                ChannelHandle h[2] = {7, 7};
                EXPECT_RC(HcclChannelAcquire(comms[r], COMM_ENGINE_CPU_TS, d, 2, h), HCCL_E_UNAVAIL);
                EX_EXPECT(h[0] == 0 && h[1] == 0);
                EX_CHECK(HcclChannelQuery(comms[r], COMM_ENGINE_CPU_TS, d, 1, h));
                EX_EXPECT(h[0] == 0);                      // the first channel of the failed request is gone too
                EX_CHECK(HcclChannelAcquire(comms[r], COMM_ENGINE_CPU_TS, d, 1, h));
                EX_EXPECT(h[0] != 0);
                EX_CHECK(HcommChannelNotifyRecord(h[0], 39));
                EX_CHECK(HcommChannelNotifyWait(h[0], 39, 10));
                d[0].notifyNum = 65;
                EXPECT_RC(HcclChannelAcquire(comms[r], COMM_ENGINE_CPU_TS, d, 1, h), HCCL_E_PARA);     // more than a channel can hold
                d[0].notifyNum = 1;
                d[0].remoteRank = r;
                EXPECT_RC(HcclChannelAcquire(comms[r], COMM_ENGINE_CPU_TS, d, 1, h), HCCL_E_PARA);     // a channel to oneself
                d[0].remoteRank = 1 - r;
                d[0].channelProtocol = COMM_PROTOCOL_ROCE;
                EXPECT_RC(HcclChannelAcquire(comms[r], COMM_ENGINE_CPU_TS, d, 1, h), HCCL_E_NOT_SUPPORT);
                d[0].header.magicWord = 0;
                EXPECT_RC(HcclChannelAcquire(comms[r], COMM_ENGINE_CPU_TS, d, 1, h), HCCL_E_PARA);
            });
        for (auto &t : ts) t.join();
        ts.clear();
        // a peer that never asks for its end of the channel: the request gives up after the connect timeout
        setenv("HCCL_CONNECT_TIMEOUT", "2", 1);
        HcommToolReloadEnv();
        HcclChannelDesc d;
        EX_CHECK(HcclChannelDescInit(&d, 1));
        d.remoteRank = 1;
        d.notifyNum = 2;
        ChannelHandle h = 0;
        const auto before = std::chrono::steady_clock::now();
        EXPECT_RC(HcclChannelAcquire(comms[0], COMM_ENGINE_CPU_TS, &d, 1, &h), HCCL_E_TIMEOUT);
        const auto took = std::chrono::steady_clock::now() - before;
        EX_EXPECT(took >= std::chrono::milliseconds(1900) && took < std::chrono::seconds(8));
        unsetenv("HCCL_CONNECT_TIMEOUT");
        HcommToolReloadEnv();
    }
    for (uint32_t r = 0; r < n; ++r) ts.emplace_back([&, r] { EX_CHECK(HcclCommDestroy(comms[r])); });
    for (auto &t : ts) t.join();
}

// --------------------------------------------------- tagged host messages with matched probe, also over a connection

static std::atomic<uint32_t> g_rawPort{0};

static void Messages(uint32_t rank, uint32_t n, HcclComm comm)
{
    if (n < 2) return;
    const int right = (int)((rank + 1) % n), left = (int)((rank + n - 1) % n);
    // two messages with different tags to the right neighbour; the receiver takes the second tag first
    std::vector<int32_t> a(100, (int32_t)rank), b(7, (int32_t)(rank + 1000));
    HcclRequest reqs[4] = {nullptr, nullptr, nullptr, nullptr};
    EX_CHECK(HcclIsend(a.data(), 100, HCCL_DATA_TYPE_INT32, right, 5, comm, &reqs[0]));
    EX_CHECK(HcclIsend(b.data(), 7, HCCL_DATA_TYPE_INT32, right, 6, comm, &reqs[1]));
    EXPECT_RC(HcclIsend(a.data(), 1, HCCL_DATA_TYPE_INT32, (int)n, 5, comm, &reqs[2]), HCCL_E_PARA);
    EXPECT_RC(HcclIsend(a.data(), 1, HCCL_DATA_TYPE_INT32, right, -2, comm, &reqs[2]), HCCL_E_PARA);
    int flag = 0, count = -1;
    HcclMessage msg = nullptr;
    HcclStatus st;
    for (int spin = 0; spin < 20000 && !flag; ++spin) {
        EX_CHECK(HcclImprobe(left, 6, comm, &flag, &msg, &st));
        if (!flag) usleep(500);
    }
    EX_EXPECT(flag == 1 && st.srcRank == left && st.tag == 6 && st.error == 0);
    EX_CHECK(HcclGetCount(&st, HCCL_DATA_TYPE_INT32, &count));
    EX_EXPECT(count == 7);
    EXPECT_RC(HcclGetCount(&st, HCCL_DATA_TYPE_INT64, &count), HCCL_E_PARA);       // 28 bytes are no whole number of those
    std::vector<int32_t> got(7, -1);
    std::vector<int32_t> tooSmall(3);
    EXPECT_RC(HcclImrecv(tooSmall.data(), 3, HCCL_DATA_TYPE_INT32, &msg, &reqs[2]), HCCL_E_MEMORY);
    EX_EXPECT(msg != nullptr);                             // still the caller's
    EX_CHECK(HcclImrecv(got.data(), 7, HCCL_DATA_TYPE_INT32, &msg, &reqs[2]));
    EX_EXPECT(msg == nullptr && got[0] == left + 1000 && got[6] == left + 1000);
    // the first message is still queued: found by a probe that names neither source nor tag
    flag = 0;
    for (int spin = 0; spin < 20000 && !flag; ++spin) {
        EX_CHECK(HcclImprobe(HCCL_ANY_SOURCE, HCCL_ANY_TAG, comm, &flag, &msg, &st));
        if (!flag) usleep(500);
    }
    EX_EXPECT(flag == 1 && st.srcRank == left && st.tag == 5 && st.count == 400);
    std::vector<int32_t> big(100, -1);
    EX_CHECK(HcclImrecv(big.data(), 100, HCCL_DATA_TYPE_INT32, &msg, &reqs[3]));
    EX_EXPECT(big[99] == left);
    EX_CHECK(HcclImprobe(left, 5, comm, &flag, &msg, &st));
    EX_EXPECT(flag == 0 && msg == nullptr);                // nothing left
    int done = 0, idx[4];
    HcclStatus sts[4];
    EX_CHECK(HcclTestSome(4, reqs, &done, idx, sts));
    EX_EXPECT(done == 4 && reqs[0] == nullptr && reqs[3] == nullptr && sts[0].count == 400 && sts[3].srcRank == left);
    EX_CHECK(HcclTestSome(4, reqs, &done, idx, sts));
    EX_EXPECT(done == 0);                                  // each completion is reported once
    EXPECT_RC(HcclImprobe((int)n, 5, comm, &flag, &msg, &st), HCCL_E_PARA);
    EX_CHECK(HcclBarrier(comm, nullptr));                  // the wildcard probes above must not meet what follows
    // an empty message is a message
    EX_CHECK(HcclIsend(nullptr, 0, HCCL_DATA_TYPE_INT8, left, 9, comm, &reqs[0]));
    flag = 0;
    for (int spin = 0; spin < 20000 && !flag; ++spin) {
        EX_CHECK(HcclImprobe(right, 9, comm, &flag, &msg, &st));
        if (!flag) usleep(500);
    }
    EX_EXPECT(flag == 1 && st.count == 0);
    EX_CHECK(HcclImrecv(nullptr, 0, HCCL_DATA_TYPE_INT8, &msg, &reqs[1]));
    EX_CHECK(HcclTestSome(2, reqs, &done, idx, sts));
    EX_EXPECT(done == 2);
    int buffer[16];
    EX_CHECK(HcclRegisterMemory(comm, buffer, sizeof(buffer)));
    EX_CHECK(HcclUnregisterMemory(comm, buffer));
    EXPECT_RC(HcclUnregisterMemory(comm, buffer), HCCL_E_NOT_FOUND);
    if (rank == 0) {
        EX_CHECK(HcclRegisterGlobalMemory(buffer, sizeof(buffer)));
        EXPECT_RC(HcclRegisterGlobalMemory(buffer, sizeof(buffer)), HCCL_E_PARA);
        EX_CHECK(HcclUnregisterGlobalMemory(buffer));
        EXPECT_RC(HcclUnregisterGlobalMemory(buffer), HCCL_E_NOT_FOUND);
    }
    EX_CHECK(HcclBarrier(comm, nullptr));

    // ---- the same between two endpoints without a communicator: rank 0 listens, rank 1 connects
    if (rank == 0) {
        HcclConn listener = nullptr, peer = nullptr;
        EX_CHECK(HcclRawOpen(&listener));
        EXPECT_RC(HcclRawListen(listener, 4), HCCL_E_PARA);                        // not bound yet
        HcclAddr addr;
        std::memset(&addr, 0, sizeof(addr));
        addr.type = HCCL_ADDR_TYPE_ROCE;
        EX_CHECK(HcclRawBind(listener, &addr));
        EX_EXPECT(addr.info.tcp.port != 0);
        EX_CHECK(HcclRawListen(listener, 4));
        g_rawPort.store(addr.info.tcp.port);
        HcclAddr from;
        EX_CHECK(HcclRawAccept(listener, &from, &peer));
        EX_EXPECT(from.info.tcp.ipv4Addr != 0);
        flag = 0;
        for (int spin = 0; spin < 20000 && !flag; ++spin) {
            EX_CHECK(HcclRawImprobe(peer, &flag, &msg, &st));
            if (!flag) usleep(500);
        }
        EX_EXPECT(flag == 1 && st.count == 40);
        EX_CHECK(HcclRawGetCount(&st, HCCL_DATA_TYPE_FP32, &count));
        EX_EXPECT(count == 10);
        float head[4] = {0}, tail[6] = {0};
        void *bufs[2] = {head, tail};
        int counts[2] = {4, 6};
        HcclRequest rr = nullptr;
        EX_CHECK(HcclRawImrecvScatter(bufs, counts, 2, HCCL_DATA_TYPE_FP32, &msg, &rr));
        EX_EXPECT(head[3] == 3.f && tail[0] == 4.f && tail[5] == 9.f);
        EX_CHECK(HcclRawIsend(tail, 6, HCCL_DATA_TYPE_FP32, peer, &reqs[0]));      // an answer
        reqs[1] = rr;
        EX_CHECK(HcclRawTestSome(2, reqs, &done, idx, sts));
        EX_EXPECT(done == 2);
        EX_CHECK(HcclRawClose(peer));
        EX_CHECK(HcclRawForceClose(listener));
        EXPECT_RC(HcclRawClose(nullptr), HCCL_E_PTR);
    } else if (rank == 1) {
        while (g_rawPort.load() == 0) usleep(1000);
        HcclConn conn = nullptr;
        EX_CHECK(HcclRawOpen(&conn));
        HcclAddr addr;
        std::memset(&addr, 0, sizeof(addr));
        addr.type = HCCL_ADDR_TYPE_ROCE;
        addr.info.tcp.port = (uint16_t)g_rawPort.load();                           // address 0: this host
        EX_CHECK(HcclRawConnect(conn, &addr));
        float ten[10];
        for (int i = 0; i < 10; ++i) ten[i] = (float)i;
        EX_CHECK(HcclRawIsend(ten, 10, HCCL_DATA_TYPE_FP32, conn, &reqs[0]));
        flag = 0;
        for (int spin = 0; spin < 20000 && !flag; ++spin) {
            EX_CHECK(HcclRawImprobe(conn, &flag, &msg, &st));
            if (!flag) usleep(500);
        }
        EX_EXPECT(flag == 1 && st.count == 24);
        float back[6] = {0};
        EX_CHECK(HcclRawImrecv(back, 6, HCCL_DATA_TYPE_FP32, &msg, &reqs[1]));
        EX_EXPECT(back[0] == 4.f && back[5] == 9.f);
        EX_CHECK(HcclRawTestSome(2, reqs, &done, idx, sts));
        EX_EXPECT(done == 2);
        EX_CHECK(HcclRawClose(conn));
    }
    EX_CHECK(HcclBarrier(comm, nullptr));
}

// ---------------------------------------------------------------------------------- argument rules of the operators

static void ArgumentRules(uint32_t rank, uint32_t n, HcclComm comm)
{
    float x[8] = {1, 2, 3, 4, 5, 6, 7, 8}, y[8] = {0};
    // nothing to do is not an error, whatever the pointers say
    EX_CHECK(HcclAllReduce(nullptr, nullptr, 0, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, comm, nullptr));
    EX_CHECK(HcclBroadcast(nullptr, 0, HCCL_DATA_TYPE_FP32, 0, comm, nullptr));
    EX_CHECK(HcclAllGather(nullptr, nullptr, 0, HCCL_DATA_TYPE_FP32, comm, nullptr));
    // missing communicator or buffers
    EXPECT_RC(HcclAllReduce(x, y, 8, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, nullptr, nullptr), HCCL_E_PTR);
    EXPECT_RC(HcclAllReduce(nullptr, y, 8, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, comm, nullptr), HCCL_E_PTR);
    EXPECT_RC(HcclAllReduce(x, nullptr, 8, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, comm, nullptr), HCCL_E_PTR);
    EXPECT_RC(HcclBroadcast(nullptr, 8, HCCL_DATA_TYPE_FP32, 0, comm, nullptr), HCCL_E_PTR);
    int notAComm[64] = {0};
    EXPECT_RC(HcclAllReduce(x, y, 8, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, (HcclComm)notAComm, nullptr), HCCL_E_PTR);
    // counts beyond the limit, undefined reductions and types, roots and peers outside the communicator
    EXPECT_RC(HcclAllReduce(x, y, 0x800000000ull, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, comm, nullptr), HCCL_E_PARA);
    EXPECT_RC(HcclAllReduce(x, y, 8, HCCL_DATA_TYPE_FP32, (HcclReduceOp)9, comm, nullptr), HCCL_E_PARA);
    EX_EXPECT(HcclAllReduce(x, y, 8, (HcclDataType)77, HCCL_REDUCE_SUM, comm, nullptr) != HCCL_SUCCESS);
    EXPECT_RC(HcclBroadcast(x, 8, HCCL_DATA_TYPE_FP32, n, comm, nullptr), HCCL_E_PARA);
    EXPECT_RC(HcclReduce(x, y, 8, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, n + 3, comm, nullptr), HCCL_E_PARA);
    EX_EXPECT(HcclSend(x, 8, HCCL_DATA_TYPE_FP32, n, comm, nullptr) != HCCL_SUCCESS);
    EX_EXPECT(HcclSend(x, 8, HCCL_DATA_TYPE_FP32, rank, comm, nullptr) != HCCL_SUCCESS);        // to oneself
    EX_EXPECT(HcclRecv(y, 8, HCCL_DATA_TYPE_FP32, n + 1, comm, nullptr) != HCCL_SUCCESS);
    // variable counts: the list must agree with the own count
    std::vector<uint64_t> counts(n, 2), displs(n);
    for (uint32_t q = 0; q < n; ++q) displs[q] = 2 * q;
    std::vector<float> in(2 * n, 1.f), out(2, 0.f);
    EXPECT_RC(HcclReduceScatterV(in.data(), counts.data(), displs.data(), out.data(), 3, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, comm, nullptr), HCCL_E_PARA);
    EXPECT_RC(HcclReduceScatterV(in.data(), nullptr, displs.data(), out.data(), 2, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, comm, nullptr), HCCL_E_PTR);
    HcclSendRecvItem item;
    item.sendRecvType = HCCL_SEND; item.buf = x; item.count = 8; item.dataType = HCCL_DATA_TYPE_FP32; item.remoteRank = n;
    EX_EXPECT(HcclBatchSendRecv(&item, 1, comm, nullptr) != HCCL_SUCCESS);
    EX_EXPECT(HcclBatchSendRecv(nullptr, 1, comm, nullptr) != HCCL_SUCCESS);
    // none of the refusals has left anything behind: the next operator runs
    EX_CHECK(HcclAllReduce(x, y, 8, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, comm, nullptr));
    EX_EXPECT(y[7] == 8.f * (float)n);
    HcclResult err = HCCL_E_INTERNAL;
    EX_CHECK(HcclGetCommAsyncError(comm, &err));
    EX_EXPECT(err == HCCL_SUCCESS);
    // a second communicator of the same name for the same rank in one process is refused
    if (n == 1) {
        char name[COMM_NAME_MAX_LENGTH] = "";
        EX_CHECK(HcclGetCommName(comm, name));
        HcclRootInfo info;
        EX_CHECK(HcclGetRootInfo(&info));
        HcclCommConfig cfg;
        HcclCommConfigInit(&cfg);
        std::snprintf(cfg.hcclCommName, sizeof(cfg.hcclCommName), "%s", name);
        HcclComm twin = nullptr;
        EXPECT_RC(HcclCommInitRootInfoConfig(1, &info, 0, &cfg, &twin), HCCL_E_PARA);
    }
}

int main(int argc, char **argv)
{
    const uint32_t n = argc > 1 ? (uint32_t)std::atoi(argv[1]) : 4;
    ExRunRanks(n, [&](uint32_t rank, HcclComm comm) {
        RankGraph(rank, n, comm);
        CommQueries(rank, n, comm);
        InnerOperators(rank, n, comm);
        Resources(rank, n, comm);
        BaseLevel(rank, n, comm);
        Teams(rank, n, comm);
        Diagnostics(rank, n, comm);
        Launch(rank, n, comm);
        Messages(rank, n, comm);
        ArgumentRules(rank, n, comm);
    });
    EdgeCases(n);
    OtherWaysToStart(n);
    std::printf("api_sweep: %u ranks ok\n", n);
    return 0;
}
