// coll_api.cc - C entry points of the operators (include/hccl/hccl.h).
//
// Argument rules follow the reference (op_base_host.cc:67-131, param_check.cc:150-343):
//   count == 0 succeeds without doing anything; counts above 0x7FFFFFFFF are rejected; null
//   communicator or buffers give HCCL_E_PTR with an EI0003 report; the reduction operator and the
//   data type must be defined and, for reducing collectives, arithmetic.
#include <cstring>

#include "../coll/ops.h"
#include "../core/dtype.h"
#include "../core/log.h"
#include "hccl/hccl.h"

using namespace hc;

namespace {

constexpr uint64_t kSysMaxCount = 0x7FFFFFFFFull;

HcclResult CheckCommon(Comm *c, uint64_t count, HcclDataType t, const char *opName)
{
    if (!c) {
        RPT_ERR("EI0003", "%s: communicator handle is null or invalid", opName);
        return HCCL_E_PTR;
    }
    if (count > kSysMaxCount) {
        RPT_ERR("EI0003", "%s: count %llu exceeds the limit %llu", opName, (unsigned long long)count, (unsigned long long)kSysMaxCount);
        return HCCL_E_PARA;
    }
    if (DtypeSize(t) == 0) {
        RPT_ERR("EI0003", "%s: data type %d is not defined", opName, (int)t);
        return HCCL_E_PARA;
    }
    return HCCL_SUCCESS;
}

HcclResult CheckReduce(HcclDataType t, HcclReduceOp op, const char *opName)
{
    if (op != HCCL_REDUCE_SUM && op != HCCL_REDUCE_PROD && op != HCCL_REDUCE_MAX && op != HCCL_REDUCE_MIN) {
        RPT_ERR("EI0003", "%s: reduction operator %d is not defined", opName, (int)op);
        return HCCL_E_PARA;
    }
    if (!DtypeReducible(t)) {
        RPT_ERR("EI0003", "%s: data type %s cannot be reduced", opName, DtypeName(t));
        return HCCL_E_NOT_SUPPORT;
    }
    return HCCL_SUCCESS;
}

std::vector<uint64_t> CopyU64(const void *p, size_t n)
{
    const uint64_t *v = (const uint64_t *)p;
    return std::vector<uint64_t>(v, v + n);
}

}  // namespace

extern "C" {

HcclResult HcclAllReduce(void *sendBuf, void *recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op, HcclComm comm, aclrtStream stream)
{
    Comm *c = AsComm(comm);
    CHK_RET(CheckCommon(c, count, dataType, "HcclAllReduce"));
    if (count == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(sendBuf);
    CHK_PTR_NULL(recvBuf);
    CHK_RET(CheckReduce(dataType, op, "HcclAllReduce"));
    OpDesc d;
    d.cmd = HCCL_CMD_ALLREDUCE; d.in = sendBuf; d.out = recvBuf; d.count = count; d.dtype = dataType; d.op = op; d.stream = stream;
    return SubmitOp(c, d);
}

HcclResult HcclAllReduceScaled(void *sendBuf, void *recvBuf, uint64_t count, HcclDataType inType, HcclDataType outType, float scale, HcclComm comm,
                               aclrtStream stream)
{
    Comm *c = AsComm(comm);
    CHK_RET(CheckCommon(c, count, inType, "HcclAllReduceScaled"));
    if (count == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(sendBuf);
    CHK_PTR_NULL(recvBuf);
    if (inType != outType) {
        RPT_ERR("EI0003", "HcclAllReduceScaled: input and output types must match (accumulation is fp32 either way)");
        return HCCL_E_NOT_SUPPORT;
    }
    if (inType != HCCL_DATA_TYPE_FP32 && inType != HCCL_DATA_TYPE_FP16 && inType != HCCL_DATA_TYPE_BFP16 && inType != HCCL_DATA_TYPE_FP64) {
        RPT_ERR("EI0003", "HcclAllReduceScaled: only floating-point types can be scaled");
        return HCCL_E_NOT_SUPPORT;
    }
    OpDesc d;
    d.cmd = HCCL_CMD_ALLREDUCE; d.in = sendBuf; d.out = recvBuf; d.count = count; d.dtype = inType; d.op = HCCL_REDUCE_SUM; d.stream = stream;
    d.useScale = true; d.scale = scale;
    return SubmitOp(c, d);
}

HcclResult HcclBroadcast(void *buf, uint64_t count, HcclDataType dataType, uint32_t root, HcclComm comm, aclrtStream stream)
{
    Comm *c = AsComm(comm);
    CHK_RET(CheckCommon(c, count, dataType, "HcclBroadcast"));
    if (count == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(buf);
    if (root >= c->nRanks) { RPT_ERR("EI0003", "HcclBroadcast: root %u outside the communicator (%u ranks)", root, c->nRanks); return HCCL_E_PARA; }
    OpDesc d;
    d.cmd = HCCL_CMD_BROADCAST; d.in = buf; d.out = buf; d.count = count; d.dtype = dataType; d.root = root; d.stream = stream;
    return SubmitOp(c, d);
}

HcclResult HcclReduceScatter(void *sendBuf, void *recvBuf, uint64_t recvCount, HcclDataType dataType, HcclReduceOp op, HcclComm comm, aclrtStream stream)
{
    Comm *c = AsComm(comm);
    CHK_RET(CheckCommon(c, recvCount, dataType, "HcclReduceScatter"));
    if (recvCount == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(sendBuf);
    CHK_PTR_NULL(recvBuf);
    CHK_RET(CheckReduce(dataType, op, "HcclReduceScatter"));
    OpDesc d;
    d.cmd = HCCL_CMD_REDUCE_SCATTER; d.in = sendBuf; d.out = recvBuf; d.count = recvCount; d.dtype = dataType; d.op = op; d.stream = stream;
    return SubmitOp(c, d);
}

HcclResult HcclReduceScatterV(void *sendBuf, const void *sendCounts, const void *sendDispls, void *recvBuf, uint64_t recvCount, HcclDataType dataType,
                              HcclReduceOp op, HcclComm comm, aclrtStream stream)
{
    Comm *c = AsComm(comm);
    CHK_RET(CheckCommon(c, recvCount, dataType, "HcclReduceScatterV"));
    CHK_PTR_NULL(sendCounts);
    CHK_PTR_NULL(sendDispls);
    CHK_RET(CheckReduce(dataType, op, "HcclReduceScatterV"));
    OpDesc d;
    d.cmd = HCCL_CMD_REDUCE_SCATTER_V; d.in = sendBuf; d.out = recvBuf; d.dtype = dataType; d.op = op; d.stream = stream;
    d.sendCounts = CopyU64(sendCounts, c->nRanks);
    d.sendDispls = CopyU64(sendDispls, c->nRanks);
    uint64_t total = 0;
    for (auto v : d.sendCounts) { if (v > kSysMaxCount) return HCCL_E_PARA; total += v; }
    if (d.sendCounts[c->rank] != recvCount) {
        RPT_ERR("EI0003", "HcclReduceScatterV: recvCount %llu differs from sendCounts[%u] = %llu", (unsigned long long)recvCount, c->rank, (unsigned long long)d.sendCounts[c->rank]);
        return HCCL_E_PARA;
    }
    if (total == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(sendBuf);
    if (recvCount) CHK_PTR_NULL(recvBuf);
    d.count = recvCount;
    return SubmitOp(c, d);
}

HcclResult HcclScatter(void *sendBuf, void *recvBuf, uint64_t recvCount, HcclDataType dataType, uint32_t root, HcclComm comm, aclrtStream stream)
{
    Comm *c = AsComm(comm);
    CHK_RET(CheckCommon(c, recvCount, dataType, "HcclScatter"));
    if (recvCount == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(recvBuf);
    if (root >= c->nRanks) return HCCL_E_PARA;
    if (c->rank == root) CHK_PTR_NULL(sendBuf);
    OpDesc d;
    d.cmd = HCCL_CMD_SCATTER; d.in = sendBuf; d.out = recvBuf; d.count = recvCount; d.dtype = dataType; d.root = root; d.stream = stream;
    return SubmitOp(c, d);
}

HcclResult HcclGather(void *sendBuf, void *recvBuf, uint64_t sendCount, HcclDataType dataType, uint32_t root, HcclComm comm, aclrtStream stream)
{
    Comm *c = AsComm(comm);
    CHK_RET(CheckCommon(c, sendCount, dataType, "HcclGather"));
    if (sendCount == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(sendBuf);
    if (root >= c->nRanks) return HCCL_E_PARA;
    if (c->rank == root) CHK_PTR_NULL(recvBuf);
    OpDesc d;
    d.cmd = HCCL_CMD_GATHER; d.in = sendBuf; d.out = recvBuf; d.count = sendCount; d.dtype = dataType; d.root = root; d.stream = stream;
    return SubmitOp(c, d);
}

HcclResult HcclAllGather(void *sendBuf, void *recvBuf, uint64_t sendCount, HcclDataType dataType, HcclComm comm, aclrtStream stream)
{
    Comm *c = AsComm(comm);
    CHK_RET(CheckCommon(c, sendCount, dataType, "HcclAllGather"));
    if (sendCount == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(sendBuf);
    CHK_PTR_NULL(recvBuf);
    OpDesc d;
    d.cmd = HCCL_CMD_ALLGATHER; d.in = sendBuf; d.out = recvBuf; d.count = sendCount; d.dtype = dataType; d.stream = stream;
    return SubmitOp(c, d);
}

HcclResult HcclAllGatherV(void *sendBuf, uint64_t sendCount, void *recvBuf, const void *recvCounts, const void *recvDispls, HcclDataType dataType,
                          HcclComm comm, aclrtStream stream)
{
    Comm *c = AsComm(comm);
    CHK_RET(CheckCommon(c, sendCount, dataType, "HcclAllGatherV"));
    CHK_PTR_NULL(recvCounts);
    CHK_PTR_NULL(recvDispls);
    OpDesc d;
    d.cmd = HCCL_CMD_ALLGATHER_V; d.in = sendBuf; d.out = recvBuf; d.dtype = dataType; d.stream = stream;
    d.recvCounts = CopyU64(recvCounts, c->nRanks);
    d.recvDispls = CopyU64(recvDispls, c->nRanks);
    uint64_t total = 0;
    for (auto v : d.recvCounts) { if (v > kSysMaxCount) return HCCL_E_PARA; total += v; }
    if (d.recvCounts[c->rank] != sendCount) {
        RPT_ERR("EI0003", "HcclAllGatherV: sendCount %llu differs from recvCounts[%u] = %llu", (unsigned long long)sendCount, c->rank, (unsigned long long)d.recvCounts[c->rank]);
        return HCCL_E_PARA;
    }
    if (total == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(recvBuf);
    if (sendCount) CHK_PTR_NULL(sendBuf);
    d.count = sendCount;
    return SubmitOp(c, d);
}

HcclResult HcclSend(void *sendBuf, uint64_t count, HcclDataType dataType, uint32_t destRank, HcclComm comm, aclrtStream stream)
{
    Comm *c = AsComm(comm);
    CHK_RET(CheckCommon(c, count, dataType, "HcclSend"));
    if (destRank >= c->nRanks || destRank == c->rank) { RPT_ERR("EI0003", "HcclSend: destination rank %u is invalid for rank %u of %u", destRank, c->rank, c->nRanks); return HCCL_E_PARA; }
    if (count == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(sendBuf);
    OpDesc d;
    d.cmd = HCCL_CMD_SEND; d.in = sendBuf; d.out = sendBuf; d.count = count; d.dtype = dataType; d.peer = destRank; d.stream = stream;
    return SubmitOp(c, d);
}

HcclResult HcclRecv(void *recvBuf, uint64_t count, HcclDataType dataType, uint32_t srcRank, HcclComm comm, aclrtStream stream)
{
    Comm *c = AsComm(comm);
    CHK_RET(CheckCommon(c, count, dataType, "HcclRecv"));
    if (srcRank >= c->nRanks || srcRank == c->rank) { RPT_ERR("EI0003", "HcclRecv: source rank %u is invalid for rank %u of %u", srcRank, c->rank, c->nRanks); return HCCL_E_PARA; }
    if (count == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(recvBuf);
    OpDesc d;
    d.cmd = HCCL_CMD_RECEIVE; d.in = recvBuf; d.out = recvBuf; d.count = count; d.dtype = dataType; d.peer = srcRank; d.stream = stream;
    return SubmitOp(c, d);
}

HcclResult HcclBatchSendRecv(HcclSendRecvItem *items, uint32_t itemNum, HcclComm comm, aclrtStream stream)
{
    Comm *c = AsComm(comm);
    if (!c) return HCCL_E_PTR;
    if (itemNum == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(items);
    OpDesc d;
    d.cmd = HCCL_CMD_BATCH_SEND_RECV; d.stream = stream;
    for (uint32_t i = 0; i < itemNum; ++i) {
        const HcclSendRecvItem &it = items[i];
        if (it.sendRecvType != HCCL_SEND && it.sendRecvType != HCCL_RECV) return HCCL_E_PARA;
        if (it.remoteRank >= c->nRanks || DtypeSize(it.dataType) == 0 || it.count > kSysMaxCount) return HCCL_E_PARA;
        if (it.remoteRank == c->rank) { RPT_ERR("EI0003", "HcclBatchSendRecv: item %u names the calling rank as its peer", i); return HCCL_E_PARA; }
        if (it.count && !it.buf) return HCCL_E_PTR;
        d.batch.push_back(it);
    }
    return SubmitOp(c, d);
}

HcclResult HcclAlltoAll(const void *sendBuf, uint64_t sendCount, HcclDataType sendType, const void *recvBuf, uint64_t recvCount, HcclDataType recvType,
                        HcclComm comm, aclrtStream stream)
{
    Comm *c = AsComm(comm);
    CHK_RET(CheckCommon(c, sendCount, sendType, "HcclAlltoAll"));
    if (sendType != recvType || sendCount != recvCount) {
        RPT_ERR("EI0003", "HcclAlltoAll: send and receive descriptions differ (%llu x %s vs %llu x %s)", (unsigned long long)sendCount, DtypeName(sendType),
                (unsigned long long)recvCount, DtypeName(recvType));
        return HCCL_E_PARA;
    }
    if (sendCount == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(sendBuf);
    CHK_PTR_NULL(recvBuf);
    OpDesc d;
    d.cmd = HCCL_CMD_ALLTOALL; d.in = sendBuf; d.out = const_cast<void *>(recvBuf); d.count = sendCount; d.dtype = sendType; d.stream = stream;
    return SubmitOp(c, d);
}

HcclResult HcclAlltoAllV(const void *sendBuf, const void *sendCounts, const void *sdispls, HcclDataType sendType, const void *recvBuf,
                         const void *recvCounts, const void *rdispls, HcclDataType recvType, HcclComm comm, aclrtStream stream)
{
    Comm *c = AsComm(comm);
    CHK_RET(CheckCommon(c, 0, sendType, "HcclAlltoAllV"));
    CHK_PTR_NULL(sendCounts); CHK_PTR_NULL(sdispls); CHK_PTR_NULL(recvCounts); CHK_PTR_NULL(rdispls);
    if (sendType != recvType) return HCCL_E_PARA;
    OpDesc d;
    d.cmd = HCCL_CMD_ALLTOALLV; d.in = sendBuf; d.out = const_cast<void *>(recvBuf); d.dtype = sendType; d.stream = stream;
    d.sendCounts = CopyU64(sendCounts, c->nRanks); d.sendDispls = CopyU64(sdispls, c->nRanks);
    d.recvCounts = CopyU64(recvCounts, c->nRanks); d.recvDispls = CopyU64(rdispls, c->nRanks);
    uint64_t sendTotal = 0, recvTotal = 0;
    for (uint32_t i = 0; i < c->nRanks; ++i) {
        if (d.sendCounts[i] > kSysMaxCount || d.recvCounts[i] > kSysMaxCount) return HCCL_E_PARA;
        sendTotal += d.sendCounts[i]; recvTotal += d.recvCounts[i];
    }
    if (d.sendCounts[c->rank] != d.recvCounts[c->rank]) {
        RPT_ERR("EI0003", "HcclAlltoAllV: what rank %u sends to itself (%llu) differs from what it expects (%llu)", c->rank,
                (unsigned long long)d.sendCounts[c->rank], (unsigned long long)d.recvCounts[c->rank]);
        return HCCL_E_PARA;
    }
    if (sendTotal) CHK_PTR_NULL(sendBuf);
    if (recvTotal) CHK_PTR_NULL(recvBuf);
    // Even a rank with nothing to move takes part: its peers cannot know.
    return SubmitOp(c, d);
}

HcclResult HcclAlltoAllVC(const void *sendBuf, const void *sendCountMatrix, HcclDataType sendType, const void *recvBuf, HcclDataType recvType,
                          HcclComm comm, aclrtStream stream)
{
    Comm *c = AsComm(comm);
    CHK_RET(CheckCommon(c, 0, sendType, "HcclAlltoAllVC"));
    CHK_PTR_NULL(sendCountMatrix);
    if (sendType != recvType) return HCCL_E_PARA;
    const uint32_t n = c->nRanks;
    const uint64_t *m = (const uint64_t *)sendCountMatrix;
    OpDesc d;
    d.cmd = HCCL_CMD_ALLTOALLVC; d.in = sendBuf; d.out = const_cast<void *>(recvBuf); d.dtype = sendType; d.stream = stream;
    d.sendCounts.resize(n); d.sendDispls.resize(n); d.recvCounts.resize(n); d.recvDispls.resize(n);
    uint64_t so = 0, ro = 0, any = 0;
    for (uint32_t q = 0; q < n; ++q) {
        d.sendCounts[q] = m[(uint64_t)c->rank * n + q]; d.sendDispls[q] = so; so += d.sendCounts[q];
        d.recvCounts[q] = m[(uint64_t)q * n + c->rank]; d.recvDispls[q] = ro; ro += d.recvCounts[q];
    }
    for (uint64_t i = 0; i < (uint64_t)n * n; ++i) { if (m[i] > kSysMaxCount) return HCCL_E_PARA; any |= m[i]; }
    if (!any) return HCCL_SUCCESS;   // the matrix is global knowledge: everyone returns together
    if (so) CHK_PTR_NULL(sendBuf);
    if (ro) CHK_PTR_NULL(recvBuf);
    return SubmitOp(c, d);
}

HcclResult HcclReduce(void *sendBuf, void *recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op, uint32_t root, HcclComm comm, aclrtStream stream)
{
    Comm *c = AsComm(comm);
    CHK_RET(CheckCommon(c, count, dataType, "HcclReduce"));
    if (count == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(sendBuf);
    if (root >= c->nRanks) return HCCL_E_PARA;
    if (c->rank == root) CHK_PTR_NULL(recvBuf);
    CHK_RET(CheckReduce(dataType, op, "HcclReduce"));
    OpDesc d;
    d.cmd = HCCL_CMD_REDUCE; d.in = sendBuf; d.out = recvBuf; d.count = count; d.dtype = dataType; d.op = op; d.root = root; d.stream = stream;
    return SubmitOp(c, d);
}

// ---- aliases used by callers that link against the reference's in-tree operator names
HcclResult HcclAllReduceInner(void *s, void *r, uint64_t n, HcclDataType t, HcclReduceOp o, HcclComm c, aclrtStream st) { return HcclAllReduce(s, r, n, t, o, c, st); }
HcclResult HcclBroadcastInner(void *b, uint64_t n, HcclDataType t, uint32_t root, HcclComm c, aclrtStream st) { return HcclBroadcast(b, n, t, root, c, st); }
HcclResult HcclReduceScatterInner(void *s, void *r, uint64_t n, HcclDataType t, HcclReduceOp o, HcclComm c, aclrtStream st) { return HcclReduceScatter(s, r, n, t, o, c, st); }
HcclResult HcclReduceScatterVInner(void *s, const void *sc, const void *sd, void *r, uint64_t n, HcclDataType t, HcclReduceOp o, HcclComm c, aclrtStream st) { return HcclReduceScatterV(s, sc, sd, r, n, t, o, c, st); }
HcclResult HcclScatterInner(void *s, void *r, uint64_t n, HcclDataType t, uint32_t root, HcclComm c, aclrtStream st) { return HcclScatter(s, r, n, t, root, c, st); }
HcclResult HcclAllGatherInner(void *s, void *r, uint64_t n, HcclDataType t, HcclComm c, aclrtStream st) { return HcclAllGather(s, r, n, t, c, st); }
HcclResult HcclAllGatherVInner(void *s, uint64_t n, void *r, const void *rc, const void *rd, HcclDataType t, HcclComm c, aclrtStream st) { return HcclAllGatherV(s, n, r, rc, rd, t, c, st); }
HcclResult HcclSendInner(void *s, uint64_t n, HcclDataType t, uint32_t dst, HcclComm c, aclrtStream st) { return HcclSend(s, n, t, dst, c, st); }
HcclResult HcclRecvInner(void *r, uint64_t n, HcclDataType t, uint32_t src, HcclComm c, aclrtStream st) { return HcclRecv(r, n, t, src, c, st); }
HcclResult HcclAlltoAllVCInner(const void *s, const void *m, HcclDataType st_, const void *r, HcclDataType rt, HcclComm c, aclrtStream st) { return HcclAlltoAllVC(s, m, st_, r, rt, c, st); }
HcclResult HcclAlltoAllVInner(const void *s, const void *sc, const void *sd, HcclDataType st_, const void *r, const void *rc, const void *rd, HcclDataType rt, HcclComm c, aclrtStream st) { return HcclAlltoAllV(s, sc, sd, st_, r, rc, rd, rt, c, st); }
HcclResult HcclAlltoAllInner(const void *s, uint64_t sn, HcclDataType st_, const void *r, uint64_t rn, HcclDataType rt, HcclComm c, aclrtStream st) { return HcclAlltoAll(s, sn, st_, r, rn, rt, c, st); }
HcclResult HcclReduceInner(void *s, void *r, uint64_t n, HcclDataType t, HcclReduceOp o, uint32_t root, HcclComm c, aclrtStream st) { return HcclReduce(s, r, n, t, o, root, c, st); }
HcclResult HcclBatchSendRecvInner(HcclSendRecvItem *items, uint32_t n, HcclComm c, aclrtStream st) { return HcclBatchSendRecv(items, n, c, st); }

}  // extern "C"
