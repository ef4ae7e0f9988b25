/*
 * hcom.h - named-group ("graph mode") API used by the python `hccl` package and by frameworks
 * that address communicators by group name (reference: pkg_inc/legacy/hccl/hcom.h:167-352).
 * The world group is called "hccl_world_group".
 */
#ifndef HCOM_H_
#define HCOM_H_

#include <stdbool.h>

#include "hccl_rank_graph.h"
#include "hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif

#define HCCL_WORLD_GROUP "hccl_world_group"

HcclResult HcomInitByRankTable(const char *rankTable, uint32_t rankId);
/* Adopt an existing communicator as the world group (for processes bootstrapped by root info). */
HcclResult HcomInitByComm(HcclComm comm);
HcclResult HcomDestroy(void);
HcclResult HcomGetInitStatus(bool *initiated);
HcclResult HcomCreateGroup(const char *group, uint32_t rankNum, uint32_t *rankIds);
HcclResult HcomDestroyGroup(const char *group);
HcclResult HcomGetCommHandleByGroup(const char *group, HcclComm *commHandle);
HcclResult HcomGetRankSize(const char *group, uint32_t *rankSize);
HcclResult HcomGetRankId(const char *group, uint32_t *rankId);
HcclResult HcomGetLocalRankSize(const char *group, uint32_t *localRankSize);
HcclResult HcomGetLocalRankId(const char *group, uint32_t *localRankId);
HcclResult HcomGetWorldRankFromGroupRank(const char *group, uint32_t groupRank, uint32_t *worldRank);
HcclResult HcomGetGroupRankFromWorldRank(uint32_t worldRank, const char *group, uint32_t *groupRank);

/* Gradient fusion split: boundaries by gradient index, or by cumulative size percentage. */
HcclResult HcomSetGradFusionByIndex(const char *group, uint32_t segmentNum, const uint32_t *idxList);
HcclResult HcomSetGradFusionBySize(const char *group, uint32_t segmentNum, const float *sizeList);
/* Resolve the stored strategy for a model with gradNum gradients of the given byte sizes into
 * segment end indices (inclusive).  segIdx must hold gradNum entries; *segNum receives the count. */
HcclResult HcomGetSplitStrategy(const char *group, uint32_t gradNum, const uint64_t *gradBytes, uint32_t *segIdx,
                                uint32_t *segNum);

HcclResult HcomGetInCCLbuffer(const char *group, void **buffer, uint64_t *size);
HcclResult HcomGetOutCCLbuffer(const char *group, void **buffer, uint64_t *size);
HcclResult HcomGetCommCCLBufferSize(const char *group, uint64_t *size);
HcclResult HcomGetBandWidthPerNPU(uint32_t level, float *bandWidthGBs);
HcclResult HcomGetServerNumAndDeviceNumPerServer(uint32_t *serverNum, uint32_t *deviceNumPerServer,
                                                 uint32_t *deviceNumPerAggregation);
HcclResult HcomGetAlgorithm(uint32_t level, char **algo);
HcclResult HcomGetL0TopoTypeEx(const char *group, CommTopo *topoType, uint32_t flag);
HcclResult HcomSupportDeterministicOptim(const char *group, bool *isDeterministicOptim);

HcclResult HcomAllReduce(const char *tag, void *in, void *out, uint64_t count, HcclDataType dataType, HcclReduceOp op,
                         const char *group, aclrtStream stream);
HcclResult HcomAllGather(const char *tag, void *in, void *out, uint64_t inCount, HcclDataType dataType,
                         const char *group, aclrtStream stream);
HcclResult HcomReduceScatter(const char *tag, void *in, void *out, uint64_t outCount, HcclDataType dataType,
                             HcclReduceOp op, const char *group, aclrtStream stream);
HcclResult HcomBroadcast(const char *tag, void *ptr, uint64_t count, HcclDataType dataType, uint32_t root,
                         const char *group, aclrtStream stream);
HcclResult HcomReduce(const char *tag, void *in, void *out, uint64_t count, HcclDataType dataType, HcclReduceOp op,
                      uint32_t root, const char *group, aclrtStream stream);
HcclResult HcomSend(const char *tag, void *in, uint64_t count, HcclDataType dataType, uint32_t destRank,
                    uint32_t srTag, const char *group, aclrtStream stream);
HcclResult HcomReceive(const char *tag, void *out, uint64_t count, HcclDataType dataType, uint32_t srcRank,
                       uint32_t srTag, const char *group, aclrtStream stream);
HcclResult HcomAllToAll(const void *in, uint64_t sendCount, HcclDataType sendType, const void *out,
                        uint64_t recvCount, HcclDataType recvType, const char *group, aclrtStream stream,
                        const char *tag);
HcclResult HcomAlltoAllV(const void *in, const void *sendCounts, const void *sdispls, HcclDataType sendType,
                         const void *out, const void *recvCounts, const void *rdispls, HcclDataType recvType,
                         const char *group, aclrtStream stream, const char *tag);
HcclResult HcomAllGatherV(const char *tag, const void *sendBuf, uint64_t sendCount, const void *recvBuf, const void *recvCounts,
                          const void *rdispls, HcclDataType dataType, const char *group, aclrtStream stream);
HcclResult HcomReduceScatterV(const char *tag, void *sendBuf, const void *sendCounts, const void *sdispls, void *recvBuf,
                              uint64_t recvCount, HcclDataType dataType, HcclReduceOp op, const char *group, aclrtStream stream);
HcclResult HcomAlltoAllVC(const void *sendBuf, const void *sendCountMatrix, HcclDataType sendType, const void *recvBuf,
                          HcclDataType recvType, const char *group, aclrtStream stream, const char *tag);

/* ---- further calls of the reference's hcom.h that have a meaning here (pkg_inc/legacy/hccl/hcom.h:205-352) ---- */

/* The world group from a rank table held in memory; `identify` is this process's rank as a decimal string. */
HcclResult HcomInitByString(const char *rankTableM, const char *identify);
/* The world group when only the master's address is known: every process calls this with the same master address, port,
 * master device and rank count, and with its own address.  The process that sits at the master's address on the master's
 * device collects the others, numbers all of them (by address, then device, then arrival) and hands out the ranks together
 * with a root-info ticket; then everybody joins as with HcclCommInitRootInfo.  All arguments are decimal strings or
 * dotted addresses, as the reference passes them (pkg_inc/legacy/hccl/hcom.h:244). */
HcclResult HcomInitByMasterInfo(const char *masterIp, const char *masterPort, const char *masterDeviceId, const char *rankSize,
                                const char *rankIp);
bool HcomFindGroup(const char *group);
HcclResult HcomGetRankSizeEx(const char *group, uint32_t *rankSize, uint32_t flag);
HcclResult HcomReleaseSubComms(void);                 /* destroys every group but the world group */
HcclResult HcomCreateCommCCLbuffer(const char *group); /* the buffer exists with the group: checks the name */

/* How operators are issued: one by one by the caller (operator base) or from a compiled graph.  Kept per process. */
typedef enum {
    HCCL_WORKFLOW_MODE_OPS_KERNEL_INFO_LIB = 0,
    HCCL_WORKFLOW_MODE_OP_BASE = 1,
    HCCL_WORKFLOW_MODE_RESERVED = 255
} HcclWorkflowMode;
HcclWorkflowMode HcomGetWorkflowMode(void);
HcclResult HcomSetWorkflowMode(HcclWorkflowMode mode);

typedef enum { PROFILING_CLOSE = 0, PROFILING_OPEN = 1, PROFILING_RESERVED } HcomProfilingMode;
/* Switches operator records and device timestamps on or off for every group. */
HcclResult HcomSetProfilingMode(HcomProfilingMode profilingMode, const char *profilingOption);

/* What the selector would pick for such an operator on the group: ifAiv tells whether a kernel of the SM engine runs it,
 * algName (at least 128 bytes) receives "operator/algorithm@engine".  counts != NULL marks a variable-count operator. */
HcclResult HcomSelectAlg(int64_t comm, const char *group, uint64_t count, void *counts, HcclDataType dataType, HcclReduceOp op,
                         HcclCMDType opType, int32_t aivCoreLimit, bool *ifAiv, char *algName);
/* The CTAs that kernel would be launched with (0 on the host engine). */
HcclResult HcomCalcAivCoreNum(const char *group, HcclCMDType opType, uint64_t count, void *counts, HcclDataType dataType,
                              int32_t aivCoreLimit, char *algName, uint32_t *numBlocks);
/* Upper bound of CTAs per collective kernel of the group, so that compute kernels keep their share of the SMs; 0 lifts it. */
HcclResult HcomSetAivCoreLimit(const char *group, uint32_t aivCoreLimit);
/* A tag that is the same on every rank for the n-th operator of a kind on a group: "<opType>_<group>_<n>". */
HcclResult HcomGenerateCclOpTag(const char *opType, int64_t hcomComm, const char *group, char *sTag);

/* Resources of fused compute + communication kernels, by group name (hccl_mc2.h). */
HcclResult HcomCreateComResourceByComm(HcclComm comm, uint32_t streamMode, bool isOpbaseMode, void **commContext);
HcclResult HcomGetAicpuOpStreamNotify(const char *group, aclrtStream *opStream, uint8_t aicpuNotifyNum, void **aicpuNotify);
HcclResult HcomMc2AiCpuStreamAllocAndGet(const char *group, uint32_t streamMode, aclrtStream *aiCpuStream);

#ifdef __cplusplus
}
#endif
#endif /* HCOM_H_ */
