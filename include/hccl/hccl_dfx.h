/*
 * hccl_dfx.h - diagnostics hooks that callers register with the library, profiling reports, operator retry control
 * and the extended ("ex" / "expt") entry points of the reference.
 * (reference: pkg_inc/hcomm/hcomm_exception.h:78, pkg_inc/hccl/hcomm_diag.h:40-55, pkg_inc/hccl/hccl_diag.h:29-51,
 *  pkg_inc/legacy/hccl/hccl_ex.h:206-232, pkg_inc/hccl/hccl_res_expt.h:44-99, pkg_inc/hcomm/hcomm_primitives_expt.h:32,
 *  framework/cluster_maintenance/recovery/operator_retry/hccl_op_retry_pub.h:30-65.)
 */
#ifndef HCCL_DFX_H
#define HCCL_DFX_H

#include <stddef.h>

#include "hccl_diag.h"
#include "hccl_res.h"
#include "hccl_types.h"
#include "../hcomm_res_defs.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ exception callbacks */

typedef enum tagHcommExceptionExpandType {
    HCOMM_EXCEPTION_INVALID = -1,
    HCOMM_EXCEPTION_STARS,      /* kept for source compatibility; never raised here */
    HCOMM_EXCEPTION_ROCE,
    HCOMM_EXCEPTION_URMA,
    HCOMM_EXCEPTION_NVLINK_WAIT /* a bounded wait on a peer's flag expired (detail.waitInfo is valid) */
} HcommExceptionExpandType;

typedef struct tagStarsExDetailInfo {
    uint32_t starsErrcode;
    uint8_t sqeType;
    uint8_t statusMerged;
    uint8_t rsvd[122];
} StarsExDetailInfo;

typedef struct tagHcommExceptionExpandInfo {
    HcommExceptionExpandType type;
    union {
        StarsExDetailInfo starsInfo;
        HcclDeviceWaitStatus waitInfo;
    } detail;
} HcommExceptionExpandInfo;

typedef struct tagHcommExceptionInfo {
    CommAbiHeader header;
    uint64_t thread;   /* thread handle the failing task ran on (0: an operator's own stream) */
    uint64_t channel;  /* channel handle involved (0: none) */
    uint32_t taskId;   /* operator ordinal on its communicator */
    uint32_t retCode;  /* HcclResult */
    uint8_t rsvd[40];
    HcommExceptionExpandInfo expandInfo;
} HcommExceptionInfo;

typedef void (*HcommExceptionCallback)(const HcommExceptionInfo *exceptionInfo, void *userData);
/* Called (from the thread that discovers it) whenever a communicator records an asynchronous failure. */
int32_t HcommExceptionRegisterCallback(HcommExceptionCallback cb, void *userData);
int32_t HcommExceptionUnregisterCallback(HcommExceptionCallback cb);

/* Operator description that the caller attaches to a communicator; on an exception the registered formatter turns it
 * into text that is logged with the failure and returned by HcclDiagDump. */
HcclResult HcommRegOpInfo(const char *commId, void *opInfo, size_t size);
typedef void (*HcommGetOpInfoCallback)(const void *opInfo, char *outPut, size_t size);
HcclResult HcommRegOpTaskException(const char *commId, HcommGetOpInfoCallback callback);

/* ------------------------------------------------------------------ profiling reports */

#define HCOMM_ALG_TAG_LENGTH 288
typedef struct HcclDfxOpInfo {
    CommAbiHeader header;
    uint64_t beginTime;
    uint64_t endTime;
    uint32_t opMode;
    uint32_t opType;
    uint32_t reduceOp;
    uint32_t dataType;
    uint32_t outputType;
    uint64_t dataCount;
    uint32_t root;
    char algTag[HCOMM_ALG_TAG_LENGTH];
    CommEngine engine;
    uint64_t cpuTsThread;
    uint32_t cpuWaitAicpuNotifyIdx;
    uint32_t cpuWaitAicpuNotifyId;
    uint64_t inputMemAddr;
    uint64_t inputMemSize;
    uint64_t outputMemAddr;
    uint64_t outputMemSize;
    int8_t reserve[96];
} HcclDfxOpInfo;

/* A profiling sink receives every report below (and one per operator the library launches while profiling is on).
 * kind: 0 operator, 1 kernel start, 2 kernel end, 3 device operator. */
typedef void (*HcclProfilingSink)(int kind, const char *group, const char *name, uint64_t beginNs, uint64_t endNs, void *userData);
HcclResult HcclProfilingSetSink(HcclProfilingSink sink, void *userData);
uint64_t HcommGetProfilingSysCycleTime(void);                 /* monotonic nanoseconds: the time base of all reports */
HcclResult HcclProfilingReportOp(HcclComm comm, uint64_t beginTime);
HcclResult HcclReportAicpuKernel(HcclComm comm, uint64_t beginTime, char *kernelName);
HcclResult HcclReportAivKernel(HcclComm comm, uint64_t beginTime);
HcclResult HcclDfxRegOpInfoByCommId(char *commId, void *hcclDfxOpInfo);
HcclResult HcommProfilingReportDeviceOp(const char *groupname);
HcclResult HcommProfilingReportKernelStartTask(uint64_t thread, const char *groupname);
HcclResult HcommProfilingReportKernelEndTask(uint64_t thread, const char *groupname);

/* ------------------------------------------------------------------ operator retry */

/* Retry is on when HCCL_OP_RETRY_ENABLE (or the communicator configuration's hcclRetryEnable) enables it; parameters come
 * from HCCL_OP_RETRY_PARAMS / hcclRetryParams ("MaxCnt:3,HoldTime:5000,IntervalTime:1000", times in milliseconds). */
typedef struct {
    uint32_t enabled;
    uint32_t maxCnt, holdTimeMs, intervalMs;
    uint64_t requests;    /* retries this rank asked for */
    uint64_t rounds;      /* retry rounds this rank took part in */
    uint64_t succeeded;   /* rounds after which the operator completed on every rank */
    uint64_t failed;      /* rounds that ended in HCCL_E_OPRETRY_FAIL */
} HcclOpRetryStats;
HcclResult HcclCommGetOpRetryStats(HcclComm comm, HcclOpRetryStats *stats);

/* ------------------------------------------------------------------ extended entry points */

typedef struct {
    uint32_t algSets;   /* bit a set: algorithm family a (HcclAlgoType order: ring, pipeline, fullmesh, H-D_R, pairwise, NHR, ...) can be forced */
    uint32_t rankSize;
} HcclTopoDescs;
/* One entry per algorithm level (level 0 = inside the NVLink domain); topoSize = entries in the caller's array. */
HcclResult HcclGetTopoDesc(HcclComm comm, HcclTopoDescs *topoDescs, uint32_t topoSize);
/* Window registration under the names of the reference's extension header. */
HcclResult HcclCommRegister(HcclComm comm, void *addr, uint64_t size, void **handle, uint32_t flag);
HcclResult HcclCommDeregister(HcclComm comm, void *handle);
HcclResult HcclCommExchangeMem(HcclComm comm, void *windowHandle, uint32_t *peerRanks, uint32_t peerRankNum);
/* Peer's CCL buffer as mapped in this process. */
HcclResult HcclGetRemoteIpcHcclBuf(HcclComm comm, uint64_t remoteRank, void **addr, uint64_t *size);
/* Device memory owned by the communicator and found again by tag (created on first use with *size bytes). */
HcclResult HcclDevMemAcquire(HcclComm comm, const char *memTag, uint64_t *size, void **addr, bool *newCreated);
/* The same execution contexts seen from another engine (here every engine drives CUDA streams: the handles are shared). */
HcclResult HcclThreadExportToCommEngine(HcclComm comm, uint32_t threadNum, const ThreadHandle *threads, CommEngine dstCommEngine,
                                        ThreadHandle *exportedThreads);
typedef int32_t(HcclTaskCallback)(uint64_t, int32_t);
/* Host callbacks by message tag: HcclTaskNotify(comm, tag, ...) queues a call on a stream. */
int32_t HcclTaskRegister(HcclComm comm, const char *msgTag, HcclTaskCallback cb);
int32_t HcclTaskUnRegister(HcclComm comm, const char *msgTag);
int32_t HcclTaskNotify(HcclComm comm, const char *msgTag, uint64_t arg0, int32_t arg1, aclrtStream stream);
/* Extra bytes that every rank contributes to the consistency exchange done when channels are created. */
HcclResult HcclCommAddExchangeInfo(HcclComm comm, const void *data, uint32_t length);
HcclResult HcclCommGetExchangeInfo(HcclComm comm, uint32_t rank, void *data, uint32_t capacity, uint32_t *length);
HcclResult HcclCommResetExchangeInfo(HcclComm comm);
/* Waits until everything queued on the thread has run (timeout in seconds, 0 = no limit). */
int32_t HcommThreadJoin(ThreadHandle thread, uint32_t timeout);

#ifdef __cplusplus
}
#endif
#endif /* HCCL_DFX_H */
