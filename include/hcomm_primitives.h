/*
 * hcomm_primitives.h - data-plane primitives issued on a Thread, optionally through a Channel.
 *
 * The same verbs exist in three places:
 *   - here, as host calls that enqueue work on the thread's engine (CUDA stream / simulator worker);
 *   - in csrc/device/hcomm_device.cuh, as __device__ functions for code running on the SM engine;
 *   - as opcodes of the schedule IR that the algorithm templates emit.
 * Verb set and batch descriptor layout follow include/hcomm_primitives.h:77-593 of the reference.
 *
 * Ordering: operations issued on one thread execute in issue order.  A *Nbi ("non-blocking
 * implicit") operation may complete later; HcommChannelFence* / HcommFenceOnThread order it.
 * Notify semantics are counting: each Record adds one to the target slot, each Wait consumes one.
 * Every Wait is bounded by `timeOut` seconds (0 = the communicator's exec timeout) and reports
 * HCCL_E_TIMEOUT through the owning communicator's async-error word instead of hanging.
 */
#ifndef HCOMM_PRIMITIVES_H
#define HCOMM_PRIMITIVES_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#include "hcomm_res_defs.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    HCOMM_REDUCE_SUM = 0,
    HCOMM_REDUCE_PROD = 1,
    HCOMM_REDUCE_MAX = 2,
    HCOMM_REDUCE_MIN = 3,
    HCOMM_REDUCE_RESERVED = 255
} HcommReduceOp;

typedef enum {
    HCOMM_DATA_TYPE_INT8 = 0,
    HCOMM_DATA_TYPE_INT16 = 1,
    HCOMM_DATA_TYPE_INT32 = 2,
    HCOMM_DATA_TYPE_FP16 = 3,
    HCOMM_DATA_TYPE_FP32 = 4,
    HCOMM_DATA_TYPE_INT64 = 5,
    HCOMM_DATA_TYPE_UINT64 = 6,
    HCOMM_DATA_TYPE_UINT8 = 7,
    HCOMM_DATA_TYPE_UINT16 = 8,
    HCOMM_DATA_TYPE_UINT32 = 9,
    HCOMM_DATA_TYPE_FP64 = 10,
    HCOMM_DATA_TYPE_BFP16 = 11,
    HCOMM_DATA_TYPE_INT128 = 12,
    HCOMM_DATA_TYPE_HIF8 = 14,
    HCOMM_DATA_TYPE_FP8E4M3 = 15,
    HCOMM_DATA_TYPE_FP8E5M2 = 16,
    HCOMM_DATA_TYPE_FP8E8M0 = 17,
    HCOMM_DATA_TYPE_RESERVED = 255
} HcommDataType;

typedef enum {
    HCOMM_TRANSFER_TYPE_INVALID = -1,
    HCOMM_TRANSFER_TYPE_WRITE = 0,
    HCOMM_TRANSFER_TYPE_WRITE_REDUCE = 1,
    HCOMM_TRANSFER_TYPE_WRITE_WITH_NOTIFY = 2,
    HCOMM_TRANSFER_TYPE_WRITE_REDUCE_WITH_NOTIFY = 3,
    HCOMM_TRANSFER_TYPE_READ = 4,
    HCOMM_TRANSFER_TYPE_READ_REDUCE = 5,
    HCOMM_TRANSFER_TYPE_NOTIFY_RECORD = 6
} HcommTransferType;

/* One element of a batch; 64 bytes. */
typedef struct {
    HcommTransferType transType;
    uint8_t reserved[4];
    union {
        uint8_t raws[56];
        struct { uint64_t len; void *dst; void *src; } write;
        struct { uint64_t len; void *dst; void *src; } read;
        struct { uint64_t count; void *dst; void *src; HcommReduceOp reduceOp; HcommDataType dataType; } reduce;
        struct { uint32_t notifyIdx; } notifyRecord;
        struct { uint64_t len; void *dst; void *src; uint32_t notifyIdx; } writeWithNotify;
        struct {
            uint64_t count; void *dst; void *src; HcommReduceOp reduceOp; HcommDataType dataType; uint32_t notifyIdx;
        } writeReduceWithNotify;
    } transferInfo;
} HcommBatchTransferDesc;

/* ---- local (same-device) operations ------------------------------------------------------- */
int32_t HcommLocalCopyOnThread(ThreadHandle thread, void *dst, const void *src, uint64_t len);
int32_t HcommLocalReduceOnThread(ThreadHandle thread, void *dst, const void *src, uint64_t count,
                                 HcommDataType dataType, HcommReduceOp reduceOp);
int32_t HcommThreadNotifyRecordOnThread(ThreadHandle thread, ThreadHandle dstThread, uint32_t dstNotifyIdx);
int32_t HcommThreadNotifyWaitOnThread(ThreadHandle thread, uint32_t notifyIdx, uint32_t timeOut);
int32_t HcommThreadNotifyWaitOnThreadWithDefaultTimeout(ThreadHandle thread, uint32_t notifyIdx);
/* Raw notify ids name a 64-bit word in the process; kept for callers that manage their own. */
int32_t HcommAclrtNotifyRecordOnThread(ThreadHandle thread, uint64_t dstNotifyId);
int32_t HcommAclrtNotifyWaitOnThread(ThreadHandle thread, uint64_t notifyId, uint32_t timeOut);

/* ---- one-sided transfers through a channel ------------------------------------------------- */
int32_t HcommWriteOnThread(ThreadHandle thread, ChannelHandle channel, void *dst, const void *src, uint64_t len);
int32_t HcommWriteReduceOnThread(ThreadHandle thread, ChannelHandle channel, void *dst, const void *src,
                                 uint64_t count, HcommDataType dataType, HcommReduceOp reduceOp);
int32_t HcommWriteWithNotifyOnThread(ThreadHandle thread, ChannelHandle channel, void *dst, const void *src,
                                     uint64_t len, uint32_t remoteNotifyIdx);
int32_t HcommWriteReduceWithNotifyOnThread(ThreadHandle thread, ChannelHandle channel, void *dst, const void *src,
                                           uint64_t count, HcommDataType dataType, HcommReduceOp reduceOp,
                                           uint32_t remoteNotifyIdx);
int32_t HcommReadOnThread(ThreadHandle thread, ChannelHandle channel, void *dst, const void *src, uint64_t len);
int32_t HcommReadReduceOnThread(ThreadHandle thread, ChannelHandle channel, void *dst, const void *src,
                                uint64_t count, HcommDataType dataType, HcommReduceOp reduceOp);
int32_t HcommWriteNbiOnThread(ThreadHandle thread, ChannelHandle channel, void *dst, const void *src, uint64_t len);
int32_t HcommWriteNbi(ChannelHandle channel, void *dst, const void *src, uint64_t len);
int32_t HcommWriteWithNotifyNbiOnThread(ThreadHandle thread, ChannelHandle channel, void *dst, const void *src,
                                        uint64_t len, uint32_t remoteNotifyIdx);
int32_t HcommWriteWithNotifyNbi(ChannelHandle channel, void *dst, const void *src, uint64_t len,
                                uint32_t remoteNotifyIdx);
int32_t HcommReadNbiOnThread(ThreadHandle thread, ChannelHandle channel, void *dst, const void *src, uint64_t len);
int32_t HcommReadNbi(ChannelHandle channel, void *dst, const void *src, uint64_t len);
int32_t HcommBatchTransferOnThread(ThreadHandle thread, ChannelHandle channel, const HcommBatchTransferDesc *descs,
                                   uint32_t descNum);

/* ---- synchronisation ------------------------------------------------------------------------ */
int32_t HcommChannelNotifyRecordOnThread(ThreadHandle thread, ChannelHandle channel, uint32_t remoteNotifyIdx);
int32_t HcommChannelNotifyRecord(ChannelHandle channel, uint32_t remoteNotifyIdx);
int32_t HcommChannelNotifyWaitOnThread(ThreadHandle thread, ChannelHandle channel, uint32_t localNotifyIdx,
                                       uint32_t timeOut);
int32_t HcommChannelNotifyWait(ChannelHandle channel, uint32_t localNotifyIdx, uint32_t timeOut);
int32_t HcommChannelNotifyWaitOnThreadWithDefaultTimeout(ThreadHandle thread, ChannelHandle channel,
                                                         uint32_t localNotifyIdx);
int32_t HcommFenceOnThread(ThreadHandle thread);
/* B200 extension: blocks the caller until everything queued on the thread so far has run (the stream of the thread is
 * synchronised) and reports an expired wait of the thread's communicator as HCCL_E_TIMEOUT. */
int32_t HcommThreadSynchronize(ThreadHandle thread);
int32_t HcommChannelFenceOnThread(ThreadHandle thread, ChannelHandle channel);
int32_t HcommChannelFence(ChannelHandle channel);
int32_t HcommChannelDrainOnThread(ThreadHandle thread, ChannelHandle channel);
int32_t HcommSetNotifyWaitTimeOut(float timeOut);
int32_t HcommThreadResAcquireTimeOut(float timeOut);

/* ---- launch batching and task replay --------------------------------------------------------
 * Batch mode defers every primitive issued between Start and End and submits them together.
 * The task cache records the expanded task list of one operator under `tag`; on a hit the list
 * is replayed with the buffer addresses patched (a CUDA graph is captured per tag on CUDA).
 */
int32_t HcommBatchModeStart(const char *batchTag);
int32_t HcommBatchModeEnd(const char *batchTag);
HcommResult HcommAicpuTsTaskCacheLookup(const char *tag, bool *isHit);
HcommResult HcommAicpuTsTaskCacheStart(const char *tag, void **addrs, uint64_t *sizes, uint64_t count);
HcommResult HcommAicpuTsTaskCacheEnd(const char *tag);
HcommResult HcommAicpuTsTaskCacheExecute(const char *tag, void **addrs, uint64_t *sizes, uint64_t count);
HcommResult HcommAicpuTsTaskCacheClear(const char *tag);
int32_t HcommAcquireComm(const char *commId);
int32_t HcommReleaseComm(const char *commId);

#ifdef __cplusplus
}
#endif
#endif /* HCOMM_PRIMITIVES_H */
