/*
 * hccl_res.h - per-communicator resources an operator needs: the CCL buffer, threads, tagged
 * engine contexts, registered memory (reference: include/hccl/hccl_res.h:39-210).
 */
#ifndef HCCL_RES_H
#define HCCL_RES_H

#include "hccl_channel.h"
#include "hccl_types.h"
#include "hcomm_res_defs.h"

#ifdef __cplusplus
extern "C" {
#endif

#define HCCL_RES_TAG_MAX_LEN 255u

/* Local CCL buffer: in-half followed by out-half, each hcclBufferSize MB, peer-visible.
 * The library's own operators stage their data in the same buffer (the stream engine's HcclBarrier included: it is a
 * one-element all-reduce), so a custom operator that keeps data there must not run a built-in operator on this
 * communicator until it has consumed the data; between its own steps it synchronises through channel notifies. */
HcclResult HcclGetHcclBuffer(HcclComm comm, void **buffer, uint64_t *size);
HcclResult HcclGetHcclBufferCleared(HcclComm comm, void **buffer, uint64_t *size);

HcclResult HcclThreadAcquire(HcclComm comm, CommEngine engine, uint32_t threadNum, uint32_t notifyNumPerThread,
                             ThreadHandle *threads);
HcclResult HcclThreadAcquireWithConfig(HcclComm comm, CommEngine engine, uint32_t threadNum, ThreadType type,
                                       const ThreadConfig *config, ThreadHandle *threads);
/* Wrap a caller-owned stream so primitives join the caller's ordering. */
HcclResult HcclThreadAcquireWithStream(HcclComm comm, CommEngine engine, aclrtStream stream, uint32_t notifyNum,
                                       ThreadHandle *thread);

typedef enum {
    HCCL_DED_THREAD_TYPE_INVALID = -1,
    HCCL_DED_THREAD_TYPE_AICPU_LAUNCH = 0,
    HCCL_DED_THREAD_TYPE_AICPU_LAUNCH_GE = 1,
    HCCL_DED_THREAD_TYPE_AICPU_ORDER_LAUNCH_OPBASE = 2,
    HCCL_DED_THREAD_TYPE_AICPU_ORDER_LAUNCH_ACLGRAPH = 3,
    HCCL_DED_THREAD_TYPE_AICPU_ORDER_LAUNCH_GE = 4,
    HCCL_DED_THREAD_TYPE_AICPU_ORDER_LAUNCH_DEVICE = 5
} HcclDedicatedThreadType;
/* One thread per use type per communicator, created on first request: keeps launches of that kind ordered. */
HcclResult HcclDedicatedThreadAcquire(HcclComm comm, HcclDedicatedThreadType useType, uint32_t notifyNumPerThread,
                                      ThreadHandle *thread);

/* Named blobs that live where `engine` can read them (device memory for SM/NVLS, host otherwise). */
HcclResult HcclEngineCtxCreate(HcclComm comm, const char *ctxTag, CommEngine engine, uint64_t size, void **ctx);
HcclResult HcclEngineCtxGet(HcclComm comm, const char *ctxTag, CommEngine engine, void **ctx, uint64_t *size);
HcclResult HcclEngineCtxCopy(HcclComm comm, CommEngine engine, const char *ctxTag, const void *srcCtx,
                             uint64_t size, uint64_t dstCtxOffset);
HcclResult HcclEngineCtxDestroy(HcclComm comm, const char *ctxTag, CommEngine engine);

HcclResult HcclCommMemReg(HcclComm comm, const char *memTag, const CommMem *mem, HcclMemHandle *memHandle);
HcclResult HcclCommMemUnreg(HcclComm comm, HcclMemHandle memHandle);

typedef aclrtStream ThreadResTypeStream;
HcclResult HcclThreadResGetInfo(HcclComm comm, ThreadHandle thread, ThreadResType resType, uint32_t infoLen,
                                void **info);

#ifdef __cplusplus
}
#endif
#endif /* HCCL_RES_H */
