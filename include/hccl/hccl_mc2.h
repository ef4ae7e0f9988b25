/*
 * hccl_mc2.h - what a fused compute + communication kernel needs from a communicator.
 * (reference: pkg_inc/legacy/hccl/hccl_ex.h:195-204, the resource calls of its matmul + collective operators: a
 * "communication context" handed to the kernel, and the stream with notifies on which the communication side runs.)
 *
 * Here the context is the communicator's device block (CommDev of hcomm_comm_dev.h: heap bases of all ranks, flag
 * pages, buffer sizes, rank and size), which the kernels of hcomm_fused.h and user kernels built on hcomm_device.cuh
 * take as their argument.  On the host simulator it is the host copy of that block.
 */
#ifndef HCCL_MC2_H
#define HCCL_MC2_H

#include "hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif

HcclResult HcclAllocComResource(HcclComm comm, uint32_t streamMode, void **commContext);
/* The tiling argument is accepted and not read: the fused kernels choose their tiles themselves. */
HcclResult HcclAllocComResourceByTiling(HcclComm comm, void *stream, void *mc2Tiling, void **commContext);
HcclResult HcclCreateComResource(const char *commName, uint32_t streamMode, void **commContext);
/* The communicator's launch thread: its stream and notify words (addresses a kernel or a host thread can signal). */
HcclResult HcclGetAicpuOpStreamNotify(const char *commName, aclrtStream *opStream, void **aicpuNotify);
HcclResult HcclGetAicpuOpStreamAndNotify(HcclComm comm, aclrtStream *opStream, uint8_t aicpuNotifyNum, void **aicpuNotify);

#ifdef __cplusplus
}
#endif
#endif /* HCCL_MC2_H */
