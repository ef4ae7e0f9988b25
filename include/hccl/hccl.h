/*
 * hccl.h - collective and point-to-point operators.
 *
 * Every call is asynchronous with respect to `stream` on a CUDA platform and blocking on the
 * host simulator.  count == 0 returns HCCL_SUCCESS without touching anything; null handles or
 * buffers return HCCL_E_PTR.  The *Inner spellings are the entry points of the reference's
 * in-tree operators (pkg_inc/legacy/hccl/hccl_inner.h:22-76) and are aliases here.
 */
#ifndef HCCL_H_
#define HCCL_H_

#include "hccl_comm.h"
#include "hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif

HcclResult HcclAllReduce(void *sendBuf, void *recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op,
                         HcclComm comm, aclrtStream stream);
HcclResult HcclBroadcast(void *buf, uint64_t count, HcclDataType dataType, uint32_t root, HcclComm comm,
                         aclrtStream stream);
HcclResult HcclReduceScatter(void *sendBuf, void *recvBuf, uint64_t recvCount, HcclDataType dataType,
                             HcclReduceOp op, HcclComm comm, aclrtStream stream);
HcclResult HcclReduceScatterV(void *sendBuf, const void *sendCounts, const void *sendDispls, void *recvBuf,
                              uint64_t recvCount, HcclDataType dataType, HcclReduceOp op, HcclComm comm,
                              aclrtStream stream);
HcclResult HcclScatter(void *sendBuf, void *recvBuf, uint64_t recvCount, HcclDataType dataType, uint32_t root,
                       HcclComm comm, aclrtStream stream);
HcclResult HcclGather(void *sendBuf, void *recvBuf, uint64_t sendCount, HcclDataType dataType, uint32_t root,
                      HcclComm comm, aclrtStream stream);
HcclResult HcclAllGather(void *sendBuf, void *recvBuf, uint64_t sendCount, HcclDataType dataType, HcclComm comm,
                         aclrtStream stream);
HcclResult HcclAllGatherV(void *sendBuf, uint64_t sendCount, void *recvBuf, const void *recvCounts,
                          const void *recvDispls, HcclDataType dataType, HcclComm comm, aclrtStream stream);
HcclResult HcclSend(void *sendBuf, uint64_t count, HcclDataType dataType, uint32_t destRank, HcclComm comm,
                    aclrtStream stream);
HcclResult HcclRecv(void *recvBuf, uint64_t count, HcclDataType dataType, uint32_t srcRank, HcclComm comm,
                    aclrtStream stream);
HcclResult HcclBatchSendRecv(HcclSendRecvItem *items, uint32_t itemNum, HcclComm comm, aclrtStream stream);
/* counts / displacements are uint64_t arrays of rankSize entries, in elements. */
HcclResult HcclAlltoAllV(const void *sendBuf, const void *sendCounts, const void *sdispls, HcclDataType sendType,
                         const void *recvBuf, const void *recvCounts, const void *rdispls, HcclDataType recvType,
                         HcclComm comm, aclrtStream stream);
/* sendCountMatrix is rankSize x rankSize uint64_t, row i = what rank i sends to each rank. */
HcclResult HcclAlltoAllVC(const void *sendBuf, const void *sendCountMatrix, HcclDataType sendType,
                          const void *recvBuf, HcclDataType recvType, HcclComm comm, aclrtStream stream);
HcclResult HcclAlltoAll(const void *sendBuf, uint64_t sendCount, HcclDataType sendType, const void *recvBuf,
                        uint64_t recvCount, HcclDataType recvType, HcclComm comm, aclrtStream stream);
HcclResult HcclReduce(void *sendBuf, void *recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op,
                      uint32_t root, HcclComm comm, aclrtStream stream);

/*
 * B200 extension: AllReduce with a scale fused into the reduction.
 * recv[i] = scale * sum_r send_r[i]; the sum and the product are formed in fp32 and rounded once to the
 * operand type.  inType and outType must be the same floating-point type (fp16, bf16, fp32, fp64); a
 * conversion on the way is not offered.  Used by the data-parallel gradient hook (divide by the world
 * size and keep bf16) without a second kernel.
 */
HcclResult HcclAllReduceScaled(void *sendBuf, void *recvBuf, uint64_t count, HcclDataType inType,
                               HcclDataType outType, float scale, HcclComm comm, aclrtStream stream);

#define HCCL_INNER_ALIAS(name) Hccl##name##Inner
HcclResult HcclAllReduceInner(void *, void *, uint64_t, HcclDataType, HcclReduceOp, HcclComm, aclrtStream);
HcclResult HcclBroadcastInner(void *, uint64_t, HcclDataType, uint32_t, HcclComm, aclrtStream);
HcclResult HcclReduceScatterInner(void *, void *, uint64_t, HcclDataType, HcclReduceOp, HcclComm, aclrtStream);
HcclResult HcclReduceScatterVInner(void *, const void *, const void *, void *, uint64_t, HcclDataType, HcclReduceOp,
                                   HcclComm, aclrtStream);
HcclResult HcclScatterInner(void *, void *, uint64_t, HcclDataType, uint32_t, HcclComm, aclrtStream);
HcclResult HcclAllGatherInner(void *, void *, uint64_t, HcclDataType, HcclComm, aclrtStream);
HcclResult HcclAllGatherVInner(void *, uint64_t, void *, const void *, const void *, HcclDataType, HcclComm,
                               aclrtStream);
HcclResult HcclSendInner(void *, uint64_t, HcclDataType, uint32_t, HcclComm, aclrtStream);
HcclResult HcclRecvInner(void *, uint64_t, HcclDataType, uint32_t, HcclComm, aclrtStream);
HcclResult HcclAlltoAllVCInner(const void *, const void *, HcclDataType, const void *, HcclDataType, HcclComm,
                               aclrtStream);
HcclResult HcclAlltoAllVInner(const void *, const void *, const void *, HcclDataType, const void *, const void *,
                              const void *, HcclDataType, HcclComm, aclrtStream);
HcclResult HcclAlltoAllInner(const void *, uint64_t, HcclDataType, const void *, uint64_t, HcclDataType, HcclComm,
                             aclrtStream);
HcclResult HcclReduceInner(void *, void *, uint64_t, HcclDataType, HcclReduceOp, uint32_t, HcclComm, aclrtStream);
HcclResult HcclBatchSendRecvInner(HcclSendRecvItem *, uint32_t, HcclComm, aclrtStream);

#ifdef __cplusplus
}
#endif
#endif /* HCCL_H_ */
