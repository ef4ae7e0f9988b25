/*
 * hccl_one_sided.h - one-sided put/get between two ranks of a communicator
 * (reference: pkg_inc/legacy/hccl/hccl_one_sided_services.h:63-181).
 *
 * Flow: both sides HcclRegisterMem their buffers (yielding opaque 512-byte descriptors), swap
 * descriptors with HcclExchangeMemDesc, HcclEnableMemAccess on the received ones to obtain a
 * usable remote address, then issue HcclBatchPut / HcclBatchGet on a stream.
 */
#ifndef HCCL_ONE_SIDED_H
#define HCCL_ONE_SIDED_H

#include "hccl_types.h"
#include "hcomm_res_defs.h"

#ifdef __cplusplus
extern "C" {
#endif

#define HCCL_MEM_DESC_LENGTH 511u
typedef struct {
    char desc[HCCL_MEM_DESC_LENGTH + 1];
} HcclMemDesc;
typedef struct {
    HcclMemDesc *array;
    uint32_t arrayLength;
} HcclMemDescs;
typedef struct {
    void *localAddr;
    void *remoteAddr;
    uint64_t count;
    HcclDataType dataType;
} HcclOneSideOpDesc;
typedef enum { HCCL_TOPO_FULLMESH = 0, HCCL_TOPO_NUM } HcclTopoType;
typedef struct {
    HcclTopoType topoType;
    uint64_t rsvd0;
    uint64_t rsvd1;
    uint64_t rsvd2;
} HcclPrepareConfig;

HcclResult HcclRegisterMem(HcclComm comm, uint32_t remoteRank, int type, void *addr, uint64_t size,
                           HcclMemDesc *desc);
HcclResult HcclDeregisterMem(HcclComm comm, HcclMemDesc *desc);
HcclResult HcclExchangeMemDesc(HcclComm comm, uint32_t remoteRank, HcclMemDescs *local, int timeout,
                               HcclMemDescs *remote, uint32_t *actualNum);
HcclResult HcclEnableMemAccess(HcclComm comm, HcclMemDesc *remoteMemDesc, CommMem *remoteMem);
HcclResult HcclDisableMemAccess(HcclComm comm, HcclMemDesc *remoteMemDesc);
HcclResult HcclBatchPut(HcclComm comm, uint32_t remoteRank, HcclOneSideOpDesc *desc, uint32_t descNum,
                        aclrtStream stream);
HcclResult HcclBatchGet(HcclComm comm, uint32_t remoteRank, HcclOneSideOpDesc *desc, uint32_t descNum,
                        aclrtStream stream);
HcclResult HcclRegisterGlobalMem(const CommMem *mem, void **memHandle);
HcclResult HcclDeregisterGlobalMem(void *memHandle);
HcclResult HcclCommBindMem(HcclComm comm, void *memHandle);
HcclResult HcclCommUnbindMem(HcclComm comm, void *memHandle);
/* Pre-build every pairwise connection so the first put/get does not pay for it. */
HcclResult HcclCommPrepare(HcclComm comm, const HcclPrepareConfig *prepareConfig, const int timeout);

#ifdef __cplusplus
}
#endif
#endif /* HCCL_ONE_SIDED_H */
