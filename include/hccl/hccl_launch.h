/*
 * hccl_launch.h - launching a user-supplied communication kernel under the communicator's rules
 * (reference: include/hccl/hccl_launch.h).
 *
 * On Ascend the kernel is an AICPU function named by {so, symbol}.  Here `kernelSoName` names a
 * shared object (or "" for the process itself) and `kernelFuncName` a host-callable symbol
 *     extern "C" int fn(void *args, uint32_t argSize, void *stream)
 * which the library resolves with dlopen/dlsym and calls on the dedicated launch thread, so that
 * user kernels are ordered with the communicator's own operators and covered by its exec timeout.
 */
#ifndef HCCL_LAUNCH_H
#define HCCL_LAUNCH_H

#include "hccl_types.h"
#include "hcomm_res_defs.h"

#ifdef __cplusplus
extern "C" {
#endif

#define P2P_MAX_ARG_SIZE 8192u
typedef struct {
    ThreadHandle sendRecvThread;
    uint8_t opParams[P2P_MAX_ARG_SIZE];
} HcclP2pKernelParam;

typedef struct {
    void *buffer;
    uint8_t reserved[8];
    HcclCMDType cmdType;
    HcclDataType dataType;
    uint64_t count;
    uint32_t remoteRank;
    void *unfoldStream;
} HcclOpP2pDesc;

#define HCCL_OP_DESC_OP_NAME_MAX_LEN 256u
#define HCCL_OPDESC_MAGIC_WORD 0x0f0f0f0fu
#define HCCL_OPDESC_VERSION 1u
typedef struct {
    CommAbiHeader header;
    uint32_t opDescType;
    char opName[HCCL_OP_DESC_OP_NAME_MAX_LEN];
    union {
        uint8_t raws[76];
        HcclOpP2pDesc p2p;
    };
} HcclOpDesc;

static inline HcclResult HcclOpDescInit(HcclOpDesc *d)
{
    if (d == NULL) {
        return HCCL_E_PTR;
    }
    memset(d, 0xFF, sizeof(*d));
    d->header.version = HCCL_OPDESC_VERSION;
    d->header.magicWord = HCCL_OPDESC_MAGIC_WORD;
    d->header.size = (uint32_t)sizeof(*d);
    d->header.reserved = 0;
    return HCCL_SUCCESS;
}

#define HCCL_KERNEL_SO_NAME_MAX_LEN 256u
#define HCCL_KERNEL_FUNC_NAME_MAX_LEN 256u
typedef struct {
    char kernelSoName[HCCL_KERNEL_SO_NAME_MAX_LEN];
    char kernelFuncName[HCCL_KERNEL_FUNC_NAME_MAX_LEN];
    void *args;
    uint32_t argSize;
} HcclKernelFuncInfo;

#define HCCL_KERNEL_LAUNCH_CFG_MAGIC_WORD 0x0f0f0f0fu
#define HCCL_KERNEL_LAUNCH_CFG_VERSION 1u
typedef struct {
    CommAbiHeader header;
    uint64_t timeOut; /* seconds */
    uint8_t reserved[104];
} HcclKernelLaunchCfg;

static inline HcclResult HcclKernelLaunchCfgInit(HcclKernelLaunchCfg *c)
{
    if (c == NULL) {
        return HCCL_E_PTR;
    }
    memset(c, 0xFF, sizeof(*c));
    c->header.version = HCCL_KERNEL_LAUNCH_CFG_VERSION;
    c->header.magicWord = HCCL_KERNEL_LAUNCH_CFG_MAGIC_WORD;
    c->header.size = (uint32_t)sizeof(*c);
    c->header.reserved = 0;
    return HCCL_SUCCESS;
}

HcclResult HcclAicpuKernelLaunch(HcclComm comm, const HcclOpDesc *opInfo, const HcclKernelFuncInfo *funcInfo,
                                 ThreadHandle launchThread, aclrtStream userStream,
                                 const HcclKernelLaunchCfg *kernelLaunchCfg);

#ifdef __cplusplus
}
#endif
#endif /* HCCL_LAUNCH_H */
