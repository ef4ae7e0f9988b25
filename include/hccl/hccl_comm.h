/*
 * hccl_comm.h - communicator life cycle, process configuration, groups, symmetric windows.
 * API surface: reference include/hccl/hccl_comm.h:36-401.
 *
 * Bring-up paths
 *   root-info : rank 0 calls HcclGetRootInfo (starts a TCP rendezvous server and returns its
 *               address in the ticket), ships the ticket to every rank by any side channel, and
 *               all ranks call HcclCommInitRootInfo(Config).
 *   rank table: every rank reads the same JSON file (v1.0 "server_list" or v2 "rank_list") and
 *               calls HcclCommInitClusterInfo(Config); the table's first rank hosts the rendezvous.
 *   init-all  : one process drives N devices (or N simulated ranks); HcclCommInitAll.
 * After rendezvous each rank maps every peer's symmetric heap (CCL buffer + flag page) and, when
 * the fabric supports it, binds the heap to an NVLS multicast object.
 */
#ifndef HCCL_COMM_H_
#define HCCL_COMM_H_

#include "hccl_launch.h"
#include "hccl_res.h"
#include "hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif

HcclResult HcclCommInitClusterInfo(const char *clusterInfo, uint32_t rank, HcclComm *comm);
HcclResult HcclCommInitClusterInfoConfig(const char *clusterInfo, uint32_t rank, HcclCommConfig *config,
                                         HcclComm *comm);
/* Derive a communicator over rankIds[] of *comm without a new rendezvous. Collective over the members. */
HcclResult HcclCreateSubCommConfig(HcclComm *comm, uint32_t rankNum, uint32_t *rankIds, uint64_t subCommId,
                                   uint32_t subCommRankId, HcclCommConfig *config, HcclComm *subComm);
HcclResult HcclGetRootInfo(HcclRootInfo *rootInfo);
HcclResult HcclCommInitRootInfo(uint32_t nRanks, const HcclRootInfo *rootInfo, uint32_t rank, HcclComm *comm);
HcclResult HcclCommInitRootInfoConfig(uint32_t nRanks, const HcclRootInfo *rootInfo, uint32_t rank,
                                      const HcclCommConfig *config, HcclComm *comm);
HcclResult HcclCommInitAll(uint32_t ndev, int32_t *devices, HcclComm *comms);
HcclResult HcclCommDestroy(HcclComm comm);

HcclResult HcclSetConfig(HcclConfig config, union HcclConfigValue configValue);
HcclResult HcclGetConfig(HcclConfig config, union HcclConfigValue *configValue);
HcclResult HcclGetCommName(HcclComm comm, char *commName);
HcclResult HcclCommGetHandleWithName(const char *commName, HcclComm *comm);
HcclResult HcclGetRankSize(HcclComm comm, uint32_t *rankSize);
HcclResult HcclGetRankId(HcclComm comm, uint32_t *rank);
HcclResult HcclBarrier(HcclComm comm, aclrtStream stream);
HcclResult HcclGetCommAsyncError(HcclComm comm, HcclResult *asyncError);
const char *HcclGetErrorString(HcclResult code);
/* Bit i set <=> HcclCommConfigCapability i is honoured. */
uint32_t HcclGetCommConfigCapability(void);

static inline void HcclCommConfigInit(HcclCommConfig *config)
{
    struct Header {
        size_t size;
        uint32_t magicWord;
        uint32_t version;
        uint64_t reserved;
    };
    if (config == NULL) {
        return;
    }
    memset(config, 0, sizeof(*config));
    struct Header *h = (struct Header *)config;
    h->size = sizeof(HcclCommConfig);
    h->magicWord = HCCL_COMM_CONFIG_MAGIC_WORD;
    h->version = HCCL_COMM_CONFIG_VERSION;
    config->hcclBufferSize = HCCL_COMM_BUFFSIZE_CONFIG_NOT_SET;
    config->hcclDeterministic = HCCL_COMM_DETERMINISTIC_CONFIG_NOT_SET;
    config->hcclOpExpansionMode = HCCL_COMM_DEFAULT_OP_EXPANSION_MODE;
    config->hcclRdmaTrafficClass = HCCL_COMM_TRAFFIC_CLASS_CONFIG_NOT_SET;
    config->hcclRdmaServiceLevel = HCCL_COMM_SERVICE_LEVEL_CONFIG_NOT_SET;
    config->hcclExecTimeOut = HCCL_COMM_EXECTIMEOUT_CONFIG_NOT_SET;
    config->hcclQos = HCCL_COMM_QOS_CONFIG_NOT_SET;
    config->hcclSymWinMaxMemSizePerRank = HCCL_DEFAULT_SYMMETRIC_MEMORY_STRIDE;
    config->hcclChannelSqDepth = HCCL_COMM_SQ_DEPTH_CONFIG_NOT_SET;
}

/* ---- fault handling ---------------------------------------------------------------------------
 * Suspend stops new launches (operators return HCCL_E_SUSPENDING), Resume re-synchronises the
 * flag pages of all ranks and re-opens the communicator.  Both are collective over live ranks.
 */
/* B200 extension: after ranks of `comm` were lost - the rank that hosted the rendezvous among them or not - the ranks
 * that are left call this together and get a new communicator over themselves, numbered in their old order.  It needs
 * neither the old rendezvous nor a ticket passed around by the caller: the lowest survivor opens a new rendezvous and
 * hands the ticket to the others over the ranks' local sockets (ranks of one host).  `oldRanks` (optional, room for the
 * old size) receives the old rank of every new rank.  The old communicator is left as it is; destroy it afterwards. */
HcclResult HcclCommRecover(HcclComm comm, uint32_t timeoutSec, HcclComm *newComm, uint32_t *newSize, uint32_t *oldRanks);
HcclResult HcclCommSuspend(HcclComm comm);
HcclResult HcclCommResume(HcclComm comm);
typedef HcclResult (*HcclCommStateCallback)(HcclComm comm, HcclCommStatePhase state, void *args);
HcclResult HcclCommRegCommStateCallback(const char *regName, HcclCommStateCallback cb, void *args);
HcclResult HcclCommGetStatus(const char *commId, HcclCommStatus *status);
HcclResult HcclCommWorkingDevNicSet(HcclComm comm, uint32_t *ranks, bool *useBackup, uint32_t nRanks);

/* ---- zero-copy user memory -----------------------------------------------------------------------
 * SetMemoryRange declares a VA range the caller manages with the CUDA VMM API; Activate tells the
 * library that `handle` (a CUmemGenericAllocationHandle) now backs [virPtr, virPtr+size) so that
 * peers can map it and operators may skip the staging copy.
 */
HcclResult HcclCommSetMemoryRange(HcclComm comm, void *baseVirPtr, size_t size, size_t alignment, uint64_t flags);
HcclResult HcclCommUnsetMemoryRange(HcclComm comm, void *baseVirPtr);
HcclResult HcclCommActivateCommMemory(HcclComm comm, void *virPtr, size_t size, size_t offset, uint64_t handle,
                                      uint64_t flags);
HcclResult HcclCommDeactivateCommMemory(HcclComm comm, void *virPtr);

/* ---- group calls: operators (and communicator inits) issued between Start and End are queued and
 * launched together at End; queued Send/Recv fuse into one BatchSendRecv. */
HcclResult HcclGroupStart(void);
HcclResult HcclGroupEnd(void);
HcclResult HcclGroupStatusGet(bool *isGroupEnabled);

/* ---- symmetric windows: the same offset names the same buffer on every rank ---------------------- */
HcclResult HcclCommSymWinRegister(HcclComm comm, void *addr, uint64_t size, HcclCommSymWindow *winHandle,
                                  uint32_t flag);
HcclResult HcclCommSymWinDeregister(HcclCommSymWindow winHandle);
HcclResult HcclCommSymWinGet(HcclComm comm, void *ptr, size_t size, HcclCommSymWindow *winHandle, size_t *offset);

typedef enum {
    HCCL_OP_EXPANSION_MODE_INVALID = -1,
    HCCL_OP_EXPANSION_MODE_AI_CPU = 0,
    HCCL_OP_EXPANSION_MODE_AIV = 1,
    HCCL_OP_EXPANSION_MODE_HOST = 2,
    HCCL_OP_EXPANSION_MODE_HOST_TS = 3,
    HCCL_OP_EXPANSION_MODE_CCU_MS = 4,
    HCCL_OP_EXPANSION_MODE_CCU_SCHED = 5,
    HCCL_OP_EXPANSION_AIV_ONLY = 6
} HcclOpExpansionMode;

typedef enum {
    HCCL_CONFIG_TYPE_INVALID = -1,
    HCCL_CONFIG_TYPE_OP_EXPANSION_MODE = 0,
    HCCL_CONFIG_TYPE_HCCL_ALGO = 1
} HcclConfigType;
typedef HcclOpExpansionMode HcclConfigTypeOpExpansionMode;
HcclResult HcclConfigGetInfo(HcclComm comm, HcclConfigType cfgType, uint32_t infoLen, void *info);

#ifdef __cplusplus
}
#endif
#endif /* HCCL_COMM_H_ */
