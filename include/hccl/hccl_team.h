/*
 * hccl_team.h - SHMEM-style teams and windows (reference: include/hccl/hccl_team.h, hcomm_team_defs.h:20-36).
 *
 * A team is an ordered subset of a communicator's ranks with per-member synchronisation words
 * (signals, counters, barriers: 64-bit slots, one set per remote member) carved out of the
 * symmetric flag page, and any number of windows: memory registered by every member so that member
 * i can address member j's copy.  The handle returned to the caller points at a device-readable
 * record {rankNum, myIndex, sync base addresses per member, window tables} usable from SM kernels.
 */
#ifndef HCCL_TEAM_H
#define HCCL_TEAM_H

#include "hccl_types.h"
#include "hcomm_res_defs.h"
#include "hcomm_team_defs.h"

#ifdef __cplusplus
extern "C" {
#endif

#define HCCL_TEAM_CREATE_DESC_MAGIC_WORD 0x0fcf0f14u
#define HCCL_TEAM_CREATE_DESC_VERSION 1u
#define HCCL_TEAM_CREATE_CHANNELS_DESC_MAGIC_WORD 0x0fcf0f15u
#define HCCL_TEAM_CREATE_CHANNELS_DESC_VERSION 1u

typedef struct {
    CommAbiHeader header;
    const uint32_t *rankIds; /* NULL + rankNum 0 = all ranks of the communicator */
    uint32_t rankNum;
    uint32_t selfRankId;
    uint32_t netLayer;
    CommProtocol protocol;
    HcommTeamSyncMemRequirement requirement;
    uint32_t reserved[4];
} HcclTeamCreateDesc;

typedef struct {
    CommAbiHeader header;
    CommEngine engine;
    uint32_t notifyNum;
    CommProtocol protocol;
    uint32_t channelCnt;
    uint32_t reserved[4];
} HcclTeamCreateChannelsDesc;

static inline HcclResult HcclTeamCreateDescInit(HcclTeamCreateDesc *d)
{
    if (d == NULL) {
        return HCCL_E_PTR;
    }
    memset(d, 0, sizeof(*d));
    d->header.version = HCCL_TEAM_CREATE_DESC_VERSION;
    d->header.magicWord = HCCL_TEAM_CREATE_DESC_MAGIC_WORD;
    d->header.size = (uint32_t)sizeof(*d);
    d->protocol = COMM_PROTOCOL_RESERVED;
    return HCCL_SUCCESS;
}

static inline HcclResult HcclTeamCreateChannelsDescInit(HcclTeamCreateChannelsDesc *d)
{
    if (d == NULL) {
        return HCCL_E_PTR;
    }
    memset(d, 0, sizeof(*d));
    d->header.version = HCCL_TEAM_CREATE_CHANNELS_DESC_VERSION;
    d->header.magicWord = HCCL_TEAM_CREATE_CHANNELS_DESC_MAGIC_WORD;
    d->header.size = (uint32_t)sizeof(*d);
    d->engine = COMM_ENGINE_RESERVED;
    d->protocol = COMM_PROTOCOL_RESERVED;
    return HCCL_SUCCESS;
}

HcclResult HcclWorldTeamCreate(HcclComm comm, const HcclTeamCreateDesc *desc, HcommTeamHandle *worldTeam);
HcclResult HcclSubTeamCreate(HcommTeamHandle worldTeam, const HcclTeamCreateDesc *desc, HcommTeamHandle *team);
HcclResult HcclTeamDestroy(HcommTeamHandle team);
HcclResult HcclTeamWindowRegister(HcclComm comm, HcommTeamHandle worldTeam, const CommMem *localMem,
                                  HcommWindowHandle *window, uint32_t flag);
HcclResult HcclTeamWindowDeregister(HcommTeamHandle worldTeam, HcommWindowHandle window);
HcclResult HcclTeamChannelsCreate(HcclComm comm, HcommTeamHandle team, const HcclTeamCreateChannelsDesc *desc);

/* Host-side team operations (same semantics as the device functions in hcomm_device.cuh). */
HcclResult HcclTeamGetInfo(HcommTeamHandle team, uint32_t *rankNum, uint32_t *myIndex);
HcclResult HcclTeamWindowGetPeerPointer(HcommTeamHandle team, HcommWindowHandle window, uint32_t memberIdx,
                                        void **ptr, uint64_t *size);
HcclResult HcclTeamSignal(HcommTeamHandle team, uint32_t memberIdx, uint32_t signalIdx, uint64_t value,
                          aclrtStream stream);
HcclResult HcclTeamSignalWait(HcommTeamHandle team, uint32_t memberIdx, uint32_t signalIdx, uint64_t value,
                              aclrtStream stream);
HcclResult HcclTeamBarrier(HcommTeamHandle team, uint32_t barrierIdx, aclrtStream stream);

#ifdef __cplusplus
}
#endif
#endif /* HCCL_TEAM_H */
