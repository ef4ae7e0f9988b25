/*
 * hccl_channel.h - channels owned by a communicator (reference: include/hccl/hccl_channel.h:39-258).
 *
 * HcclChannelAcquire is lazy and idempotent per (engine, remoteRank, protocol, notifyNum): the
 * first request performs the handshake (memory table exchange + consistency check against the
 * peer over the bootstrap network), later identical requests return the same handle.
 */
#ifndef HCCL_CHANNEL_H
#define HCCL_CHANNEL_H

#include "hccl_types.h"
#include "hcomm_channel.h"
#include "hcomm_res_defs.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef void *HcclMemHandle;

#define HCCL_CHANNEL_MAGIC_WORD 0x0f0f0f0fu
#define HCCL_CHANNEL_VERSION 1u
#define HCCL_CHANNEL_DESC_RAW_MAX_LEN 128u

typedef struct {
    CommAbiHeader header;
    uint32_t remoteRank;
    CommProtocol channelProtocol; /* take it from HcclRankGraphGetLinks; NVLINK on B200 */
    EndpointDesc localEndpoint;
    EndpointDesc remoteEndpoint;
    uint32_t notifyNum;
    HcclMemHandle *memHandles;
    uint32_t memHandleNum;
    union {
        uint8_t raws[HCCL_CHANNEL_DESC_RAW_MAX_LEN];
        struct {
            uint32_t queueNum;
            uint32_t retryCnt;
            uint32_t retryInterval;
            uint8_t tc;
            uint8_t sl;
        } roceAttr;
        struct {
            uint8_t pathMode;
        } ubMemAttr;
    };
} HcclChannelDesc;

#ifndef LIKELY
#define LIKELY(x) (__builtin_expect(!!(x), 1))
#define UNLIKELY(x) (__builtin_expect(!!(x), 0))
#endif

static inline HcclResult HcclChannelDescInit(HcclChannelDesc *d, uint32_t descNum)
{
    if (d == NULL) {
        return HCCL_E_PTR;
    }
    for (uint32_t i = 0; i < descNum; ++i, ++d) {
        memset(d, 0xFF, sizeof(*d));
        d->header.version = HCCL_CHANNEL_VERSION;
        d->header.magicWord = HCCL_CHANNEL_MAGIC_WORD;
        d->header.size = (uint32_t)sizeof(*d);
        d->header.reserved = 0;
        d->remoteRank = ~0u;
        d->channelProtocol = COMM_PROTOCOL_RESERVED;
        d->notifyNum = 0;
        d->memHandles = NULL;
        d->memHandleNum = 0;
        (void)EndpointDescInit(&d->localEndpoint, 1);
        (void)EndpointDescInit(&d->remoteEndpoint, 1);
    }
    return HCCL_SUCCESS;
}

HcclResult HcclChannelAcquire(HcclComm comm, CommEngine engine, const HcclChannelDesc *descs, uint32_t channelNum,
                              ChannelHandle *channels);

typedef void *HcclChannelConfig;
#define HCCL_CHANNEL_CONFIG_SHARED_QUEUE_TAG_MAX_LEN 255u
typedef enum {
    HCCL_CHANNEL_CONFIG_TYPE_INVALID = -1,
    HCCL_CHANNEL_CONFIG_TYPE_IS_SHARED_QUEUE = 0,
    HCCL_CHANNEL_CONFIG_TYPE_SHARED_QUEUE_TAG = 1
} HcclChannelConfigType;
HcclResult HcclChannelConfigCreate(HcclChannelConfig *config);
HcclResult HcclChannelConfigDestroy(HcclChannelConfig config);
HcclResult HcclChannelConfigSetInt(HcclChannelConfig config, HcclChannelConfigType type, uint32_t value);
HcclResult HcclChannelConfigSetStr(HcclChannelConfig config, HcclChannelConfigType type, const char *value);
HcclResult HcclChannelAcquireWithConfig(HcclComm comm, CommEngine engine, const HcclChannelDesc *descs,
                                        uint32_t channelNum, HcclChannelConfig config, ChannelHandle *channels);
/* Returns existing handles only; entries that were never acquired come back as 0. */
HcclResult HcclChannelQuery(HcclComm comm, CommEngine engine, const HcclChannelDesc *descs, uint32_t channelNum,
                            ChannelHandle *channels);
HcclResult HcclChannelDestroy(HcclComm comm, const ChannelHandle *channels, uint32_t channelNum);
/* The peer's CCL buffer as seen from this rank (tag "HcclBuffer"). */
HcclResult HcclChannelGetHcclBuffer(HcclComm comm, ChannelHandle channel, void **buffer, uint64_t *size);
HcclResult HcclChannelGetRemoteMems(HcclComm comm, ChannelHandle channel, uint32_t *memNum, CommMem **remoteMems,
                                    char ***memTags);
/* For the SM engine: device-resident descriptor {peer window table, notify slots} of the channel. */
HcclResult HcclChannelGetDeviceView(HcclComm comm, ChannelHandle channel, void **deviceChannel);

#ifdef __cplusplus
}
#endif
#endif /* HCCL_CHANNEL_H */
