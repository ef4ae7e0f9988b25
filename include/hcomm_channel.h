/*
 * hcomm_channel.h - channel creation at the base-communication level.
 *
 * A channel is a one-to-one data path between a local endpoint and a remote endpoint.  On B200
 * a channel is a window onto the peer's memory mapped over NVLink plus a set of 64-bit notify
 * slots in the peer's flag page; there are no queue pairs.  The descriptor keeps the HCOMM v4
 * layout so that code which fills the RoCE / UB attribute unions still compiles; those
 * attributes are ignored (reference: include/hcomm_channel.h:26-190).
 */
#ifndef HCOMM_CHANNEL_H
#define HCOMM_CHANNEL_H

#include "hcomm_res_defs.h"

#ifdef __cplusplus
extern "C" {
#endif

#define HCOMM_CHANNEL_MAGIC_WORD 0x0fcf0f0fu
#define HCOMM_CHANNEL_VERSION_ONE 1u
#define HCOMM_CHANNEL_VERSION 4u
#define HCOMM_CHANNEL_NAME_MAX_LEN 191u
#define HCOMM_CHANNEL_DESC_RAW_MAX_LEN 128u
#define HCOMM_CHANNEL_MAX_NOTIFY 64u
#define HCOMM_CHANNEL_MAX_MEM_HANDLES 256u

typedef struct {
    CommAbiHeader header;
    EndpointDesc remoteEndpoint;
    uint32_t notifyNum;         /* notify slots on this channel, at most 64 */
    bool exchangeAllMems;       /* true: every registered memory is made visible to the peer */
    HcommMemHandle *memHandles; /* memories to exchange when exchangeAllMems is false */
    uint32_t memHandleNum;
    HcommSocket socket;         /* optional pre-connected control socket */
    HcommSocketRole role;
    uint16_t port;
    union {
        uint8_t raws[HCOMM_CHANNEL_DESC_RAW_MAX_LEN];
        struct {
            uint32_t queueNum;
            uint32_t retryCnt;
            uint32_t retryInterval;
            uint8_t tc;
            uint8_t sl;
            uint32_t qpThreshold;
            uint32_t cqAttrFlags;
            uint16_t *srcPortList;
        } roceAttr;
        struct {
            uint32_t qos;
        } hccsAttr;
        struct {
            uint32_t sqDepth;
        } ubAttr;
        struct {
            uint8_t pathMode;
        } ubMemAttr;
    };
    uint32_t qos;
    const char *channelName; /* both ends must pass the same name; NULL = anonymous */
} HcommChannelDesc;

#define HCOMM_CHANNEL_DESC_ABI_V1_SIZE (offsetof(HcommChannelDesc, qos))

static inline HcommResult HcommChannelDescInit(HcommChannelDesc *d, uint32_t num)
{
    if (d == NULL) {
        return 2;
    }
    for (uint32_t i = 0; i < num; ++i, ++d) {
        memset(d, 0xFF, sizeof(*d));
        d->header.version = HCOMM_CHANNEL_VERSION;
        d->header.magicWord = HCOMM_CHANNEL_MAGIC_WORD;
        d->header.size = (uint32_t)sizeof(*d);
        d->header.reserved = 0;
        d->notifyNum = 0;
        d->exchangeAllMems = false;
        d->memHandles = NULL;
        d->memHandleNum = 0;
        d->socket = NULL;
        d->role = HCOMM_SOCKET_ROLE_RESERVED;
        d->port = 0;
        d->roceAttr.srcPortList = NULL;
        d->channelName = NULL;
        (void)EndpointDescInit(&d->remoteEndpoint, 1);
    }
    return 0;
}

/* Channel life cycle as reported by HcommChannelGetStatus. */
typedef enum {
    HCOMM_CHANNEL_STATUS_INIT = 0,
    HCOMM_CHANNEL_STATUS_SOCKET_OK = 1,
    HCOMM_CHANNEL_STATUS_READY = 2,
    HCOMM_CHANNEL_STATUS_SOCKET_TIMEOUT = 3,
    HCOMM_CHANNEL_STATUS_FAILED = 4,
    HCOMM_CHANNEL_STATUS_RES_UNAVAIL = 5
} HcommChannelStatus;

typedef void *HcommChannelConfig;
typedef enum {
    HCOMM_CHANNEL_CONFIG_TYPE_INVALID = -1,
    HCOMM_CHANNEL_CONFIG_TYPE_IS_SHARED_QUEUE = 0
} HcommChannelConfigType;

HcommResult HcommChannelCreate(EndpointHandle endpoint, CommEngine engine, HcommChannelDesc *descs,
                               uint32_t channelNum, ChannelHandle *channels);
HcommResult HcommChannelConfigCreate(HcommChannelConfig *config);
HcommResult HcommChannelConfigDestroy(HcommChannelConfig config);
HcommResult HcommChannelConfigSetInt(HcommChannelConfig config, HcommChannelConfigType type, uint32_t value);
HcommResult HcommChannelCreateWithConfig(EndpointHandle endpoint, CommEngine engine, HcommChannelDesc *descs,
                                         uint32_t channelNum, HcommChannelConfig config, ChannelHandle *channels);
HcommResult HcommChannelGetStatus(const ChannelHandle *channels, uint32_t num, int32_t *statusList);
HcommResult HcommChannelDestroy(const ChannelHandle *channels, uint32_t num);

#ifdef __cplusplus
}
#endif
#endif /* HCOMM_CHANNEL_H */
