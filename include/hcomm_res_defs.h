/*
 * hcomm_res_defs.h - resource-level vocabulary: ABI header, engines, protocols, endpoints, memory.
 *
 * Values of the enums and the sizes of the descriptor structs follow the HCOMM ABI
 * (reference: include/hcomm_res_defs.h:57-271).  The B200 build adds one protocol value,
 * COMM_PROTOCOL_NVLINK, which is what every link of an NVSwitch box reports.
 */
#ifndef HCOMM_RES_DEFS_H
#define HCOMM_RES_DEFS_H

#include <arpa/inet.h>
#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#ifdef __cplusplus
extern "C" {
#endif

#define COMM_ADDR_EID_LEN 16U

typedef int32_t HcommResult;
typedef void *EndpointHandle;
typedef void *HcommMemHandle;
typedef void *HcommSocket;

#ifndef CHANNEL_HANDLE_DEFINED
#define CHANNEL_HANDLE_DEFINED
typedef uint64_t ChannelHandle;
#endif
#ifndef THREAD_HANDLE_DEFINED
#define THREAD_HANDLE_DEFINED
typedef uint64_t ThreadHandle;
#endif

/* Every descriptor that crosses the API starts with this header so layouts can grow. */
typedef struct {
    uint32_t version;
    uint32_t magicWord;
    uint32_t size;
    uint32_t reserved;
} CommAbiHeader;

typedef enum {
    THREAD_TYPE_INVALID = -1,
    THREAD_TYPE_TS = 0
} ThreadType;

#define HCOMM_THREAD_CONFIG_MAGIC_WORD 0x0f0f0f2fu
#define HCOMM_THREAD_CONFIG_VERSION 1u

typedef struct {
    CommAbiHeader header;
    uint16_t notifyNumPerThread;
    uint8_t reserved[14];
} ThreadConfig;

static inline HcommResult ThreadConfigInit(ThreadConfig *cfg, uint32_t num)
{
    if (cfg == NULL) {
        return 2; /* HCCL_E_PTR */
    }
    for (uint32_t i = 0; i < num; ++i) {
        memset(&cfg[i], 0, sizeof(ThreadConfig));
        cfg[i].header.version = HCOMM_THREAD_CONFIG_VERSION;
        cfg[i].header.magicWord = HCOMM_THREAD_CONFIG_MAGIC_WORD;
        cfg[i].header.size = (uint32_t)sizeof(ThreadConfig);
    }
    return 0;
}

/*
 * Execution engines.  Mapping on B200:
 *   CPU      host thread touching mapped memory directly (simulator and debugging)
 *   CPU_TS   host enqueues copies / reduce kernels / flag ops on CUDA streams
 *   AICPU(_TS)  accepted as aliases of CPU_TS (there is no device control CPU)
 *   AIV      "SM engine": the work runs inside one persistent CUDA kernel
 *   CCU      NVLS: in-switch reduction / multicast through multimem instructions
 */
typedef enum {
    COMM_ENGINE_RESERVED = -1,
    COMM_ENGINE_CPU = 0,
    COMM_ENGINE_CPU_TS = 1,
    COMM_ENGINE_AICPU = 2,
    COMM_ENGINE_AICPU_TS = 3,
    COMM_ENGINE_AIV = 4,
    COMM_ENGINE_CCU = 5
} CommEngine;
#define COMM_ENGINE_SM COMM_ENGINE_AIV
#define COMM_ENGINE_NVLS COMM_ENGINE_CCU

typedef enum {
    COMM_PROTOCOL_RESERVED = -1,
    COMM_PROTOCOL_HCCS = 0,
    COMM_PROTOCOL_ROCE = 1,
    COMM_PROTOCOL_PCIE = 2,
    COMM_PROTOCOL_SIO = 3,
    COMM_PROTOCOL_UB_CTP = 4,
    COMM_PROTOCOL_UBC_CTP = COMM_PROTOCOL_UB_CTP,
    COMM_PROTOCOL_UBC_TP = 5,
    COMM_PROTOCOL_UB_MEM = 6,
    COMM_PROTOCOL_UBOE = 7,
    COMM_PROTOCOL_HCCS_ONLY = 8,
    COMM_PROTOCOL_UB_RTP = 9,
    COMM_PROTOCOL_UBG = COMM_PROTOCOL_UB_RTP,
    COMM_PROTOCOL_NVLINK = 16, /* NVLink 5 through NVSwitch (B200 extension) */
    COMM_PROTOCOL_SHM = 17     /* host shared memory (simulator) */
} CommProtocol;

typedef enum {
    COMM_ADDR_TYPE_RESERVED = -1,
    COMM_ADDR_TYPE_IP_V4 = 0,
    COMM_ADDR_TYPE_IP_V6 = 1,
    COMM_ADDR_TYPE_ID = 2,
    COMM_ADDR_TYPE_EID = 3
} CommAddrType;

typedef struct {
    CommAddrType type;
    union {
        uint8_t raws[36];
        struct in_addr addr;
        struct in6_addr addr6;
        uint32_t id;
        uint8_t eid[COMM_ADDR_EID_LEN];
    };
} CommAddr;

typedef enum {
    ENDPOINT_LOC_TYPE_RESERVED = -1,
    ENDPOINT_LOC_TYPE_DEVICE = 0,
    ENDPOINT_LOC_TYPE_HOST = 1
} EndpointLocType;

typedef struct {
    EndpointLocType locType;
    union {
        uint8_t raws[60];
        struct {
            uint32_t devPhyId;    /* CUDA device ordinal as NVML numbers it */
            uint32_t superDevId;
            uint32_t serverIdx;   /* index of the host in the job */
            uint32_t superPodIdx; /* NVLink domain (clique) index */
        } device;
        struct {
            uint32_t id;
        } host;
    };
} EndpointLoc;

typedef struct {
    CommProtocol protocol;
    CommAddr commAddr;
    EndpointLoc loc;
    union {
        uint8_t raws[52];
    };
} EndpointDesc;

static inline HcommResult EndpointDescInit(EndpointDesc *ep, uint32_t num)
{
    if (ep == NULL) {
        return 2;
    }
    for (uint32_t i = 0; i < num; ++i) {
        memset(&ep[i], 0xFF, sizeof(EndpointDesc));
        ep[i].protocol = COMM_PROTOCOL_RESERVED;
        ep[i].commAddr.type = COMM_ADDR_TYPE_RESERVED;
        ep[i].loc.locType = ENDPOINT_LOC_TYPE_RESERVED;
    }
    return 0;
}

typedef enum {
    COMM_MEM_TYPE_INVALID = -1,
    COMM_MEM_TYPE_DEVICE = 0,
    COMM_MEM_TYPE_HOST = 1
} CommMemType;

typedef struct {
    CommMemType type;
    void *addr;
    uint64_t size;
} CommMem;

typedef enum {
    HCOMM_SOCKET_ROLE_RESERVED = -1,
    HCOMM_SOCKET_ROLE_CLIENT = 0,
    HCOMM_SOCKET_ROLE_SERVER = 1
} HcommSocketRole;

typedef enum {
    HCOMM_ENDPOINT_FEATURE_INVALID = -1,
    HCOMM_ENDPOINT_FEATURE_NDA = 0,      /* device-initiated async transfer: true for NVLINK */
    HCOMM_ENDPOINT_FEATURE_MULTICAST = 1 /* NVLS multicast objects available */
} HcommEndpointFeatureType;

typedef enum {
    THREAD_RES_TYPE_INVALID = -1,
    THREAD_RES_TYPE_STREAM = 0
} ThreadResType;

#ifdef __cplusplus
}
#endif
#endif /* HCOMM_RES_DEFS_H */
