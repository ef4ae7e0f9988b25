/*
 * hccl_types.h - scalar types, enums and plain structs shared by every HCCL entry point.
 *
 * Binary layout contract: the numeric values of HcclResult / HcclDataType / HcclReduceOp,
 * the 4108-byte HcclRootInfo blob and the HcclCommConfig v11 field order follow the HCCL ABI
 * (reference: include/hccl/hccl_types.h:23-235) so that callers compiled against HCCL keep
 * working.  Everything behind these types is a CUDA / NVLink implementation.
 */
#ifndef HCCL_TYPES_H_
#define HCCL_TYPES_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Stream handle.  On a CUDA platform it is a cudaStream_t; the host simulator ignores it. */
#ifndef HCCL_STREAM_TYPE_DEFINED
#define HCCL_STREAM_TYPE_DEFINED
typedef void *aclrtStream;
typedef void *hcclStream_t;
#endif

typedef enum {
    HCCL_SUCCESS = 0,
    HCCL_E_PARA = 1,              /* bad argument value */
    HCCL_E_PTR = 2,               /* null pointer */
    HCCL_E_MEMORY = 3,            /* memory operation failed */
    HCCL_E_INTERNAL = 4,          /* invariant broken inside the library */
    HCCL_E_NOT_SUPPORT = 5,       /* feature not available on this platform */
    HCCL_E_NOT_FOUND = 6,         /* named resource does not exist */
    HCCL_E_UNAVAIL = 7,           /* resource exhausted, caller may fall back */
    HCCL_E_SYSCALL = 8,           /* OS call failed */
    HCCL_E_TIMEOUT = 9,           /* bounded wait expired */
    HCCL_E_OPEN_FILE_FAILURE = 10,
    HCCL_E_TCP_CONNECT = 11,
    HCCL_E_ROCE_CONNECT = 12,
    HCCL_E_TCP_TRANSFER = 13,
    HCCL_E_ROCE_TRANSFER = 14,
    HCCL_E_RUNTIME = 15,          /* CUDA runtime call failed */
    HCCL_E_DRV = 16,              /* CUDA driver / NVML call failed */
    HCCL_E_PROFILING = 17,
    HCCL_E_CCE = 18,
    HCCL_E_NETWORK = 19,
    HCCL_E_AGAIN = 20,            /* retry later */
    HCCL_E_REMOTE = 21,           /* a peer reported an error */
    HCCL_E_SUSPENDING = 22,       /* communicator is suspended */
    HCCL_E_OPRETRY_FAIL = 23,
    HCCL_E_OOM = 24,
    HCCL_E_IN_STATUS = 1041,
    HCCL_E_RESERVED
} HcclResult;

typedef void *HcclComm;
typedef void *HcclConn;
typedef void *HcclCommSymWindow;

typedef enum {
    HCCL_REDUCE_SUM = 0,
    HCCL_REDUCE_PROD = 1,
    HCCL_REDUCE_MAX = 2,
    HCCL_REDUCE_MIN = 3,
    HCCL_REDUCE_RESERVED = 255
} HcclReduceOp;

typedef enum {
    HCCL_DATA_TYPE_INT8 = 0,
    HCCL_DATA_TYPE_INT16 = 1,
    HCCL_DATA_TYPE_INT32 = 2,
    HCCL_DATA_TYPE_FP16 = 3,
    HCCL_DATA_TYPE_FP32 = 4,
    HCCL_DATA_TYPE_INT64 = 5,
    HCCL_DATA_TYPE_UINT64 = 6,
    HCCL_DATA_TYPE_UINT8 = 7,
    HCCL_DATA_TYPE_UINT16 = 8,
    HCCL_DATA_TYPE_UINT32 = 9,
    HCCL_DATA_TYPE_FP64 = 10,
    HCCL_DATA_TYPE_BFP16 = 11,
    HCCL_DATA_TYPE_INT128 = 12,
    HCCL_DATA_TYPE_HIF8 = 14,
    HCCL_DATA_TYPE_FP8E4M3 = 15,
    HCCL_DATA_TYPE_FP8E5M2 = 16,
    HCCL_DATA_TYPE_FP8E8M0 = 17,
    HCCL_DATA_TYPE_RESERVED = 255
} HcclDataType;

/* Process-wide knobs reachable through HcclSetConfig / HcclGetConfig. */
typedef enum {
    HCCL_DETERMINISTIC = 0, /* 0 fastest, 1 fixed reduction order, 2 strict order preserving */
    HCCL_CONFIG_RESERVED
} HcclConfig;

union HcclConfigValue {
    int32_t value;
};
#ifndef __cplusplus
typedef union HcclConfigValue HcclConfigValue;
#endif

enum {
    HCCL_ROOT_INFO_BYTES = 4108,
    COMM_NAME_MAX_LENGTH = 128,
    BUFFER_NAME_MAX_LENGTH = 128,
    UDI_MAX_LENGTH = 128,
    HCCL_COMM_ALGO_MAX_LENGTH = 1600,
    HCCL_COMM_RETRY_ENABLE_MAX_LENGTH = 50,
    HCCL_COMM_RETRY_PARAMS_MAX_LENGTH = 128,
    HCCL_COMM_CONFIG_INFO_BYTES = 24,
    HCCL_COMM_CONFIG_VERSION = 11,
    HCCL_COMM_DEFAULT_BUFFSIZE = 200, /* MB, each of the in and out halves */
    HCCL_COMM_DEFAULT_DETERMINISTIC = 0,
    HCCL_COMM_DEFAULT_OP_EXPANSION_MODE = 0
};
#define HCCL_COMM_CONFIG_MAGIC_WORD 0xf0f0f0f0u
#define HCCL_COMM_BUFFSIZE_CONFIG_NOT_SET 0xffffffffu
#define HCCL_COMM_DETERMINISTIC_CONFIG_NOT_SET 0xffffffffu
#define HCCL_COMM_TRAFFIC_CLASS_CONFIG_NOT_SET 0xffffffffu
#define HCCL_COMM_SERVICE_LEVEL_CONFIG_NOT_SET 0xffffffffu
#define HCCL_COMM_EXECTIMEOUT_CONFIG_NOT_SET ((int32_t)0xffffffff)
#define HCCL_COMM_QOS_CONFIG_NOT_SET 0xffffffffu
#define HCCL_COMM_SQ_DEPTH_CONFIG_NOT_SET 0xffffffffu
#define HCCL_DEFAULT_SYMMETRIC_MEMORY_STRIDE 16ULL /* GB of VA reserved per rank */

/* Opaque rendezvous ticket produced by HcclGetRootInfo and shipped to every rank out of band. */
typedef struct HcclRootInfoDef {
    char internal[HCCL_ROOT_INFO_BYTES];
} HcclRootInfo;

/*
 * Per-communicator configuration.  The first 24 bytes are a private header
 * {size_t size; u32 magic; u32 version; u64 reserved} written by HcclCommConfigInit.
 */
typedef struct HcclCommConfigDef {
    char reserved[HCCL_COMM_CONFIG_INFO_BYTES];
    uint32_t hcclBufferSize;      /* MB per half of the CCL buffer */
    uint32_t hcclDeterministic;
    char hcclCommName[COMM_NAME_MAX_LENGTH];
    char hcclUdi[UDI_MAX_LENGTH];
    uint32_t hcclOpExpansionMode; /* 0 default, 1 host, 2 host-TS, 3 SM kernels w/ fallback, 4 SM only, 5 NVLS */
    uint32_t hcclRdmaTrafficClass;
    uint32_t hcclRdmaServiceLevel;
    uint32_t hcclWorldRankID;
    uint64_t hcclJobID;
    uint8_t aclGraphZeroCopyEnable;
    int32_t hcclExecTimeOut;      /* seconds; bounds every device-side wait */
    char hcclAlgo[HCCL_COMM_ALGO_MAX_LENGTH];
    char hcclRetryEnable[HCCL_COMM_RETRY_ENABLE_MAX_LENGTH];
    char hcclRetryParams[HCCL_COMM_RETRY_PARAMS_MAX_LENGTH];
    char hcclBufferName[BUFFER_NAME_MAX_LENGTH];
    uint32_t hcclQos;
    uint64_t hcclSymWinMaxMemSizePerRank; /* GB of VA per rank for symmetric windows */
    uint32_t hcclChannelSqDepth;
} HcclCommConfig;

typedef enum {
    HCCL_COMM_CONFIG_BUFFER_SIZE = 0,
    HCCL_COMM_CONFIG_DETERMINISTIC = 1,
    HCCL_COMM_CONFIG_COMM_NAME = 2,
    HCCL_COMM_CONFIG_OP_EXPANSION_MODE = 3,
    HCCL_COMM_CONFIG_SUPPORT_INIT_BY_ENV = 4,
    HCCL_COMM_CONFIG_WORLD_RANKID = 5,
    HCCL_COMM_CONFIG_JOBID = 6,
    HCCL_COMM_CONFIG_ACLGRAPH_ZEROCOPY_ENABLE = 7,
    HCCL_COMM_CONFIG_EXEC_TIMEOUT = 8,
    HCCL_COMM_CONFIG_ALGO = 9,
    HCCL_COMM_CONFIG_RETRY = 10,
    HCCL_COMM_CONFIG_BUFFER_NAME = 11,
    HCCL_COMM_CONFIG_RESERVED
} HcclCommConfigCapability;

typedef enum { HCCL_SEND = 0, HCCL_RECV = 1, HCCL_SEND_RECV_RESERVED } HcclSendRecvType;

typedef struct HcclSendRecvItemDef {
    HcclSendRecvType sendRecvType;
    void *buf;
    uint64_t count;
    HcclDataType dataType;
    uint32_t remoteRank;
} HcclSendRecvItem;

typedef enum {
    HCCL_CMD_INVALID = 0,
    HCCL_CMD_BROADCAST = 1,
    HCCL_CMD_ALLREDUCE,
    HCCL_CMD_REDUCE,
    HCCL_CMD_SEND,
    HCCL_CMD_RECEIVE,
    HCCL_CMD_ALLGATHER,
    HCCL_CMD_REDUCE_SCATTER,
    HCCL_CMD_ALLTOALLV,
    HCCL_CMD_ALLTOALLVC,
    HCCL_CMD_ALLTOALL,
    HCCL_CMD_GATHER,
    HCCL_CMD_SCATTER,
    HCCL_CMD_BATCH_SEND_RECV,
    HCCL_CMD_BATCH_PUT,
    HCCL_CMD_BATCH_GET,
    HCCL_CMD_ALLGATHER_V,
    HCCL_CMD_REDUCE_SCATTER_V,
    HCCL_CMD_BATCH_WRITE,
    HCCL_CMD_HALF_ALLTOALLV = 20,
    HCCL_CMD_ALL,
    HCCL_CMD_FINALIZE = 100,
    HCCL_CMD_INTER_GROUP_SYNC,
    HCCL_CMD_INIT,
    HCCL_CMD_BARRIER,
    HCCL_CMD_MAX
} HcclCMDType;

typedef enum {
    HCCL_COMM_STATUS_READY = 0,
    HCCL_COMM_STATUS_SUSPENDING = 1,
    HCCL_COMM_STATUS_INVALID = 254,
    HCCL_COMM_STATUS_RESERVED = 255
} HcclCommStatus;

typedef enum {
    HCCL_COMM_STATE_PHASE_INVALID = -1,
    HCCL_COMM_STATE_PHASE_DESTROY_PRE = 0,
    HCCL_COMM_STATE_PHASE_DESTROY_POST = 1,
    HCCL_COMM_STATE_PHASE_RESUME_PRE = 2,
    HCCL_COMM_STATE_PHASE_RESUME_POST = 3
} HcclCommStatePhase;

#ifdef __cplusplus
}
#endif
#endif /* HCCL_TYPES_H_ */
