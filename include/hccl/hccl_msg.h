/*
 * hccl_msg.h - host-side tagged messages in the style of MPI's matched probe, and the same over plain connections.
 * (reference: pkg_inc/legacy/hccl/hccl_ex.h:29-190 with the types of pkg_inc/legacy/hccl/base.h:225-379; there the
 * calls serve parameter-server style jobs whose ranks exchange host buffers of sizes the receiver does not know.)
 *
 * Messages between ranks of a communicator travel over its control plane (TCP through the rendezvous hub): they are
 * meant for control data, not for tensors.  A send copies the buffer and completes at once.  The receiver first probes
 * ({source, tag}, either may be a wildcard), learns the size from the status, then receives the probed message.
 * The Raw calls do the same between two endpoints that are connected like sockets, without a communicator.
 */
#ifndef HCCL_MSG_H
#define HCCL_MSG_H

#include "hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    HCCL_MODE_NORMAL = 0, /* exact probes */
    HCCL_MODE_ANY = 1,    /* probes with HCCL_ANY_SOURCE / HCCL_ANY_TAG */
    HCCL_MODE_PS = 2,
    HCCL_MODE_AI_CPU = 3,
    HCCL_MODE_SCHED_OS = 4
} WorkMode;

typedef struct tagCommAttr {
    WorkMode mode;
    uint32_t deviceId;
} CommAttr;

#define HCCL_ANY_SOURCE (-1)
#define HCCL_ANY_TAG (-1)

typedef void *HcclMessage;
typedef void *HcclRequest;

typedef struct {
    int srcRank;   /* sender of the probed / received message */
    int tag;
    int error;     /* 0: none */
    int cancelled;
    int count;     /* payload in bytes; HcclGetCount converts to elements */
} HcclStatus;

typedef enum { HCCL_ADDR_TYPE_ROCE = 0, HCCL_ADDR_TYPE_NUM } HcclAddrType;
typedef struct {
    HcclAddrType type;
    union {
        struct {
            uint32_t ipv4Addr; /* network byte order, as inet_pton writes it; 0 = any local address */
            uint16_t port;     /* host byte order; 0 when binding = pick one (HcclRawBind writes it back) */
        } tcp;
        uint8_t bytes[28];
    } info;
} HcclAddr;

/* A communicator from a rank table held in memory (JSON text), and its end. */
HcclResult HcclInitComm(const char *rankTableM, uint32_t rank, const CommAttr *attr, HcclComm *comm);
HcclResult HcclFinalizeComm(HcclComm comm);

/* Buffers the message calls will use; kept for source compatibility (sends copy, so nothing has to be pinned). */
HcclResult HcclRegisterGlobalMemory(void *addr, uint64_t size);
HcclResult HcclUnregisterGlobalMemory(void *addr);
HcclResult HcclRegisterMemory(HcclComm comm, void *buffer, uint64_t size);
HcclResult HcclUnregisterMemory(HcclComm comm, void *buffer);

int HcclIsend(void *buffer, int count, HcclDataType dataType, int dstRank, int tag, HcclComm comm, HcclRequest *request);
int HcclImprobe(int srcRank, int tag, HcclComm comm, int *flag, HcclMessage *msg, HcclStatus *status);
int HcclImrecv(void *buffer, int count, HcclDataType dataType, HcclMessage *msg, HcclRequest *request);
int HcclGetCount(const HcclStatus *status, HcclDataType dataType, int *count);
/* Completed requests are reported once, freed, and their array entries set to NULL. */
int HcclTestSome(int count, HcclRequest requestArray[], int *compCount, int compIndices[], HcclStatus compStatus[]);

/* The same between two connected endpoints. */
HcclResult HcclRawOpen(HcclConn *conn);
HcclResult HcclRawClose(HcclConn conn);
HcclResult HcclRawForceClose(HcclConn conn);
HcclResult HcclRawBind(HcclConn conn, HcclAddr *bindAddr);
HcclResult HcclRawConnect(HcclConn conn, HcclAddr *connectAddr);
HcclResult HcclRawListen(HcclConn conn, int backLog);
HcclResult HcclRawAccept(HcclConn listenConn, HcclAddr *acceptAddr, HcclConn *acceptConn);
HcclResult HcclRawIsend(const void *buf, int count, HcclDataType dataType, HcclConn conn, HcclRequest *request);
HcclResult HcclRawImprobe(HcclConn conn, int *flag, HcclMessage *msg, HcclStatus *status);
HcclResult HcclRawImrecv(void *buf, int count, HcclDataType datatype, HcclMessage *msg, HcclRequest *request);
HcclResult HcclRawImrecvScatter(void *buf[], int count[], int bufCount, HcclDataType datatype, HcclMessage *msg, HcclRequest *request);
HcclResult HcclRawGetCount(const HcclStatus *status, HcclDataType dataType, int *count);
HcclResult HcclRawTestSome(int count, HcclRequest requestArray[], int *compCount, int compIndices[], HcclStatus compStatus[]);

#ifdef __cplusplus
}
#endif
#endif /* HCCL_MSG_H */
