/*
 * hccl_diag.h - diagnostics: operator trace ring, exec counters, per-op profiling records, the
 * device status block that bounded waits fill in, heartbeat state, communicator snapshots.
 * (reference: pkg_inc/hccl/hccl_diag.h, pkg_inc/hccl/hcomm_diag.h, dfx directories.)
 */
#ifndef HCCL_DIAG_H
#define HCCL_DIAG_H

#include "hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif

/* One record per operator launch, kept in a per-communicator ring (newest overwrites oldest). */
typedef struct {
    uint64_t seq;          /* operator ordinal on this communicator */
    uint32_t cmdType;      /* HcclCMDType */
    uint32_t dataType;
    uint64_t count;
    uint32_t reduceOp;
    uint32_t root;
    char algName[48];      /* what the selector picked */
    uint64_t hostStartNs;  /* CLOCK_MONOTONIC */
    uint64_t hostEndNs;    /* launch returned */
    uint64_t devStartNs;   /* %globaltimer at kernel start, 0 if not sampled */
    uint64_t devEndNs;
} HcclOpRecord;

/* What a device-side bounded wait writes when it gives up. */
typedef struct {
    uint32_t valid;      /* 0 = nothing recorded */
    uint32_t rank;       /* the waiting rank */
    uint32_t peer;       /* the rank that never signalled */
    uint32_t kind;       /* 1 barrier, 2 channel notify, 3 thread notify, 4 tile flag, 5 mbarrier */
    uint32_t slot;       /* flag index */
    uint32_t block;      /* CTA that gave up */
    uint64_t expected;
    uint64_t seen;
    uint64_t seq;        /* operator ordinal */
} HcclDeviceWaitStatus;

HcclResult HcclDiagGetOpRecords(HcclComm comm, HcclOpRecord *records, uint32_t capacity, uint32_t *written);
HcclResult HcclDiagGetOpCounters(HcclComm comm, uint64_t *launched, uint64_t *headCount, uint64_t *tailCount);
/* Device-side durations of the most recent kernels of the communicator (GPU global timer, nanoseconds), oldest first;
 * at most 16 are kept, recorded while profiling is on (HcclDiagSetProfiling).  A kernel that is still running reports end = 0. */
HcclResult HcclDiagGetKernelTimes(HcclComm comm, uint64_t *startNs, uint64_t *endNs, uint32_t capacity, uint32_t *written);
HcclResult HcclDiagGetWaitStatus(HcclComm comm, HcclDeviceWaitStatus *status);
HcclResult HcclDiagClearWaitStatus(HcclComm comm);
/* rank -> milliseconds since its last heartbeat (UINT64_MAX: never seen); lostMask bit r = LOST.  The mask joins
 * what the control plane's hub reports with what the ring monitor found (each rank pings its nearest live
 * neighbours and passes on the losses it knows of), so it keeps growing after the hub's own process is gone. */
HcclResult HcclDiagGetHeartbeat(HcclComm comm, uint64_t *ageMs, uint32_t capacity, uint64_t *lostMask);
/* Stops this rank's heartbeat thread: to the others it looks like a rank that hangs (its sockets stay open).  For
 * tests of the lost-rank paths; the thread is not started again. */
HcclResult HcclDiagPauseHeartbeat(HcclComm comm);
HcclResult HcclDiagSetProfiling(HcclComm comm, int enable);
/* Human-readable dump of the newest operator records and the wait status. */
HcclResult HcclDiagDump(HcclComm comm, char *buf, uint32_t bufLen);

/* Snapshot: enough state to rebuild the communicator in a restarted process without rendezvous.
 * Layout: "HCSN" u32 version, then length-prefixed sections {config, params, rank table, op count}. */
HcclResult HcclCommSnapshotSize(HcclComm comm, uint64_t *size);
HcclResult HcclCommSnapshotSave(HcclComm comm, void *buf, uint64_t bufLen, uint64_t *written);
HcclResult HcclCommSnapshotInfo(const void *buf, uint64_t len, uint32_t *rankSize, uint32_t *rank,
                                char *commName, uint64_t *opCount);

/* Quiesce every communicator of the process around an external process snapshot. */
HcclResult HcclSnapshotPre(void);
HcclResult HcclSnapshotPost(void);
HcclResult HcclSnapshotRestore(void);

#ifdef __cplusplus
}
#endif
#endif /* HCCL_DIAG_H */
