// hcomm_comm_dev.h - layout shared by the host runtime and the CUDA kernels.
//
// Every rank owns one "symmetric heap": a physical block that all ranks of the communicator map
// at  heapBase + rank * heapStride  in their own address space, so the address of byte `off` on
// rank r is computed, not looked up.  The heap starts with a control region (flags and notify
// slots, never cleared between operators: all synchronisation values only grow) followed by the
// CCL buffer, two halves that operators use alternately (launch parity) so that a fast rank can
// start the next operator while a slow one still reads the previous one's data - the same
// ping-pong the reference applies to its AIV staging buffer
// (algorithm/base/alg_aiv_template/aiv_communication_base.h:166-168).
#pragma once
#include <stdint.h>

#include "hccl/hccl_diag.h"

#define HC_MAX_RANKS 64          /* sizing of flag tables */
#define HC_KERNEL_MAX_RANKS 16   /* rank count the SM kernels accept (one NVLink domain) */
#define HC_MAX_CTAS 256          /* CTAs per rank that can take part in a cross-rank barrier */
#define HC_IR_MAX_CTAS 128       /* CTAs of the schedule-interpreter kernel */
#define HC_IR_RANKS 16           /* ranks the interpreter's notify tables are laid out for (= HC_KERNEL_MAX_RANKS) */
#define HC_IR_NOTIFY 8           /* notify slots per (CTA, peer) in the interpreter */
#define HC_CHAN_NOTIFY 64        /* notify slots per channel on the host engines */

#define HC_CTRL_BYTES (4ull << 20)
#define HC_OFF_BARRIER 0ull                       /* u32  [HC_MAX_CTAS][HC_MAX_RANKS]                */
#define HC_OFF_IR_NOTIFY (64ull << 10)            /* u64  [HC_IR_MAX_CTAS][HC_IR_RANKS][HC_IR_NOTIFY]: 128 KB */
#define HC_OFF_CHAN_NOTIFY (384ull << 10)         /* u64  [HC_MAX_RANKS][HC_CHAN_NOTIFY]              */
#define HC_OFF_P2P (448ull << 10)                 /* u64  [HC_MAX_RANKS][8] send/recv handshakes      */
#define HC_OFF_META (480ull << 10)                /* u64  [HC_MAX_RANKS] per-operator values agreed in-kernel */
#define HC_OFF_THREAD_NOTIFY (512ull << 10)       /* u64  [1024] local thread notifies                */
#define HC_OFF_FUSED (576ull << 10)               /* u32  [8192] tile-ready flags of fused ops        */
#define HC_OFF_TEAM_SYNC (1ull << 20)             /* u64  team signal / counter / barrier words, 1 MB */
#define HC_OFF_ONESIDED (2ull << 20)              /* scratch for one-sided services, 2 MB             */

/* Kinds recorded in HcclDeviceWaitStatus::kind */
#define HC_WAIT_BARRIER 1
#define HC_WAIT_CHAN_NOTIFY 2
#define HC_WAIT_THREAD_NOTIFY 3
#define HC_WAIT_TILE_FLAG 4
#define HC_WAIT_MBARRIER 5
#define HC_WAIT_BOUNDS 6       /* not a wait: a range check of the bounds-checking build failed */

/* Device-resident description of one communicator (one per rank). */
struct CommDev {
    int32_t rank;
    int32_t nRanks;
    char *heapBase;          /* address of rank 0's heap in THIS rank's address space */
    uint64_t heapStride;
    char *mcBase;            /* NVLS multicast alias of the heap, or NULL */
    uint64_t bufOffset;      /* = HC_CTRL_BYTES */
    uint64_t halfBytes;      /* size of one CCL half */
    uint32_t *epoch;         /* device-local: last barrier epoch consumed */
    uint32_t *launches;      /* device-local: operators launched (parity picks the CCL half) */
    uint32_t *blocksDone;    /* device-local scratch counter */
    uint32_t profile;        /* non-zero: kernels record start / end timestamps in the ring at HC_DEV_TIMES_OFFSET */
    uint32_t heapMB;         /* size of one rank's heap in MB (range checks of the bounds-checking build) */
    uint64_t *irConsumed;    /* device-local [HC_IR_MAX_CTAS][HC_IR_RANKS][HC_IR_NOTIFY]: posts consumed by the interpreter's waits */
    uint32_t *abortWord;     /* host-pinned: non-zero makes every wait return immediately */
    HcclDeviceWaitStatus *status; /* host-pinned record of the first wait that expired */
    uint64_t *opCounters;    /* device-local {head, tail}: bumped at kernel start / end (the host peeks at them to tell which operator hangs) */
    uint64_t timeoutNs;      /* budget of every device-side wait */
    uint64_t llOffset;       /* heap offset of the flag-in-data (LL) area: [2 parities][HC_KERNEL_MAX_RANKS sources][HC_LL_SLOT_BYTES] */
};

/* The structure, the launch counters and the head/tail counters share one device allocation so that a kernel
 * finds its counters at a fixed distance from the structure (no dependent pointer load on the cold path):
 *   [0, 128) CommDev   [128, 640) u32 counters[128]: 0 epoch, 1 launches, 2 blocksDone, ...   [640, 656) u64 {head, tail} */
/* LL area: every 8 bytes carry 4 bytes of payload and a 4-byte tag; a slot takes HC_LL_MAX_PAYLOAD payload bytes. */
#define HC_LL_MAX_PAYLOAD (1024ull << 10)
#define HC_LL_SLOT_BYTES (2 * HC_LL_MAX_PAYLOAD)

#define HC_DEV_COUNTERS_OFFSET 128
#define HC_DEV_OPCOUNTERS_OFFSET 640
/* [704, 960): ring of HC_DEV_TIME_SLOTS {start ns, end ns} pairs (GPU global timer) of the most recent kernels; slot = head count % slots */
#define HC_DEV_TIMES_OFFSET 704
#define HC_DEV_TIME_SLOTS 16
#define HC_DEV_BLOCK_BYTES 1024

#ifdef __CUDACC__
#define HC_HD __host__ __device__ __forceinline__
#elif defined(__cplusplus)
#define HC_HD inline
#else
#define HC_HD static inline
typedef struct CommDev CommDev;   /* C programs read the layout too */
#endif

HC_HD char *HcPeerHeap(const CommDev *d, int r) { return d->heapBase + (uint64_t)r * d->heapStride; }
