// coll_kernels.h - host-side interface of the specialised collective kernels (engine "sm" / "nvls").
//
// One kernel per (collective, regime); all share the argument block below.  A launch normally has
// gridDim.y == 1 and takes its arguments by value.  When several ranks of one process share a GPU
// (tests on a single device) the ranks' argument blocks are placed in a device table and ONE
// cooperative launch with gridDim.y == nRanks runs all of them, because kernels that wait on each
// other must never be separate launches on one GPU.
#pragma once
#include <stdint.h>

#include "comm_dev.h"
#include "hccl/hccl_types.h"

namespace hc {

enum FastKind : int32_t {
    FK_ALLREDUCE_ONESHOT = 0,
    FK_ALLREDUCE_TWOSHOT,
    FK_ALLREDUCE_NVLS,
    FK_REDUCE_SCATTER,
    FK_ALLGATHER,
    FK_ALLTOALL,
    FK_BROADCAST_PUSH,
    FK_BROADCAST_TWOSHOT,
    FK_BROADCAST_NVLS,
    FK_REDUCE,
    FK_SCATTER,
    FK_GATHER,
    FK_SEND,
    FK_RECV,
    FK_BARRIER,
    FK_SMALL_LL,             // flag-in-data exchange for small all-reduce / all-gather / all-to-all / reduce-scatter
    FK_REDUCE_SCATTER_NVLS,  // in-switch reduce-scatter (multimem.ld_reduce of the rank's own block)
    FK_ALLGATHER_NVLS,       // all-gather by multicast stores
    FK_ALLREDUCE_TWOSHOT_WIN,   // two-shot all-reduce of an operand beyond the staging: windows inside one launch
    FK_REDUCE_SCATTER_WIN,      // reduce-scatter of blocks beyond a staging slot: column windows inside one launch
    FK_REDUCE_SCATTER_INPLACE,  // reduce-scatter that reads the peers' registered inputs in place
    FK_ALLREDUCE_NVLS_PIPE,     // in-switch all-reduce of a large unregistered operand: copy-in / reduce / copy-out of different windows overlap
    FK_COUNT
};
const char *FastKindName(int32_t k);

enum LlMode : int32_t { LL_ALLREDUCE = 0, LL_ALLGATHER = 1, LL_ALLTOALL = 2, LL_REDUCE_SCATTER = 3 };

struct CollArgs {
    CommDev *dev;
    const void *in;
    void *out;
    uint64_t count;          // elements; meaning depends on the collective (see coll_kernels.cu)
    uint64_t sliceElems;     // elements per slot / slice (host-computed, 16-byte multiple)
    int32_t dtype;
    int32_t op;
    int32_t root;
    int32_t peer;            // send / recv partner; FK_SMALL_LL: which collective (LlMode)
    float scale;             // applied to the reduced value when useScale != 0
    int32_t useScale;
    int32_t preBarrier;      // 1: synchronise all ranks before touching peer memory
    uint32_t elemSize;
    // variable-count collectives (elements); unused entries are zero
    uint64_t sendCounts[HC_KERNEL_MAX_RANKS], sendDispls[HC_KERNEL_MAX_RANKS];
    uint64_t recvCounts[HC_KERNEL_MAX_RANKS], recvDispls[HC_KERNEL_MAX_RANKS];
    uint64_t col0, col1;     // column window of this launch for chunked all-to-all style ops
    uint64_t winElems;       // all-reduce: elements per in-kernel window (0 = the whole operand is one window)
    // Registered (zero-copy) buffers: the operand's address in every rank's memory as this rank maps it, and the
    // multicast alias of the operand; NULL when the buffer is not inside a registered window (or has no alias).
    const void *inPeer[HC_KERNEL_MAX_RANKS];
    const void *inMc;
    void *outMc;
    // point-to-point bookkeeping (values before this operator)
    uint64_t p2pDataBase, p2pAckBase;
    uint64_t p2pOffset;      // offset of the point-to-point landing area in the heap
    uint64_t p2pSlotBytes;   // bytes per source rank in that area (two sub-slots)
};

struct FastLaunch {
    int32_t kind;
    CollArgs args;
    int ctas;                // CTAs per rank
    int threads;
    void *stream;
    // shared-GPU emulation
    const CollArgs *emuTable;   // device pointer to nRanks argument blocks, or NULL
    int emuRanks;
};

// ---- schedule interpreter (engine "sm-ir"): one kernel runs this rank's program of a Schedule
struct IrLayoutDev { uint64_t sliceCount, total; };       // uniform slice geometry of INPUT / OUTPUT / SCRATCH
struct IrArgs {
    CommDev *dev;
    const void *prims;       // DevPrim[nPrims] in device memory
    uint32_t nPrims;
    int32_t dtype, op;
    uint32_t elemSize;
    const void *in;
    void *out;
    IrLayoutDev lay[3];
    uint64_t cap;            // elements per scratch slot in this pass
    uint64_t col0, col1;     // column window of this pass
    int32_t preBarrier;
};
// Launches the interpreter for one pass; `emuTable` as in FastLaunch.  HCCL_E_NOT_SUPPORT for a data type without a kernel.
HcclResult LaunchIrKernel(const IrArgs &args, int ctas, void *stream, const IrArgs *emuTable, int emuRanks);
void *IrKernelFor(int dtype);

// Forces every kernel of this file to be loaded on the current device (call once per device before any launch).
void PreloadFastKernels();
// Returns HCCL_E_NOT_SUPPORT for a (kind, dtype) pair without a kernel.
HcclResult LaunchFastKernel(const FastLaunch &l);
// Barriers a kernel of this kind consumes (the epoch advance), so callers can reason about it.
uint32_t FastKindBarriers(int32_t kind, int preBarrier);
// Upper bound of CTAs per rank for which all CTAs of `ranksOnDevice` ranks are co-resident.
int FastMaxCoResidentCtas(int32_t kind, int threads, int ranksOnDevice);

}  // namespace hc
