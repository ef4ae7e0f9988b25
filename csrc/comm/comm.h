// comm.h - the communicator: everything one rank holds for one group of ranks.
//
// Counterpart of the reference's CollComm (src/coll_communicator_mgr/communicator/coll_comm.h:54-187)
// with its collaborators folded in:
//   control plane     Bootstrap (shared with sub-communicators) + a gather group
//   topology          RankTable / RankGraph
//   symmetric heap    control region + CCL buffer of every rank mapped at heapBase + r*stride,
//                     optional NVLS multicast alias
//   resources         threads, channels, engine contexts, registered memories, windows, teams
//   execution state   operator ordinal, host-side notify bookkeeping, READY/SUSPENDED state machine
//   diagnostics       operator record ring, wait-status block, counters
#pragma once
#include <atomic>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../alg/ir.h"
#include "../alg/templates.h"
#include "../core/bootstrap.h"
#include "../device/comm_dev.h"
#include "../plat/platform.h"
#include "../topo/rank_graph.h"
#include "hccl/hccl_comm.h"
#include "hccl/hccl_diag.h"
#include "hccl/hccl_team.h"

namespace hc {

struct ResolvedConfig {
    uint32_t bufferMB = 200;
    uint32_t deterministic = 0;
    std::string name;
    std::string udi;
    uint32_t opExpansionMode = 0;
    int32_t execTimeoutSec = 1836;
    std::string algo;
    std::string bufferName;
    uint32_t worldRankId = 0;
    uint64_t jobId = 0;
    uint64_t symStrideGB = 16;
    uint8_t graphZeroCopy = 0;
    std::string retryEnable, retryParams;
};

// A registered memory (HcclCommMemReg / HcommMemReg) and, after exchange, its peer views.
struct RegMem {
    std::string tag;
    CommMem mem{};
    bool symmetric = false;          // part of the heap: peers compute its address
    uint64_t heapOffset = 0;
};

struct Window {
    uint32_t magic = 0x57494e44;     // "WIND"
    struct Comm *comm = nullptr;
    void *localAddr = nullptr;       // the registered range [localAddr, localAddr+size)
    uint64_t size = 0;
    std::vector<void *> peerPtr;     // address of the same range on rank r, valid in this process
    void *mcPtr = nullptr;
    // how the peer views were obtained (for teardown)
    enum Kind { HEAP, VMM, IPC } kind = HEAP;
    void *vaBase = nullptr;
    size_t vaBytes = 0;
    size_t mapStride = 0;
    std::vector<PhysMem> imported;
    std::vector<void *> ipcBases;
    uint64_t allocOffset = 0;        // offset of localAddr inside its allocation
    // multicast alias of a virtual-memory window (the heap's own alias serves HEAP windows)
    PhysMem mcPhys;
    void *mcVa = nullptr;
    size_t mcBytes = 0;
    bool mcBound = false;
};

// The registered window that holds [ptr, ptr + bytes), or NULL; *offset receives the distance from the window's start.
struct Comm;
Window *FindWindow(Comm *c, const void *ptr, uint64_t bytes, uint64_t *offset);

struct ThreadRes {
    uint32_t magic = 0x54485244;     // "THRD"
    struct Comm *comm = nullptr;     // may be null for HcommThreadAlloc threads
    Platform *plat = nullptr;
    CommEngine engine = COMM_ENGINE_CPU_TS;
    Stream stream = nullptr;
    bool ownsStream = false;
    uint32_t notifyNum = 0;
    uint64_t *notify = nullptr;      // notifyNum 64-bit words the device can see
    std::vector<uint64_t> waited;    // waits issued per slot (host-side expectation)
    bool ownsNotify = false;
};

struct ChannelRes {
    uint32_t magic = 0x4348414e;     // "CHAN"
    struct Comm *comm = nullptr;
    CommEngine engine = COMM_ENGINE_CPU_TS;
    uint32_t remoteRank = 0;
    CommProtocol protocol = COMM_PROTOCOL_NVLINK;
    uint32_t notifyNum = 0;
    uint32_t notifyBase = 0;         // first slot of this channel in the per-peer notify table
    std::vector<uint64_t> waited;    // waits issued per local slot
    std::atomic<int> status{0};      // HcommChannelStatus
    std::vector<CommMem> remoteMems;
    std::vector<std::string> remoteTags;
    std::vector<char *> tagPtrs;
    void *devView = nullptr;
    // where records go and where they arrive; filled from the heap for communicator channels and from
    // exchanged descriptors for base-level channels
    uint64_t *remoteNotify = nullptr, *localNotify = nullptr;
    Platform *plat = nullptr;
    int sock = -1;                   // base-level channels keep their control socket
    std::vector<void *> importedBases;
};

enum class CommState { READY = 0, SUSPENDING = 1, SUSPENDED = 2, DESTROYED = 3 };
struct RetryState;       // coll/ops.h

struct Comm {
    uint32_t magic = 0x434f4d4d;     // "COMM"
    Platform *plat = nullptr;
    int device = 0;
    uint32_t rank = 0, nRanks = 0;
    ResolvedConfig cfg;
    std::string identifier;

    std::shared_ptr<Bootstrap> boot;
    std::shared_ptr<BootstrapHub> hub;       // only on the process that started the rendezvous
    Bootstrap::Group group;                  // gather group of this communicator on `boot`
    std::vector<uint32_t> worldRanks;        // bootstrap rank of each member
    RankTable table;
    RankGraph graph;

    // ---- symmetric heap
    PhysMem heapPhys;
    std::vector<PhysMem> peerPhys;
    char *heapBase = nullptr;
    uint64_t heapStride = 0, heapBytes = 0, halfBytes = 0;
    uint64_t p2pOffset = 0, p2pSlotBytes = 0;    // landing area of the send/recv kernels: one slot per source rank
    uint64_t llOffset = 0, llBytes = 0;          // flag-in-data area of the small-message kernels
    std::vector<uint64_t> p2pSent, p2pRecvd;     // chunks exchanged so far with each peer
    // Fused GEMM kernels: tile flags in the control region hold launch sequence numbers (kept on the device), so the
    // host keeps no per-call state for them.
    void *fusedLocal = nullptr;                  // device-local scratch: push chunk counters, phase clocks
    bool fusedPhaseClocks = false;               // record per-CTA phase clocks in the CTA-pair fused kernels
    int fusedLastCtas = 0;                       // CTAs of the most recent CTA-pair fused launch
    void *fusedTemp = nullptr;                   // GEMM result of the split GEMM + reduce-scatter form
    size_t fusedTempBytes = 0;
    void *irPrimRing = nullptr;                  // device ring of interpreter programs (8 slots of 2048 primitives)
    int irPrimNext = 0;
    bool lastOpOnHost = true;                    // the next specialised kernel must start with a barrier
    PhysMem mcPhys;
    char *mcBase = nullptr;
    bool mcBound = false;
    bool emuSameDevice = false;              // several ranks of this process share one GPU

    // ---- device-visible state
    CommDev *devStruct = nullptr;            // device memory
    CommDev hostDev{};                       // host copy
    uint32_t *devCounters = nullptr;         // epoch, launches, blocksDone (+ pad)
    uint64_t *devIrCounters = nullptr;       // irSent + irConsumed
    uint32_t *abortWord = nullptr;           // pinned host
    HcclDeviceWaitStatus *waitStatus = nullptr;
    uint64_t *opCounters = nullptr;          // device {head, tail} (inside the devStruct block); read with Platform::PeekSync

    // ---- execution state
    std::mutex opMu;                         // operators of one communicator are issued one at a time
    uint64_t opSeq = 0;
    uint32_t hostLaunches = 0;               // parity of the CCL half used by host-engine operators
    std::vector<uint64_t> chanWaited;        // [HC_MAX_RANKS][HC_CHAN_NOTIFY] waits issued on the internal slots
    std::atomic<int> state{(int)CommState::READY};
    std::atomic<int> asyncError{0};
    std::vector<Stream> auxStreams;

    // ---- resources handed to users
    std::mutex resMu;
    std::vector<std::unique_ptr<ThreadRes>> threads;
    std::map<int, ThreadRes *> dedicatedThreads;
    std::vector<std::unique_ptr<ChannelRes>> channels;
    // Channel notify slots are numbered per peer (both ends of a pair acquire their k-th channel with the same
    // base); slots 0..7 of every peer belong to the library's own schedules.
    std::vector<uint32_t> nextChanNotify;    // [nRanks], starts at 8
    struct EngineCtx { void *ptr; uint64_t size; CommEngine engine; };
    std::map<std::string, EngineCtx> engineCtxs;
    std::vector<std::unique_ptr<RegMem>> regMems;
    std::vector<std::unique_ptr<Window>> windows;
    uint64_t teamSyncUsed = 0;               // bytes of HC_OFF_TEAM_SYNC handed out
    uint32_t ctaLimit = 0;                   // upper bound of CTAs per collective kernel of this communicator (HcomSetAivCoreLimit); 0 = none
    uint32_t subCommSeq = 0;

    // ---- diagnostics
    std::shared_ptr<RetryState> retry;       // operator retry agent, when switched on
    // what the caller attached for diagnostics (HcommRegOpInfo / HcommRegOpTaskException / HcclDfxRegOpInfoByCommId)
    std::vector<uint8_t> userOpInfo;
    void (*userOpInfoFormatter)(const void *, char *, size_t) = nullptr;
    std::vector<uint8_t> exchangeInfo;                       // HcclCommAddExchangeInfo: this rank's extra bytes
    std::vector<std::vector<uint8_t>> peerExchangeInfo;      // what the peers contributed, filled by the channel exchange
    std::map<std::string, int32_t (*)(uint64_t, int32_t)> taskCallbacks;
    std::map<std::string, std::pair<void *, uint64_t>> taggedDevMem;
    std::mutex diagMu;
    std::vector<HcclOpRecord> opRing;
    uint64_t opRingNext = 0;
    bool profiling = false;

    // ---- schedule cache: key -> built schedule for this rank
    std::map<std::string, std::shared_ptr<Schedule>> schedCache;

    ~Comm();
    char *PeerHeap(uint32_t r) const { return heapBase + (uint64_t)r * heapStride; }
    char *LocalHeap() const { return PeerHeap(rank); }
    char *CclBuffer() const { return LocalHeap() + HC_CTRL_BYTES; }
    uint32_t TimeoutMs() const { return cfg.execTimeoutSec <= 0 ? 0x7fffffffu : (uint32_t)cfg.execTimeoutSec * 1000u; }
};

// Validates a handle coming from C.
inline Comm *AsComm(HcclComm h)
{
    Comm *c = (Comm *)h;
    return (c && c->magic == 0x434f4d4d) ? c : nullptr;
}

struct CommInitArgs {
    Platform *plat = nullptr;
    int device = -1;                               // -1: the calling thread's current device
    std::shared_ptr<Bootstrap> boot;               // already connected
    std::shared_ptr<BootstrapHub> hub;
    Bootstrap::Group group;
    std::vector<Blob> memberInfo;                  // rank record of each member (RankEntry streams)
    const HcclCommConfig *config = nullptr;
    std::string defaultName;
};

// Builds the local rank record that a rank contributes to the rendezvous.
Blob MakeRankRecord(Platform *plat, int device, uint32_t rank);
HcclResult CommCreate(const CommInitArgs &args, Comm **out);
void CommDestroy(Comm *c);
HcclResult ResolveConfig(const HcclCommConfig *cfg, const std::string &defaultName, ResolvedConfig *out);

// Registry of live communicators of the process (name -> comm), state callbacks.
HcclResult RegistryAdd(Comm *c);
void RegistryRemove(Comm *c);
Comm *RegistryFind(const std::string &name);
void RegistryForEach(const std::function<void(Comm *)> &fn);

// Operator retry agent (coll/retry.cc).
void RetrySetup(Comm *c);
void RetryTeardown(Comm *c);
// Collective (two barriers on `g`): every synchronisation value of the communicator back to its initial state.
HcclResult CommClearSyncState(Comm *c, Bootstrap::Group &g);
// Diagnostics hooks (api/dfx_api.cc): exception callbacks fire when a communicator records a failure, the profiling
// sink receives one report per operator while profiling is on.
void DfxFireException(Comm *c, HcclResult err);
void DfxReportOp(Comm *c, const char *name, uint64_t beginNs, uint64_t endNs);

// Clears the device-local scratch of the fused GEMM kernels (fused_gemm.cu) when a communicator resumes.
void FusedResetLocal(Comm *c);

// Records an asynchronous failure: stores it, tells the peers, logs the wait status.
void CommSetAsyncError(Comm *c, HcclResult err);
// Checks the pinned abort word / status after an operator and converts it into an error.
HcclResult CommPollDeviceStatus(Comm *c);

}  // namespace hc
