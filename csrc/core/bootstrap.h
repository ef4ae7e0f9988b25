// bootstrap.h - rendezvous and host control plane of a communicator.
//
// Topology of the control plane: a star.  The root (started by HcclGetRootInfo, or implied by a
// rank table) runs a hub thread; every rank, the root's own rank included, is an agent with one TCP
// connection to the hub.  Bring-up follows the reference's root-info flow
// (src/coll_communicator_mgr/rank_info_detect/rank_info_detect_service.cc:183-272): each agent sends
// its id string, the world size and a rank-info record; the hub waits until all ranks have
// reported (or the connect timeout expires -> HCCL_E_TIMEOUT / EI0015), orders the records by rank
// and broadcasts the full table with a step number.  After that the hub stays up and serves
//   - gathers over any subset of ranks (all-gather / barrier / broadcast are built on it),
//   - relayed point-to-point messages (channel handshakes, descriptor exchange),
//   - heartbeats: it tracks the last time each rank was heard and broadcasts the set of lost ranks;
//     a connection that closes without a goodbye marks the rank lost at once,
//   - asynchronous error broadcast (a rank that hits a device timeout tells everyone).
// File descriptors (exported memory) travel rank-to-rank over abstract Unix sockets.
//
// Beside the star, when heartbeats are on, the ranks watch each other in a ring that does not need the hub (the
// reference's cluster monitor is a double ring, src/coll_communicator_mgr/dfx/cluster_monitor/README_en.md:9-20):
// every interval a rank pings its nearest live neighbour in both directions over that neighbour's Unix socket.  A
// neighbour whose socket refuses connections (its process is gone) or that has been silent for the lost time is marked
// lost; every ping carries the sender's set of lost ranks, so the news travels round the ring also after the hub's
// process has died.  A rank that closes its communicator says goodbye first and is skipped from then on.
#pragma once
#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "hccl/hccl_types.h"
#include "net.h"

namespace hc {

constexpr uint32_t kRootHandleMagic = 0x48434c52;  // "HCLR"

// Contents of HcclRootInfo::internal.
struct RootHandle {
    char ip[64];
    uint32_t port;
    uint32_t netMode;        // 0 = TCP over IPv4
    char identifier[128];    // "ip_port_pid_timestamp": also the default communicator name
    uint32_t magic;
    uint32_t version;
};

using Blob = std::vector<uint8_t>;

class BootstrapHub {
public:
    ~BootstrapHub();
    // Binds and starts the hub thread.  port 0 picks HCCL_HOST_SOCKET_PORT_RANGE, else
    // HCCL_IF_BASE_PORT, else an ephemeral port.
    HcclResult Start(const std::string &ip, int port, const std::string &identifierHint);
    const RootHandle &handle() const { return handle_; }
    // 0 running, 1 finished cleanly, <0 failed (value = -HcclResult).
    int status() const { return status_.load(); }
    void Stop();
    // Test hook: drop the next n relay messages addressed to `dst` (simulates a lost handshake).
    void DropRelayTo(uint32_t dst, int n) { dropDst_ = dst; dropCount_ = n; }

private:
    void Run();
    RootHandle handle_{};
    int listenFd_ = -1;
    std::thread thread_;
    std::atomic<int> status_{0};
    std::atomic<bool> stop_{false};
    std::atomic<uint32_t> dropDst_{0};
    std::atomic<int> dropCount_{0};
};

class Bootstrap {
public:
    Bootstrap();
    ~Bootstrap();

    // Joins the rendezvous.  `info` is this rank's record; on success table[r] is rank r's record.
    HcclResult Connect(const RootHandle &root, uint32_t rank, uint32_t nRanks, const Blob &info,
                       std::vector<Blob> *table);
    void Close();

    uint32_t rank() const { return rank_; }
    uint32_t nRanks() const { return nRanks_; }
    const std::string &identifier() const { return identifier_; }

    // A subset of ranks that gathers among itself.  groupId 0 is the world.
    struct Group {
        uint32_t id = 0;
        std::vector<uint32_t> ranks;  // world ranks, ascending position = group index
        uint32_t myIndex = 0;
        uint32_t seq = 0;
    };
    Group WorldGroup() const;
    Group MakeGroup(uint32_t id, const std::vector<uint32_t> &ranks) const;

    HcclResult AllGather(Group &g, const Blob &mine, std::vector<Blob> *all, int timeoutMs = -1);
    HcclResult Barrier(Group &g, int timeoutMs = -1);
    // The barrier in two steps: Arrive tells the others that this rank is there and returns at once; Wait returns when all
    // have arrived.  A Wait that ran out of time (HCCL_E_TIMEOUT) leaves the barrier pending and may be repeated.
    HcclResult BarrierArrive(Group &g, uint64_t *ticket);
    HcclResult BarrierWait(uint64_t ticket, int timeoutMs, bool quiet = false);
    HcclResult Broadcast(Group &g, uint32_t rootIndex, Blob *data, int timeoutMs = -1);
    // Relayed datagrams; (src, tag) streams are FIFO.
    HcclResult Send(uint32_t dstRank, uint64_t tag, const Blob &data);
    HcclResult Recv(uint32_t srcRank, uint64_t tag, Blob *data, int timeoutMs = -1);
    // File descriptor passing.  The received descriptor belongs to the caller.
    // Takes the oldest queued relay message from `srcRank` (~0u: from anybody) whose tag agrees with `want` in the bits
    // of `mask`, without waiting.  HCCL_E_AGAIN when there is none.
    HcclResult TryRecv(uint32_t srcRank, uint64_t want, uint64_t mask, Blob *data, uint32_t *fromRank, uint64_t *fromTag);
    // Rank-to-rank bytes over the ranks' Unix sockets, without the hub (ranks of one host).  Used where the hub is gone.
    HcclResult SendDirect(uint32_t dstRank, const Blob &data);
    HcclResult RecvDirect(uint32_t srcRank, Blob *data, int timeoutMs);
    HcclResult SendFd(uint32_t dstRank, uint64_t tag, int fd);
    HcclResult RecvFd(uint32_t srcRank, uint64_t tag, int *fd, int timeoutMs = -1);

    // Heartbeat: starts a thread that pings the hub every intervalMs.
    void StartHeartbeat(int intervalMs);
    void StopHeartbeat();   // also what a test uses to make this rank fall silent
    uint64_t LostMask() const { return lostMask_.load() | ringLost_.load(); }
    // The connection to the hub (rank 0's process) broke without this side closing it: that process is gone, and with
    // it the heartbeat view, the relays and the retry rounds.
    bool HubGone() const { return hubGone_.load(); }
    // Milliseconds since rank r was last heard by the hub, as of the newest state broadcast.
    void HeartbeatAges(std::vector<uint64_t> *ages) const;
    // Async error fan-out.
    HcclResult NotifyError(HcclResult code);
    HcclResult RemoteError() const { return (HcclResult)remoteError_.load(); }
    void ClearRemoteError() { remoteError_.store(0); }

    int defaultTimeoutMs() const { return timeoutMs_; }

private:
    struct Key {
        uint32_t src;
        uint64_t tag;
        bool operator<(const Key &o) const { return src != o.src ? src < o.src : tag < o.tag; }
    };
    void ReaderLoop();
    void FdAcceptLoop();
    // ring monitor (runs on the heartbeat thread; messages arrive on the descriptor-accept thread)
    void RingTick(int lostAfterMs);
    void RingHeard(uint32_t src, uint32_t kind, uint64_t lostSeen);
    bool RingSend(uint32_t dst, uint32_t kind, int deadlineMs);
    int RingNeighbour(int dir) const;
    HcclResult SendMsg(uint16_t type, uint32_t dst, uint64_t tag, const void *data, size_t len);

    uint32_t rank_ = 0, nRanks_ = 0;
    std::string identifier_;
    int sock_ = -1;
    int udsFd_ = -1;
    int timeoutMs_ = 120000;
    std::mutex sendMu_;
    std::mutex mu_;
    std::condition_variable cv_;
    std::map<uint64_t, std::vector<Blob>> gatherDone_;
    std::map<Key, std::deque<Blob>> inbox_;
    std::map<Key, std::deque<int>> fdInbox_;
    std::map<uint32_t, std::deque<Blob>> directInbox_;   // guarded by mu_: SendDirect messages by sender
    std::thread reader_, fdAcceptor_, heart_;
    std::atomic<bool> closing_{false};
    std::atomic<bool> heartStop_{false};
    std::atomic<bool> hubGone_{false};
    std::atomic<uint64_t> lostMask_{0};
    std::atomic<int> remoteError_{0};
    mutable std::mutex hbMu_;
    std::vector<uint64_t> ages_;
    std::atomic<uint64_t> ringLost_{0}, ringLeft_{0};
    std::vector<int64_t> ringHeardMs_;       // guarded by hbMu_: when each rank's ping last arrived
    std::vector<int> ringRefused_;           // heartbeat thread only: consecutive refused connections per rank
};

}  // namespace hc
