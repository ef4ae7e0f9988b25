#include "bootstrap.h"

#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstring>

#include "env.h"
#include "log.h"

namespace hc {
namespace {

constexpr uint32_t kMsgMagic = 0x4d434348;  // "HCCM"
constexpr uint64_t kMaxMsgBytes = 100ull << 20;  // same cap as the reference's rank-table buffer

// Messages of the ring monitor travel over the descriptor-passing sockets without a descriptor: the header's second
// word says which kind, the set of ranks the sender holds for lost rides in its tag.
constexpr uint32_t kRingPing = 1, kRingBye = 2;
// The same sockets carry rank-to-rank bytes that must not depend on the hub (Bootstrap::SendDirect).
constexpr uint32_t kDirectBytes = 3;
constexpr uint64_t kMaxDirectBytes = 1 << 20;

enum MsgType : uint16_t {
    MSG_HELLO = 1,
    MSG_TABLE = 2,
    MSG_GATHER = 3,
    MSG_GATHER_REPLY = 4,
    MSG_RELAY = 5,
    MSG_HEARTBEAT = 6,
    MSG_HB_STATE = 7,
    MSG_ERROR = 8,
    MSG_BYE = 9,
    MSG_REJECT = 10,
};

struct MsgHdr {
    uint32_t magic;
    uint16_t type;
    uint16_t flags;
    uint32_t src;
    uint32_t dst;
    uint64_t tag;
    uint64_t len;
};

void Put32(Blob &b, uint32_t v) { b.insert(b.end(), (uint8_t *)&v, (uint8_t *)&v + 4); }
void Put64(Blob &b, uint64_t v) { b.insert(b.end(), (uint8_t *)&v, (uint8_t *)&v + 8); }
void PutBlob(Blob &b, const Blob &x) { Put64(b, x.size()); b.insert(b.end(), x.begin(), x.end()); }
struct Reader {
    const uint8_t *p, *e;
    bool ok = true;
    Reader(const Blob &b) : p(b.data()), e(b.data() + b.size()) {}
    uint32_t u32() { uint32_t v = 0; if (e - p < 4) { ok = false; return 0; } memcpy(&v, p, 4); p += 4; return v; }
    uint64_t u64() { uint64_t v = 0; if (e - p < 8) { ok = false; return 0; } memcpy(&v, p, 8); p += 8; return v; }
    Blob blob() { uint64_t n = u64(); if (!ok || (uint64_t)(e - p) < n) { ok = false; return {}; } Blob b(p, p + n); p += n; return b; }
};

HcclResult WriteMsg(int fd, uint16_t type, uint32_t src, uint32_t dst, uint64_t tag, const void *data, size_t len)
{
    MsgHdr h{kMsgMagic, type, 0, src, dst, tag, len};
    Blob buf(sizeof(h) + len);
    memcpy(buf.data(), &h, sizeof(h));
    if (len) memcpy(buf.data() + sizeof(h), data, len);
    return net::SendAll(fd, buf.data(), buf.size());
}

HcclResult ReadMsg(int fd, MsgHdr *h, Blob *payload, int64_t deadline)
{
    HcclResult r = net::RecvAll(fd, h, sizeof(*h), deadline);
    if (r != HCCL_SUCCESS) return r;
    if (h->magic != kMsgMagic || h->len > kMaxMsgBytes) return HCCL_E_TCP_TRANSFER;
    payload->resize(h->len);
    if (h->len) r = net::RecvAll(fd, payload->data(), h->len, deadline);
    return r;
}

}  // namespace

// ------------------------------------------------------------------------------------------ hub

BootstrapHub::~BootstrapHub() { Stop(); }

void BootstrapHub::Stop()
{
    stop_.store(true);
    if (thread_.joinable()) thread_.join();
    net::Close(listenFd_);
}

HcclResult BootstrapHub::Start(const std::string &ip, int port, const std::string &identifierHint)
{
    const EnvConfig &env = EnvConfig::Get();
    int lo = port, hi = port;
    if (port == 0) {
        if (!env.hostPortRange.value.empty() && env.hostPortRange.value != "auto") {
            ParsePortRange(env.hostPortRange.value, lo, hi);
        } else if (env.ifBasePort.fromEnv) {
            lo = env.ifBasePort.value;
            hi = lo + 15;  // the reference pre-empts a 16-port window above the base port
        }
    }
    int boundPort = 0;
    HcclResult r = net::TcpListen(ip, lo, hi, &listenFd_, &boundPort);
    if (r != HCCL_SUCCESS) return r;
    memset(&handle_, 0, sizeof(handle_));
    snprintf(handle_.ip, sizeof(handle_.ip), "%s", ip.c_str());
    handle_.port = (uint32_t)boundPort;
    handle_.netMode = 0;
    handle_.magic = kRootHandleMagic;
    handle_.version = 1;
    if (identifierHint.empty()) {
        snprintf(handle_.identifier, sizeof(handle_.identifier), "%s_%d_%d_%lld", ip.c_str(), boundPort, (int)getpid(),
                 (long long)net::NowMs());
    } else {
        snprintf(handle_.identifier, sizeof(handle_.identifier), "%s", identifierHint.c_str());
    }
    thread_ = std::thread([this] { Run(); });
    HCCL_INFO("bootstrap hub listening on %s:%d id=%s", ip.c_str(), boundPort, handle_.identifier);
    return HCCL_SUCCESS;
}

void BootstrapHub::Run()
{
    const EnvConfig &env = EnvConfig::Get();
    net::Whitelist wl;
    if (!env.whitelistDisable.value) wl.Load(env.whitelistFile.value);
    const int64_t deadline = net::NowMs() + (int64_t)env.connectTimeoutSec.value * 1000;

    struct Agent {
        int fd = -1;
        bool alive = false;
        bool bye = false;
        int64_t lastSeen = 0;
        Blob info;
    };
    std::vector<Agent> agents;
    uint32_t nRanks = 0, joined = 0;
    auto failAll = [&](HcclResult code) {
        for (auto &a : agents)
            if (a.fd >= 0) { WriteMsg(a.fd, MSG_REJECT, 0, 0, (uint64_t)code, nullptr, 0); net::Close(a.fd); }
        status_.store(-(int)code);
    };

    // Phase 1: collect one HELLO per rank.
    while (nRanks == 0 || joined < nRanks) {
        if (stop_.load()) { failAll(HCCL_E_INTERNAL); return; }
        int fd = -1;
        std::string peer;
        int64_t now = net::NowMs();
        if (now >= deadline) {
            std::string missing;
            for (uint32_t r = 0; r < nRanks; ++r)
                if (!agents[r].alive) missing += std::to_string(r) + " ";
            RPT_ERR("EI0015", "rendezvous timed out after %d s: %u of %u ranks joined, missing ranks: %s",
                    env.connectTimeoutSec.value, joined, nRanks, missing.c_str());
            failAll(HCCL_E_TIMEOUT);
            return;
        }
        HcclResult r = net::TcpAccept(listenFd_, std::min<int64_t>(deadline, now + 100), &fd, &peer);
        if (r == HCCL_E_TIMEOUT) continue;
        if (r != HCCL_SUCCESS) { failAll(r); return; }
        if (!wl.Allows(peer)) {
            HCCL_WARNING("connection from %s refused by whitelist", peer.c_str());
            net::Close(fd);
            continue;
        }
        MsgHdr h;
        Blob pl;
        // A rank sends its HELLO right after connecting.  Whatever else connects (a port scan, a health check) and stays
        // silent must not hold up the ranks that queue behind it: it gets a few seconds, not the rendezvous' whole time.
        if (ReadMsg(fd, &h, &pl, std::min<int64_t>(deadline, net::NowMs() + 3000)) != HCCL_SUCCESS || h.type != MSG_HELLO) { net::Close(fd); continue; }
        Reader rd(pl);
        uint32_t size = rd.u32(), rank = rd.u32();
        Blob agentId = rd.blob();
        Blob info = rd.blob();
        if (!rd.ok || size == 0 || rank >= size || (nRanks != 0 && size != nRanks)) {
            RPT_ERR("EI0014", "rank %u reports world size %u but the rendezvous expects %u", rank, size, nRanks);
            WriteMsg(fd, MSG_REJECT, 0, rank, HCCL_E_PARA, nullptr, 0);
            net::Close(fd);
            failAll(HCCL_E_PARA);
            return;
        }
        if (nRanks == 0) { nRanks = size; agents.resize(nRanks); }
        if (agents[rank].alive) {
            RPT_ERR("EI0014", "rank %u joined the rendezvous twice", rank);
            WriteMsg(fd, MSG_REJECT, 0, rank, HCCL_E_PARA, nullptr, 0);
            net::Close(fd);
            failAll(HCCL_E_PARA);
            return;
        }
        agents[rank].fd = fd;
        agents[rank].alive = true;
        agents[rank].lastSeen = net::NowMs();
        agents[rank].info = std::move(info);
        ++joined;
        HCCL_DEBUG_CAT(CAT_BOOT, "hub: rank %u/%u joined from %s (%.*s)", rank, nRanks, peer.c_str(), (int)agentId.size(),
                       (const char *)agentId.data());
    }
    {   // broadcast the ordered table, step 1
        Blob table;
        Put32(table, 1);
        Put32(table, nRanks);
        for (auto &a : agents) PutBlob(table, a.info);
        for (uint32_t r = 0; r < nRanks; ++r) WriteMsg(agents[r].fd, MSG_TABLE, 0, r, 0, table.data(), table.size());
    }

    // Phase 2: serve.
    struct Gather {
        uint32_t size = 0, got = 0;
        std::vector<Blob> parts;
        std::vector<uint32_t> members;
    };
    std::map<uint64_t, Gather> gathers;
    uint64_t lostMask = 0;
    int64_t lastHbBroadcast = 0;
    const int lostMs = env.heartbeatLostMs.value;
    bool heartbeatSeen = false;
    auto broadcastHb = [&]() {
        Blob st;
        Put64(st, lostMask);
        int64_t now = net::NowMs();
        Put32(st, nRanks);
        for (auto &a : agents) Put64(st, a.alive || a.bye ? (uint64_t)(now - a.lastSeen) : UINT64_MAX);
        for (uint32_t r = 0; r < nRanks; ++r)
            if (agents[r].fd >= 0) WriteMsg(agents[r].fd, MSG_HB_STATE, 0, r, 0, st.data(), st.size());
        lastHbBroadcast = now;
    };
    for (;;) {
        uint32_t live = 0;
        std::vector<struct pollfd> pfds;
        std::vector<uint32_t> idx;
        for (uint32_t r = 0; r < nRanks; ++r)
            if (agents[r].fd >= 0) { pfds.push_back({agents[r].fd, POLLIN, 0}); idx.push_back(r); ++live; }
        if (live == 0) break;
        if (stop_.load()) break;
        int pr = poll(pfds.data(), pfds.size(), 50);
        int64_t now = net::NowMs();
        if (pr > 0) {
            for (size_t i = 0; i < pfds.size(); ++i) {
                if (!(pfds[i].revents & (POLLIN | POLLHUP | POLLERR))) continue;
                uint32_t r = idx[i];
                Agent &a = agents[r];
                MsgHdr h;
                Blob pl;
                HcclResult rr = ReadMsg(a.fd, &h, &pl, now + 5000);
                if (rr != HCCL_SUCCESS) {
                    net::Close(a.fd);
                    a.alive = false;
                    if (!a.bye) {   // vanished without goodbye: tell everyone now
                        lostMask |= (1ull << (r & 63));
                        HCCL_WARNING("hub: rank %u disconnected without goodbye, marked LOST", r);
                        broadcastHb();
                    }
                    continue;
                }
                a.lastSeen = now;
                switch (h.type) {
                    case MSG_GATHER: {
                        Reader rd(pl);
                        uint32_t gsize = rd.u32(), gidx = rd.u32();
                        Blob part = rd.blob();
                        Gather &g = gathers[h.tag];
                        if (g.size == 0) { g.size = gsize; g.parts.resize(gsize); g.members.assign(gsize, ~0u); }
                        if (gidx < g.size && g.members[gidx] == ~0u) {
                            g.parts[gidx] = std::move(part);
                            g.members[gidx] = r;
                            ++g.got;
                        }
                        if (g.got == g.size) {
                            Blob out;
                            Put32(out, g.size);
                            for (auto &p : g.parts) PutBlob(out, p);
                            for (uint32_t m : g.members)
                                if (agents[m].fd >= 0) WriteMsg(agents[m].fd, MSG_GATHER_REPLY, 0, m, h.tag, out.data(), out.size());
                            gathers.erase(h.tag);
                        }
                        break;
                    }
                    case MSG_RELAY:
                        if (dropCount_.load() > 0 && dropDst_.load() == h.dst) { dropCount_.fetch_sub(1); break; }
                        if (h.dst < nRanks && agents[h.dst].fd >= 0)
                            WriteMsg(agents[h.dst].fd, MSG_RELAY, r, h.dst, h.tag, pl.data(), pl.size());
                        break;
                    case MSG_HEARTBEAT:
                        heartbeatSeen = true;
                        break;
                    case MSG_ERROR:
                        for (uint32_t m = 0; m < nRanks; ++m)
                            if (m != r && agents[m].fd >= 0) WriteMsg(agents[m].fd, MSG_ERROR, r, m, h.tag, nullptr, 0);
                        break;
                    case MSG_BYE:
                        a.bye = true;
                        net::Close(a.fd);
                        a.alive = false;
                        break;
                    default:
                        break;
                }
            }
        }
        if (heartbeatSeen) {
            uint64_t mask = lostMask;
            for (uint32_t r = 0; r < nRanks; ++r)
                if (agents[r].alive && now - agents[r].lastSeen > lostMs) mask |= (1ull << (r & 63));
            if (mask != lostMask || now - lastHbBroadcast > 1000) { lostMask = mask; broadcastHb(); }
        }
    }
    for (auto &a : agents) net::Close(a.fd);
    status_.store(1);
}

// ---------------------------------------------------------------------------------------- agent

Bootstrap::Bootstrap() {}
Bootstrap::~Bootstrap() { Close(); }

HcclResult Bootstrap::SendMsg(uint16_t type, uint32_t dst, uint64_t tag, const void *data, size_t len)
{
    std::lock_guard<std::mutex> lk(sendMu_);
    if (sock_ < 0) return HCCL_E_NETWORK;
    return WriteMsg(sock_, type, rank_, dst, tag, data, len);
}

HcclResult Bootstrap::Connect(const RootHandle &root, uint32_t rank, uint32_t nRanks, const Blob &info,
                              std::vector<Blob> *table)
{
    if (root.magic != kRootHandleMagic) {
        RPT_ERR("EI0003", "root info was not produced by HcclGetRootInfo (bad magic)");
        return HCCL_E_PARA;
    }
    const EnvConfig &env = EnvConfig::Get();
    rank_ = rank;
    nRanks_ = nRanks;
    identifier_ = root.identifier;
    timeoutMs_ = env.connectTimeoutSec.value * 1000;
    int64_t deadline = net::NowMs() + timeoutMs_;
    HcclResult r = net::TcpConnect(root.ip, (int)root.port, deadline, &sock_);
    if (r != HCCL_SUCCESS) {
        RPT_ERR("EI0006", "rank %u cannot reach the rendezvous server %s:%u within %d s", rank, root.ip, root.port,
                env.connectTimeoutSec.value);
        return r == HCCL_E_TCP_CONNECT ? HCCL_E_TIMEOUT : r;
    }
    // Unix socket for descriptor passing must exist before anyone learns we joined.
    r = net::UdsListen("hccl-" + identifier_ + "-" + std::to_string(rank), &udsFd_);
    if (r != HCCL_SUCCESS) return r;

    Blob hello;
    Put32(hello, nRanks);
    Put32(hello, rank);
    std::string agentId = std::string(root.identifier) + "/" + std::to_string(rank);
    PutBlob(hello, Blob(agentId.begin(), agentId.end()));
    PutBlob(hello, info);
    r = SendMsg(MSG_HELLO, 0, 0, hello.data(), hello.size());
    if (r != HCCL_SUCCESS) return r;

    MsgHdr h;
    Blob pl;
    r = ReadMsg(sock_, &h, &pl, deadline + 2000);
    if (r != HCCL_SUCCESS) {
        RPT_ERR("EI0015", "rank %u: no rank table from the rendezvous server (%s)", rank, HcclResult(r) == HCCL_E_TIMEOUT ? "timeout" : "connection lost");
        return r == HCCL_E_TCP_TRANSFER ? HCCL_E_TIMEOUT : r;
    }
    if (h.type == MSG_REJECT) return (HcclResult)h.tag;
    if (h.type != MSG_TABLE) return HCCL_E_INTERNAL;
    Reader rd(pl);
    uint32_t step = rd.u32(), n = rd.u32();
    if (step != 1 || n != nRanks) return HCCL_E_INTERNAL;
    table->clear();
    for (uint32_t i = 0; i < n; ++i) table->push_back(rd.blob());
    if (!rd.ok) return HCCL_E_INTERNAL;
    ages_.assign(nRanks, 0);

    reader_ = std::thread([this] { ReaderLoop(); });
    fdAcceptor_ = std::thread([this] { FdAcceptLoop(); });
    if (env.heartbeatMs.value > 0) StartHeartbeat(env.heartbeatMs.value);
    return HCCL_SUCCESS;
}

void Bootstrap::Close()
{
    if (closing_.exchange(true)) return;
    const bool monitored = heart_.joinable();
    StopHeartbeat();
    if (monitored && nRanks_ >= 2 && nRanks_ <= 64) {
        // Leave the ring: every rank still there skips this one from now on instead of finding its socket closed.
        // Everyone is told, not only the neighbours, because two neighbours that leave at the same moment would
        // otherwise each tell only the other.  One connection attempt per rank: a rank that is gone costs nothing.
        const uint64_t skip = LostMask() | ringLeft_.load();
        for (uint32_t r = 0; r < nRanks_; ++r)
            if (r != rank_ && !((skip >> r) & 1)) RingSend(r, kRingBye, 0);
    }
    if (sock_ >= 0) {
        {
            std::lock_guard<std::mutex> lk(sendMu_);
            WriteMsg(sock_, MSG_BYE, rank_, 0, 0, nullptr, 0);
            ::shutdown(sock_, SHUT_RDWR);
        }
    }
    if (reader_.joinable()) reader_.join();
    if (fdAcceptor_.joinable()) fdAcceptor_.join();
    {
        std::lock_guard<std::mutex> lk(sendMu_);
        net::Close(sock_);
    }
    net::Close(udsFd_);
    std::lock_guard<std::mutex> lk(mu_);
    for (auto &kv : fdInbox_)
        for (int fd : kv.second) ::close(fd);
    fdInbox_.clear();
}

void Bootstrap::ReaderLoop()
{
    while (!closing_.load()) {
        // Wait for the first byte with a short timeout (to notice closing_), then read the whole message with a long one:
        // a deadline that expires between the header and the payload would drop the header and leave the stream out of
        // step - the rest of that message would be taken for the next header, and a reply would never be delivered.
        struct pollfd pf = {sock_, POLLIN, 0};
        int pr = poll(&pf, 1, 200);
        if (pr == 0 || (pr < 0 && errno == EINTR)) continue;
        MsgHdr h;
        Blob pl;
        HcclResult r = ReadMsg(sock_, &h, &pl, net::NowMs() + 30000);
        if (r != HCCL_SUCCESS) {
            if (!closing_.load()) {
                hubGone_.store(true);
                cv_.notify_all();
            }
            return;
        }
        switch (h.type) {
            case MSG_GATHER_REPLY: {
                Reader rd(pl);
                uint32_t n = rd.u32();
                std::vector<Blob> parts;
                for (uint32_t i = 0; i < n; ++i) parts.push_back(rd.blob());
                std::lock_guard<std::mutex> lk(mu_);
                gatherDone_[h.tag] = std::move(parts);
                cv_.notify_all();
                break;
            }
            case MSG_RELAY: {
                std::lock_guard<std::mutex> lk(mu_);
                inbox_[Key{h.src, h.tag}].push_back(std::move(pl));
                cv_.notify_all();
                break;
            }
            case MSG_HB_STATE: {
                Reader rd(pl);
                uint64_t mask = rd.u64();
                uint32_t n = rd.u32();
                std::lock_guard<std::mutex> lk(hbMu_);
                ages_.resize(n);
                for (uint32_t i = 0; i < n; ++i) ages_[i] = rd.u64();
                lostMask_.store(mask);
                break;
            }
            case MSG_ERROR:
                remoteError_.store((int)h.tag);
                HCCL_WARNING("rank %u reported asynchronous error %d", h.src, (int)h.tag);
                break;
            default:
                break;
        }
    }
}

void Bootstrap::FdAcceptLoop()
{
    while (!closing_.load()) {
        struct pollfd pf = {udsFd_, POLLIN, 0};
        int r = poll(&pf, 1, 100);
        if (r <= 0) continue;
        int c = accept(udsFd_, nullptr, nullptr);
        if (c < 0) continue;
        struct { uint32_t src; uint32_t pad; uint64_t tag; } meta;
        int fd = -1;
        // the sender writes its header right after connecting: a connection that stays silent is dropped soon, because
        // descriptors, pings and direct messages of the other ranks queue behind it
        if (net::UdsRecvFd(c, &meta, sizeof(meta), &fd, net::NowMs() + 2000) == HCCL_SUCCESS) {
            if (fd < 0 && meta.pad == kDirectBytes) {
                // bytes for this rank: the length rides in the tag, the payload follows on the same connection
                Blob data(meta.tag <= kMaxDirectBytes ? (size_t)meta.tag : 0);
                if (meta.tag <= kMaxDirectBytes && (data.empty() || net::RecvAll(c, data.data(), data.size(), net::NowMs() + 5000) == HCCL_SUCCESS)) {
                    std::lock_guard<std::mutex> lk(mu_);
                    directInbox_[meta.src].push_back(std::move(data));
                    cv_.notify_all();
                }
            } else if (fd < 0) {
                RingHeard(meta.src, meta.pad, meta.tag);      // no descriptor: a message of the ring monitor
            } else {
                std::lock_guard<std::mutex> lk(mu_);
                fdInbox_[Key{meta.src, meta.tag}].push_back(fd);
                cv_.notify_all();
            }
        }
        ::close(c);
    }
}

Bootstrap::Group Bootstrap::WorldGroup() const
{
    Group g;
    g.id = 0;
    g.ranks.resize(nRanks_);
    for (uint32_t i = 0; i < nRanks_; ++i) g.ranks[i] = i;
    g.myIndex = rank_;
    return g;
}

Bootstrap::Group Bootstrap::MakeGroup(uint32_t id, const std::vector<uint32_t> &ranks) const
{
    Group g;
    g.id = id;
    g.ranks = ranks;
    g.myIndex = ~0u;
    for (uint32_t i = 0; i < ranks.size(); ++i)
        if (ranks[i] == rank_) g.myIndex = i;
    return g;
}

HcclResult Bootstrap::AllGather(Group &g, const Blob &mine, std::vector<Blob> *all, int timeoutMs)
{
    if (g.myIndex == ~0u) return HCCL_E_PARA;
    uint64_t tag = ((uint64_t)g.id << 32) | (uint64_t)(g.seq++);
    Blob msg;
    Put32(msg, (uint32_t)g.ranks.size());
    Put32(msg, g.myIndex);
    PutBlob(msg, mine);
    HcclResult r = SendMsg(MSG_GATHER, 0, tag, msg.data(), msg.size());
    if (r != HCCL_SUCCESS) return r;
    if (timeoutMs < 0) timeoutMs = timeoutMs_;
    std::unique_lock<std::mutex> lk(mu_);
    bool ok = cv_.wait_for(lk, std::chrono::milliseconds(timeoutMs), [&] { return gatherDone_.count(tag) || hubGone_.load(); });
    if (!ok || !gatherDone_.count(tag)) {
        HCCL_ERROR("rank %u: control-plane gather (group %u, seq %u) did not complete: %s", rank_, g.id, g.seq - 1,
                   hubGone_.load() ? "rendezvous server is gone" : "timeout");
        return hubGone_.load() ? HCCL_E_NETWORK : HCCL_E_TIMEOUT;
    }
    if (all) *all = std::move(gatherDone_[tag]);
    gatherDone_.erase(tag);
    return HCCL_SUCCESS;
}

HcclResult Bootstrap::Barrier(Group &g, int timeoutMs) { return AllGather(g, Blob(), nullptr, timeoutMs); }

HcclResult Bootstrap::BarrierArrive(Group &g, uint64_t *ticket)
{
    if (g.myIndex == ~0u || !ticket) return HCCL_E_PARA;
    *ticket = ((uint64_t)g.id << 32) | (uint64_t)(g.seq++);
    Blob msg;
    Put32(msg, (uint32_t)g.ranks.size());
    Put32(msg, g.myIndex);
    PutBlob(msg, Blob());
    return SendMsg(MSG_GATHER, 0, *ticket, msg.data(), msg.size());
}

HcclResult Bootstrap::BarrierWait(uint64_t ticket, int timeoutMs, bool quiet)
{
    if (timeoutMs < 0) timeoutMs = timeoutMs_;
    std::unique_lock<std::mutex> lk(mu_);
    cv_.wait_for(lk, std::chrono::milliseconds(timeoutMs), [&] { return gatherDone_.count(ticket) || hubGone_.load(); });
    if (gatherDone_.count(ticket)) {
        gatherDone_.erase(ticket);
        return HCCL_SUCCESS;
    }
    if (!quiet)
        HCCL_ERROR("rank %u: control-plane barrier (group %u, seq %u) did not complete: %s", rank_, (uint32_t)(ticket >> 32), (uint32_t)ticket,
                   hubGone_.load() ? "rendezvous server is gone" : "timeout");
    return hubGone_.load() ? HCCL_E_NETWORK : HCCL_E_TIMEOUT;
}

HcclResult Bootstrap::Broadcast(Group &g, uint32_t rootIndex, Blob *data, int timeoutMs)
{
    std::vector<Blob> all;
    HcclResult r = AllGather(g, g.myIndex == rootIndex ? *data : Blob(), &all, timeoutMs);
    if (r != HCCL_SUCCESS) return r;
    if (rootIndex >= all.size()) return HCCL_E_PARA;
    *data = all[rootIndex];
    return HCCL_SUCCESS;
}

HcclResult Bootstrap::Send(uint32_t dstRank, uint64_t tag, const Blob &data)
{
    return SendMsg(MSG_RELAY, dstRank, tag, data.data(), data.size());
}

HcclResult Bootstrap::Recv(uint32_t srcRank, uint64_t tag, Blob *data, int timeoutMs)
{
    if (timeoutMs < 0) timeoutMs = timeoutMs_;
    Key k{srcRank, tag};
    std::unique_lock<std::mutex> lk(mu_);
    bool ok = cv_.wait_for(lk, std::chrono::milliseconds(timeoutMs),
                           [&] { auto it = inbox_.find(k); return (it != inbox_.end() && !it->second.empty()) || hubGone_.load(); });
    auto it = inbox_.find(k);
    if (!ok || it == inbox_.end() || it->second.empty()) return hubGone_.load() ? HCCL_E_NETWORK : HCCL_E_TIMEOUT;
    *data = std::move(it->second.front());
    it->second.pop_front();
    if (it->second.empty()) inbox_.erase(it);
    return HCCL_SUCCESS;
}

HcclResult Bootstrap::TryRecv(uint32_t srcRank, uint64_t want, uint64_t mask, Blob *data, uint32_t *fromRank, uint64_t *fromTag)
{
    std::lock_guard<std::mutex> lk(mu_);
    for (auto it = inbox_.begin(); it != inbox_.end(); ++it) {
        if (it->second.empty()) continue;
        if (srcRank != ~0u && it->first.src != srcRank) continue;
        if ((it->first.tag & mask) != (want & mask)) continue;
        if (data) *data = std::move(it->second.front());
        if (fromRank) *fromRank = it->first.src;
        if (fromTag) *fromTag = it->first.tag;
        it->second.pop_front();
        if (it->second.empty()) inbox_.erase(it);
        return HCCL_SUCCESS;
    }
    return hubGone_.load() ? HCCL_E_NETWORK : HCCL_E_AGAIN;
}

HcclResult Bootstrap::SendDirect(uint32_t dstRank, const Blob &data)
{
    if (data.size() > kMaxDirectBytes) return HCCL_E_PARA;
    int c = -1;
    HcclResult r = net::UdsConnect("hccl-" + identifier_ + "-" + std::to_string(dstRank), net::NowMs() + 2000, &c);
    if (r != HCCL_SUCCESS) return r;
    struct { uint32_t src; uint32_t pad; uint64_t tag; } meta{rank_, kDirectBytes, (uint64_t)data.size()};
    r = net::SendAll(c, &meta, sizeof(meta));
    if (r == HCCL_SUCCESS && !data.empty()) r = net::SendAll(c, data.data(), data.size());
    ::close(c);
    return r;
}

HcclResult Bootstrap::RecvDirect(uint32_t srcRank, Blob *data, int timeoutMs)
{
    std::unique_lock<std::mutex> lk(mu_);
    bool ok = cv_.wait_for(lk, std::chrono::milliseconds(timeoutMs), [&] { auto it = directInbox_.find(srcRank); return it != directInbox_.end() && !it->second.empty(); });
    if (!ok) return HCCL_E_TIMEOUT;
    auto it = directInbox_.find(srcRank);
    *data = std::move(it->second.front());
    it->second.pop_front();
    return HCCL_SUCCESS;
}

HcclResult Bootstrap::SendFd(uint32_t dstRank, uint64_t tag, int fd)
{
    int c = -1;
    HcclResult r = net::UdsConnect("hccl-" + identifier_ + "-" + std::to_string(dstRank), net::NowMs() + timeoutMs_, &c);
    if (r != HCCL_SUCCESS) return r;
    struct { uint32_t src; uint32_t pad; uint64_t tag; } meta{rank_, 0, tag};
    r = net::UdsSendFd(c, &meta, sizeof(meta), fd);
    ::close(c);
    return r;
}

HcclResult Bootstrap::RecvFd(uint32_t srcRank, uint64_t tag, int *fd, int timeoutMs)
{
    if (timeoutMs < 0) timeoutMs = timeoutMs_;
    Key k{srcRank, tag};
    std::unique_lock<std::mutex> lk(mu_);
    bool ok = cv_.wait_for(lk, std::chrono::milliseconds(timeoutMs),
                           [&] { auto it = fdInbox_.find(k); return it != fdInbox_.end() && !it->second.empty(); });
    if (!ok) return HCCL_E_TIMEOUT;
    auto it = fdInbox_.find(k);
    *fd = it->second.front();
    it->second.pop_front();
    if (it->second.empty()) fdInbox_.erase(it);
    return HCCL_SUCCESS;
}

// ---- ring monitor

// Nearest rank in direction dir (+1 / -1) that is neither lost nor gone; -1 if there is none.
int Bootstrap::RingNeighbour(int dir) const
{
    const uint64_t skip = LostMask() | ringLeft_.load();
    for (uint32_t k = 1; k < nRanks_; ++k) {
        const uint32_t r = (rank_ + nRanks_ + (dir > 0 ? k : nRanks_ - k)) % nRanks_;
        if (r == rank_) break;
        if (nRanks_ <= 64 && (skip >> r) & 1) continue;
        return (int)r;
    }
    return -1;
}

bool Bootstrap::RingSend(uint32_t dst, uint32_t kind, int deadlineMs)
{
    int c = -1;
    if (net::UdsConnect("hccl-" + identifier_ + "-" + std::to_string(dst), net::NowMs() + deadlineMs, &c) != HCCL_SUCCESS) return false;
    struct { uint32_t src; uint32_t pad; uint64_t tag; } meta{rank_, kind, LostMask()};
    ssize_t n;
    do { n = send(c, &meta, sizeof(meta), MSG_NOSIGNAL); } while (n < 0 && errno == EINTR);
    ::close(c);
    return n == (ssize_t)sizeof(meta);
}

void Bootstrap::RingHeard(uint32_t src, uint32_t kind, uint64_t lostSeen)
{
    if (src >= nRanks_ || nRanks_ > 64) return;
    if (kind == kRingBye) { ringLeft_.fetch_or(1ull << src); return; }
    if (kind != kRingPing) return;
    {
        std::lock_guard<std::mutex> lk(hbMu_);
        if (src < ringHeardMs_.size()) ringHeardMs_[src] = net::NowMs();
    }
    // what the sender knows travels on; nobody talks this rank, or the sender itself, into being lost
    ringLost_.fetch_or(lostSeen & ~(1ull << rank_) & ~(1ull << src));
}

void Bootstrap::RingTick(int lostAfterMs)
{
    if (nRanks_ < 2 || nRanks_ > 64) return;
    const int64_t now = net::NowMs();
    int done = -1;
    for (int dir : {+1, -1}) {
        const int nb = RingNeighbour(dir);
        if (nb < 0 || nb == done) continue;         // two ranks: both directions meet the same neighbour
        done = nb;
        if (RingSend((uint32_t)nb, kRingPing, 100)) {
            ringRefused_[nb] = 0;
        } else if (++ringRefused_[nb] >= 2) {
            // nobody listens on the neighbour's socket any more: its process is gone
            ringLost_.fetch_or(1ull << nb);
            HCCL_WARNING("ring monitor: rank %d does not accept connections, marked LOST by rank %u", nb, rank_);
            continue;
        }
        int64_t heard;
        {
            std::lock_guard<std::mutex> lk(hbMu_);
            heard = ringHeardMs_[nb];
        }
        if (now - heard > lostAfterMs) {
            ringLost_.fetch_or(1ull << nb);
            HCCL_WARNING("ring monitor: rank %d silent for %lld ms, marked LOST by rank %u", nb, (long long)(now - heard), rank_);
        }
    }
}

void Bootstrap::StartHeartbeat(int intervalMs)
{
    if (heart_.joinable()) return;
    heartStop_.store(false);
    {
        std::lock_guard<std::mutex> lk(hbMu_);
        ringHeardMs_.assign(nRanks_, net::NowMs());        // silence counts from now
    }
    ringRefused_.assign(nRanks_, 0);
    const int lostAfterMs = EnvConfig::Get().heartbeatLostMs.value;
    heart_ = std::thread([this, intervalMs, lostAfterMs] {
        while (!heartStop_.load() && !closing_.load()) {
            if (!hubGone_.load()) SendMsg(MSG_HEARTBEAT, 0, 0, nullptr, 0);
            RingTick(lostAfterMs);
            for (int waited = 0; waited < intervalMs && !heartStop_.load(); waited += 10) usleep(10000);
        }
    });
}

void Bootstrap::StopHeartbeat()
{
    heartStop_.store(true);
    if (heart_.joinable()) heart_.join();
}

void Bootstrap::HeartbeatAges(std::vector<uint64_t> *ages) const
{
    std::lock_guard<std::mutex> lk(hbMu_);
    *ages = ages_;
}

HcclResult Bootstrap::NotifyError(HcclResult code) { return SendMsg(MSG_ERROR, 0, (uint64_t)code, nullptr, 0); }

}  // namespace hc
