// msg_api.cc - host-side tagged messages with matched probe (include/hccl/hccl_msg.h): between ranks of a communicator
// over its control plane, and between two endpoints connected like sockets.
// Reference: the hccd flow, src/legacy/ascend910/hccd/hccd.cc:300-420 (HcclIsend / Improbe / Imrecv / GetCount / TestSome
// on a communicator) and its raw-connection twin declared in pkg_inc/legacy/hccl/hccl_ex.h:82-190.
//
// A send copies the payload and is complete when the call returns, so its request only carries the status.  A probe takes
// the matching message out of the queue and hands it to the caller as an HcclMessage; the receive that follows copies it
// into the caller's buffer (MPI's matched probe: no other receive can steal it in between).
#include <arpa/inet.h>
#include <poll.h>
#include <unistd.h>

#include <cstdio>
#include <cstring>
#include <fstream>
#include <mutex>
#include <set>
#include <string>
#include <vector>

#include "../comm/comm.h"
#include "../core/dtype.h"
#include "../core/env.h"
#include "../core/log.h"
#include "../core/net.h"
#include "hccl/hccl_comm.h"
#include "hccl/hccl_msg.h"
#include "hccl/hccl_res.h"

using namespace hc;

namespace {

constexpr uint32_t kReqMagic = 0x51455248;   // "HREQ"
constexpr uint32_t kMsgMagic = 0x47534d48;   // "HMSG"
constexpr uint32_t kConnMagic = 0x4e4e4f43;  // "CONN"
constexpr uint32_t kFrameMagic = 0x4d415246; // "FRAM"
constexpr int kMaxMessageBytes = 64 << 20;

struct Request {
    uint32_t magic = kReqMagic;
    HcclStatus status{};
};
struct Message {
    uint32_t magic = kMsgMagic;
    HcclStatus status{};
    Blob data;
};
struct Conn {
    uint32_t magic = kConnMagic;
    int fd = -1, listenFd = -1;
    std::string bindIp = "0.0.0.0";
    int bindPort = 0;
    std::mutex mu;
};

Request *AsRequest(HcclRequest r) { Request *q = (Request *)r; return q && q->magic == kReqMagic ? q : nullptr; }
Message *AsMessage(HcclMessage m) { Message *q = (Message *)m; return q && q->magic == kMsgMagic ? q : nullptr; }
Conn *AsConn(HcclConn c) { Conn *q = (Conn *)c; return q && q->magic == kConnMagic ? q : nullptr; }

// Relay tags of the message calls: a space of their own, the communicator's group and the caller's tag.
constexpr uint64_t kTagSpace = 0x4dull << 56;
uint64_t RelayTag(const Comm *c, int tag) { return kTagSpace | ((uint64_t)(c->group.id & 0xffffffu) << 32) | (uint32_t)tag; }

int CheckPayload(int count, HcclDataType dt, uint64_t *bytes)
{
    if (count < 0) return HCCL_E_PARA;
    const uint32_t esz = DtypeSize(dt);
    if (esz == 0) return HCCL_E_NOT_SUPPORT;
    *bytes = (uint64_t)count * esz;
    return *bytes > (uint64_t)kMaxMessageBytes ? HCCL_E_PARA : HCCL_SUCCESS;
}

// Copies the probed payload into the caller's buffer(s) and turns the message into a completed request.
HcclResult Deliver(Message *m, void *const bufs[], const uint64_t sizes[], int n, HcclRequest *request)
{
    uint64_t room = 0;
    for (int i = 0; i < n; ++i) room += sizes[i];
    if (room < m->data.size()) {
        RPT_ERR("EI0003", "a message of %zu bytes does not fit the %llu bytes offered", m->data.size(), (unsigned long long)room);
        return HCCL_E_MEMORY;        // the message stays with the caller, who may offer a larger buffer
    }
    uint64_t off = 0;
    for (int i = 0; i < n && off < m->data.size(); ++i) {
        const uint64_t k = std::min<uint64_t>(sizes[i], m->data.size() - off);
        if (k) memcpy(bufs[i], m->data.data() + off, k);
        off += k;
    }
    Request *q = new Request();
    q->status = m->status;
    *request = q;
    m->magic = 0;
    delete m;
    return HCCL_SUCCESS;
}

int TestSome(int count, HcclRequest requestArray[], int *compCount, int compIndices[], HcclStatus compStatus[])
{
    if (count < 0 || (count && !requestArray) || !compCount) return HCCL_E_PTR;
    int done = 0;
    for (int i = 0; i < count; ++i) {
        if (!requestArray[i]) continue;                        // reported earlier
        Request *q = AsRequest(requestArray[i]);
        if (!q) return HCCL_E_PARA;
        if (compIndices) compIndices[done] = i;
        if (compStatus) compStatus[done] = q->status;
        ++done;
        q->magic = 0;
        delete q;
        requestArray[i] = nullptr;
    }
    *compCount = done;
    return HCCL_SUCCESS;
}

int GetCount(const HcclStatus *status, HcclDataType dt, int *count)
{
    if (!status || !count) return HCCL_E_PTR;
    const uint32_t esz = DtypeSize(dt);
    if (esz == 0) return HCCL_E_NOT_SUPPORT;
    if (status->count % (int)esz != 0) return HCCL_E_PARA;     // the payload is not a whole number of such elements
    *count = status->count / (int)esz;
    return HCCL_SUCCESS;
}

std::mutex g_memMu;
std::set<void *> g_globalBuffers;

}  // namespace

extern "C" {

// ------------------------------------------------------------------------------ communicator from a table in memory

HcclResult HcclInitComm(const char *rankTableM, uint32_t rank, const CommAttr *attr, HcclComm *comm)
{
    CHK_PTR_NULL(rankTableM); CHK_PTR_NULL(comm);
    if (attr && (attr->mode < HCCL_MODE_NORMAL || attr->mode > HCCL_MODE_SCHED_OS)) return HCCL_E_PARA;
    // the table loader reads files: the text goes through a private temporary one
    char path[] = "/tmp/hccl_table_XXXXXX";
    int fd = mkstemp(path);
    if (fd < 0) return HCCL_E_OPEN_FILE_FAILURE;
    const size_t len = strlen(rankTableM);
    const bool written = write(fd, rankTableM, len) == (ssize_t)len;
    close(fd);
    HcclResult r = written ? HcclCommInitClusterInfo(path, rank, comm) : HCCL_E_OPEN_FILE_FAILURE;
    unlink(path);
    return r;
}

HcclResult HcclFinalizeComm(HcclComm comm) { return HcclCommDestroy(comm); }

HcclResult HcclRegisterGlobalMemory(void *addr, uint64_t size)
{
    CHK_PTR_NULL(addr);
    if (size == 0) return HCCL_E_PARA;
    std::lock_guard<std::mutex> lk(g_memMu);
    return g_globalBuffers.insert(addr).second ? HCCL_SUCCESS : HCCL_E_PARA;
}
HcclResult HcclUnregisterGlobalMemory(void *addr)
{
    CHK_PTR_NULL(addr);
    std::lock_guard<std::mutex> lk(g_memMu);
    return g_globalBuffers.erase(addr) ? HCCL_SUCCESS : HCCL_E_NOT_FOUND;
}
HcclResult HcclRegisterMemory(HcclComm comm, void *buffer, uint64_t size)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(buffer);
    if (size == 0) return HCCL_E_PARA;
    CommMem m{COMM_MEM_TYPE_HOST, buffer, size};
    HcclMemHandle h;
    char tag[64];
    snprintf(tag, sizeof(tag), "msg:%p", buffer);
    return HcclCommMemReg(comm, tag, &m, &h);
}
HcclResult HcclUnregisterMemory(HcclComm comm, void *buffer)
{
    Comm *c = AsComm(comm);
    CHK_PTR_NULL(c); CHK_PTR_NULL(buffer);
    char tag[64];
    snprintf(tag, sizeof(tag), "msg:%p", buffer);
    std::lock_guard<std::mutex> lk(c->resMu);
    for (auto it = c->regMems.begin(); it != c->regMems.end(); ++it)
        if ((*it)->tag == tag) { c->regMems.erase(it); return HCCL_SUCCESS; }
    return HCCL_E_NOT_FOUND;
}

// --------------------------------------------------------------------------------- messages between ranks

int HcclIsend(void *buffer, int count, HcclDataType dataType, int dstRank, int tag, HcclComm comm, HcclRequest *request)
{
    Comm *c = AsComm(comm);
    if (!c || !request || (count > 0 && !buffer)) return HCCL_E_PTR;
    if (dstRank < 0 || (uint32_t)dstRank >= c->nRanks || tag < 0) { RPT_ERR("EI0003", "HcclIsend: destination %d or tag %d out of range", dstRank, tag); return HCCL_E_PARA; }
    uint64_t bytes = 0;
    int rc = CheckPayload(count, dataType, &bytes);
    if (rc) return rc;
    Blob data(bytes);
    if (bytes) CHK_RET(c->plat->MemcpySync(data.data(), buffer, bytes));       // the buffer may be device memory
    if ((uint32_t)dstRank == c->rank) return HCCL_E_NOT_SUPPORT;               // the control plane has no loop-back
    CHK_RET(c->boot->Send(c->worldRanks[dstRank], RelayTag(c, tag), data));
    Request *q = new Request();
    q->status.srcRank = (int)c->rank; q->status.tag = tag; q->status.count = (int)bytes;
    *request = q;
    return HCCL_SUCCESS;
}

int HcclImprobe(int srcRank, int tag, HcclComm comm, int *flag, HcclMessage *msg, HcclStatus *status)
{
    Comm *c = AsComm(comm);
    if (!c || !flag || !msg || !status) return HCCL_E_PTR;
    if ((srcRank != HCCL_ANY_SOURCE && (srcRank < 0 || (uint32_t)srcRank >= c->nRanks)) || (tag != HCCL_ANY_TAG && tag < 0)) return HCCL_E_PARA;
    *flag = 0;
    *msg = nullptr;
    const uint64_t want = RelayTag(c, tag == HCCL_ANY_TAG ? 0 : tag);
    const uint64_t mask = tag == HCCL_ANY_TAG ? ~0xffffffffull : ~0ull;
    Blob data;
    uint32_t fromWorld = 0;
    uint64_t fromTag = 0;
    HcclResult r = HCCL_E_AGAIN;
    if (srcRank != HCCL_ANY_SOURCE) {
        r = c->boot->TryRecv(c->worldRanks[srcRank], want, mask, &data, &fromWorld, &fromTag);
    } else {
        // any member of this communicator (the control plane may carry other groups' ranks as well)
        for (uint32_t q = 0; q < c->nRanks && r == HCCL_E_AGAIN; ++q)
            if (q != c->rank) r = c->boot->TryRecv(c->worldRanks[q], want, mask, &data, &fromWorld, &fromTag);
    }
    if (r == HCCL_E_AGAIN) return HCCL_SUCCESS;                                 // nothing there yet
    if (r != HCCL_SUCCESS) return r;
    Message *m = new Message();
    m->data = std::move(data);
    for (uint32_t q = 0; q < c->nRanks; ++q)
        if (c->worldRanks[q] == fromWorld) m->status.srcRank = (int)q;
    m->status.tag = (int)(uint32_t)fromTag;
    m->status.count = (int)m->data.size();
    *status = m->status;
    *msg = m;
    *flag = 1;
    return HCCL_SUCCESS;
}

int HcclImrecv(void *buffer, int count, HcclDataType dataType, HcclMessage *msg, HcclRequest *request)
{
    if (!msg || !request) return HCCL_E_PTR;
    Message *m = AsMessage(*msg);
    if (!m) return HCCL_E_PARA;
    uint64_t bytes = 0;
    int rc = CheckPayload(count, dataType, &bytes);
    if (rc) return rc;
    if (bytes && !buffer) return HCCL_E_PTR;
    void *bufs[1] = {buffer};
    HcclResult r = Deliver(m, bufs, &bytes, 1, request);
    if (r == HCCL_SUCCESS) *msg = nullptr;
    return r;
}

int HcclGetCount(const HcclStatus *status, HcclDataType dataType, int *count) { return GetCount(status, dataType, count); }

int HcclTestSome(int count, HcclRequest requestArray[], int *compCount, int compIndices[], HcclStatus compStatus[])
{
    return TestSome(count, requestArray, compCount, compIndices, compStatus);
}

// ------------------------------------------------------------------------------- the same over a connection

HcclResult HcclRawOpen(HcclConn *conn)
{
    CHK_PTR_NULL(conn);
    *conn = new Conn();
    return HCCL_SUCCESS;
}

HcclResult HcclRawForceClose(HcclConn conn)
{
    Conn *c = AsConn(conn);
    CHK_PTR_NULL(c);
    net::Close(c->fd);
    net::Close(c->listenFd);
    c->magic = 0;
    delete c;
    return HCCL_SUCCESS;
}
HcclResult HcclRawClose(HcclConn conn) { return HcclRawForceClose(conn); }    // sends are complete when they return: nothing to drain

HcclResult HcclRawBind(HcclConn conn, HcclAddr *bindAddr)
{
    Conn *c = AsConn(conn);
    CHK_PTR_NULL(c); CHK_PTR_NULL(bindAddr);
    if (bindAddr->type != HCCL_ADDR_TYPE_ROCE) return HCCL_E_NOT_SUPPORT;
    if (c->listenFd >= 0 || c->fd >= 0) return HCCL_E_PARA;
    char ip[INET_ADDRSTRLEN] = "0.0.0.0";
    if (bindAddr->info.tcp.ipv4Addr) inet_ntop(AF_INET, &bindAddr->info.tcp.ipv4Addr, ip, sizeof(ip));
    // bind and listen are one step underneath: the port is taken now so that it can be written back
    int port = 0;
    CHK_RET(net::TcpListen(ip, bindAddr->info.tcp.port, bindAddr->info.tcp.port, &c->listenFd, &port));
    c->bindIp = ip;
    c->bindPort = port;
    bindAddr->info.tcp.port = (uint16_t)port;
    return HCCL_SUCCESS;
}

HcclResult HcclRawListen(HcclConn conn, int backLog)
{
    Conn *c = AsConn(conn);
    CHK_PTR_NULL(c);
    (void)backLog;
    if (c->listenFd < 0) { RPT_ERR("EI0003", "HcclRawListen on a connection that was not bound"); return HCCL_E_PARA; }
    return HCCL_SUCCESS;
}

HcclResult HcclRawAccept(HcclConn listenConn, HcclAddr *acceptAddr, HcclConn *acceptConn)
{
    Conn *l = AsConn(listenConn);
    CHK_PTR_NULL(l); CHK_PTR_NULL(acceptConn);
    if (l->listenFd < 0) return HCCL_E_PARA;
    int fd = -1;
    std::string peer;
    HcclResult r = net::TcpAccept(l->listenFd, net::NowMs() + (int64_t)EnvConfig::Get().connectTimeoutSec.value * 1000, &fd, &peer);
    if (r != HCCL_SUCCESS) return r;
    Conn *c = new Conn();
    c->fd = fd;
    if (acceptAddr) {
        memset(acceptAddr, 0, sizeof(*acceptAddr));
        acceptAddr->type = HCCL_ADDR_TYPE_ROCE;
        inet_pton(AF_INET, peer.c_str(), &acceptAddr->info.tcp.ipv4Addr);
    }
    *acceptConn = c;
    return HCCL_SUCCESS;
}

HcclResult HcclRawConnect(HcclConn conn, HcclAddr *connectAddr)
{
    Conn *c = AsConn(conn);
    CHK_PTR_NULL(c); CHK_PTR_NULL(connectAddr);
    if (connectAddr->type != HCCL_ADDR_TYPE_ROCE) return HCCL_E_NOT_SUPPORT;
    if (c->fd >= 0 || c->listenFd >= 0) return HCCL_E_PARA;
    char ip[INET_ADDRSTRLEN] = "127.0.0.1";
    if (connectAddr->info.tcp.ipv4Addr) inet_ntop(AF_INET, &connectAddr->info.tcp.ipv4Addr, ip, sizeof(ip));
    return net::TcpConnect(ip, connectAddr->info.tcp.port, net::NowMs() + (int64_t)EnvConfig::Get().connectTimeoutSec.value * 1000, &c->fd);
}

HcclResult HcclRawIsend(const void *buf, int count, HcclDataType dataType, HcclConn conn, HcclRequest *request)
{
    Conn *c = AsConn(conn);
    CHK_PTR_NULL(c); CHK_PTR_NULL(request);
    if (c->fd < 0) return HCCL_E_PARA;
    uint64_t bytes = 0;
    int rc = CheckPayload(count, dataType, &bytes);
    if (rc) return (HcclResult)rc;
    if (bytes && !buf) return HCCL_E_PTR;
    uint32_t hdr[2] = {kFrameMagic, (uint32_t)bytes};
    std::lock_guard<std::mutex> lk(c->mu);
    CHK_RET(net::SendAll(c->fd, hdr, sizeof(hdr)));
    if (bytes) CHK_RET(net::SendAll(c->fd, buf, bytes));
    Request *q = new Request();
    q->status.count = (int)bytes;
    *request = q;
    return HCCL_SUCCESS;
}

HcclResult HcclRawImprobe(HcclConn conn, int *flag, HcclMessage *msg, HcclStatus *status)
{
    Conn *c = AsConn(conn);
    CHK_PTR_NULL(c); CHK_PTR_NULL(flag); CHK_PTR_NULL(msg); CHK_PTR_NULL(status);
    if (c->fd < 0) return HCCL_E_PARA;
    *flag = 0;
    *msg = nullptr;
    std::lock_guard<std::mutex> lk(c->mu);
    struct pollfd p = {c->fd, POLLIN, 0};
    if (poll(&p, 1, 0) <= 0 || !(p.revents & (POLLIN | POLLHUP))) return HCCL_SUCCESS;      // nothing has arrived
    // a frame has begun: its sender writes header and payload in one go, so the rest follows at once
    uint32_t hdr[2];
    const int64_t deadline = net::NowMs() + 10000;
    HcclResult r = net::RecvAll(c->fd, hdr, sizeof(hdr), deadline);
    if (r != HCCL_SUCCESS) return r == HCCL_E_TIMEOUT ? HCCL_E_TIMEOUT : HCCL_E_TCP_TRANSFER;
    if (hdr[0] != kFrameMagic || hdr[1] > (uint32_t)kMaxMessageBytes) { RPT_ERR("EI0003", "the peer of this connection does not speak its framing"); return HCCL_E_TCP_TRANSFER; }
    Message *m = new Message();
    m->data.resize(hdr[1]);
    if (hdr[1] && net::RecvAll(c->fd, m->data.data(), hdr[1], deadline) != HCCL_SUCCESS) { delete m; return HCCL_E_TCP_TRANSFER; }
    m->status.count = (int)hdr[1];
    *status = m->status;
    *msg = m;
    *flag = 1;
    return HCCL_SUCCESS;
}

HcclResult HcclRawImrecv(void *buf, int count, HcclDataType datatype, HcclMessage *msg, HcclRequest *request)
{
    return (HcclResult)HcclImrecv(buf, count, datatype, msg, request);
}

HcclResult HcclRawImrecvScatter(void *buf[], int count[], int bufCount, HcclDataType datatype, HcclMessage *msg, HcclRequest *request)
{
    CHK_PTR_NULL(buf); CHK_PTR_NULL(count); CHK_PTR_NULL(msg); CHK_PTR_NULL(request);
    Message *m = AsMessage(*msg);
    if (!m || bufCount <= 0 || bufCount > 1024) return HCCL_E_PARA;
    std::vector<uint64_t> sizes(bufCount);
    for (int i = 0; i < bufCount; ++i) {
        int rc = CheckPayload(count[i], datatype, &sizes[i]);
        if (rc) return (HcclResult)rc;
        if (sizes[i] && !buf[i]) return HCCL_E_PTR;
    }
    HcclResult r = Deliver(m, buf, sizes.data(), bufCount, request);
    if (r == HCCL_SUCCESS) *msg = nullptr;
    return r;
}

HcclResult HcclRawGetCount(const HcclStatus *status, HcclDataType dataType, int *count) { return (HcclResult)GetCount(status, dataType, count); }

HcclResult HcclRawTestSome(int count, HcclRequest requestArray[], int *compCount, int compIndices[], HcclStatus compStatus[])
{
    return (HcclResult)TestSome(count, requestArray, compCount, compIndices, compStatus);
}

}  // extern "C"
