// net.h - blocking TCP and Unix-domain socket helpers with deadlines.
// TCP carries the control plane (rendezvous, handshakes, heartbeats); the Unix-domain side exists
// to pass file descriptors (SCM_RIGHTS) that name exported device or shared memory.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#include "hccl/hccl_types.h"

namespace hc {
namespace net {

int64_t NowMs();

// Picks the address the rendezvous server binds to: HCCL_IF_IP, else the first address of
// HCCL_SOCKET_IFNAME, else the first non-loopback IPv4 address, else 127.0.0.1.
std::string PickLocalIp();

// Listens on ip:port; port 0 = ephemeral, or the first free port of [lo,hi] when lo>0.
HcclResult TcpListen(const std::string &ip, int lo, int hi, int *fdOut, int *portOut);
// Retries until deadlineMs (absolute, NowMs clock) so that clients may start before the server.
HcclResult TcpConnect(const std::string &ip, int port, int64_t deadlineMs, int *fdOut);
// Accept with deadline; peerIp receives the dotted address.
HcclResult TcpAccept(int listenFd, int64_t deadlineMs, int *fdOut, std::string *peerIp);

HcclResult SendAll(int fd, const void *buf, size_t len);
HcclResult RecvAll(int fd, void *buf, size_t len, int64_t deadlineMs);  // deadlineMs<0: no deadline
void Close(int &fd);

// Abstract-namespace Unix sockets (no filesystem entry, vanish with the process).
HcclResult UdsListen(const std::string &name, int *fdOut);
HcclResult UdsConnect(const std::string &name, int64_t deadlineMs, int *fdOut);
HcclResult UdsSendFd(int sock, const void *meta, size_t metaLen, int fdToSend);
HcclResult UdsRecvFd(int sock, void *meta, size_t metaLen, int *fdOut, int64_t deadlineMs);

// One-IP-per-line allow list; empty file name = allow all.
class Whitelist {
public:
    HcclResult Load(const std::string &path);
    bool Allows(const std::string &ip) const;
private:
    bool enabled_ = false;
    std::vector<std::string> ips_;
};

}  // namespace net
}  // namespace hc
