#include "net.h"

#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <ifaddrs.h>
#include <net/if.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <cstring>
#include <fstream>

#include "env.h"
#include "log.h"

namespace hc {
namespace net {

int64_t NowMs()
{
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (int64_t)ts.tv_sec * 1000 + ts.tv_nsec / 1000000;
}

std::string PickLocalIp()
{
    const EnvConfig &env = EnvConfig::Get();
    if (!env.ifIp.value.empty()) return env.ifIp.value;
    std::string want = env.socketIfname.value;
    bool exclude = false;
    if (!want.empty() && want[0] == '^') { exclude = true; want = want.substr(1); }
    if (!want.empty() && want[0] == '=') want = want.substr(1);
    struct ifaddrs *ifs = nullptr;
    std::string best;
    if (getifaddrs(&ifs) == 0) {
        for (struct ifaddrs *i = ifs; i; i = i->ifa_next) {
            if (!i->ifa_addr || i->ifa_addr->sa_family != AF_INET) continue;
            if (!(i->ifa_flags & IFF_UP)) continue;
            std::string name = i->ifa_name;
            bool match = want.empty() ? !(i->ifa_flags & IFF_LOOPBACK) : (name.compare(0, want.size(), want) == 0) != exclude;
            if (!match) continue;
            char buf[INET_ADDRSTRLEN];
            inet_ntop(AF_INET, &((struct sockaddr_in *)i->ifa_addr)->sin_addr, buf, sizeof(buf));
            best = buf;
            break;
        }
        freeifaddrs(ifs);
    }
    return best.empty() ? std::string("127.0.0.1") : best;
}

static void SetCommonOpts(int fd)
{
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    int fl = fcntl(fd, F_GETFD);
    fcntl(fd, F_SETFD, fl | FD_CLOEXEC);
}

HcclResult TcpListen(const std::string &ip, int lo, int hi, int *fdOut, int *portOut)
{
    if (lo <= 0) lo = hi = 0;
    for (int port = lo; port <= hi; ++port) {
        int fd = socket(AF_INET, SOCK_STREAM, 0);
        if (fd < 0) return HCCL_E_SYSCALL;
        int one = 1;
        setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
        struct sockaddr_in sa;
        memset(&sa, 0, sizeof(sa));
        sa.sin_family = AF_INET;
        sa.sin_port = htons((uint16_t)port);
        if (inet_pton(AF_INET, ip.c_str(), &sa.sin_addr) != 1) sa.sin_addr.s_addr = htonl(INADDR_ANY);
        if (bind(fd, (struct sockaddr *)&sa, sizeof(sa)) == 0 && listen(fd, 1024) == 0) {
            socklen_t len = sizeof(sa);
            getsockname(fd, (struct sockaddr *)&sa, &len);
            SetCommonOpts(fd);
            *fdOut = fd;
            *portOut = ntohs(sa.sin_port);
            return HCCL_SUCCESS;
        }
        ::close(fd);
        if (port == 0) break;
    }
    RPT_ERR("EI0019", "no free port to listen on %s in [%d,%d]", ip.c_str(), lo, hi);
    return HCCL_E_UNAVAIL;
}

HcclResult TcpConnect(const std::string &ip, int port, int64_t deadlineMs, int *fdOut)
{
    struct sockaddr_in sa;
    memset(&sa, 0, sizeof(sa));
    sa.sin_family = AF_INET;
    sa.sin_port = htons((uint16_t)port);
    if (inet_pton(AF_INET, ip.c_str(), &sa.sin_addr) != 1) return HCCL_E_PARA;
    int backoffMs = 5;
    for (;;) {
        int fd = socket(AF_INET, SOCK_STREAM, 0);
        if (fd < 0) return HCCL_E_SYSCALL;
        if (connect(fd, (struct sockaddr *)&sa, sizeof(sa)) == 0) {
            SetCommonOpts(fd);
            *fdOut = fd;
            return HCCL_SUCCESS;
        }
        ::close(fd);
        if (NowMs() >= deadlineMs) break;
        usleep((useconds_t)backoffMs * 1000);
        if (backoffMs < 200) backoffMs *= 2;
    }
    return HCCL_E_TCP_CONNECT;
}

HcclResult TcpAccept(int listenFd, int64_t deadlineMs, int *fdOut, std::string *peerIp)
{
    for (;;) {
        int64_t left = deadlineMs - NowMs();
        if (left <= 0) return HCCL_E_TIMEOUT;
        struct pollfd p = {listenFd, POLLIN, 0};
        int r = poll(&p, 1, (int)(left > 200 ? 200 : left));
        if (r < 0 && errno != EINTR) return HCCL_E_SYSCALL;
        if (r <= 0) continue;
        if (p.revents & (POLLERR | POLLNVAL | POLLHUP)) return HCCL_E_NETWORK;
        struct sockaddr_in sa;
        socklen_t len = sizeof(sa);
        int fd = accept(listenFd, (struct sockaddr *)&sa, &len);
        if (fd < 0) {
            if (errno == EINTR || errno == EAGAIN) continue;
            return HCCL_E_SYSCALL;
        }
        SetCommonOpts(fd);
        if (peerIp) {
            char buf[INET_ADDRSTRLEN];
            inet_ntop(AF_INET, &sa.sin_addr, buf, sizeof(buf));
            *peerIp = buf;
        }
        *fdOut = fd;
        return HCCL_SUCCESS;
    }
}

HcclResult SendAll(int fd, const void *buf, size_t len)
{
    const char *p = (const char *)buf;
    while (len > 0) {
        ssize_t n = ::send(fd, p, len, MSG_NOSIGNAL);
        if (n < 0) {
            if (errno == EINTR) continue;
            return HCCL_E_TCP_TRANSFER;
        }
        p += n;
        len -= (size_t)n;
    }
    return HCCL_SUCCESS;
}

HcclResult RecvAll(int fd, void *buf, size_t len, int64_t deadlineMs)
{
    char *p = (char *)buf;
    while (len > 0) {
        if (deadlineMs >= 0) {
            int64_t left = deadlineMs - NowMs();
            if (left <= 0) return HCCL_E_TIMEOUT;
            struct pollfd pf = {fd, POLLIN, 0};
            int r = poll(&pf, 1, (int)(left > 200 ? 200 : left));
            if (r < 0 && errno != EINTR) return HCCL_E_SYSCALL;
            if (r <= 0) continue;
        }
        ssize_t n = ::recv(fd, p, len, 0);
        if (n == 0) return HCCL_E_TCP_TRANSFER;  // peer closed
        if (n < 0) {
            if (errno == EINTR || errno == EAGAIN) continue;
            return HCCL_E_TCP_TRANSFER;
        }
        p += n;
        len -= (size_t)n;
    }
    return HCCL_SUCCESS;
}

void Close(int &fd)
{
    if (fd >= 0) {
        ::shutdown(fd, SHUT_RDWR);
        ::close(fd);
        fd = -1;
    }
}

static socklen_t FillAbstract(struct sockaddr_un &sa, const std::string &name)
{
    memset(&sa, 0, sizeof(sa));
    sa.sun_family = AF_UNIX;
    size_t n = name.size();
    if (n > sizeof(sa.sun_path) - 2) n = sizeof(sa.sun_path) - 2;
    sa.sun_path[0] = '\0';
    memcpy(sa.sun_path + 1, name.data(), n);
    return (socklen_t)(offsetof(struct sockaddr_un, sun_path) + 1 + n);
}

HcclResult UdsListen(const std::string &name, int *fdOut)
{
    int fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd < 0) return HCCL_E_SYSCALL;
    struct sockaddr_un sa;
    socklen_t len = FillAbstract(sa, name);
    if (bind(fd, (struct sockaddr *)&sa, len) != 0 || listen(fd, 256) != 0) {
        HCCL_ERROR("unix listen on @%s failed: %s", name.c_str(), strerror(errno));
        ::close(fd);
        return HCCL_E_SYSCALL;
    }
    *fdOut = fd;
    return HCCL_SUCCESS;
}

HcclResult UdsConnect(const std::string &name, int64_t deadlineMs, int *fdOut)
{
    struct sockaddr_un sa;
    socklen_t len = FillAbstract(sa, name);
    for (;;) {
        int fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
        if (fd < 0) return HCCL_E_SYSCALL;
        if (connect(fd, (struct sockaddr *)&sa, len) == 0) {
            *fdOut = fd;
            return HCCL_SUCCESS;
        }
        ::close(fd);
        if (NowMs() >= deadlineMs) return HCCL_E_TIMEOUT;
        usleep(2000);
    }
}

HcclResult UdsSendFd(int sock, const void *meta, size_t metaLen, int fdToSend)
{
    struct msghdr msg;
    memset(&msg, 0, sizeof(msg));
    struct iovec iov = {const_cast<void *>(meta), metaLen};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    char ctrl[CMSG_SPACE(sizeof(int))];
    memset(ctrl, 0, sizeof(ctrl));
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    struct cmsghdr *c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(c), &fdToSend, sizeof(int));
    ssize_t n;
    do { n = sendmsg(sock, &msg, MSG_NOSIGNAL); } while (n < 0 && errno == EINTR);
    return n == (ssize_t)metaLen ? HCCL_SUCCESS : HCCL_E_SYSCALL;
}

HcclResult UdsRecvFd(int sock, void *meta, size_t metaLen, int *fdOut, int64_t deadlineMs)
{
    for (;;) {
        int64_t left = deadlineMs - NowMs();
        if (left <= 0) return HCCL_E_TIMEOUT;
        struct pollfd pf = {sock, POLLIN, 0};
        int r = poll(&pf, 1, (int)(left > 200 ? 200 : left));
        if (r < 0 && errno != EINTR) return HCCL_E_SYSCALL;
        if (r > 0) break;
    }
    struct msghdr msg;
    memset(&msg, 0, sizeof(msg));
    struct iovec iov = {meta, metaLen};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    char ctrl[CMSG_SPACE(sizeof(int))];
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    ssize_t n;
    do { n = recvmsg(sock, &msg, MSG_CMSG_CLOEXEC); } while (n < 0 && errno == EINTR);
    if (n != (ssize_t)metaLen) return HCCL_E_SYSCALL;
    struct cmsghdr *c = CMSG_FIRSTHDR(&msg);
    if (!c || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) {
        *fdOut = -1;              // a message without a descriptor (the ring monitor's pings)
        return HCCL_SUCCESS;
    }
    memcpy(fdOut, CMSG_DATA(c), sizeof(int));
    return HCCL_SUCCESS;
}

HcclResult Whitelist::Load(const std::string &path)
{
    enabled_ = false;
    ips_.clear();
    if (path.empty()) return HCCL_SUCCESS;
    std::ifstream f(path);
    if (!f) {
        RPT_ERR("EI0004", "whitelist file %s cannot be opened", path.c_str());
        return HCCL_E_OPEN_FILE_FAILURE;
    }
    std::string line;
    while (std::getline(f, line)) {
        size_t a = line.find_first_not_of(" \t\r\",[]");
        size_t b = line.find_last_not_of(" \t\r\",[]");
        if (a == std::string::npos) continue;
        ips_.push_back(line.substr(a, b - a + 1));
    }
    enabled_ = true;
    return HCCL_SUCCESS;
}

bool Whitelist::Allows(const std::string &ip) const
{
    if (!enabled_) return true;
    for (auto &s : ips_)
        if (s == ip) return true;
    return false;
}

}  // namespace net
}  // namespace hc
