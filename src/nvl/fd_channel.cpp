#include "nvl/fd_channel.h"

#include <errno.h>
#include <poll.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include "megray/debug.h"

namespace MegRay {

namespace {
// abstract namespace: sun_path[0] == 0, the name follows
socklen_t make_addr(struct sockaddr_un* addr, const std::string& group, uint32_t rank) {
    memset(addr, 0, sizeof(*addr));
    addr->sun_family = AF_UNIX;
    char name[96];
    int n = snprintf(name, sizeof(name), "megray-%s-%u", group.c_str(), rank);
    if (n > static_cast<int>(sizeof(addr->sun_path)) - 2)
        n = sizeof(addr->sun_path) - 2;
    memcpy(addr->sun_path + 1, name, static_cast<size_t>(n));
    return static_cast<socklen_t>(offsetof(struct sockaddr_un, sun_path) + 1 + n);
}
struct Msg {
    uint32_t from;
    uint32_t tag;
};
}  // namespace

FdChannel::~FdChannel() { close(); }

void FdChannel::close() {
    if (m_sock >= 0) {
        ::close(m_sock);
        m_sock = -1;
    }
}

Status FdChannel::open(const std::string& group, uint32_t rank) {
    m_group = group;
    m_rank = rank;
    m_sock = ::socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
    if (m_sock < 0) {
        MEGRAY_ERROR("unix socket: %s", strerror(errno));
        return MEGRAY_SYS_ERROR;
    }
    struct sockaddr_un addr;
    socklen_t len = make_addr(&addr, group, rank);
    if (::bind(m_sock, reinterpret_cast<struct sockaddr*>(&addr), len) != 0) {
        MEGRAY_ERROR("bind unix socket: %s", strerror(errno));
        close();
        return MEGRAY_SYS_ERROR;
    }
    return MEGRAY_OK;
}

Status FdChannel::send_fd(uint32_t peer, int fd, uint32_t tag) {
    struct sockaddr_un addr;
    socklen_t alen = make_addr(&addr, m_group, peer);
    Msg m = {m_rank, tag};
    struct iovec iov = {&m, sizeof(m)};
    char ctrl[CMSG_SPACE(sizeof(int))];
    memset(ctrl, 0, sizeof(ctrl));
    struct msghdr msg = {};
    msg.msg_name = &addr;
    msg.msg_namelen = alen;
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    struct cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(c), &fd, sizeof(int));
    for (int attempt = 0; attempt < 200; ++attempt) {
        if (::sendmsg(m_sock, &msg, 0) >= 0)
            return MEGRAY_OK;
        if (errno != ECONNREFUSED && errno != ENOENT && errno != EAGAIN && errno != EINTR)
            break;
        usleep(10 * 1000);  // the peer has not bound its socket yet
    }
    MEGRAY_ERROR("sendmsg(fd) to rank %u: %s", peer, strerror(errno));
    return MEGRAY_SYS_ERROR;
}

Status FdChannel::recv_fd(int* fd, uint32_t* from, uint32_t* tag, int64_t timeout_ms) {
    struct pollfd p = {m_sock, POLLIN, 0};
    int r;
    do {
        r = ::poll(&p, 1, timeout_ms > 0 ? static_cast<int>(timeout_ms) : -1);
    } while (r < 0 && errno == EINTR);
    if (r == 0)
        return MEGRAY_TIMEOUT;
    if (r < 0)
        return MEGRAY_SYS_ERROR;
    Msg m = {};
    struct iovec iov = {&m, sizeof(m)};
    char ctrl[CMSG_SPACE(sizeof(int))];
    struct msghdr msg = {};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    ssize_t n = ::recvmsg(m_sock, &msg, MSG_CMSG_CLOEXEC);
    if (n != static_cast<ssize_t>(sizeof(m))) {
        MEGRAY_ERROR("recvmsg(fd): %s", n < 0 ? strerror(errno) : "short message");
        return MEGRAY_SYS_ERROR;
    }
    struct cmsghdr* c = CMSG_FIRSTHDR(&msg);
    if (c == nullptr || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS) {
        MEGRAY_ERROR("recvmsg(fd): no descriptor attached");
        return MEGRAY_SYS_ERROR;
    }
    memcpy(fd, CMSG_DATA(c), sizeof(int));
    *from = m.from;
    *tag = m.tag;
    return MEGRAY_OK;
}

}  // namespace MegRay
