#include "rendezvous/net.h"

#include <errno.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <time.h>
#include <unistd.h>

namespace MegRay {
namespace net {

int64_t now_ms() {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return static_cast<int64_t>(ts.tv_sec) * 1000 + ts.tv_nsec / 1000000;
}

int64_t deadline_after(int64_t timeout_ms) { return timeout_ms > 0 ? now_ms() + timeout_ms : -1; }

void tune_socket(int fd) {
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    int fl = fcntl(fd, F_GETFL, 0);
    if (fl >= 0)
        fcntl(fd, F_SETFL, fl | O_NONBLOCK);
    int fdfl = fcntl(fd, F_GETFD, 0);
    if (fdfl >= 0)
        fcntl(fd, F_SETFD, fdfl | FD_CLOEXEC);
}

namespace {
// Wait until fd is ready for `events`; 1 ready, 0 deadline passed, -1 error, -2 cancelled.
int wait_fd(int fd, short events, int64_t deadline_ms, int cancel_fd) {
    for (;;) {
        int to = -1;
        if (deadline_ms >= 0) {
            int64_t left = deadline_ms - now_ms();
            if (left <= 0)
                return 0;
            to = left > 1000 ? 1000 : static_cast<int>(left);
        }
        struct pollfd p[2] = {{fd, events, 0}, {cancel_fd, POLLIN, 0}};
        int r = ::poll(p, cancel_fd >= 0 ? 2 : 1, to);
        if (r > 0 && cancel_fd >= 0 && p[1].revents)
            return -2;
        if (r > 0)
            return 1;  // readable/writable or HUP/ERR: let the I/O call report it
        if (r < 0 && errno != EINTR)
            return -1;
    }
}
}  // namespace

Status send_all(int fd, const void* buf, size_t len, int64_t deadline_ms, int cancel_fd) {
    const char* p = static_cast<const char*>(buf);
    size_t done = 0;
    while (done < len) {
        ssize_t n = ::send(fd, p + done, len - done, MSG_NOSIGNAL);
        if (n > 0) {
            done += static_cast<size_t>(n);
            continue;
        }
        if (n < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) {
            int w = wait_fd(fd, POLLOUT, deadline_ms, cancel_fd);
            if (w == 0)
                return MEGRAY_TIMEOUT;
            if (w == -2)
                return MEGRAY_ABORTED;
            if (w < 0)
                return MEGRAY_SYS_ERROR;
            continue;
        }
        if (n < 0 && errno == EINTR)
            continue;
        return MEGRAY_SYS_ERROR;
    }
    return MEGRAY_OK;
}

Status recv_all(int fd, void* buf, size_t len, int64_t deadline_ms, bool* eof_at_start,
                int cancel_fd) {
    char* p = static_cast<char*>(buf);
    size_t done = 0;
    if (eof_at_start)
        *eof_at_start = false;
    while (done < len) {
        ssize_t n = ::recv(fd, p + done, len - done, 0);
        if (n > 0) {
            done += static_cast<size_t>(n);
            continue;
        }
        if (n == 0) {
            if (eof_at_start && done == 0)
                *eof_at_start = true;
            return MEGRAY_SYS_ERROR;
        }
        if (errno == EAGAIN || errno == EWOULDBLOCK) {
            int w = wait_fd(fd, POLLIN, deadline_ms, cancel_fd);
            if (w == 0)
                return MEGRAY_TIMEOUT;
            if (w == -2)
                return MEGRAY_ABORTED;
            if (w < 0)
                return MEGRAY_SYS_ERROR;
            continue;
        }
        if (errno == EINTR)
            continue;
        return MEGRAY_SYS_ERROR;
    }
    return MEGRAY_OK;
}

}  // namespace net
}  // namespace MegRay
