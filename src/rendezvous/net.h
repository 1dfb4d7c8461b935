// Socket helpers shared by the rendezvous client and server: deadline-aware
// full reads/writes on blocking-free sockets.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include "megray/types.h"

namespace MegRay {
namespace net {

/** Monotonic milliseconds. */
int64_t now_ms();

/** Absolute deadline `timeout_ms` from now; <= 0 means none (returns -1). */
int64_t deadline_after(int64_t timeout_ms);

/** Write exactly `len` bytes. MEGRAY_OK, MEGRAY_TIMEOUT or MEGRAY_SYS_ERROR. */
Status send_all(int fd, const void* buf, size_t len, int64_t deadline_ms, int cancel_fd = -1);

/** Read exactly `len` bytes.  `*eof_at_start` (optional) is set when the peer
 *  closed before the first byte; the call then returns MEGRAY_SYS_ERROR. */
Status recv_all(int fd, void* buf, size_t len, int64_t deadline_ms, bool* eof_at_start = nullptr,
                int cancel_fd = -1);

/** `cancel_fd` (optional): when it becomes readable the call returns MEGRAY_ABORTED. */

/** TCP_NODELAY + close-on-exec + non-blocking. */
void tune_socket(int fd);

}  // namespace net
}  // namespace MegRay
