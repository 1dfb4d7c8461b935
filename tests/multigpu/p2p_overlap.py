"""send / recv on the communicator's own stream.  Default: stream-ordered (the received data is
there when the caller's stream gets to the next kernel).  With set_p2p_async: the caller's stream
does not wait for the transfer, so a native all_reduce enqueued right after a large send / recv
pair finishes long before the pair does; p2p_join() then orders the stream after the transfer."""
import torch
from common import setup

rank, n, dev, comm, server = setup()
peer = rank ^ 1
big = 256 << 20       # bytes of the point-to-point message
small = 1 << 20       # elements of the all_reduce
a = torch.full((big // 4,), float(rank + 1), device=dev)
b = torch.zeros_like(a)
x = torch.full((small,), float(rank + 1), device=dev)
y = torch.empty_like(x)


def pair():
    if peer < n:
        comm.group_start()
        comm.send(a, peer)
        comm.recv(b, peer)
        comm.group_end()


def timed(fn, reps=3):
    fn()
    torch.cuda.synchronize()
    comm.stream_barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


# stream-ordered by default: the next kernel on the stream sees the received data
b.zero_()
pair()
total = b.sum()          # enqueued on the same stream right after the pair
torch.cuda.synchronize()
if peer < n:
    assert float(total) == float(peer + 1) * (big // 4), float(total)

t_pair = timed(pair)
t_ar = timed(lambda: comm.all_reduce(x, y))

comm.set_p2p_async(True)


def overlapped():
    pair()                      # the stream does not wait for this transfer ...
    comm.all_reduce(x, y)       # ... so the all_reduce starts at once


def overlapped_joined():
    overlapped()
    comm.p2p_join()


t_user = timed(lambda: (overlapped(), None)[1])   # time on the caller's stream, transfers still in flight
comm.p2p_join()
torch.cuda.synchronize()
b.zero_()
t_both = timed(overlapped_joined)
torch.cuda.synchronize()
assert float(y[0]) == n * (n + 1) / 2
if peer < n:
    assert float(b[0]) == float(peer + 1) and float(b[-1]) == float(peer + 1)
    # the caller's stream was not held up by the transfer, and the two together take less than one after the other
    assert t_user < 0.6 * (t_pair + t_ar), (t_user, t_pair, t_ar)
    assert t_both < 0.97 * (t_pair + t_ar) + 0.02, (t_both, t_pair, t_ar)
print(f"RANK_OK {rank} pair {t_pair:.3f} ms all_reduce {t_ar:.3f} ms, stream time {t_user:.3f} ms, both joined {t_both:.3f} ms",
      flush=True)
comm.set_p2p_async(False)
comm.close()
