"""Operation tracing: with tracing on, every collective call of every rank leaves a span in a
Chrome-trace JSON file (name, rank as the process id of the trace viewer, duration, byte count)."""
import ctypes as C
import json

import numpy as np

from helpers import with_group
from megray_b200 import _lib


def test_host_collectives_leave_spans_in_the_trace_file(tmp_path):
    lib = _lib.load()
    path = tmp_path / "trace.json"
    lib.megray_trace_enable(str(path).encode())

    def body(comm, rank):
        x = np.full(1000, rank + 1, np.float32)
        out = np.empty_like(x)
        comm.all_reduce(x, out, "sum")
        g = np.empty(2 * 1000, np.float32)
        comm.all_gather(x, g)
        comm.broadcast(x, out, 0)
        return float(out[0])

    assert with_group(2, "shm", body) == [1.0, 1.0]
    written = lib.megray_trace_dump()
    assert written >= 6
    events = json.loads(path.read_text())
    events = events["traceEvents"] if isinstance(events, dict) else events
    names = [e["name"] for e in events]
    for op in ("all_reduce", "all_gather", "broadcast"):
        assert sum(op in n for n in names) >= 2, names  # one per rank
    one = next(e for e in events if "all_reduce" in e["name"])
    assert one["ph"] == "X" and one["dur"] >= 0 and "bytes" in json.dumps(one)
    assert {e["pid"] for e in events if "all_reduce" in e["name"]} == {0, 1}
