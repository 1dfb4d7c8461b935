"""The bounds-checked build of the collective kernels (``python -m megray_b200.build
--debug-bounds``): every CTA-level copy or reduction checks its range against the call's buffers
and the ranks' heaps before touching it.  Two runs of the C++ test runner built that way:

* the sweep of all ten operations must pass with no range refused (and with the guard zones
  around the staging workspaces intact);
* in self-test mode the communicator declares its buffers half as long as they are, and the guard
  must refuse, skip and report the ranges beyond the declared half.  No access that is really out
  of bounds is made anywhere.

compute-sanitizer is not available on the machines this was written on; these two runs are the
device-side bounds evidence."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu


def _run(filter_, env):
    from megray_b200 import build

    binary = build.build_debug_bounds()
    e = dict(os.environ, MEGRAY_LOG_LEVEL="3", MEGRAY_EXPECT_BOUNDS_BUILD="1")
    e.update(env)
    out = subprocess.run([binary, filter_], capture_output=True, text=True, timeout=900, env=e)
    assert out.returncode == 0, out.stdout[-4000:] + out.stderr[-2000:]
    return out.stdout


def test_sweep_passes_in_the_bounds_checked_build():
    out = _run("Nvl_SingleRank", {})
    assert "0 failed" in out and "[   OK    ] Nvl_SingleRankGroupRunsEveryOperation" in out, out[-3000:]


def test_range_guard_refuses_ranges_outside_the_declared_buffers():
    out = _run("Nvl_RangeGuard", {"MEGRAY_DEBUG_BOUNDS_SELFTEST": "1"})
    assert "[   OK    ] Nvl_RangeGuardRefusesWhatLiesOutsideTheDeclaredBuffers" in out, out[-3000:]
