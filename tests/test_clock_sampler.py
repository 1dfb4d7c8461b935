"""ClockSampler against a fake nvidia-smi on PATH: median SM clock, maximum power, and the list of
throttle reasons that were active in any sample.  (The sampler only reads; nothing about a GPU is
ever changed.)"""
import os
import stat
import time

from megray_b200.utils.clocks import ClockSampler

FAKE = """#!/bin/sh
# prints one CSV line per call, cycling through three states kept in a counter file
n=$(cat "$FAKE_SMI_COUNTER" 2>/dev/null || echo 0)
echo $((n + 1)) > "$FAKE_SMI_COUNTER"
case $((n % 3)) in
  0) echo "1965, 1965, 612.5, Not Active, Not Active, Not Active, Not Active" ;;
  1) echo "1320, 1965, 998.0, Not Active, Not Active, Not Active, Active" ;;
  2) echo "1275, 1965, 1001.2, Not Active, Not Active, Not Active, Active" ;;
esac
"""


def test_sampler_summarises_what_nvidia_smi_printed(tmp_path, monkeypatch):
    exe = tmp_path / "nvidia-smi"
    exe.write_text(FAKE)
    exe.chmod(exe.stat().st_mode | stat.S_IXUSR)
    monkeypatch.setenv("PATH", f"{tmp_path}{os.pathsep}{os.environ['PATH']}")
    monkeypatch.setenv("FAKE_SMI_COUNTER", str(tmp_path / "count"))
    s = ClockSampler(0, period_s=0.01).start()
    deadline = time.time() + 10
    while len(s.rows) < 6 and time.time() < deadline:
        time.sleep(0.02)
    out = s.stop()
    assert out["samples"] >= 6
    assert out["sm_max_mhz"] == 1965.0
    assert out["sm_mhz"] in (1275.0, 1320.0, 1965.0) and out["power_w_max"] == 1001.2
    assert out["reasons"] == ["sw_power_cap"]


def test_sampler_without_nvidia_smi_reports_nothing(tmp_path, monkeypatch):
    monkeypatch.setenv("PATH", str(tmp_path))  # no nvidia-smi anywhere
    out = ClockSampler(0, period_s=0.01).start().stop()
    assert out == {"sm_mhz": None, "sm_max_mhz": None, "power_w_max": None, "reasons": [], "samples": 0}
