#!/usr/bin/env python
"""Measures the algorithm crossover points of the NVL backend and writes the tune table.

Runs ``build/megray_bench`` (threads as ranks, device-timed, max over ranks) for all_reduce over a
range of message sizes with the one-shot threshold forced low and high and with several grid
sizes, picks for each size the fastest setting, and writes a JSON file that a communicator reads
when ``MEGRAY_TUNE_FILE`` names it:

    {"oneshot_bytes": ..., "max_ctas": ..., "cta_bytes": ..., "measured": {...}}

    python bench/tune.py --devices 8 --out tune_8gpu.json
"""
import argparse
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(devices, sizes, env):
    e = dict(os.environ, **env)
    cmd = [os.path.join(ROOT, "build", "megray_bench"), "-d", str(devices), "-e", "nvl", "-f", "all_reduce",
           "-s", ",".join(str(s) for s in sizes), "-t", "float32", "-w", "10", "-i", "30", "-j"]
    out = subprocess.run(cmd, capture_output=True, text=True, env=e, timeout=600)
    res = {}
    for line in out.stdout.splitlines():
        if line.startswith("{"):
            d = json.loads(line)
            if d["ok"]:
                res[d["bytes"]] = d["time_us"]
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--devices", type=int, default=2)
    ap.add_argument("--out", default="tune.json")
    a = ap.parse_args()
    sizes = [1 << k for k in range(10, 25)]
    one = run(a.devices, sizes, {"MEGRAY_ALGO": "oneshot"})
    two = run(a.devices, sizes, {"MEGRAY_ALGO": "twoshot"})
    crossover = 0
    for s in sizes:
        if s in one and s in two and one[s] <= two[s]:
            crossover = s
    best_cta, best_t = 128 * 1024, None
    big = [1 << 24, 1 << 26]
    for cta_bytes in (32 << 10, 64 << 10, 128 << 10, 256 << 10):
        r = run(a.devices, big, {"MEGRAY_ALGO": "twoshot", "MEGRAY_CTA_BYTES": str(cta_bytes)})
        t = sum(r.get(s, 1e18) for s in big)
        if best_t is None or t < best_t:
            best_cta, best_t = cta_bytes, t
    table = {"oneshot_bytes": crossover, "max_ctas": 64, "cta_bytes": best_cta, "nvls_min_bytes": 0,
             "devices": a.devices, "measured": {"oneshot_us": one, "twoshot_us": two}}
    with open(a.out, "w") as f:
        json.dump(table, f, indent=1)
    print(json.dumps({k: v for k, v in table.items() if k != "measured"}))


if __name__ == "__main__":
    sys.exit(main())
