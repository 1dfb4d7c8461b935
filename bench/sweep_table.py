#!/usr/bin/env python
"""Turns JSON lines of `megray_bench -j` runs into one markdown table: one row per (operation,
size), one column pair (time, bus bandwidth) per labelled run, and the time ratio of every run
against the first one.

    build/megray_bench -d 8 -e nccl -f all_reduce,all_gather -s 1K,1M,1G -j > nccl.json
    build/megray_bench -d 8 -e nvl -R -f all_reduce,all_gather -s 1K,1M,1G -j > nvl.json
    python bench/sweep_table.py reference=nccl.json registered=nvl.json

A file may hold several backends; `label=file:backend` keeps only that backend's lines.
"""
import json
import sys


def human(nbytes: int) -> str:
    for unit, name in ((1 << 30, "GiB"), (1 << 20, "MiB"), (1 << 10, "KiB")):
        if nbytes >= unit and nbytes % unit == 0:
            return f"{nbytes // unit} {name}"
    return f"{nbytes} B"


def load(spec: str):
    label, _, rest = spec.partition("=")
    path, _, backend = rest.partition(":")
    rows = {}
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line.startswith("{"):
                continue
            r = json.loads(line)
            if backend and r.get("backend") != backend:
                continue
            rows[(r["op"], int(r["bytes"]))] = r
    return label, rows


def table(specs) -> str:
    runs = [load(s) for s in specs]
    keys = []
    for _, rows in runs:
        for k in rows:
            if k not in keys:
                keys.append(k)
    head = "| op | bytes | " + " | ".join(f"{label} us / GB/s" for label, _ in runs)
    if len(runs) > 1:
        head += " | " + " | ".join(f"{runs[0][0]} / {label}" for label, _ in runs[1:])
    lines = [head + " |", "|" + "---|" * (2 + len(runs) + max(0, len(runs) - 1))]
    for op, nbytes in keys:
        cells = []
        for _, rows in runs:
            r = rows.get((op, nbytes))
            cells.append(f"{r['time_us']:.1f} / {r['busbw_gbs']:.0f}" + ("" if r.get("ok", True) else " (failed)")
                         if r else "-")
        base = runs[0][1].get((op, nbytes))
        for _, rows in runs[1:]:
            r = rows.get((op, nbytes))
            cells.append(f"{base['time_us'] / r['time_us']:.2f}x" if base and r and r["time_us"] > 0 else "-")
        lines.append(f"| {op} | {human(nbytes)} | " + " | ".join(cells) + " |")
    return "\n".join(lines)


if __name__ == "__main__":
    if len(sys.argv) < 2 or any("=" not in a for a in sys.argv[1:]):
        sys.exit(__doc__)
    print(table(sys.argv[1:]))
