#!/usr/bin/env python
"""Turns JSON lines of `megray_bench -j` runs into markdown tables.

One row per (operation, dtype, reduce op, size); one column pair (time, bus bandwidth) per labelled
run, the algorithm the last run took, and the time ratio of every run against the first one.

    build/megray_bench -d 8 -e nvl -f all -t all -o all -s 1K:1G -c -j > nvl.json
    baseline/_ref/megray_bench_ref -d 8 -e nccl -f all -t all -o all -s 1K:1G -c -j > ref.json
    python bench/sweep_table.py reference=ref.json nvl=nvl.json            # every row
    python bench/sweep_table.py --summary reference=ref.json nvl=nvl.json  # per operation: bus bandwidth by size
                                                                           # (float32 sum) and the range of the ratio
                                                                           # over all dtypes and reduce ops

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
            rows[(r["op"], r.get("dtype", "float32"), r.get("reduce", "sum"), int(r["bytes"]))] = r
    return label, rows


def all_keys(runs):
    keys = []
    seen = set()
    for _, rows in runs:
        for k in rows:
            if k not in seen:
                seen.add(k)
                keys.append(k)
    return keys


def table(specs) -> str:
    runs = [load(s) for s in specs]
    head = "| op | dtype | reduce | bytes | " + " | ".join(f"{label} us / GB/s" for label, _ in runs)
    head += " | algorithm"
    if len(runs) > 1:
        head += " | " + " | ".join(f"{runs[0][0]} / {label}" for label, _ in runs[1:])
    lines = [head + " |", "|" + "---|" * (5 + len(runs) + max(0, len(runs) - 1))]
    for key in all_keys(runs):
        op, dtype, red, nbytes = key
        cells = []
        for _, rows in runs:
            r = rows.get(key)
            cells.append(f"{r['time_us']:.1f} / {r['busbw_gbs']:.0f}" + ("" if r.get("ok", True) else " (FAILED)")
                         if r else "-")
        last = runs[-1][1].get(key)
        cells.append(last.get("algo", "-") if last else "-")
        base = runs[0][1].get(key)
        for _, rows in runs[1:]:
            r = rows.get(key)
            cells.append(f"{base['time_us'] / r['time_us']:.2f}x" if base and r and r["time_us"] > 0 else "-")
        lines.append(f"| {op} | {dtype} | {red} | {human(nbytes)} | " + " | ".join(cells) + " |")
    return "\n".join(lines)


def summary(specs) -> str:
    """Per operation and size: bus bandwidth of the float32 sum rows of every run, and over all
    dtypes and reduce ops the lowest and highest time ratio (first run / last run) and the number of
    rows, checked rows and failed rows."""
    runs = [load(s) for s in specs]
    base, last = runs[0][1], runs[-1][1]
    keys = all_keys(runs)
    ops = []
    for k in keys:
        if k[0] not in ops:
            ops.append(k[0])
    sizes = sorted({k[3] for k in keys})
    head = ("| op | bytes | " + " | ".join(f"{label} GB/s (float32 sum)" for label, _ in runs) +
            f" | {runs[0][0]} / {runs[-1][0]}: min .. max over dtypes and ops | rows | failed |")
    lines = [head, "|" + "---|" * (5 + len(runs))]
    for op in ops:
        for nbytes in sizes:
            mine = [k for k in keys if k[0] == op and k[3] == nbytes]
            if not mine:
                continue
            f32 = next((k for k in mine if k[1] == "float32" and k[2] in ("sum", "-")), mine[0])
            cells = []
            for _, rows in runs:
                r = rows.get(f32)
                cells.append(f"{r['busbw_gbs']:.1f}" if r else "-")
            ratios = [base[k]["time_us"] / last[k]["time_us"] for k in mine
                      if k in base and k in last and last[k]["time_us"] > 0]
            failed = sum(1 for _, rows in runs for k in mine if k in rows and not rows[k].get("ok", True))
            span = f"{min(ratios):.2f}x .. {max(ratios):.2f}x" if ratios else "-"
            lines.append(f"| {op} | {human(nbytes)} | " + " | ".join(cells) + f" | {span} | {len(mine)} | {failed} |")
    return "\n".join(lines)


if __name__ == "__main__":
    args = sys.argv[1:]
    want_summary = "--summary" in args
    args = [a for a in args if a != "--summary"]
    if not args or any("=" not in a for a in args):
        sys.exit(__doc__)
    print(summary(args) if want_summary else table(args))
