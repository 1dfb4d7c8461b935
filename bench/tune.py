#!/usr/bin/env python
"""Measures the algorithm crossover points of the NVL backend on this machine and writes the
tune table a communicator loads (MEGRAY_TUNE_FILE, or megray_b200/tune/tune_b200_n<ranks>.json
when that file exists).

For every operation it runs ``build/megray_bench`` (threads as ranks, device-timed, max over
ranks, float32) over the small and middle sizes with each algorithm forced in turn and keeps, per
operation, the largest size up to which the flagged-word kernel is the fastest; for all_reduce
also the size up to which the one-shot kernel beats the single-pass one; and, when the NVSwitch
multicast object can be set up (``--nvls``: MEGRAY_NVLS=1 in the benchmark processes only), the
size from which the multimem kernels beat plain peer loads and stores on heap buffers.  It also
picks the grid size, the bytes per CTA of the single-pass kernels and the chunk of the pipelined
broadcast by the summed time over a few sizes, and the size from which a reduce has its root push.

    python bench/tune.py --devices 8 --out megray_b200/tune/tune_b200_n8.json
"""
import argparse
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KINDS = ["all_reduce", "reduce_scatter", "all_gather", "all_to_all", "broadcast", "reduce", "gather", "scatter"]


def run(devices, funcs, sizes, env, extra=()):
    e = dict(os.environ, MEGRAY_NVL_P2P="0", **env)  # (no send/recv here: skip setting up its engine)
    cmd = [os.path.join(ROOT, "build", "megray_bench"), "-d", str(devices), "-e", "nvl", "-f", ",".join(funcs),
           "-s", ",".join(str(s) for s in sizes), "-t", "float32", "-w", "5", "-i", "25", "-j", *extra]
    out = subprocess.run(cmd, capture_output=True, text=True, env=e, timeout=900)
    res = {}
    for line in out.stdout.splitlines():
        if line.startswith("{"):
            d = json.loads(line)
            if d["ok"]:
                res[(d["op"], d["bytes"])] = (d["time_us"], d.get("algo", "-"))
    if not res:
        sys.stderr.write(out.stderr[-2000:])
    return res


def crossover(sizes, a, b, func, margin=1.0):
    """Largest size s at which a is at least as fast as b (times `margin`), provided a is not
    slower than b by more than 10 % anywhere below s (one noisy sample at a small size does not
    switch a off altogether; a real loss does)."""
    best = 0
    for s in sizes:
        ta, tb = a.get((func, s)), b.get((func, s))
        if ta is None or tb is None or ta[0] > tb[0] * 1.10:
            break
        if ta[0] <= tb[0] * margin:
            best = s
    return best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--devices", type=int, default=2)
    ap.add_argument("--out", default=None)
    ap.add_argument("--nvls", action="store_true", help="also measure the NVSwitch multimem kernels (heap buffers)")
    ap.add_argument("--crossovers-only", action="store_true",
                    help="measure the algorithm crossovers only; keep the default grid and chunk sizes")
    a = ap.parse_args()
    out_path = a.out or os.path.join(ROOT, "megray_b200", "tune", f"tune_b200_n{a.devices}.json")
    table = {"devices": a.devices, "measured": {}}

    # flagged words against what would run otherwise (one-shot / single pass / staged)
    small = [1 << k for k in range(10, 21)]  # 1 KiB .. 1 MiB per source / destination pair
    with_ll = run(a.devices, KINDS, small, {"MEGRAY_LL_BYTES": str(1 << 20), "MEGRAY_TUNE_DEFAULT": "0"})
    without = run(a.devices, KINDS, small, {"MEGRAY_LL_BYTES": "0", "MEGRAY_TUNE_DEFAULT": "0"})
    for k in KINDS:
        table[f"ll_{k}"] = crossover(small, with_ll, without, k, margin=1.02)
        table["measured"][f"us_ll_vs_other_{k}"] = {str(s): [with_ll.get((k, s), [None])[0], without.get((k, s), [None])[0]]
                                        for s in small}

    # all_reduce: one-shot (one barrier, staging slots) against single pass (two barriers, no staging)
    mid = [1 << k for k in range(15, 23)]  # 32 KiB .. 4 MiB
    one = run(a.devices, ["all_reduce"], mid, {"MEGRAY_LL_BYTES": "0", "MEGRAY_ONESHOT_BYTES": str(1 << 30),
                                               "MEGRAY_TUNE_DEFAULT": "0"})
    two = run(a.devices, ["all_reduce"], mid, {"MEGRAY_LL_BYTES": "0", "MEGRAY_ONESHOT_BYTES": "0",
                                               "MEGRAY_TUNE_DEFAULT": "0"})
    table["oneshot_bytes"] = crossover(mid, one, two, "all_reduce")
    table["measured"]["us_oneshot_vs_single_pass"] = {str(s): [one.get(("all_reduce", s), [None])[0], two.get(("all_reduce", s), [None])[0]]
                                    for s in mid}

    # grid size of the single-pass kernels at a bandwidth-bound size
    big = [64 << 20]
    best_ctas, best_t = 64, None
    for ctas in (() if a.crossovers_only else (32, 64)):
        r = run(a.devices, ["all_reduce", "all_gather"], big, {"MEGRAY_MAX_CTAS": str(ctas)})
        t = sum(v[0] for v in r.values()) if len(r) == 2 else None
        table["measured"][f"us_sum_at_{ctas}_ctas"] = t
        if t is not None and (best_t is None or t < best_t):
            best_ctas, best_t = ctas, t
    table["max_ctas"] = best_ctas

    def pick(key, values, funcs, sizes, env_name):
        """The value of one knob with the smallest summed time over `funcs` x `sizes`."""
        if a.crossovers_only:
            return
        best_v, best_sum = None, None
        for v in values:
            r = run(a.devices, funcs, sizes, {env_name: str(v), "MEGRAY_TUNE_DEFAULT": "0", "MEGRAY_MAX_CTAS": str(best_ctas)})
            t = sum(x[0] for x in r.values()) if len(r) == len(funcs) * len(sizes) else None
            table["measured"][f"us_sum_{key}_{v}"] = t
            if t is not None and (best_sum is None or t < best_sum):
                best_v, best_sum = v, t
        if best_v is not None:
            table[key] = best_v

    # bytes per CTA of the single-pass kernels in the middle sizes (more CTAs: more bytes in
    # flight, but a longer barrier), chunk of the pipelined broadcast
    pick("direct_cta_bytes", (16 << 10, 32 << 10, 128 << 10), KINDS, [1 << 20, 4 << 20, 16 << 20], "MEGRAY_DIRECT_CTA_BYTES")
    if a.devices > 2:
        pick("bcast_chunk_bytes", (32 << 10, 64 << 10, 256 << 10, 1 << 20), ["broadcast"], [4 << 20, 64 << 20, 1 << 30],
             "MEGRAY_BCAST_CHUNK")

    # reduce on more than two ranks: the reducers load everything and store to the root (0), the root
    # pushes its input into the reducers' slots (1), or loads only, the root loading the reduced
    # chunks from the reducers' slots (2), or the same in steps separated by barriers (3): the
    # staged form that is fastest at the largest size, and
    # the size from which it beats form 0 at every larger size
    if a.devices > 2:
        rsizes = [1 << k for k in range(20, 31, 2)]  # 1 MiB .. 1 GiB
        base_env = {"MEGRAY_TUNE_DEFAULT": "0", "MEGRAY_LL_BYTES": "0", "MEGRAY_MAX_CTAS": str(best_ctas)}
        forms = {0: run(a.devices, ["reduce"], rsizes, dict(base_env, MEGRAY_REDUCE_MODE="0"))}
        for mode in (1, 2, 3):
            forms[mode] = run(a.devices, ["reduce"], rsizes, dict(base_env, MEGRAY_REDUCE_MODE=str(mode), MEGRAY_REDUCE_STAGED_MIN="0"))
        t = lambda mode, sz: forms[mode].get(("reduce", sz), [float("inf")])[0]
        staged = min((1, 2, 3), key=lambda mode: t(mode, rsizes[-1]))
        first = 1 << 62
        for sz in reversed(rsizes):
            if t(staged, sz) > t(0, sz):
                break
            first = sz
        table["reduce_mode"] = staged if first < (1 << 62) else 0
        table["reduce_staged_min_bytes"] = first
        table["measured"]["us_reduce_forms_0_1_2_3"] = {str(sz): [t(0, sz), t(1, sz), t(2, sz), t(3, sz)] for sz in rsizes}

    # broadcast: stores (root and slice owners push) against loads alone (everybody pulls)
    bsizes = [1 << k for k in range(20, 31, 2)]  # 1 MiB .. 1 GiB
    benv = {"MEGRAY_TUNE_DEFAULT": "0", "MEGRAY_LL_BYTES": "0", "MEGRAY_MAX_CTAS": str(best_ctas)}
    pushed = run(a.devices, ["broadcast"], bsizes, dict(benv, MEGRAY_BCAST_PULL="0"))
    pulled = run(a.devices, ["broadcast"], bsizes, dict(benv, MEGRAY_BCAST_PULL="1"))
    first = 1 << 62
    for sz in reversed(bsizes):
        tl, tp = pulled.get(("broadcast", sz)), pushed.get(("broadcast", sz))
        if tl is None or tp is None or tl[0] > tp[0]:
            break
        first = sz
    table["bcast_pull"] = 1 if first < (1 << 62) else 0
    table["bcast_pull_min_bytes"] = first if first < (1 << 62) else 0
    table["measured"]["us_broadcast_pushed_vs_pulled"] = {str(sz): [pushed.get(("broadcast", sz), [None])[0],
                                                                   pulled.get(("broadcast", sz), [None])[0]] for sz in bsizes}

    if a.nvls:
        sizes = [1 << k for k in range(18, 29, 2)]  # 256 KiB .. 256 MiB
        env = {"MEGRAY_NVLS": "1", "NCCL_NVLS_ENABLE": "1", "MEGRAY_HEAP_MB": "2048"}
        mc = run(a.devices, ["all_reduce"], sizes, dict(env), extra=("-H",))
        p2p = run(a.devices, ["all_reduce"], sizes, dict(env, MEGRAY_NVLS="0"), extra=("-H",))
        first = 0
        for s in reversed(sizes):
            if (("all_reduce", s) in mc and ("all_reduce", s) in p2p and mc[("all_reduce", s)][1] == "nvls" and
                    mc[("all_reduce", s)][0] <= p2p[("all_reduce", s)][0]):
                first = s
            else:
                break
        table["nvls_min_bytes"] = first if first else (1 << 62)
        table["measured"]["us_nvls_vs_p2p"] = {str(s): [mc.get(("all_reduce", s), [None])[0], p2p.get(("all_reduce", s), [None])[0]]
                                     for s in sizes}
    table["measured"] = table.pop("measured")  # the raw timings go last: the library reads the first match of a key
    os.makedirs(os.path.dirname(out_path), exist_ok=True)
    with open(out_path, "w") as f:
        json.dump(table, f, indent=1)
    print(json.dumps({k: v for k, v in table.items() if k != "measured"}))


if __name__ == "__main__":
    sys.exit(main())
