"""Builds the reference library, unmodified, into ``baseline/_ref``.

The reference has no Python packaging (``pip install <reference checkout>`` ends with "Neither
'setup.py' nor 'pyproject.toml' found") and its own CMake needs the absent
``third_party/nccl`` sources, so its translation units are compiled in place against the
installed NCCL: ``src/megray.cpp``, ``src/core/*.cpp``, ``src/nccl/*.cpp`` with a
hand-written ``config.h`` that mirrors ``include/megray/config.h.in`` for a CUDA + NCCL
build.  Products:

    baseline/_ref/libmegray_ref.so   reference objects + baseline/ref_shim.cpp (C doorway)
    baseline/_ref/performance        the reference's own benchmark (test/performance.cpp)
    baseline/_ref/megray_bench_ref   bench/megray_bench.cpp built against the reference (device-timed sweep)

    python baseline/build_ref.py [--reference <reference checkout>]
"""
import argparse
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")

CONFIG_H = """#pragma once
#define MEGRAY_WITH_CUDA
#define MEGRAY_WITH_NCCL
#define MEGRAY_LOG_LEVEL 2
"""


def nccl_flags():
    if os.path.exists("/usr/include/nccl.h"):
        return [], ["-L/usr/lib/x86_64-linux-gnu", "-l:libnccl.so.2"]
    import nvidia.nccl as n  # type: ignore

    base = os.path.dirname(n.__file__)
    return [f"-I{base}/include"], [f"-L{base}/lib", "-l:libnccl.so.2", f"-Wl,-rpath,{base}/lib"]


def build(ref: str) -> str:
    if not os.path.isdir(os.path.join(ref, "src", "nccl")):
        raise RuntimeError(f"no reference sources under {ref}")
    inc_dir = os.path.join(OUT, "include", "megray")
    os.makedirs(inc_dir, exist_ok=True)
    with open(os.path.join(inc_dir, "config.h"), "w") as f:
        f.write(CONFIG_H)
    ninc, nlib = nccl_flags()
    # g++ 13 no longer pulls <cstdint> in through other headers, which the reference's headers
    # rely on (include/megray/server.h:24): force-include it instead of touching the sources.
    common = ["g++", "-std=c++14", "-O2", "-fPIC", "-w", "-include", "cstdint", f"-I{OUT}/include", f"-I{ref}/include", f"-I{ref}/src",
              f"-I{CUDA}/include"] + ninc
    srcs = [os.path.join(ref, "src", "megray.cpp")] + sorted(glob.glob(os.path.join(ref, "src", "core", "*.cpp"))) \
        + sorted(glob.glob(os.path.join(ref, "src", "nccl", "*.cpp")))
    objs = []
    for s in srcs:
        o = os.path.join(OUT, os.path.relpath(s, ref).replace(os.sep, "_") + ".o")
        subprocess.check_call(common + ["-c", s, "-o", o])
        objs.append(o)
    shim = os.path.join(OUT, "ref_shim.o")
    subprocess.check_call(common + ["-c", os.path.join(HERE, "ref_shim.cpp"), "-o", shim])
    lib = os.path.join(OUT, "libmegray_ref.so")
    link = [f"-L{CUDA}/lib64", "-lcudart", "-lpthread", "-ldl"] + nlib
    subprocess.check_call(["g++", "-shared", "-o", lib] + objs + [shim] + link)
    perf_objs = []
    for s in ("test/performance.cpp", "test/test_cuda.cpp", "test/test_hip.cpp"):
        o = os.path.join(OUT, s.replace("/", "_") + ".o")
        subprocess.check_call(common + [f"-I{ref}/test", "-c", os.path.join(ref, s), "-o", o])
        perf_objs.append(o)
    subprocess.check_call(["g++", "-o", os.path.join(OUT, "performance")] + perf_objs + objs + link)
    # the device-timed sweep tool of this repository, compiled against the reference's headers and
    # linked with the reference's objects: the like-for-like collective baseline
    bench_src = os.path.join(os.path.dirname(HERE), "bench", "megray_bench.cpp")
    if os.path.exists(bench_src):
        bo = os.path.join(OUT, "megray_bench_ref.o")
        subprocess.check_call(common + ["-DMEGRAY_BENCH_REFERENCE", "-c", bench_src, "-o", bo])
        subprocess.check_call(["g++", "-o", os.path.join(OUT, "megray_bench_ref"), bo] + objs + link)
    return lib


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("MEGRAY_REFERENCE"),
                    help="checkout of the reference library (or set MEGRAY_REFERENCE)")
    a = ap.parse_args()
    if not a.reference:
        ap.error("name the reference checkout with --reference or MEGRAY_REFERENCE")
    print(build(a.reference))
    sys.exit(0)
