"""In-tree native build of ``libmegray.so`` (and the C++ test / benchmark binaries).

The library is plain C++17 + CUDA for sm_100a with no dependency on PyTorch: the
Python layer talks to it through its ``extern "C"`` interface with ctypes.  The
build is driven by ninja from a generated ``build/build.ninja`` so that repeated
calls only recompile what changed.  NCCL is not linked: the NCCL engine opens
``libnccl.so.2`` at run time.

    python -m megray_b200.build            # library only
    python -m megray_b200.build --all      # + megray_test, megray_bench binaries
"""
from __future__ import annotations

import argparse
import glob
import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BUILD_DIR = os.path.join(ROOT, "build")
LIB_DIR = os.path.join(ROOT, "megray_b200", "lib")
LIB_PATH = os.path.join(LIB_DIR, "libmegray.so")

CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")
GENCODE = "-gencode arch=compute_100a,code=sm_100a"


def _sources():
    cpp = sorted(glob.glob(os.path.join(ROOT, "src", "**", "*.cpp"), recursive=True))
    cu = sorted(glob.glob(os.path.join(ROOT, "src", "**", "*.cu"), recursive=True))
    return cpp, cu


def _nccl_include():
    """Directory holding nccl.h (only the header is needed at build time)."""
    for cand in ("/usr/include",):
        if os.path.exists(os.path.join(cand, "nccl.h")):
            return cand
    try:
        import nvidia.nccl  # type: ignore

        d = os.path.join(os.path.dirname(nvidia.nccl.__file__), "include")
        if os.path.exists(os.path.join(d, "nccl.h")):
            return d
    except Exception:
        pass
    return None


def write_ninja(with_bins: bool) -> str:
    os.makedirs(BUILD_DIR, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    cpp, cu = _sources()
    inc = f"-I{ROOT}/include -I{ROOT}/src -I{CUDA_HOME}/include"
    nccl_inc = _nccl_include()
    defs = "-DMEGRAY_WITH_CUDA -DMEGRAY_WITH_NVL -DMEGRAY_WITH_SHM"
    if nccl_inc:
        defs += " -DMEGRAY_WITH_NCCL"
        if nccl_inc != "/usr/include":
            inc += f" -I{nccl_inc}"
    lines = [
        "ninja_required_version = 1.3",
        f"cxxflags = -std=c++17 -O2 -g -fPIC -Wall -Wno-unused-function {defs} {inc}",
        f"nvccflags = -std=c++17 -O3 {GENCODE} -lineinfo -Xcompiler -fPIC "
        f"--expt-relaxed-constexpr {defs} {inc}",
        "rule cxx",
        "  command = g++ -MMD -MF $out.d $cxxflags -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "  description = CXX $in",
        "rule nvcc",
        f"  command = {NVCC} -MD -MF $out.d $nvccflags -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "  description = NVCC $in",
        "rule link_so",
        f"  command = {NVCC} -shared {GENCODE} -o $out $in -lpthread -ldl -lrt",
        "  description = LINK $out",
        "rule link_bin",
        f"  command = g++ -o $out $in -L{LIB_DIR} -lmegray -Wl,-rpath,{LIB_DIR} "
        f"-Wl,-rpath,$$ORIGIN/../megray_b200/lib -L{CUDA_HOME}/lib64 -lcudart -lpthread -ldl",
        "  description = LINK $out",
        "",
    ]
    objs = []
    for src in cpp + cu:
        rel = os.path.relpath(src, ROOT).replace(os.sep, "_")
        obj = os.path.join(BUILD_DIR, rel + ".o")
        rule = "nvcc" if src.endswith(".cu") else "cxx"
        lines.append(f"build {obj}: {rule} {src}")
        objs.append(obj)
    lines.append(f"build {LIB_PATH}: link_so {' '.join(objs)}")
    targets = [LIB_PATH]
    if with_bins:
        for name, srcs in (
            ("megray_test", sorted(glob.glob(os.path.join(ROOT, "tests", "cpp", "*.cpp")))),
            ("megray_bench", sorted(glob.glob(os.path.join(ROOT, "bench", "*.cpp")))),
            ("all_reduce_threads", [os.path.join(ROOT, "examples", "all_reduce_threads.cpp")]),
        ):
            if not srcs:
                continue
            bobjs = []
            for src in srcs:
                rel = os.path.relpath(src, ROOT).replace(os.sep, "_")
                obj = os.path.join(BUILD_DIR, rel + ".o")
                lines.append(f"build {obj}: cxx {src}")
                bobjs.append(obj)
            out = os.path.join(BUILD_DIR, name)
            lines.append(f"build {out}: link_bin {' '.join(bobjs)} | {LIB_PATH}")
            targets.append(out)
    lines.append("default " + " ".join(targets))
    path = os.path.join(BUILD_DIR, "build.ninja")
    text = "\n".join(lines) + "\n"
    old = open(path).read() if os.path.exists(path) else None
    if old != text:
        with open(path, "w") as f:
            f.write(text)
    return path


def build_sanitized(kind: str = "thread") -> str:
    """Builds the C++ test runner with the host code under a sanitizer (``thread``, or
    ``address,undefined``) into ``build/san_<kind>/megray_test`` and returns its path.  The host
    sources (rendezvous, host backend, factory, options, tracing, C++ tests) are compiled with
    ``-fsanitize``; the device objects of the normal build are linked as they are.  The runner
    is meant for CPU ranks: rendezvous, host backend and selection logic."""
    build(with_bins=True)
    tag = kind.replace(",", "_")
    out_dir = os.path.join(BUILD_DIR, "san_" + tag)
    os.makedirs(out_dir, exist_ok=True)
    cpp, cu = _sources()
    cpp += sorted(glob.glob(os.path.join(ROOT, "tests", "cpp", "*.cpp")))
    inc = f"-I{ROOT}/include -I{ROOT}/src -I{ROOT}/tests/cpp -I{CUDA_HOME}/include"
    nccl_inc = _nccl_include()
    defs = "-DMEGRAY_WITH_CUDA -DMEGRAY_WITH_NVL -DMEGRAY_WITH_SHM"
    if nccl_inc:
        defs += " -DMEGRAY_WITH_NCCL"
        if nccl_inc != "/usr/include":
            inc += f" -I{nccl_inc}"
    flags = f"-std=c++17 -O1 -g -fno-omit-frame-pointer -fPIC -fsanitize={kind} {defs} {inc}"
    lines = [
        "ninja_required_version = 1.3",
        f"cxxflags = {flags}",
        "rule cxx",
        "  command = g++ -MMD -MF $out.d $cxxflags -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "rule link",
        f"  command = g++ -fsanitize={kind} -o $out $in -L{CUDA_HOME}/lib64 -lcudart -lpthread -ldl -lrt",
        "",
    ]
    objs = []
    for src in cpp:
        obj = os.path.join(out_dir, os.path.relpath(src, ROOT).replace(os.sep, "_") + ".o")
        lines.append(f"build {obj}: cxx {src}")
        objs.append(obj)
    for src in cu:  # device objects of the normal build
        objs.append(os.path.join(BUILD_DIR, os.path.relpath(src, ROOT).replace(os.sep, "_") + ".o"))
    target = os.path.join(out_dir, "megray_test")
    lines.append(f"build {target}: link {' '.join(objs)}")
    lines.append(f"default {target}")
    path = os.path.join(out_dir, "build.ninja")
    text = "\n".join(lines) + "\n"
    if not os.path.exists(path) or open(path).read() != text:
        with open(path, "w") as f:
            f.write(text)
    res = subprocess.run([shutil.which("ninja"), "-f", path, "-C", out_dir], stdout=subprocess.PIPE,
                         stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout)
        raise RuntimeError("sanitizer build failed")
    return target


def build_debug_bounds() -> str:
    """Builds the C++ test runner with the collective kernels compiled under
    ``-DMEGRAY_DEBUG_BOUNDS`` into ``build/debug_bounds/megray_test`` and returns its path.  In
    that build every CTA-level copy or reduction first checks its whole range against the call's
    buffers and the heaps; a range outside them is skipped, recorded, and reported as
    MEGRAY_OUT_OF_BOUNDS.  All other objects are those of the normal build."""
    build(with_bins=True)
    out_dir = os.path.join(BUILD_DIR, "debug_bounds")
    if os.environ.get("MEGRAY_SKIP_BUILD") == "1" and os.path.exists(os.path.join(out_dir, "megray_test")):
        return os.path.join(out_dir, "megray_test")
    os.makedirs(out_dir, exist_ok=True)
    cpp, cu = _sources()
    inc = f"-I{ROOT}/include -I{ROOT}/src -I{CUDA_HOME}/include"
    nccl_inc = _nccl_include()
    defs = "-DMEGRAY_WITH_CUDA -DMEGRAY_WITH_NVL -DMEGRAY_WITH_SHM"
    if nccl_inc:
        defs += " -DMEGRAY_WITH_NCCL"
        if nccl_inc != "/usr/include":
            inc += f" -I{nccl_inc}"
    checked = [s for s in cu if os.path.basename(s) == "collectives.cu"]
    lines = [
        "ninja_required_version = 1.3",
        f"nvccflags = -std=c++17 -O3 {GENCODE} -lineinfo -Xcompiler -fPIC --expt-relaxed-constexpr "
        f"-DMEGRAY_DEBUG_BOUNDS {defs} {inc}",
        "rule nvcc",
        f"  command = {NVCC} -MD -MF $out.d $nvccflags -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "rule link",
        f"  command = {NVCC} {GENCODE} -o $out $in -L{CUDA_HOME}/lib64 -lcudart -lpthread -ldl -lrt",
        "",
    ]

    def normal_obj(src):
        return os.path.join(BUILD_DIR, os.path.relpath(src, ROOT).replace(os.sep, "_") + ".o")

    objs = []
    for src in cpp + cu:
        if src in checked:
            obj = os.path.join(out_dir, os.path.relpath(src, ROOT).replace(os.sep, "_") + ".o")
            lines.append(f"build {obj}: nvcc {src}")
            objs.append(obj)
        else:
            objs.append(normal_obj(src))
    for src in sorted(glob.glob(os.path.join(ROOT, "tests", "cpp", "*.cpp"))):
        objs.append(normal_obj(src))
    target = os.path.join(out_dir, "megray_test")
    lines.append(f"build {target}: link {' '.join(objs)}")
    lines.append(f"default {target}")
    path = os.path.join(out_dir, "build.ninja")
    text = "\n".join(lines) + "\n"
    if not os.path.exists(path) or open(path).read() != text:
        with open(path, "w") as f:
            f.write(text)
    res = subprocess.run([shutil.which("ninja"), "-f", path, "-C", out_dir], stdout=subprocess.PIPE,
                         stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout)
        raise RuntimeError("bounds-checked build failed")
    return target


def build(with_bins: bool = False, verbose: bool = False) -> str:
    """Compile everything that is stale; returns the path of libmegray.so.  With
    MEGRAY_SKIP_BUILD=1 in the environment nothing is compiled (a machine that received the
    binaries ready-made and should spend its time on something else)."""
    if os.environ.get("MEGRAY_SKIP_BUILD") == "1" and os.path.exists(LIB_PATH):
        return LIB_PATH
    ninja = shutil.which("ninja")
    if ninja is None:
        raise RuntimeError("ninja not found on PATH")
    path = write_ninja(with_bins)
    cmd = [ninja, "-f", path, "-C", BUILD_DIR]
    if verbose:
        cmd.append("-v")
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout)
        raise RuntimeError("native build failed")
    if verbose:
        print(res.stdout)
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--all", action="store_true", help="also build megray_test and megray_bench")
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("--sanitize", default=None, metavar="KIND",
                    help="build the C++ test runner with the host code under -fsanitize=KIND "
                         "(thread, or address,undefined) instead")
    ap.add_argument("--debug-bounds", action="store_true",
                    help="build the C++ test runner with range-checked collective kernels instead")
    a = ap.parse_args()
    if a.debug_bounds:
        print(build_debug_bounds())
    elif a.sanitize:
        print(build_sanitized(a.sanitize))
    else:
        print(build(with_bins=a.all, verbose=a.verbose))
