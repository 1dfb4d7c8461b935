"""The CMake build for C++ users configures for sm_100a by default (tcgen05 / TMEM / TMA code does
not assemble for anything else) and lets the caller override the architecture."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NVCC = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")


def _configure(tmp_path, *extra):
    if shutil.which("cmake") is None or not os.path.exists(NVCC):
        pytest.skip("cmake or nvcc not available")
    out = subprocess.run(["cmake", "-S", ROOT, "-B", str(tmp_path), f"-DCMAKE_CUDA_COMPILER={NVCC}", *extra],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    cache = open(os.path.join(str(tmp_path), "CMakeCache.txt")).read()
    return [line for line in cache.splitlines() if line.startswith("CMAKE_CUDA_ARCHITECTURES")]


def test_default_architecture_is_sm_100a(tmp_path):
    lines = _configure(tmp_path)
    assert lines == [] or all(line.endswith("=100a") for line in lines), lines
    # the generated compile rules carry the architecture
    flags = subprocess.run(["grep", "-rl", "100a", str(tmp_path)], capture_output=True, text=True).stdout
    assert flags.strip(), "no generated file mentions 100a"


def test_architecture_can_be_overridden(tmp_path):
    lines = _configure(tmp_path, "-DCMAKE_CUDA_ARCHITECTURES=100a-real")
    assert any(line.endswith("=100a-real") for line in lines), lines
