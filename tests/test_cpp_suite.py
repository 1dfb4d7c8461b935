"""Runs the C++ test binary (tests/cpp/megray_test.cpp).  Without a GPU it covers the
rendezvous and the host backend; on a GPU box the same binary adds the NCCL and NVL cases
when one GPU per rank is available."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _binary():
    from megray_b200 import build

    build.build(with_bins=True)
    path = os.path.join(ROOT, "build", "megray_test")
    assert os.path.exists(path)
    return path


def _run(extra_env=None):
    env = dict(os.environ, MEGRAY_LOG_LEVEL="3")
    env.update(extra_env or {})
    out = subprocess.run([_binary()], capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stdout[-4000:] + out.stderr[-2000:]
    return out.stdout


def test_cpp_suite_on_cpu():
    out = _run({"CUDA_VISIBLE_DEVICES": ""})
    assert "0 failed" in out


@pytest.mark.gpu
def test_cpp_suite_with_gpus():
    out = _run()
    assert "0 failed" in out


def test_example_program_runs_on_the_host_backend():
    _binary()  # builds the example along with the test runner
    exe = os.path.join(ROOT, "build", "all_reduce_threads")
    out = subprocess.run([exe, "3", "shm"], capture_output=True, text=True, timeout=120,
                         env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert out.returncode == 0 and "ok" in out.stdout, out.stdout + out.stderr
