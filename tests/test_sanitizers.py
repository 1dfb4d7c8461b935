"""The host code (rendezvous server / client, host backend with its atomics, ring mailboxes and
shared regions, factory, options) under ThreadSanitizer and under AddressSanitizer +
UndefinedBehaviorSanitizer: the C++ test runner is rebuilt with -fsanitize and run with CPU ranks
as threads.  Any report fails the test.  (Device code cannot run under these tools; its checks are
the CPU oracles and the exhaustive small cases of the GPU tests.)"""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(kind, extra_env):
    from megray_b200 import build

    if shutil.which("g++") is None:
        pytest.skip("no g++")
    try:
        binary = build.build_sanitized(kind)
    except RuntimeError as e:  # a toolchain without the sanitizer runtime
        pytest.skip(f"sanitizer build unavailable: {e}")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", MEGRAY_LOG_LEVEL="3")
    env.update(extra_env)
    out = subprocess.run([binary], capture_output=True, text=True, timeout=900, env=env)
    text = out.stdout + out.stderr
    assert out.returncode == 0, text[-5000:]
    assert "0 failed" in out.stdout
    return text


def test_host_code_under_thread_sanitizer():
    text = _run("thread", {"TSAN_OPTIONS": "halt_on_error=0 second_deadlock_stack=1"})
    assert "ThreadSanitizer" not in text, text[-5000:]


def test_host_code_under_address_and_undefined_behaviour_sanitizers():
    text = _run("address,undefined", {"ASAN_OPTIONS": "detect_leaks=1", "UBSAN_OPTIONS": "print_stacktrace=1"})
    for marker in ("AddressSanitizer", "LeakSanitizer", "runtime error"):
        assert marker not in text, text[-5000:]
