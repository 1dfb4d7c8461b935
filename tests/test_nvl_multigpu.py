"""Native NVL backend on real GPUs, one process per GPU (launched here with torchrun on
2 GPUs; NVLS is off and kernels use plain peer loads/stores).  Covers: every collective against
a CPU reference over dtypes and ragged sizes, the fused scale/cast all_reduce, send/recv, the
tensor-parallel model against its single-GPU evaluation (fused and unfused paths), and the
device-side wait limit: a rank that skips a collective makes its peer's kernel give up after the
limit and report MEGRAY_TIMEOUT, with the GPU still usable."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


NPROC = int(os.environ.get("MEGRAY_TEST_NPROC", "2"))  # ranks (= GPUs) per test; 2, 4 or 8


def torchrun(script, nproc=None, env=None, timeout=600):
    nproc = nproc or NPROC
    e = dict(os.environ, NCCL_NVLS_ENABLE="0", MEGRAY_NVLS="0", MEGRAY_LOG_LEVEL="2")
    e.update(env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", "29641", os.path.join(ROOT, "tests", "multigpu", script)]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=e, cwd=ROOT)
    assert out.returncode == 0, out.stdout[-5000:] + out.stderr[-3000:]
    return out.stdout


def test_collectives_against_cpu_reference():
    out = torchrun("collectives.py")
    assert out.count("RANK_OK") == NPROC, out[-3000:]


def test_collectives_with_the_pull_form_of_small_exchanges():
    # the default is the push form for small all_gather / all_to_all
    out = torchrun("collectives.py", env={"MEGRAY_PUSH_EXCHANGE": "0"})
    assert out.count("RANK_OK") == NPROC, out[-3000:]


def test_tensor_parallel_model_matches_single_gpu():
    out = torchrun("tp_model.py", env={"MEGRAY_HEAP_MB": "1024"})
    assert out.count("RANK_OK") == NPROC, out[-3000:]


def test_tensor_parallel_model_on_the_wide_gemm_tile():
    # the 512-row tile: per-sub-tile shard flags and owners, both epilogue groups, late-joining
    # second group behind the fused all_gather
    out = torchrun("tp_model.py", env={"MEGRAY_HEAP_MB": "1024", "MEGRAY_GEMM_VARIANT": "3"})
    assert out.count("RANK_OK") == NPROC, out[-3000:]


@pytest.mark.parametrize("variant", ["2", "3"])
def test_fused_kernels_with_many_tiles_per_cta_pair(variant):
    # the gather is still in flight while tiles retire; on the wide tile (variant 3) the second
    # epilogue group joins in the middle of the tile sequence
    out = torchrun("fused_many_tiles.py", env={"MEGRAY_HEAP_MB": "1024", "MEGRAY_GEMM_VARIANT": variant})
    assert out.count("RANK_OK") == NPROC, out[-3000:]


def test_expert_parallel_moe_matches_single_gpu():
    out = torchrun("moe.py", env={"MEGRAY_HEAP_MB": "1024"})
    assert out.count("RANK_OK") == NPROC, out[-3000:]


def test_single_pass_collectives_on_heap_tensors():
    out = torchrun("direct.py", env={"MEGRAY_HEAP_MB": "4096"})
    print("\n".join(l for l in out.splitlines() if l.startswith(("BW", "RANK_OK"))))
    assert out.count("RANK_OK") == NPROC, out[-3000:]
    assert "nvls_calls=0" in out


@pytest.mark.parametrize("ipc_cache", ["0", "1"])
def test_single_pass_collectives_on_registered_user_buffers(ipc_cache):
    # "0": explicit registration maps the buffers (one host exchange per buffer); "1": allocations
    # are exported on first use and registering only does that ahead of time
    out = torchrun("registered.py", env={"MEGRAY_IPC_CACHE": ipc_cache})
    assert out.count("RANK_OK") == NPROC, out[-3000:]


def test_single_pass_collectives_through_nvswitch_multimem():
    # falls back to peer loads/stores (with a warning) where multicast is unavailable
    out = torchrun("direct.py", env={"MEGRAY_HEAP_MB": "4096", "MEGRAY_NVLS": "1", "NCCL_NVLS_ENABLE": "1"})
    print("\n".join(l for l in out.splitlines() if l.startswith(("BW", "RANK_OK"))))
    assert out.count("RANK_OK") == NPROC, out[-3000:]


def test_device_wait_limit_reports_timeout_and_keeps_the_gpu_usable():
    out = torchrun("timeout.py")
    assert out.count("RANK_OK") == NPROC, out[-3000:]


def test_fused_call_wait_limit_reports_timeout_and_keeps_the_gpu_usable():
    out = torchrun("fused_timeout.py", nproc=2, env={"MEGRAY_HEAP_MB": "512"})
    assert out.count("RANK_OK") == 2, out[-3000:]


def test_fused_reduce_scatter_on_a_recreated_communicator():
    out = torchrun("recreate.py", env={"MEGRAY_HEAP_MB": "512"})
    assert out.count("RANK_OK") == NPROC, out[-3000:]


def test_send_recv_overlaps_a_native_collective_when_its_join_is_postponed():
    out = torchrun("p2p_overlap.py", nproc=2)
    print("\n".join(l for l in out.splitlines() if l.startswith("RANK_OK")))
    assert out.count("RANK_OK") == 2, out[-3000:]


def test_full_size_fused_step_matches_the_unfused_step_elementwise():
    out = torchrun("tp_fullsize_fused_vs_unfused.py", env={"MEGRAY_HEAP_MB": "6144"}, timeout=900)
    print("\n".join(l for l in out.splitlines() if "differ" in l))
    assert out.count("RANK_OK") == NPROC, out[-3000:]


def test_ordinary_tensors_of_separate_processes_take_the_single_pass_kernels():
    # allocations are exported and mapped on first use (asymmetric first use, freed and
    # re-allocated memory, views at odd offsets)
    out = torchrun("ipc_cache.py")
    assert out.count("RANK_OK") == NPROC, out[-3000:]


def test_collectives_on_the_staged_paths_when_nothing_is_exported():
    out = torchrun("collectives.py", env={"MEGRAY_IPC_CACHE": "0"})
    assert out.count("RANK_OK") == NPROC, out[-3000:]
