"""The fused tensor-parallel kernels on a group of one rank (one GPU): all_gather -> GEMM gathers
only its own shard, and GEMM -> reduce_scatter owns every row, so all its tiles take the path
that waits for the (zero) other ranks' partial tiles, adds the residual and writes the shard.
Compared with a float32 PyTorch evaluation.  The multi-rank versions of these checks are in
tests/multigpu/."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def group():
    import megray_b200 as mr

    torch.cuda.set_device(0)
    port = mr.get_free_port()
    server = mr.Server(1, port)
    comm = mr.Communicator(1, 0, "nvl").init("127.0.0.1", port)
    yield comm
    comm.close()
    server.close()


def _close(got, want, tol=3e-2):
    torch.cuda.synchronize()
    scale = max(float(want.float().abs().max()), 1e-6)
    return float((got.float() - want.float()).abs().max()) / scale < tol


@pytest.mark.parametrize("variant", [0, 2, 3])
def test_fused_calls_on_a_single_rank_group(group, variant):
    from megray_b200.ops import gemm_error_flag
    from megray_b200.parallel.tensor_parallel import TensorParallelOps

    comm = group
    dev = torch.device("cuda", 0)
    T, d, fl = 2048, 1024, 768
    g = torch.Generator(device=dev).manual_seed(7)
    x = (torch.randn(T, d, device=dev, generator=g) * 0.5).to(torch.bfloat16)
    w_gu = (torch.randn(2 * fl, d, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    w_dn = (torch.randn(d, fl, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    res = (torch.randn(T, d, device=dev, generator=g) * 0.5).to(torch.bfloat16)
    tp = TensorParallelOps(comm, T, d, fused=True)
    assert tp.fused
    tp.variant = variant
    xg = tp.full_buffer()
    xg.copy_(x)
    gu = torch.empty(T, 2 * fl, dtype=torch.bfloat16, device=dev)
    h = torch.empty(T, fl, dtype=torch.bfloat16, device=dev)
    out = torch.empty(T, d, dtype=torch.bfloat16, device=dev)
    gu_ref = x.float() @ w_gu.float().t()
    h_ref = torch.nn.functional.silu(gu_ref[:, :fl]) * gu_ref[:, fl:]
    for rep in range(3):  # the delivery counters and flag epochs are reused call after call
        tp.ag_gemm_swiglu(xg, w_gu, gu, h, fl)
        assert _close(gu, gu_ref) and _close(h, h_ref)
        out.zero_()
        tp.gemm_rs(h, w_dn, None, out, residual=res if rep == 1 else None)
        want = h.float() @ w_dn.float().t() + (res.float() if rep == 1 else 0)
        assert _close(out, want), f"gemm_rs rep {rep}"
        assert int(gemm_error_flag(dev).item()) == 0 and comm.status == 0
