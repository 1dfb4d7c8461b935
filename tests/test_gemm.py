"""tcgen05 GEMM kernel against float32 PyTorch: all four operand layouts, ragged sizes, the
accumulate / SwiGLU / dSwiGLU epilogues, grouped (per-expert) problems."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def mk(r, c, scale=0.5):
    return (torch.randn(r, c, device="cuda") * scale).to(torch.bfloat16)


def close(got, want, tol=2e-2):
    from megray_b200.ops import gemm_error_flag

    torch.cuda.synchronize()
    assert int(gemm_error_flag().item()) == 0
    scale = max(float(want.abs().max()), 1.0)
    err = float((got.float() - want.float()).abs().max())
    assert err <= tol * scale, f"max error {err} vs scale {scale}"


# variant 0 picks a CTA-pair kernel (cta_group::2; 256 x 256 tiles, or 512 x 256 for large
# problems) when M > 128, 1 forces the single-CTA kernel (128 x 256 tiles), 2 the 256-row
# pair tile, 3 the 512-row pair tile (two sub-tiles with one accumulator each)
@pytest.mark.parametrize("variant", [0, 1, 2, 3])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (300, 264, 200), (1024, 2048, 512),
                                   (129, 8, 8), (64, 1000, 72), (2048, 1024, 1536)])
def test_nt(M, N, K, variant):
    from megray_b200.ops import gemm

    torch.manual_seed(0)
    a, b = mk(M, K), mk(N, K)
    close(gemm(a, b, variant=variant), a.float() @ b.float().t())


@pytest.mark.parametrize("variant", [0, 1, 3])
@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (True, True)])
def test_transposed_operands(a_mn, b_mn, variant):
    from megray_b200.ops import gemm

    torch.manual_seed(1)
    M, N, K = 384, 520, 320
    a = mk(K, M) if a_mn else mk(M, K)
    b = mk(K, N) if b_mn else mk(N, K)
    want = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
    close(gemm(a, b, a_mn=a_mn, b_mn=b_mn, variant=variant), want)


@pytest.mark.parametrize("variant,sm_limit", [(0, 0), (2, 0), (3, 0), (3, 16)])
def test_many_tiles_per_cta_pair_exercise_the_ring_and_both_accumulators(variant, sm_limit):
    from megray_b200.ops import gemm

    torch.manual_seed(7)
    M, N, K = 4096, 6144, 1088  # 16 x 24 tiles over <= 74 pairs: several tiles each, 17 k-steps
    a, b = mk(M, K), mk(N, K)
    out = gemm(a, b, variant=variant, sm_limit=sm_limit)
    idx = torch.randint(0, M, (64,), device="cuda")
    close(out[idx], a[idx].float() @ b.float().t(), tol=3e-2)


@pytest.mark.parametrize("variant", [0, 1, 3])
@pytest.mark.parametrize("M,N,K", [(300, 264, 200), (1024, 2048, 512), (129, 8, 64)])
def test_row_segment_store_epilogue(M, N, K, variant):
    from megray_b200.ops import EPI_STORE_ROWS, gemm

    torch.manual_seed(8)
    a, b = mk(M, K), mk(N, K)
    out = torch.full((M, N), 3.0, device="cuda", dtype=torch.bfloat16)
    gemm(a, b, out, epilogue=EPI_STORE_ROWS, variant=variant)
    close(out, a.float() @ b.float().t())


def test_accumulate():
    from megray_b200.ops import EPI_ACCUM, gemm

    torch.manual_seed(2)
    a, b, d = mk(256, 128), mk(512, 128), mk(256, 512)
    d0 = d.clone()
    gemm(a, b, d, epilogue=EPI_ACCUM)
    close(d, a.float() @ b.float().t() + d0.float())


@pytest.mark.parametrize("variant", [0, 1, 3])
def test_swiglu_and_its_derivative(variant):
    from megray_b200.ops import EPI_DSWIGLU, EPI_SWIGLU, gemm

    torch.manual_seed(3)
    M, F, K = 384, 640, 256
    x, w = mk(M, K), mk(2 * F, K, 0.1)
    gu, h = gemm(x, w, epilogue=EPI_SWIGLU, n=F, variant=variant)
    ref = x.float() @ w.float().t()
    close(gu, ref)
    close(h, torch.nn.functional.silu(ref[:, :F]) * ref[:, F:])
    # backward of h = silu(g) * u through the fused epilogue of dH = dY @ Wd
    dy, wd = mk(M, K), mk(K, F, 0.1)
    dgu = gemm(dy, wd, b_mn=True, epilogue=EPI_DSWIGLU, aux=gu, n=F, variant=variant)
    g = gu[:, :F].float().requires_grad_()
    u = gu[:, F:].float().requires_grad_()
    (torch.nn.functional.silu(g) * u).backward(dy.float() @ wd.float())
    close(dgu, torch.cat([g.grad, u.grad], 1))


def test_grouped_rows_pick_their_expert_weights():
    from megray_b200.ops import gemm

    torch.manual_seed(4)
    E, N, K = 3, 256, 192
    blocks = [0, 2, 2, -1, 1]  # group of each 128-row block; -1 = padding block (left untouched)
    M = 128 * len(blocks)
    x, w = mk(M, K), mk(E * N, K)
    out = torch.full((M, N), 7.0, device="cuda", dtype=torch.bfloat16)
    gemm(x, w, out, n=N, m_block_group=torch.tensor(blocks, device="cuda", dtype=torch.int32),
         group_rows_b=N, groups=E)
    torch.cuda.synchronize()
    for i, e in enumerate(blocks):
        rows = slice(128 * i, 128 * (i + 1))
        if e < 0:
            assert float((out[rows].float() - 7.0).abs().max()) == 0.0
        else:
            close(out[rows], x[rows].float() @ w[e * N:(e + 1) * N].float().t())


def test_grouped_k_ranges_give_one_weight_gradient_per_expert():
    from megray_b200.ops import gemm

    torch.manual_seed(5)
    E, M, N = 3, 256, 384
    kb = [0, 256, 256]      # expert 1 has no rows: its gradient must be zero
    ke = [256, 256, 640]
    T = 640
    dy, x = mk(T, M), mk(T, N)
    out = gemm(dy, x, a_mn=True, b_mn=True, groups=E,
               k_begin=torch.tensor(kb, device="cuda", dtype=torch.int32),
               k_end=torch.tensor(ke, device="cuda", dtype=torch.int32))
    assert out.shape == (E * M, N)
    for e in range(E):
        want = dy[kb[e]:ke[e]].float().t() @ x[kb[e]:ke[e]].float()
        close(out[e * M:(e + 1) * M], want)


def test_bad_arguments_are_rejected_not_launched():
    from megray_b200.ops import gemm

    a, b = mk(128, 64), mk(256, 72)
    with pytest.raises(ValueError):
        gemm(a, b)
    with pytest.raises(ValueError):
        gemm(a.float(), b)


@pytest.mark.parametrize("M,N,K,splits", [(1024, 512, 8192, 2), (1024, 512, 8192 + 64, 3), (512, 264, 4096, 8),
                                          (768, 256, 4096, 4)])
@pytest.mark.parametrize("a_mn,b_mn", [(True, True), (False, False)])
def test_split_k_matches_the_plain_product(M, N, K, splits, a_mn, b_mn):
    """K cut into ranges, one float32 partial product per range on the kernel's grouped-K form
    (512-row tile when M allows), summed in float32 by the N-way reduce kernel and rounded once."""
    from megray_b200.ops import gemm_split_k

    torch.manual_seed(11)
    a = mk(K, M) if a_mn else mk(M, K)
    b = mk(K, N) if b_mn else mk(N, K)
    out = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    gemm_split_k(a, b, out, splits, a_mn=a_mn, b_mn=b_mn)
    want = (a.float().t() if a_mn else a.float()) @ (b.float() if b_mn else b.float().t())
    close(out, want, tol=1e-2)
