"""The GEMM kernel's tile raster, evaluated on the host (no GPU): for every variant, epilogue
tiling, rotation and ragged size, the tiles of a problem cover the output exactly once, start on
the tile grid, and the rotation puts the asked row block first."""
import ctypes as C

import pytest

from megray_b200 import _lib
from megray_b200._lib import GemmArgs

EPI_STORE, EPI_SWIGLU = 0, 1


def schedule(M, N, K, variant=0, epilogue=EPI_STORE, m_rot=0, sms=148):
    lib = _lib.load()
    a = GemmArgs()
    a.M, a.N, a.K = M, N, K
    a.variant, a.epilogue, a.m_rot = variant, epilogue, m_rot
    a.aux_off = N
    cap = 1 << 16
    buf = (C.c_int * (4 * cap))()
    n = lib.megray_gemm_tile_schedule(C.byref(a), sms, buf, cap)
    assert 0 <= n <= cap
    return [(buf[4 * t], buf[4 * t + 1], buf[4 * t + 2], buf[4 * t + 3]) for t in range(n)]


@pytest.mark.parametrize("variant,tile_m", [(1, 128), (2, 256), (3, 512)])
@pytest.mark.parametrize("M,N", [(4096, 8192), (3584, 2048), (300, 264), (8192 + 128, 512 + 8)])
@pytest.mark.parametrize("epilogue,tile_n", [(EPI_STORE, 256), (EPI_SWIGLU, 128)])
@pytest.mark.parametrize("m_rot", [0, 1024])
def test_tiles_cover_the_output_exactly_once(variant, tile_m, M, N, epilogue, tile_n, m_rot):
    if M <= 128:
        tile_m = 128
    tiles = schedule(M, N, 4096, variant, epilogue, m_rot % M)
    assert all(t[2] == tile_m and t[3] == tile_n for t in tiles)
    mb, nb = -(-M // tile_m), -(-N // tile_n)
    assert len(tiles) == mb * nb
    seen = {(m0, n0) for m0, n0, _, _ in tiles}
    assert len(seen) == len(tiles)
    assert seen == {(i * tile_m, j * tile_n) for i in range(mb) for j in range(nb)}


def test_rotation_starts_with_the_asked_row_block_and_keeps_column_sweeps_together():
    tiles = schedule(32768, 8192, 8192, variant=3, m_rot=3 * 4096)
    assert tiles[0][0] == 3 * 4096
    # a sweep of group_m = 8 row blocks x all 32 column tiles comes before the next row blocks
    first = tiles[: 8 * 32]
    assert {t[0] for t in first} == {3 * 4096 + 512 * i for i in range(8)}


def test_automatic_variant_picks_the_wide_tile_only_for_large_dense_problems():
    assert schedule(32768, 8192, 8192)[0][2] == 512
    assert schedule(32768, 8192, 1024)[0][2] == 256     # short K loop: epilogue would show
    assert schedule(512, 8192, 8192)[0][2] == 256       # M below 1024
    assert schedule(2048, 1024, 8192)[0][2] == 256      # too few tiles for 74 CTA pairs
    assert schedule(128, 1024, 8192)[0][2] == 128


def test_grouped_problems_have_no_host_schedule():
    lib = _lib.load()
    a = GemmArgs()
    a.M, a.N, a.K = 1024, 1024, 1024
    a.k_begin = 16  # any non-null device address: grouped-K ranges live on the device
    buf = (C.c_int * 16)()
    assert lib.megray_gemm_tile_schedule(C.byref(a), 148, buf, 4) == -1


def test_split_k_choice_follows_the_wave_arithmetic():
    """No GPU: the number of K ranges picked for the weight gradients of the sharded MLP."""
    from megray_b200.ops.gemm import pick_split_k

    T, d, F = 32768, 8192, 28672
    # plenty of tiles: no split
    assert pick_split_k(d, F, T) == 1 and pick_split_k(2 * F, d, T) == 1
    # 8-way shard: 224 tiles on 74 CTA pairs would take 4 waves for the work of 3.03
    assert pick_split_k(d, F // 8, T) > 1
    # 448 tiles lose half a wave in seven: not worth writing and re-reading float32 partial products
    assert pick_split_k(2 * F // 8, d, T) == 1
    # short K or ragged M: never
    assert pick_split_k(d, F // 8, 2048) == 1 and pick_split_k(d + 8, F // 8, T) == 1
