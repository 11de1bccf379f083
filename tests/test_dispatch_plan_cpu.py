"""The matmul dispatch's planning, checked without a GPU: which path a shape takes and how much
scratch it asks for (the queries read shapes only; with no device they assume B200's 148 SMs).
The expected values restate the plans: k cut into work units, stream-mode teams and slots,
256-row tiles, rows past a tile boundary on the bandwidth-bound kernel."""
import ctypes
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as ge  # noqa: E402

pkg = ge.load_package()
from polarai_framework_b200.capi import Arg  # noqa: E402

TC, SKINNY, FFMA = 0, 1, 2
SMS = 148


@pytest.fixture(scope="module")
def lib():
    return pkg.lib()


def ws(lib, tl, tr, m, n, k):
    return int(lib.cdll.polar_b200_fmatmul_workspace_bytes(tl, tr, m, n, k))


def test_paths(lib):
    path = lib.cdll.polar_b200_fmatmul_path
    assert path(0, 0, 65536, 4096, 784) == TC           # MLP layer 1
    assert path(1, 0, 784, 4096, 65536) == TC           # its weight gradient
    assert path(0, 0, 65536, 10, 4096) == SKINNY        # 10 outputs: small n, K-major left
    assert path(1, 0, 4096, 10, 65536) == SKINNY        # small n, split k
    assert path(0, 1, 65536, 4096, 10) == SKINNY        # small k
    assert path(0, 0, 33, 17, 50) == FFMA               # below one tile
    assert path(0, 0, 512, 510, 512) == FFMA            # row pitch TMA cannot describe (n % 4 != 0, right stored [k, n])


def tc_plan(lib, tl, tr, m, n, k):
    rows, exchanged, splits = ctypes.c_int(-1), ctypes.c_int(-1), ctypes.c_int(-1)
    lib.cdll.polar_b200_fmatmul_tc_plan(tl, tr, m, n, k, ctypes.byref(rows), ctypes.byref(exchanged),
                                        ctypes.byref(splits))
    return rows.value, exchanged.value, splits.value


def test_tile_height_and_orientation(lib):
    # MLP layer 1 (k = 784: the epilogue is a visible share of a tile): 256-row tiles, operands in
    # exchanged roles so that the epilogue stores whole lines, whole tiles - at the full batch and
    # at the per-GPU batch of the 8-GPU run (512 tiles in four waves still beat 1024 128-row tiles)
    assert tc_plan(lib, 0, 0, 65536, 4096, 784) == (256, 1, 1)
    assert tc_plan(lib, 0, 0, 8192, 4096, 784) == (256, 1, 1)
    # long sums: the epilogue does not matter, the plain orientation stays
    assert tc_plan(lib, 0, 0, 8192, 8192, 8192)[:2] == (256, 0)
    # the weight gradient (stream mode or fixed cuts; rows past the tile boundary beside it)
    assert tc_plan(lib, 1, 0, 784, 4096, 8192) == (256, 0, 0)
    rows, exchanged, splits = tc_plan(lib, 1, 0, 784, 4096, 65536)
    assert (rows, exchanged) == (256, 0) and splits == 3
    # a short sum below the exchange's range, and one tile row only: 128-row tiles
    assert tc_plan(lib, 0, 0, 128, 512, 64) == (128, 0, 1)


def test_whole_waves_need_no_scratch(lib):
    assert ws(lib, 0, 0, 65536, 4096, 784) == 0
    assert ws(lib, 0, 0, 8192, 8192, 8192) == 0
    assert ws(lib, 0, 1, 8192, 4096, 784) == 0


def test_weight_gradient_of_the_full_batch(lib):
    # 784 = 3 * 256 + 16 rows, k = 65536: 768 rows on the tensor cores in 256-row tiles (48 tiles,
    # three work units each fill 144 of 148 SMs), 16 rows on the split-k small-n kernel AT THE
    # SAME TIME on the library's side stream: the two scratch areas follow one another
    tc = 3 * 768 * 4096 * 4
    splits_ragged = min((2 * SMS + 3) // 4, 65536 // 128)          # two CTAs per SM over 4 column blocks
    ragged = splits_ragged * 4096 * 16 * 4
    assert tc % 256 == 0
    assert ws(lib, 1, 0, 784, 4096, 65536) == tc + ragged


def test_weight_gradient_of_an_eighth_of_the_batch(lib):
    # k = 8192 (the per-GPU shape of the 8-GPU run): the same division - 768 rows in 256-row tiles,
    # stream mode (49 teams of 3 CTAs, slots [row tile][team + column] of 256 x 256 floats), the
    # 16 rows beside it
    teams = SMS // 3
    tc = 3 * (teams + 16) * 256 * 256 * 4
    ragged = min((2 * SMS + 3) // 4, 8192 // 128) * 4096 * 16 * 4
    assert ws(lib, 1, 0, 784, 4096, 8192) == tc + ragged
    # below 4096 the extra pass over the right operand would outlast the tiles: no division
    assert ws(lib, 1, 0, 784, 4096, 2048) != 0
    assert ws(lib, 1, 0, 784, 4096, 2048) % (128 * 256 * 4) == 0


def test_long_k_and_few_tiles_use_fixed_cuts(lib):
    # 1024 x 1024 x 65536: 256-row tiles -> 16 tiles; k too long for stream mode; 8 cuts fill 128 SMs
    got = ws(lib, 0, 0, 1024, 1024, 65536)
    assert got % (1024 * 1024 * 4) == 0 and 2 <= got // (1024 * 1024 * 4) <= 8


def test_by_name_query_agrees_and_knows_the_fused_forms(lib):
    q = lib.cdll.polar_b200_launch_workspace_bytes

    def args(*shapes):
        arr = (Arg * len(shapes))()
        keep = []
        for i, shp in enumerate(shapes):
            s = (ctypes.c_uint64 * len(shp))(*shp)
            keep.append(s)
            arr[i].is_tensor, arr[i].tensor.dims, arr[i].tensor.shape = 1, len(shp), s
        return arr, keep

    a, keep = args((65536, 784), (65536, 4096), (784, 4096))
    assert int(q(b"fmatmul_t_f", a, 3)) == ws(lib, 1, 0, 784, 4096, 65536)
    # with the sigmoid in the tensor-core epilogue the ragged rows stay on the tensor cores:
    # 784 rows pad to four 256-row tiles, 64 tiles, two cuts fill 128 SMs
    fused = int(q(b"fmatmul_t_f_sigmoid", a, 3))
    assert fused != ws(lib, 1, 0, 784, 4096, 65536) and fused % (784 * 4096 * 4) == 0
    b, keep2 = args((65536, 4096), (4096, 10), (65536, 10))
    assert int(q(b"fmatmul_f_f", b, 3)) == 0 and int(q(b"fadd", b, 3)) == 0
    assert int(q(b"fmatmul_f_f_nonsense", b, 3)) == 0
