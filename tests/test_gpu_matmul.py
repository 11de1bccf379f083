"""GPU parity of fmatmul (all four transpose forms) against the CPU oracle.

Error metric: |c - ref| / sum_k |a||b| with ref accumulated in double; the bound
is 1e-4 (the fp32-sequential reference order itself lies within it).  Small
integer cases are bit-exact."""
import numpy as np
import pytest

from conftest import expected_of, run_kat

pytestmark = pytest.mark.gpu

TOL = 1e-4


@pytest.fixture(scope="module")
def gpu():
    import __graft_entry__ as ge
    ge.load_package()
    from polarai_framework_b200.device_builtins import HostBuiltins
    return HostBuiltins("cuda:0")


@pytest.fixture(scope="module")
def par_oracle():
    from oracle import oracle as orc
    o = orc.Oracle()
    o.set_threads(o.max_threads())
    return o


def operands(rng, tl, tr, m, n, k):
    left = rng.uniform(-1, 1, (k, m) if tl else (m, k)).astype(np.float32)
    right = rng.uniform(-1, 1, (n, k) if tr else (k, n)).astype(np.float32)
    return left, right


def rel_err(got, ref, mag):
    return float(np.max(np.abs(got.astype(np.float64) - ref) / mag))


def test_reference_kats_bit_exact(gpu, kats):
    for case in kats:
        if case["builtin"] != "fmatmul":
            continue
        got = run_kat(gpu, case)
        assert np.array_equal(got.ravel(), expected_of(case)), case["name"]


@pytest.mark.parametrize("tl", [0, 1])
@pytest.mark.parametrize("tr", [0, 1])
def test_seeded_fixture(gpu, seeded, par_oracle, tl, tr):
    tag = f"mm_{'t' if tl else 'f'}_{'t' if tr else 'f'}"
    l, r = seeded[tag + "_left"], seeded[tag + "_right"]
    ref, mag = par_oracle.fmatmul_f64(tl, tr, l, r)
    for which in ("auto", "ffma"):
        assert rel_err(gpu.fmatmul(tl, tr, l, r, which=which), ref, mag) <= TOL
    assert rel_err(seeded[tag + "_out"], ref, mag) <= TOL


SHAPES = [
    (128, 256, 32), (128, 128, 64), (64, 32, 32),          # one tile, one or two slabs
    (200, 300, 100), (260, 516, 36), (1000, 40, 2000),      # ragged m/n/k tails (multiples of 4)
    (512, 512, 512), (256, 784, 128), (784, 128, 256),      # sizes from the logistic-regression / MLP configs
    (1024, 1024, 1024),
    (2304, 2048, 96),                                       # 144 or 288 tiles: several tiles per persistent CTA
    (4224, 1280, 64),
    (1024, 1024, 2048), (784, 512, 4096),                   # few tiles, long k: the default path cuts k into work units
    (1280, 4096, 64), (2560, 4000, 48),                     # 160 tiles on 148 SMs: the 12 tiles of the last wave run as column halves
]


@pytest.mark.parametrize("tl", [0, 1])
@pytest.mark.parametrize("tr", [0, 1])
@pytest.mark.parametrize("shape", SHAPES)
def test_tensor_core_path(gpu, par_oracle, tl, tr, shape):
    m, n, k = shape
    rng = np.random.default_rng(m * 7 + n * 3 + k + tl * 2 + tr)
    l, r = operands(rng, tl, tr, m, n, k)
    ref, mag = par_oracle.fmatmul_f64(tl, tr, l, r)
    # 512: the 256 x 256 tile configuration; + 1000: the operands exchange roles (the transposed
    # product is computed and its tiles are stored transposed)
    for tile_n in (256, 128, 512, 1256, 1128, 1512):
        for slab_k in ((16,) if tile_n % 1000 == 512 else (16, 32)):
            got = gpu.fmatmul(tl, tr, l, r, which="tc", tile_n=tile_n, slab_k=slab_k)
            err = rel_err(got, ref, mag)
            assert err <= TOL, (tile_n, slab_k, err)
            assert err <= 5e-6, (tile_n, slab_k, err)   # what the three-product split actually delivers
    auto = gpu.fmatmul(tl, tr, l, r)
    assert rel_err(auto, ref, mag) <= TOL
    assert gpu.d.device_status() == 0


@pytest.mark.parametrize("tl", [0, 1])
@pytest.mark.parametrize("tr", [0, 1])
@pytest.mark.parametrize("shape", SHAPES + [(784, 4096, 8192), (300, 700, 5000), (128, 256, 16 * 1000)])
def test_k_cut_into_work_units_and_stream_mode(gpu, par_oracle, tl, tr, shape):
    # fixed cuts of k (2, 3, 8 units per tile) and stream mode (-1: equal shares of all slabs per
    # CTA, tiles continued by the next CTA) give the product to the same accuracy, run to run
    # the same bits, for every transpose form and ragged shape
    m, n, k = shape
    if m * n * k > 1 << 33 and (tl, tr) != (1, 0):
        pytest.skip("the large case runs in the form the MLP's weight gradient uses")
    rng = np.random.default_rng(m * 5 + n * 3 + k + tl * 2 + tr)
    l, r = operands(rng, tl, tr, m, n, k)
    ref, mag = par_oracle.fmatmul_f64(tl, tr, l, r)
    for splits in (-1, 2, 3, 8):
        if splits > 1 and ((m * n) & 3 or (k + 15) // 16 < splits):
            continue
        for tile_n, slab_k in (((256, 16), (256, 32), (512, 16)) if splits == -1 else
                               ((256, 16), (512, 16), (1256, 16), (1512, 16))):
            got = gpu.fmatmul(tl, tr, l, r, which="tc", tile_n=tile_n, slab_k=slab_k, splits=splits)
            assert rel_err(got, ref, mag) <= 5e-6, (splits, tile_n, slab_k)
            again = gpu.fmatmul(tl, tr, l, r, which="tc", tile_n=tile_n, slab_k=slab_k, splits=splits)
            assert np.array_equal(got.view(np.uint32), again.view(np.uint32)), (splits, tile_n, slab_k)
    assert gpu.d.device_status() == 0


@pytest.mark.parametrize("tl,tr,m,n,k", [
    (0, 0, 256, 1, 784),      # logistic regression forward
    (1, 0, 784, 1, 256),      # X^T dZ
    (0, 0, 1024, 10, 4096),   # hidden -> 10 outputs
    (1, 0, 4096, 10, 1024),   # H^T dZ2
    (0, 1, 1024, 4096, 10),   # dZ2 W2^T
    (0, 0, 33, 17, 5), (1, 1, 7, 9, 1027), (0, 1, 1, 1, 1),
    # one tiny dimension: the bandwidth-bound CUDA-core kernels
    (0, 0, 1000, 3, 512), (0, 1, 1000, 16, 260), (0, 0, 5, 10, 4096), (0, 0, 4099, 10, 2052),
    (1, 0, 1028, 5, 1000), (1, 1, 516, 2, 300), (1, 0, 4096, 10, 30000), (1, 0, 4, 1, 33),
    (0, 0, 100, 300, 16), (1, 1, 100, 302, 7), (1, 0, 64, 4096, 4), (0, 1, 70000, 64, 10),
])
def test_shapes_tma_cannot_describe(gpu, par_oracle, tl, tr, m, n, k):
    rng = np.random.default_rng(m + n + k)
    l, r = operands(rng, tl, tr, m, n, k)
    ref, mag = par_oracle.fmatmul_f64(tl, tr, l, r)
    assert rel_err(gpu.fmatmul(tl, tr, l, r), ref, mag) <= TOL


@pytest.mark.parametrize("m,n,k", [(784, 512, 49152), (260, 256, 65536), (1296, 128, 50000), (144, 1024, 49156)])
def test_rows_past_a_tile_boundary_of_t_f_products(gpu, par_oracle, m, n, k):
    # left stored [k, m] with m a few rows past a multiple of 128: whole tile rows on the tensor
    # cores, the rest on the bandwidth-bound kernel; with the library's own scratch and with a
    # caller workspace of exactly the size the library asks for
    import torch
    rng = np.random.default_rng(m + n + k)
    l, r = operands(rng, 1, 0, m, n, k)
    ref, mag = par_oracle.fmatmul_f64(1, 0, l, r)
    got = gpu.fmatmul(1, 0, l, r)
    assert rel_err(got, ref, mag) <= 5e-6
    lib = gpu.d.lib
    need = int(lib.cdll.polar_b200_fmatmul_workspace_bytes(1, 0, m, n, k))
    assert need > 0
    L, R = torch.from_numpy(l).cuda(), torch.from_numpy(r).cuda()
    out = torch.full((m, n), float("nan"), device="cuda")
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    lib.call("polar_b200_fmatmul", 1, 0, m, n, k, L.data_ptr(), R.data_ptr(), out.data_ptr(), ws.data_ptr(), need, st)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint32), got.view(np.uint32))   # deterministic
    assert lib.cdll.polar_b200_fmatmul(1, 0, m, n, k, L.data_ptr(), R.data_ptr(), out.data_ptr(), ws.data_ptr(),
                                       need - 16, st) != 0                            # too small: a status
    assert gpu.d.device_status() == 0


def test_empty_dimensions(gpu):
    assert gpu.fmatmul(0, 0, np.empty((0, 8), np.float32), np.empty((8, 4), np.float32)).shape == (0, 4)
    out = gpu.fmatmul(0, 0, np.empty((3, 0), np.float32), np.empty((0, 4), np.float32))
    assert np.array_equal(out, np.zeros((3, 4), np.float32))


def test_plain_tf32_is_not_enough(gpu, par_oracle):
    # the single-product mode misses the tolerance the split meets: the split is needed
    rng = np.random.default_rng(9)
    l, r = operands(rng, 0, 1, 256, 256, 1024)
    ref, mag = par_oracle.fmatmul_f64(0, 1, l, r)
    e1 = rel_err(gpu.fmatmul(0, 1, l, r, which="tc", passes=1), ref, mag)
    e3 = rel_err(gpu.fmatmul(0, 1, l, r, which="tc", passes=3), ref, mag)
    assert e1 > 2e-5 and e3 < 5e-6


@pytest.mark.parametrize("tl,tr", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_large_sampled_against_f64(gpu, par_oracle, tl, tr):
    # 4096^3 and the skinny 65536 x 784 x 1024 case: sampled entries, full rows and columns
    import torch
    for (m, n, k) in ((4096, 4096, 4096), (65536, 1024, 784)):
        torch.manual_seed(m + tl * 2 + tr)
        L = torch.empty((k, m) if tl else (m, k), device="cuda").uniform_(-1, 1)
        R = torch.empty((n, k) if tr else (k, n), device="cuda").uniform_(-1, 1)
        out = torch.empty((m, n), device="cuda")
        gpu.d.fmatmul(tl, tr, L, R, out)
        torch.cuda.synchronize()
        assert gpu.d.device_status() == 0
        l, r, got = L.cpu().numpy(), R.cpu().numpy(), out.cpu().numpy()
        rng = np.random.default_rng(1)
        rows = rng.integers(0, m, 4096).astype(np.uint64)
        cols = rng.integers(0, n, 4096).astype(np.uint64)
        # plus 8 full rows and 8 full columns, first/last included
        fr = np.array([0, m - 1] + list(rng.integers(0, m, 6)), np.uint64)
        fc = np.array([0, n - 1] + list(rng.integers(0, n, 6)), np.uint64)
        rows = np.concatenate([rows, np.repeat(fr, n), np.tile(np.arange(m, dtype=np.uint64), 8)])
        cols = np.concatenate([cols, np.tile(np.arange(n, dtype=np.uint64), 8), np.repeat(fc, m)])
        ref, mag = par_oracle.fmatmul_entries_f64(tl, tr, l, r, rows, cols)
        g = got[rows.astype(np.int64), cols.astype(np.int64)].astype(np.float64)
        assert float(np.max(np.abs(g - ref) / mag)) <= TOL


def test_linearity_at_8192(gpu):
    # full-size property check: (A1 + A2) B == A1 B + A2 B within the tolerance, and the
    # tensor-core result agrees with the FFMA kernel on a strip of rows
    import torch
    d = gpu.d
    n = 8192
    torch.manual_seed(0)
    A1 = torch.empty((n, n), device="cuda").uniform_(-1, 1)
    A2 = torch.empty((n, n), device="cuda").uniform_(-1, 1)
    B = torch.empty((n, n), device="cuda").uniform_(-1, 1)
    C1, C2, C12 = (torch.empty((n, n), device="cuda") for _ in range(3))
    d.fmatmul(0, 0, A1, B, C1)
    d.fmatmul(0, 0, A2, B, C2)
    d.fmatmul(0, 0, A1 + A2, B, C12)
    torch.cuda.synchronize()
    scale = float(n) * 0.25 * 2                     # E|a||b| summed over k, both terms
    assert float((C12 - (C1 + C2)).abs().max()) / scale <= TOL
    strip = torch.empty((256, n), device="cuda")
    d.fmatmul_ffma(0, 0, A1[:256].contiguous(), B, strip)
    torch.cuda.synchronize()
    assert float((strip - C1[:256]).abs().max()) / (n * 0.25) <= TOL
    assert d.device_status() == 0


@pytest.mark.parametrize("tl,tr", [(0, 0), (1, 1)])
def test_full_compare_at_2048(gpu, par_oracle, tl, tr):
    # every entry of a 2048^3 product against the double-accumulated oracle
    m = n = k = 2048
    rng = np.random.default_rng(2048 + 2 * tl + tr)
    l, r = operands(rng, tl, tr, m, n, k)
    ref, mag = par_oracle.fmatmul_f64(tl, tr, l, r)
    got = gpu.fmatmul(tl, tr, l, r)
    err = rel_err(got, ref, mag)
    assert err <= TOL and err <= 5e-6, err
    assert gpu.d.device_status() == 0


@pytest.mark.parametrize("tl,tr", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_8192_sampled_against_f64(gpu, par_oracle, tl, tr):
    # 8192^3 in the configuration the dispatch picks (256 x 256 tiles): 4096 seeded entries,
    # 4 full rows and 4 full columns (first and last included) against double dot products
    import torch
    m = n = k = 8192
    torch.manual_seed(8192 + tl * 2 + tr)
    L = torch.empty((k, m) if tl else (m, k), device="cuda").uniform_(-1, 1)
    R = torch.empty((n, k) if tr else (k, n), device="cuda").uniform_(-1, 1)
    out = torch.empty((m, n), device="cuda")
    gpu.d.fmatmul(tl, tr, L, R, out)
    torch.cuda.synchronize()
    assert gpu.d.device_status() == 0
    l, r, got = L.cpu().numpy(), R.cpu().numpy(), out.cpu().numpy()
    del L, R, out
    rng = np.random.default_rng(2)
    rows = rng.integers(0, m, 4096).astype(np.uint64)
    cols = rng.integers(0, n, 4096).astype(np.uint64)
    fr = np.array([0, m - 1] + list(rng.integers(0, m, 2)), np.uint64)
    fc = np.array([0, n - 1] + list(rng.integers(0, n, 2)), np.uint64)
    rows = np.concatenate([rows, np.repeat(fr, n), np.tile(np.arange(m, dtype=np.uint64), 4)])
    cols = np.concatenate([cols, np.tile(np.arange(n, dtype=np.uint64), 4), np.repeat(fc, m)])
    ref, mag = par_oracle.fmatmul_entries_f64(tl, tr, l, r, rows, cols)
    g = got[rows.astype(np.int64), cols.astype(np.int64)].astype(np.float64)
    err = float(np.max(np.abs(g - ref) / mag))
    assert err <= TOL and err <= 1e-5, err


def test_result_that_is_only_4_byte_aligned(gpu, par_oracle):
    # `out` one float past a 16-byte boundary, on shapes whose k range is cut into work units
    # (fixed cuts: the partial products are summed by a second kernel; stream mode: slots) and
    # on the whole-tile path: every store to the result must fall back to 4-byte stores
    import torch
    d = gpu.d
    for (tl, tr, m, n, k, splits) in ((0, 1, 512, 512, 4096, 4), (1, 0, 512, 256, 8192, 8), (0, 0, 640, 512, 2048, -1),
                                      (0, 0, 384, 512, 512, 1)):
        rng = np.random.default_rng(m + n + k)
        l, r = operands(rng, tl, tr, m, n, k)
        ref, mag = par_oracle.fmatmul_f64(tl, tr, l, r)
        L, R = torch.from_numpy(l).cuda(), torch.from_numpy(r).cuda()
        for tile_n in (256, 512) if splits == -1 else (256, 512, 1256, 1512):
            base = torch.full((m * n + 8,), float("nan"), device="cuda")
            out = base[1:1 + m * n].view(m, n)
            assert out.data_ptr() % 16 == 4
            d.fmatmul_tc(tl, tr, L, R, out, tile_n=tile_n, slab_k=16, splits=splits)
            torch.cuda.synchronize()
            assert d.device_status() == 0
            assert rel_err(out.cpu().numpy(), ref, mag) <= 5e-6, (m, n, k, splits, tile_n)
            assert bool(torch.isnan(base[0])) and bool(torch.isnan(base[1 + m * n:]).all())   # nothing outside
        # and through the dispatch, which plans the cuts itself
        base = torch.full((m * n + 8,), float("nan"), device="cuda")
        out = base[1:1 + m * n].view(m, n)
        d.fmatmul(tl, tr, L, R, out)
        torch.cuda.synchronize()
        assert rel_err(out.cpu().numpy(), ref, mag) <= 5e-6


@pytest.mark.parametrize("m,n,k,row0,rows", [(784, 4096, 8192, 0, 512), (784, 4096, 8192, 512, 272), (1024, 512, 2048, 256, 768),
                                            (784, 512, 4096, 0, 784)])
def test_block_of_rows_of_a_t_f_product(gpu, par_oracle, m, n, k, row0, rows):
    # out[row0 : row0+rows] of left^T.right, the other rows untouched; through the entry point and by name
    import ctypes
    import torch
    from polarai_framework_b200.capi import Arg
    rng = np.random.default_rng(m + n + k + row0)
    l, r = operands(rng, 1, 0, m, n, k)
    ref, mag = par_oracle.fmatmul_f64(1, 0, np.ascontiguousarray(l[:, row0:row0 + rows]), r)
    L, R = torch.from_numpy(l).cuda(), torch.from_numpy(r).cuda()
    lib = gpu.d.lib
    st = torch.cuda.current_stream().cuda_stream
    out = torch.full((m, n), float("nan"), device="cuda")
    lib.call("polar_b200_fmatmul_t_f_rows", m, row0, rows, n, k, L.data_ptr(), R.data_ptr(), out.data_ptr(), None, 0, st)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    assert rel_err(got[row0:row0 + rows], ref, mag) <= 5e-6
    assert np.isnan(got[:row0]).all() and np.isnan(got[row0 + rows:]).all()
    # by name, with a caller workspace of the size the library asks for
    args = (Arg * 5)()
    shapes = [(ctypes.c_uint64 * 2)(k, m), (ctypes.c_uint64 * 2)(k, n), None, None, (ctypes.c_uint64 * 2)(m, n)]
    out2 = torch.full((m, n), float("nan"), device="cuda")
    for a, t, shp in zip(args, (L, R, None, None, out2), shapes):
        if t is not None:
            a.is_tensor, a.tensor.data, a.tensor.dims, a.tensor.shape = 1, t.data_ptr(), 2, shp
    args[2].scalar, args[3].scalar = float(row0), float(rows)
    need = int(lib.cdll.polar_b200_launch_workspace_bytes(b"fmatmul_t_f_rows", args, 5))
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    lib.call("polar_b200_launch_by_name", b"fmatmul_t_f_rows", args, 5, ws.data_ptr() if need else None, need, st)
    torch.cuda.synchronize()
    assert np.array_equal(out2.cpu().numpy()[row0:row0 + rows].view(np.uint32), got[row0:row0 + rows].view(np.uint32))
    assert gpu.d.device_status() == 0
    # a block that does not start on a multiple of 4, or runs past the result: statuses
    assert lib.cdll.polar_b200_fmatmul_t_f_rows(m, 2, 64, n, k, L.data_ptr(), R.data_ptr(), out.data_ptr(), None, 0, st) == 1
    assert lib.cdll.polar_b200_fmatmul_t_f_rows(m, 0, m + 4, n, k, L.data_ptr(), R.data_ptr(), out.data_ptr(), None, 0, st) == 1
