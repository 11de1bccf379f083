"""GPU parity of the elementwise builtins against the CPU oracle and the golden
fixtures.  Everything goes through the C ABI (ctypes)."""
import numpy as np
import pytest

from conftest import expected_of, run_kat

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu():
    import torch
    import __graft_entry__ as ge
    ge.load_package()
    from polarai_framework_b200.device_builtins import HostBuiltins
    assert torch.cuda.is_available()
    return HostBuiltins("cuda:0")


def bits(a):
    return np.ascontiguousarray(a, np.float32).ravel().view(np.uint32)


def max_rel(got, want):
    want = want.astype(np.float64)
    got = got.astype(np.float64)
    denom = np.where(want == 0, 1.0, np.abs(want))
    return float(np.max(np.abs(got - want) / denom))


EXACT = {"fadd", "fmul", "fdivide", "fmulconcat"}


def test_reference_kats(gpu, kats):
    for case in kats:
        if case["builtin"] == "fmatmul":
            continue
        got = run_kat(gpu, case)
        want = expected_of(case)
        if case["builtin"] in EXACT:
            assert np.array_equal(bits(got), bits(want)), case["name"]
        else:
            assert max_rel(got, want) <= 1e-5, case["name"]


def test_seeded_fixture(gpu, seeded):
    d = seeded
    n = d["a"].size
    assert np.array_equal(bits(gpu.ffill(1.234, n)), bits(d["out_fill"]))
    assert np.array_equal(bits(gpu.fcopy(d["a"])), bits(d["out_copy"]))
    assert np.array_equal(bits(gpu.fadd(d["a"], 1.0, d["b"], 1.0)), bits(d["out_add"]))
    assert np.array_equal(bits(gpu.fadd(d["a"], 0.34, d["b"], -0.21)), bits(d["out_combine"]))
    assert np.array_equal(bits(gpu.fmul(d["a"], d["b"])), bits(d["out_mul"]))
    assert np.array_equal(bits(gpu.fdivide(d["a"], d["den"])), bits(d["out_divide"]))
    assert np.array_equal(bits(gpu.fmulconcat(d["grad"], d["a"])), bits(d["out_mulconcat"]))
    assert max_rel(gpu.fsigmoid(d["xs"]), d["out_sigmoid"]) <= 1e-5
    # log-loss: p = 0 or 1 gives log(1e-5)-sized terms; relative tolerance still holds
    assert max_rel(gpu.flogloss(d["p"], d["y"]), d["out_logloss"]) <= 1e-5
    assert max_rel(gpu.flogloss(d["p"], d["ysoft"]), d["out_logloss_soft"]) <= 1e-5


@pytest.mark.parametrize("n", [0, 1, 3, 4, 5, 1023, 1025, 4096 * 256 + 7, 1 << 20])
def test_sizes_against_oracle(gpu, oracle, n):
    rng = np.random.default_rng(n)
    a = rng.uniform(-1, 1, n).astype(np.float32)
    b = rng.uniform(-1, 1, n).astype(np.float32)
    den = rng.uniform(0.5, 2, n).astype(np.float32)
    p = rng.uniform(0.01, 0.99, n).astype(np.float32)
    y = (rng.random(n) < 0.5).astype(np.float32)
    g = np.array([0.37], np.float32)
    assert np.array_equal(bits(gpu.ffill(-2.5, n)), bits(oracle.ffill(-2.5, n)))
    assert np.array_equal(bits(gpu.fcopy(a)), bits(a))
    assert np.array_equal(bits(gpu.fadd(a, 0.7, b, -1.3)), bits(oracle.fadd(a, 0.7, b, -1.3)))
    assert np.array_equal(bits(gpu.fmul(a, b)), bits(oracle.fmul(a, b)))
    assert np.array_equal(bits(gpu.fdivide(a, den)), bits(oracle.fdivide(a, den)))
    assert np.array_equal(bits(gpu.fmulconcat(g, a)), bits(oracle.fmulconcat(g, a)))
    if n:
        assert max_rel(gpu.fsigmoid(a * 12), oracle.fsigmoid(a * 12)) <= 1e-5
        assert max_rel(gpu.fsigmoid(a * 12, clamp=False), oracle.fsigmoid(a * 12, clamp=False)) <= 1e-5
        assert max_rel(gpu.flogloss(p, y), oracle.flogloss(p, y)) <= 1e-5


def test_logloss_edge_cases_match_the_oracle_class_by_class(gpu, oracle):
    # Labels that are exactly 0 or 1 take a one-logarithm path whose result must be the bits of
    # the two-logarithm formula; everything around the places where that could differ is checked
    # against the oracle: p at and around 0, 1, 1 - eps (p + eps == 1: log == +0), eps
    # (1 - p + eps == 1), arguments <= 0 (log = -inf / NaN: 0 * log must stay NaN), inf and NaN
    # inputs, labels -0.0, 0.5 and 2 (general form).
    eps = np.float32(1e-5)
    one = np.float32(1.0)
    ps = [0.0, 1.0, 1e-5, 1.0 - 1e-5, float(one - eps), float(np.nextafter(one - eps, 0)), float(np.nextafter(one - eps, 2)),
          float(eps), float(np.nextafter(eps, 0)), float(np.nextafter(eps, 1)), 0.5, 0.25, 0.999, 1e-3,
          -1e-5, float(-eps), -0.5, 1.00001, 1.5, 2.0, -0.0, np.inf, -np.inf, np.nan, 1e-30, 0.6, 0.2, 0.8, 0.3]
    ys = [0.0, 1.0, -0.0, 0.5, 2.0, 1e-3, np.nan]
    P, Y = np.meshgrid(np.array(ps, np.float32), np.array(ys, np.float32))
    P, Y = np.ascontiguousarray(P.ravel()), np.ascontiguousarray(Y.ravel())
    # pad so that vector and tail paths are both exercised
    P, Y = np.tile(P, 41)[:8003], np.tile(Y, 41)[:8003]
    with np.errstate(all="ignore"):
        got, want = gpu.flogloss(P, Y), oracle.flogloss(P, Y)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    inf = np.isinf(want)
    assert np.array_equal(np.isinf(got), inf) and np.array_equal(got[inf], want[inf])
    zero = want == 0
    assert np.array_equal(got == 0, zero) and np.array_equal(np.signbit(got[zero]), np.signbit(want[zero]))
    rest = ~(np.isnan(want) | inf | zero)
    assert np.max(np.abs(got[rest].astype(np.float64) - want[rest]) / np.abs(want[rest])) <= 1e-5
    # binary labels at scale: the same tolerance on two million elements
    rng = np.random.default_rng(77)
    p = rng.uniform(0, 1, 1 << 21).astype(np.float32)
    y = (rng.random(1 << 21) < 0.5).astype(np.float32)
    assert max_rel(gpu.flogloss(p, y), oracle.flogloss(p, y)) <= 1e-5


def test_fill_and_copy_special_bit_patterns(gpu):
    # bit-exact means NaN payloads, -0.0, denormals and infinities survive
    pats = np.array([0x7FC00001, 0xFFC12345, 0x80000000, 0x00000001, 0x7F800000, 0xFF800000, 0x3F9DF3B6],
                    np.uint32)
    src = np.resize(pats, 10007).view(np.float32)
    assert np.array_equal(bits(gpu.fcopy(src)), bits(src))
    for pat in pats:
        v = np.array([pat], np.uint32).view(np.float32)[0]
        out = gpu.ffill(v, 1001)
        assert np.all(bits(out) == pat)


def test_misaligned_pointers_take_the_scalar_kernel(gpu, oracle):
    import torch
    d = gpu.d
    n = 5001
    rng = np.random.default_rng(3)
    a = rng.uniform(-1, 1, n + 3).astype(np.float32)
    b = rng.uniform(-1, 1, n + 3).astype(np.float32)
    ta, tb = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    out = torch.zeros(n + 3, device="cuda")
    d.fadd(ta[1:n + 1], 0.5, tb[3:n + 3], 2.0, out[2:n + 2])
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    assert np.array_equal(bits(got[2:n + 2]), bits(oracle.fadd(a[1:n + 1], 0.5, b[3:n + 3], 2.0)))
    assert got[0] == 0 and got[1] == 0 and got[n + 2] == 0      # nothing outside the range


def test_in_place_update(gpu, oracle):
    import torch
    d = gpu.d
    rng = np.random.default_rng(5)
    w = rng.uniform(-1, 1, 784 * 10).astype(np.float32)
    dw = rng.uniform(-1, 1, 784 * 10).astype(np.float32)
    tw, tdw = torch.from_numpy(w).cuda(), torch.from_numpy(dw).cuda()
    d.fadd(tw, 1.0, tdw, -0.1, tw)                       # W <- W - 0.1 dW
    torch.cuda.synchronize()
    assert np.array_equal(bits(tw.cpu().numpy()), bits(oracle.fadd(w, 1.0, dw, -0.1)))


def test_fsum(gpu):
    import torch
    x = torch.rand(1_000_003, device="cuda")
    acc = torch.zeros(1, dtype=torch.float64, device="cuda")
    gpu.d.fsum(x, acc)
    torch.cuda.synchronize()
    want = float(x.double().sum())
    assert abs(float(acc) - want) <= 1e-9 * want
    gpu.d.fsum(x[1:], acc)                                # misaligned view, adds on top
    torch.cuda.synchronize()
    assert abs(float(acc) - (want + float(x[1:].double().sum()))) <= 1e-9 * want


def test_fsum_as_a_builtin_with_a_tensor_result(gpu):
    # "fsum" by name: the float of a double-accumulated sum, the same bits run to run, with the
    # library's own scratch and with a caller workspace of exactly the size it asks for
    import ctypes
    import torch
    from polarai_framework_b200.capi import Arg
    lib = gpu.d.lib
    st = torch.cuda.current_stream().cuda_stream
    for n in (1, 3, 4, 1_000_003, 65536 * 10):
        x = torch.rand(n + 1, device="cuda")[1:] if n == 1_000_003 else torch.rand(n, device="cuda")   # one unaligned case
        out = torch.full((1,), float("nan"), device="cuda")
        args = (Arg * 2)()
        shapes = [(ctypes.c_uint64 * 1)(n), (ctypes.c_uint64 * 1)(1)]
        for a, t, shp in zip(args, (x, out), shapes):
            a.is_tensor, a.tensor.data, a.tensor.dims, a.tensor.shape = 1, t.data_ptr(), 1, shp
        lib.call("polar_b200_launch_by_name", b"fsum", args, 2, None, 0, st)
        torch.cuda.synchronize()
        want = float(x.double().sum())
        first = float(out)
        assert abs(first - want) <= 1e-6 * max(want, 1.0), n
        need = int(lib.cdll.polar_b200_launch_workspace_bytes(b"fsum", args, 2))
        assert need == int(lib.cdll.polar_b200_fsum_f32_workspace_bytes(n)) and need % 8 == 0 and need > 0
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        out.fill_(float("nan"))
        lib.call("polar_b200_launch_by_name", b"fsum", args, 2, ws.data_ptr(), need, st)
        torch.cuda.synchronize()
        assert float(out) == first, n                                  # deterministic
        assert lib.cdll.polar_b200_launch_by_name(b"fsum", args, 2, ws.data_ptr(), need - 8, st) == 5   # too small


def test_large_stream_properties(gpu):
    # 2^28 elements: too slow for the scalar oracle in a test, so use properties.
    import torch
    d = gpu.d
    n = 1 << 28
    a = torch.empty(n, device="cuda").uniform_(-1, 1)
    b = torch.empty(n, device="cuda").uniform_(0.5, 2)
    out = torch.empty(n, device="cuda")
    d.fcopy(a, out)
    assert torch.equal(out.view(torch.int32), a.view(torch.int32))
    d.fadd(a, 1.0, b, 0.0, out)                           # a*1 + b*0 == a exactly
    assert torch.equal(out, a)
    d.fmul(a, b, out)
    assert torch.equal(out, a * b)
    d.fdivide(a, b, out)
    assert torch.equal(out, a / b)
    d.ffill(1.234, out)
    assert bool((out == 1.234).all())
    acc = torch.zeros(1, dtype=torch.float64, device="cuda")
    d.fsum(out, acc)
    torch.cuda.synchronize()
    assert abs(float(acc) - n * float(np.float32(1.234))) < 1e-3
