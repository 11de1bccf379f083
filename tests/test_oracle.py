"""CPU tests: the oracle restatement against the reference's golden vectors and
against the reference's own OpenCL C kernels compiled as C."""
import numpy as np
import pytest

from conftest import expected_of, run_kat
from oracle import oracle as orc


def bits(a):
    return np.ascontiguousarray(a, np.float32).ravel().view(np.uint32)


def test_kats_bit_exact(oracle, kats):
    assert len(kats) == 13
    for case in kats:
        got = run_kat(oracle, case)
        assert np.array_equal(bits(got), bits(expected_of(case))), case["name"]


def test_kats_match_targets_written_in_reference_tests(kats):
    # AddOperation.cpp:24,69 write the expected numbers out; the others compute
    # them with an in-file loop.
    for case in kats:
        t = case["inputs"].get("stated_target")
        if t is not None:
            assert np.array_equal(expected_of(case), np.array(t, np.float32))


def test_kat_values_by_hand(kats):
    by = {c["name"]: expected_of(c) for c in kats}
    assert by["MatMulNN"][0] == 3 * 6 + 4 * 7 + 5 * 8 + 10 * 11
    assert list(by["MatMulNNRect"]) == [127, 104, 131, 233, 133, 176]
    assert list(by["MatMulTN"]) == list(by["MatMulNNRect"]) == list(by["MatMulNT"])
    # both sigmoid clamps are exercised by the reference's vector
    assert by["Sigmoid"][0] == np.float32(1e-5)
    assert by["Sigmoid"][3] == np.float32(1.0) - np.float32(1e-5)


@pytest.mark.parametrize("name,call", [
    ("out_fill", lambda o, d: o.ffill(1.234, d["a"].size)),
    ("out_copy", lambda o, d: o.fcopy(d["a"])),
    ("out_add", lambda o, d: o.fadd(d["a"], 1.0, d["b"], 1.0)),
    ("out_combine", lambda o, d: o.fadd(d["a"], 0.34, d["b"], -0.21)),
    ("out_mul", lambda o, d: o.fmul(d["a"], d["b"])),
    ("out_divide", lambda o, d: o.fdivide(d["a"], d["den"])),
    ("out_sigmoid", lambda o, d: o.fsigmoid(d["xs"])),
    ("out_logloss", lambda o, d: o.flogloss(d["p"], d["y"])),
    ("out_logloss_soft", lambda o, d: o.flogloss(d["p"], d["ysoft"])),
    ("out_mulconcat", lambda o, d: o.fmulconcat(d["grad"], d["a"])),
])
def test_seeded_bit_exact(oracle, seeded, name, call):
    assert np.array_equal(bits(call(oracle, seeded)), bits(seeded[name]))


@pytest.mark.parametrize("tl", [0, 1])
@pytest.mark.parametrize("tr", [0, 1])
def test_seeded_matmul_bit_exact(oracle, seeded, tl, tr):
    tag = f"mm_{'t' if tl else 'f'}_{'t' if tr else 'f'}"
    got = oracle.fmatmul(tl, tr, seeded[tag + "_left"], seeded[tag + "_right"])
    assert np.array_equal(bits(got), bits(seeded[tag + "_out"]))
    # transposed storage of the same logical operands gives the same product
    l = seeded[tag + "_left"]
    r = seeded[tag + "_right"]
    a = l.T if tl else l
    b = r.T if tr else r
    plain = oracle.fmatmul(0, 0, np.ascontiguousarray(a), np.ascontiguousarray(b))
    assert np.array_equal(bits(plain), bits(got))


def test_f64_matmul_bounds_fp32_sum(oracle, seeded):
    l, r = seeded["mm_f_f_left"], seeded["mm_f_f_right"]
    ref, mag = oracle.fmatmul_f64(0, 0, l, r)
    assert np.allclose(ref, l.astype(np.float64) @ r.astype(np.float64), rtol=1e-12, atol=1e-12)
    seq = oracle.fmatmul(0, 0, l, r)
    assert np.max(np.abs(seq - ref) / mag) < 1e-5
    rows = np.array([0, 5, 36], np.uint64)
    cols = np.array([28, 0, 7], np.uint64)
    e, m = oracle.fmatmul_entries_f64(0, 0, l, r, rows, cols)
    assert np.array_equal(e, ref[rows.astype(int), cols.astype(int)])
    assert np.array_equal(m, mag[rows.astype(int), cols.astype(int)])


def test_sigmoid_unclamped_differs_only_at_the_ends(oracle):
    x = np.array([-100, -12, -5, 0, 5, 12, 100], np.float32)
    c, u = oracle.fsigmoid(x, True), oracle.fsigmoid(x, False)
    assert np.array_equal(c[2:5], u[2:5])
    assert c[0] == np.float32(1e-5) and u[0] == 0.0
    assert c[-1] == np.float32(1) - np.float32(1e-5) and u[-1] == 1.0


def test_empty_inputs(oracle):
    e = np.empty(0, np.float32)
    assert oracle.fadd(e, 1, e, 1).size == 0
    assert oracle.fsigmoid(e).size == 0
    assert oracle.fmatmul(0, 0, np.empty((0, 3), np.float32), np.empty((3, 2), np.float32)).shape == (0, 2)
    assert np.array_equal(oracle.fmatmul(0, 0, np.empty((2, 0), np.float32), np.empty((0, 2), np.float32)),
                          np.zeros((2, 2), np.float32))


def test_threads_do_not_change_results(seeded):
    o1, o4 = orc.Oracle(1), orc.Oracle(4)
    assert np.array_equal(o1.flogloss(seeded["p"], seeded["y"]), o4.flogloss(seeded["p"], seeded["y"]))
    l, r = seeded["mm_t_t_left"], seeded["mm_t_t_right"]
    assert np.array_equal(o1.fmatmul(1, 1, l, r), o4.fmatmul(1, 1, l, r))


@pytest.mark.skipif(not orc.RefOcl.available(), reason="oracle/_ref not built (no reference tree)")
def test_restatement_equals_compiled_reference_on_random_inputs(oracle):
    ref = orc.RefOcl(threads=2)
    rng = np.random.default_rng(7)
    n = 50_003
    a = rng.uniform(-1, 1, n).astype(np.float32)
    b = rng.uniform(-1, 1, n).astype(np.float32)
    den = rng.uniform(0.5, 2, n).astype(np.float32)
    x = rng.uniform(-30, 30, n).astype(np.float32)
    p = rng.uniform(0, 1, n).astype(np.float32)
    y = (rng.random(n) < 0.5).astype(np.float32)
    g = np.array([1.7], np.float32)
    assert np.array_equal(bits(oracle.ffill(-3.5, n)), bits(ref.ffill(-3.5, n)))
    assert np.array_equal(bits(oracle.fcopy(a)), bits(ref.fcopy(a)))
    assert np.array_equal(bits(oracle.fadd(a, 0.3, b, -1.1)), bits(ref.fadd(a, 0.3, b, -1.1)))
    assert np.array_equal(bits(oracle.fmul(a, b)), bits(ref.fmul(a, b)))
    assert np.array_equal(bits(oracle.fdivide(a, den)), bits(ref.fdivide(a, den)))
    assert np.array_equal(bits(oracle.fsigmoid(x)), bits(ref.fsigmoid(x)))
    assert np.array_equal(bits(oracle.flogloss(p, y)), bits(ref.flogloss(p, y)))
    assert np.array_equal(bits(oracle.fmulconcat(g, a)), bits(ref.fmulconcat(g, a)))
    for tl in (0, 1):
        for tr in (0, 1):
            l = rng.uniform(-1, 1, (65, 41) if tl else (41, 65)).astype(np.float32)
            r = rng.uniform(-1, 1, (33, 65) if tr else (65, 33)).astype(np.float32)
            assert np.array_equal(bits(oracle.fmatmul(tl, tr, l, r)), bits(ref.fmatmul(tl, tr, l, r)))
