"""GPU tests of the device-runtime plugin: builtins launched by native kernel name
through Device::launch with LaunchCommand/ArgDesc/TensorInfo, data entering and
leaving through host buffers."""
import numpy as np
import pytest

from conftest import expected_of, run_kat

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rtb():
    import __graft_entry__ as ge
    ge.load_package()
    from polarai_framework_b200.runtime import RuntimeBuiltins
    b = RuntimeBuiltins()
    assert b.rt.device_count() >= 1
    yield b
    b.rt.close()


def bits(a):
    return np.ascontiguousarray(a, np.float32).ravel().view(np.uint32)


def test_device_names_are_unique(rtb):
    names = [rtb.rt.device_name(i) for i in range(rtb.rt.device_count())]
    assert len(set(names)) == len(names)
    assert all("#" in n for n in names)


def test_reference_kats_through_launch(rtb, kats):
    for case in kats:
        got = run_kat(rtb, case)
        want = expected_of(case)
        if case["builtin"] in ("fsigmoid", "flogloss"):
            assert np.max(np.abs(got.ravel() - want) / np.abs(want)) <= 1e-5, case["name"]
        else:
            # small integers and exactly rounded operations: bit-exact, matmul included
            assert np.array_equal(bits(got), bits(want)), case["name"]


def test_seeded_matmuls_through_launch(rtb, seeded, oracle):
    for tl in (0, 1):
        for tr in (0, 1):
            tag = f"mm_{'t' if tl else 'f'}_{'t' if tr else 'f'}"
            got = rtb.fmatmul(tl, tr, seeded[tag + "_left"], seeded[tag + "_right"])
            ref, mag = oracle.fmatmul_f64(tl, tr, seeded[tag + "_left"], seeded[tag + "_right"])
            assert np.max(np.abs(got - ref) / mag) <= 1e-4
            assert np.max(np.abs(seeded[tag + "_out"] - ref) / mag) <= 1e-4


def test_graph_like_sequence_stays_on_device(rtb, oracle):
    # out = sigmoid((a+b)*c/d): four launches, one upload per input, one download
    rt = rtb.rt
    rng = np.random.default_rng(0)
    n = 1 << 20
    a, b, c = (rng.uniform(-1, 1, n).astype(np.float32) for _ in range(3))
    d = rng.uniform(0.5, 2, n).astype(np.float32)
    ta, tb, tc, td = (rt.tensor((n,)) for _ in range(4))
    for t, x in ((ta, a), (tb, b), (tc, c), (td, d)):
        rt.write(t, x)
    t1, t2, t3, t4 = (rt.tensor((n,)) for _ in range(4))
    rt.launch("fadd", [ta, 1.0, tb, 1.0, t1])
    rt.launch("fmul", [t1, tc, t2])
    rt.launch("fdivide", [t2, td, t3])
    rt.launch("fsigmoid", [t3, t4])
    got = rt.read(t4)
    want = oracle.fsigmoid(oracle.fdivide(oracle.fmul(oracle.fadd(a, 1.0, b, 1.0), c), d))
    assert np.max(np.abs(got - want) / np.abs(want)) <= 1e-5
    # intermediate results are readable too and bit-exact
    assert np.array_equal(bits(rt.read(t3)), bits(oracle.fdivide(oracle.fmul(oracle.fadd(a, 1.0, b, 1.0), c), d)))
    for t in (ta, tb, tc, td, t1, t2, t3, t4):
        rt.free(t)


def test_in_place_weight_update(rtb, oracle):
    rt = rtb.rt
    rng = np.random.default_rng(1)
    w = rng.uniform(-1, 1, (784, 10)).astype(np.float32)
    dw = rng.uniform(-1, 1, (784, 10)).astype(np.float32)
    tw, tdw = rt.tensor(w.shape), rt.tensor(w.shape)
    rt.write(tw, w)
    rt.write(tdw, dw)
    for _ in range(3):
        rt.launch("fadd", [tw, 1.0, tdw, -0.1, tw])
        w = oracle.fadd(w, 1.0, dw, -0.1)
    assert np.array_equal(bits(rt.read(tw)), bits(w))
    rt.free(tw)
    rt.free(tdw)


def test_errors_are_statuses(rtb):
    from polarai_framework_b200.capi import PolarB200Error
    rt = rtb.rt
    a, b = rt.tensor((8,)), rt.tensor((9,))
    with pytest.raises(PolarB200Error):
        rt.launch("fcopy", [a, b])                 # sizes differ
    with pytest.raises(PolarB200Error):
        rt.launch("fnotakernel", [a, a])
    with pytest.raises(PolarB200Error):
        rt.launch("fadd", [a, a])                  # wrong argument pattern
    rt.launch("ffill", [2.0, a])                   # the device is still usable
    assert np.all(rt.read(a) == 2.0)
    rt.free(a)
    rt.free(b)


def test_memory_limit_offloads_released_records(rtb):
    rt = rtb.rt
    base = rt.bytes_in_use()
    n = 1 << 20
    rt.set_memory_limit(base + 3 * 4 * n)
    ts = []
    for i in range(6):                              # twice the cap
        t = rt.tensor((n,))
        rt.launch("ffill", [float(i + 1), t])
        ts.append(t)
    assert rt.bytes_in_use() <= base + 3 * 4 * n
    for i, t in enumerate(ts):                      # evicted records were saved to host memory
        assert np.all(rt.read(t) == float(i + 1))
    rt.set_memory_limit(0)
    for t in ts:
        rt.free(t)


def test_mlp_program_through_the_plugin_equals_the_direct_executor(rtb):
    # the same builtin program (extended builtins included) driven through Device::launch with
    # host buffers on both sides gives the bits of the direct C-ABI path
    from polarai_framework_b200.program import DeviceExecutor, fuse_program, mlp_program
    from polarai_framework_b200.runtime import RuntimeProgramExecutor
    rng = np.random.default_rng(3)
    batch, hidden = 512, 1024
    X = rng.standard_normal((batch, 784)).astype(np.float32)
    Y = np.eye(10, dtype=np.float32)[rng.integers(0, 10, batch)]
    W1 = rng.uniform(-0.05, 0.05, (784, hidden)).astype(np.float32)
    W2 = rng.uniform(-0.2, 0.2, (hidden, 10)).astype(np.float32)
    for prog in (mlp_program(batch, 784, hidden, 10, 0.1), fuse_program(mlp_program(batch, 784, hidden, 10, 0.1))):
        direct = DeviceExecutor(prog)
        direct.set_inputs(X=X, Y=Y, W1=W1, W2=W2)
        plugin = RuntimeProgramExecutor(prog, rtb.rt)
        plugin.set_inputs(X=X, Y=Y, W1=W1, W2=W2)
        for _ in range(2):
            direct.run(), plugin.run()
        for k in prog.outputs:
            assert np.array_equal(bits(direct.output(k)), bits(plugin.output(k))), k
        plugin.close()
