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


def _cuda_current_device():
    """The calling thread's current device as the CUDA runtime torch uses reports it."""
    import ctypes
    import torch
    cur = ctypes.c_int(-1)
    for name in ("libcudart.so.12", "libcudart.so"):
        try:
            rc = ctypes.CDLL(name).cudaGetDevice(ctypes.byref(cur))
        except OSError:
            continue
        assert rc == 0
        assert cur.value == torch.cuda.current_device()
        return cur.value
    return torch.cuda.current_device()


def test_write_launch_write_again_keeps_the_first_launch_input(rtb):
    # A host write returns before the upload of the previous version has necessarily run (the
    # upload is asynchronous, from pinned memory): the second write must not disturb what the
    # first launch reads.  Large enough that the copies take milliseconds.
    rt = rtb.rt
    n = 16 << 20
    v1 = np.arange(n, dtype=np.float32)
    v2 = -v1
    x, a, b = rt.tensor((n,)), rt.tensor((n,)), rt.tensor((n,))
    for _ in range(3):                                     # repeated: buffers alternate
        rt.write(x, v1)
        rt.launch("fcopy", [x, a])
        rt.write(x, v2)
        rt.launch("fcopy", [x, b])
        assert np.array_equal(rt.read(a), v1)
        assert np.array_equal(rt.read(b), v2)
    # in-place production through the record's own pinned buffer
    import ctypes
    host = ctypes.c_void_p()
    rt._check(rt.cdll.polar_b200_rt_host_begin_write(rt.h, x.virt_addr, x.bytes, ctypes.byref(host)))
    np.ctypeslib.as_array(ctypes.cast(host, ctypes.POINTER(ctypes.c_float)), (n,))[:] = 7.0
    rt._check(rt.cdll.polar_b200_rt_host_end_write(rt.h, x.virt_addr, x.bytes))
    rt.launch("fcopy", [x, a])
    assert np.all(rt.read(a) == 7.0)
    for t in (x, a, b):
        rt.free(t)


def test_read_waits_for_the_writer_of_the_record_not_for_later_launches(rtb):
    # the value read is the one the record had when read() was called, whatever was queued
    # for OTHER records afterwards
    rt = rtb.rt
    n = 8 << 20
    s, big1, big2 = rt.tensor((4,)), rt.tensor((n,)), rt.tensor((n,))
    rt.launch("ffill", [1.5, big1])
    rt.launch("ffill", [2.5, s])
    for _ in range(20):                                    # work queued behind the writer of `s`
        rt.launch("fcopy", [big1, big2])
    assert np.all(rt.read(s) == 2.5)
    assert np.all(rt.read(big2) == 1.5)
    for t in (s, big1, big2):
        rt.free(t)


def test_plugin_leaves_the_callers_device_alone():
    # A host that enumerates all GPUs through the plugin, computes on the LAST one and closes
    # must find its own current device unchanged after every call: the reference's driver
    # calls initContext() on the host's thread (RuntimeDriver.cpp:39-50) and a changed device
    # makes the host's next launch run on the wrong GPU.
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import __graft_entry__ as ge
    ge.load_package()
    from polarai_framework_b200.runtime import Runtime
    torch.cuda.set_device(0)
    mine = torch.ones(1024, device="cuda:0")
    assert _cuda_current_device() == 0
    rt = Runtime()
    assert _cuda_current_device() == 0
    last = rt.device_count() - 1
    assert last >= 1
    t = rt.tensor((1 << 16,), device=last)
    assert _cuda_current_device() == 0
    rt.launch("ffill", [3.0, t], device=last)
    assert _cuda_current_device() == 0
    assert np.all(rt.read(t) == 3.0)
    assert _cuda_current_device() == 0
    rt.barrier(last)
    rt.free(t)
    rt.close()
    assert _cuda_current_device() == 0
    assert float((mine * 2).sum().item()) == 2048.0      # the host's own tensors still work


def test_record_written_on_one_gpu_is_read_on_another():
    # device-to-device refresh: ordered after the producer kernel on the source GPU's stream
    # and before the consumer on the destination's, with no host synchronisation in between
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import __graft_entry__ as ge
    ge.load_package()
    from polarai_framework_b200.runtime import Runtime
    rt = Runtime()
    n = 32 << 20
    a = rt.tensor((n,), device=0)
    b = rt.tensor((n,), device=0)
    out = rt.tensor((n,), device=1)
    rt.cdll.polar_b200_rt_allocate(rt.h, 1, b.virt_addr, b.bytes)      # the same record, known to GPU 1 as well
    for k in range(3):
        rt.launch("ffill", [float(k + 1), a], device=0)
        rt.launch("fadd", [a, 1.0, a, 1.0, b], device=0)               # b = 2(k+1), produced on GPU 0
        rt.launch("fadd", [b, 1.0, b, 0.5, out], device=1)             # consumed on GPU 1: 3(k+1)
        rt.launch("ffill", [-1.0, b], device=0)                        # GPU 0 overwrites b right away
        assert np.all(rt.read(out) == 3.0 * (k + 1))
    for t in (a, b, out):
        rt.free(t)
    rt.close()
