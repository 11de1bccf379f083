"""The reference project's own integration tests - all twelve files of
tests/integration/operations/ in the reference (Add, Combine, Conv2D, Divide, LogLoss,
MatMul, MulConcat, Mul, Pool2D, ReLU, Sigmoid, Softmax) - compiled unmodified against this
package's Executor and run against the B200 device plugin.

The binary is built by polarai-framework_b200/build.py from the reference tree
where it lies (with the stand-in gtest header in tests/ref_integration/); it is not
tracked, and on a machine without the reference tree the prebuilt file is used.
Each test builds a graph with the unchanged Context/Graph/Node/Loader API,
Executor::addGraph + evaluate, and compares with the test's in-file CPU loop with
EXPECT_FLOAT_EQ (4 units in the last place)."""
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "polarai-framework_b200", "lib", "ref", "ref_integration_tests")


def run(*flags):
    out = subprocess.run([BIN, *flags], capture_output=True, text=True, timeout=300)
    m = re.search(r"(\d+) ran, (\d+) failed, (\d+) skipped, (\d+) disabled", out.stdout)
    assert m, out.stdout + out.stderr
    return out, tuple(int(x) for x in m.groups())


@pytest.mark.skipif(not os.path.exists(BIN), reason="reference integration tests are not built")
def test_binary_loads_the_plugin_and_skips_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("covered by the GPU test")
    out, (ran, failed, skipped, disabled) = run("--also_run_disabled_tests")
    assert out.returncode == 0 and ran == 17 and failed == 0 and skipped == 17


@pytest.mark.gpu
def test_reference_integration_tests_pass_on_the_b200_device():
    assert os.path.exists(BIN), "build the package where the reference tree is present"
    out, (ran, failed, skipped, disabled) = run()
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-2000:]
    assert (ran, failed, skipped, disabled) == (15, 0, 0, 2), out.stdout[-3000:]
    # the two tests the reference ships DISABLED_ (Sigmoid, LogLoss) pass as well
    out, (ran, failed, skipped, disabled) = run("--also_run_disabled_tests")
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-2000:]
    assert (ran, failed, skipped, disabled) == (17, 0, 0, 0), out.stdout[-3000:]


PARITY = os.path.join(ROOT, "polarai-framework_b200", "lib", "ref", "autograd_parity")


@pytest.mark.skipif(not os.path.exists(PARITY), reason="autograd parity binary is not built")
@pytest.mark.parametrize("batch", [1, 256])
def test_reference_autograd_runs_through_the_executor_on_the_oracle_device(batch):
    # CPU part: Graph::getGradient's gradient and weight-update graphs execute through the
    # direct Executor on the oracle device; at batch 1 the result equals the analytic SGD step.
    out = subprocess.run([PARITY, str(batch)], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    # 18 builtins of the two graphs + 7 constant tensors (ones/zeros of the gradient graph, the
    # learning rate) filled on the device by ffill instead of the reference's host loop
    assert "oracle device: 25 launches" in out.stdout
    if batch == 1:
        assert "analytic SGD step" in out.stdout
    # with the reference's host-side constant fill the same numbers come out of 18 launches
    env = dict(os.environ, POLAR_B200_HOST_CONSTANTS="1")
    host = subprocess.run([PARITY, str(batch)], capture_output=True, text=True, timeout=300, env=env)
    assert host.returncode == 0, host.stdout + host.stderr
    assert "oracle device: 18 launches" in host.stdout
    assert host.stdout.split("launches", 1)[1] == out.stdout.split("launches", 1)[1]


@pytest.mark.gpu
@pytest.mark.parametrize("batch", [1, 256])
def test_logistic_regression_with_reference_autograd_matches_the_oracle_device(batch):
    assert os.path.exists(PARITY), "build the package where the reference tree is present"
    out = subprocess.run([PARITY, str(batch)], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "PARITY OK" in out.stdout, out.stdout


LSPOLAR = os.path.join(ROOT, "polarai-framework_b200", "lib", "ref", "lspolar")


@pytest.mark.skipif(not os.path.exists(LSPOLAR), reason="lspolar is not built")
def test_reference_lspolar_loads_the_plugin():
    # utils/lspolar/main.cpp of the reference, unmodified: RuntimeDriver dlopens libpolar_rt_cuda.so
    import torch
    out = subprocess.run([LSPOLAR], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "Total device count:" in out.stdout
    if torch.cuda.is_available():
        n = torch.cuda.device_count()
        assert f"Total device count: {n}" in out.stdout
        for i in range(n):
            assert f"#{i}" in out.stdout
        assert "Provider   : CUDA" in out.stdout and "Kind       : GPU" in out.stdout
    else:
        assert "Total device count: 0" in out.stdout


ALLOC_TEST = os.path.join(ROOT, "polarai-framework_b200", "lib", "ref", "pool_allocator_test")


@pytest.mark.skipif(not os.path.exists(ALLOC_TEST), reason="allocator unit tests are not built")
def test_pool_backend_allocator_host_logic():
    # coherence, lock conflicts and error statuses of the BackendAllocator, with fake devices (no CUDA needed)
    out = subprocess.run([ALLOC_TEST], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "6 ran, 0 failed, 0 skipped" in out.stdout


@pytest.mark.skipif(not os.path.exists(PARITY), reason="autograd parity binary is not built")
def test_recorded_program_has_the_call_sequence_the_reference_lowering_pins():
    # The reference pins, per node, the order of runtime calls its graph lowering emits
    # (utils/dialects/test/conversion/graph_to_runtime.mlir:52-110): an input node is
    # alloc, lock read_write, invoke_loader, release; an operation node is alloc(out),
    # lock read_write(out), lock read per operand, the launch with arguments in builtin order,
    # release per operand, release(out); a barrier closes each cluster.  The Executor of this
    # package replays exactly that, recorded through the reference's own Generator.
    env = dict(os.environ, POLAR_B200_DUMP_PROGRAM="1")
    out = subprocess.run([PARITY, "1"], capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0, out.stdout + out.stderr
    text = out.stdout
    first = text[text.index("program logreg\n"):text.index("program GradientGraph")]
    lines = [l.strip() for l in first.splitlines()[1:]]
    nodes, cur = {}, None
    order = []
    for l in lines:
        if l.startswith("node "):
            cur = l.split()[1]
            nodes[cur] = []
            order.append(cur)
        elif l.startswith("barrier"):
            order.append(l)
        else:
            nodes[cur].append(l)
    va = {n: nodes[n][0].split("va=")[1] for n in nodes}            # every node allocates its result first
    for n in ("X", "W", "Y"):
        assert nodes[n] == [f"alloc va={va[n]}", f"lock read_write va={va[n]}", f"load va={va[n]}",
                            f"release va={va[n]}"], n
    assert nodes["matmul"] == [f"alloc va={va['matmul']}", f"lock read_write va={va['matmul']}",
                               f"lock read va={va['W']}", f"lock read va={va['X']}",
                               f"launch fmatmul_f_f T{va['X']} T{va['W']} T{va['matmul']}",
                               f"release va={va['W']}", f"release va={va['X']}", f"release va={va['matmul']}"]
    assert nodes["sigmoid"][3] == f"launch fsigmoid T{va['matmul']} T{va['sigmoid']}"
    # LogLoss: predicted first, ground truth second, whatever the edge marks' numbering
    assert f"launch flogloss T{va['sigmoid']} T{va['Y']} T{va['logloss']}" in nodes["logloss"]
    # clusters: the three inputs, then one operation per cluster, a barrier after each
    assert order[:4] == ["X", "W", "Y", "barrier cluster=0"]
    assert order[4:10] == ["matmul", "barrier cluster=1", "sigmoid", "barrier cluster=2", "logloss",
                           "barrier cluster=3"]
    # the gradient graph's constants are recorded as loads too (they become ffill at run time)
    grad = text[text.index("program GradientGraph"):]
    assert "launch fmulconcat" in grad and "launch fdivide" in grad and "launch fadd" in grad
    # fadd's argument order: tensor, scale, tensor, scale, result (kernel_materialize.mlir:36,73)
    fadd = next(l.split()[2:] for l in grad.splitlines() if l.strip().startswith("launch fadd"))
    assert [t[0] for t in fadd] == ["T", "f", "T", "f", "T"], fadd


DP_EXEC = os.path.join(ROOT, "polarai-framework_b200", "lib", "ref", "data_parallel_executor")


@pytest.mark.skipif(not os.path.exists(DP_EXEC), reason="data-parallel executor test is not built")
def test_executor_splits_the_batch_over_fake_devices():
    # The Executor given 2 and 4 (fake, oracle-computing) devices and told which inputs are
    # batch-shaped: every device receives the whole program on its rows, the batch contraction is
    # summed over the devices, results equal the one-device run; undeclared, only the first
    # device works (the reference's behaviour).
    out = subprocess.run([DP_EXEC], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "DATA PARALLEL OK" in out.stdout
    assert "2 devices 5 5 | 4 devices 5 5 5 5" in out.stdout
    assert "undeclared: second device got 0 launches" in out.stdout


@pytest.mark.gpu
def test_executor_splits_the_batch_over_the_b200_devices():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    assert os.path.exists(DP_EXEC), "build the package where the reference tree is present"
    out = subprocess.run([DP_EXEC], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "B200 devices vs the oracle on one device" in out.stdout and "DATA PARALLEL OK" in out.stdout
