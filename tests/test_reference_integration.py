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
    assert "4 ran, 0 failed, 0 skipped" in out.stdout
