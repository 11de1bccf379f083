"""GPU parity of whole builtin programs (the benchmark configurations) against the
same programs run on the CPU oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import __graft_entry__ as ge
    ge.load_package()
    from oracle import oracle as orc
    o = orc.Oracle()
    o.set_threads(o.max_threads())
    return o


def run_both(program, oracle, inputs):
    from polarai_framework_b200.program import DeviceExecutor
    from oracle.program_executor import OracleExecutor
    dev = DeviceExecutor(program)
    dev.set_inputs(**inputs)
    dev.run()
    cpu = OracleExecutor(program, oracle)
    cpu.set_inputs(**inputs)
    cpu.run()
    return dev, cpu


def max_rel(got, want):
    return float(np.max(np.abs(got.astype(np.float64) - want) / np.maximum(np.abs(want), 1e-30)))


def test_elementwise_chain_2pow20(env):
    from polarai_framework_b200.program import elementwise_chain_program
    rng = np.random.default_rng(0)
    n = 1 << 20
    ins = {k: rng.uniform(-1, 1, n).astype(np.float32) for k in "abc"}
    ins["d"] = rng.uniform(0.5, 2, n).astype(np.float32)
    dev, cpu = run_both(elementwise_chain_program(n), env, ins)
    assert np.array_equal(dev.output("t3"), cpu.output("t3"))          # add, mul, divide: bit-exact
    assert max_rel(dev.output("out"), cpu.output("out")) <= 1e-5


def test_logistic_regression_step(env):
    from polarai_framework_b200.program import logreg_program
    rng = np.random.default_rng(0)
    X = rng.standard_normal((256, 784)).astype(np.float32)
    W = (rng.standard_normal((784, 1)) * 0.01).astype(np.float32)
    Y = (rng.random((256, 1)) < 0.5).astype(np.float32)
    dev, cpu = run_both(logreg_program(256, 784, 0.1), env, dict(X=X, W=W, Y=Y))
    assert max_rel(dev.output("L"), cpu.output("L")) <= 1e-4
    scale = np.abs(cpu.output("dW")).max()
    assert np.max(np.abs(dev.output("dW") - cpu.output("dW"))) / scale <= 1e-4
    assert np.max(np.abs(dev.output("W") - cpu.output("W"))) / np.abs(cpu.output("W")).max() <= 1e-4


@pytest.mark.parametrize("batch,hidden", [(512, 4096), (1000, 256)])
def test_mlp_step(env, batch, hidden):
    from polarai_framework_b200.program import mlp_program
    rng = np.random.default_rng(0)
    X = rng.standard_normal((batch, 784)).astype(np.float32)
    Y = np.eye(10, dtype=np.float32)[rng.integers(0, 10, batch)]
    a1, a2 = np.sqrt(6 / (784 + hidden)), np.sqrt(6 / (hidden + 10))
    W1 = rng.uniform(-a1, a1, (784, hidden)).astype(np.float32)
    W2 = rng.uniform(-a2, a2, (hidden, 10)).astype(np.float32)
    dev, cpu = run_both(mlp_program(batch, 784, hidden, 10, 0.1), env, dict(X=X, Y=Y, W1=W1, W2=W2))
    assert max_rel(dev.output("L"), cpu.output("L")) <= 1e-4
    assert abs(dev.output("L").mean() - cpu.output("L").mean()) / cpu.output("L").mean() <= 1e-4
    for g in ("dW1", "dW2", "W1", "W2"):
        want = cpu.output(g)
        assert np.max(np.abs(dev.output(g) - want)) / np.abs(want).max() <= 1e-4, g


def test_full_batch_mlp_step_is_the_sum_of_its_halves():
    # Config 4 at its full size (65536 rows on one GPU), checked through a property the CPU
    # oracle is too slow to check directly: every row's loss is independent of the other rows,
    # and the weight gradients (batch sums) of the whole batch equal the sum of the gradients
    # of its two halves - the identity the data-parallel split relies on.
    import torch
    from polarai_framework_b200.program import DeviceExecutor, fuse_program, mlp_program
    batch, hidden = 65536, 4096
    g = torch.Generator(device="cuda").manual_seed(4)
    X = torch.randn((batch, 784), device="cuda", generator=g)
    Y = torch.nn.functional.one_hot(torch.randint(0, 10, (batch,), device="cuda", generator=g), 10).float()
    a1, a2 = (6 / (784 + hidden)) ** 0.5, (6 / (hidden + 10)) ** 0.5
    W1 = (torch.rand((784, hidden), device="cuda", generator=g) * 2 - 1) * a1
    W2 = (torch.rand((hidden, 10), device="cuda", generator=g) * 2 - 1) * a2

    def step(rows, fused):
        prog = mlp_program(rows.stop - rows.start, 784, hidden, 10, 0.1)
        ex = DeviceExecutor(fuse_program(prog) if fused else prog)
        ex.set_inputs(X=X[rows], Y=Y[rows], W1=W1, W2=W2)
        ex.run()
        torch.cuda.synchronize()
        out = {k: ex.t[k].clone() for k in ("L", "dW1", "dW2", "W1", "W2", "dZ1", "dZ2", "H")}
        del ex
        return out

    whole = step(slice(0, batch), True)
    lo, hi = step(slice(0, batch // 2), True), step(slice(batch // 2, batch), True)
    assert torch.equal(torch.cat([lo["L"], hi["L"]]), whole["L"])
    # Tolerance in the matmul tests' metric, |error| / sum_k |a||b|: the tensor-core accumulator
    # rounds toward zero at every step, so a 65536-term sum carries about 4e-6 of it (measured
    # against float64), far more than the 2e-8 of a round-to-nearest fp32 sum and still 20x inside 1e-4.
    torch.backends.cuda.matmul.allow_tf32 = False
    for k, left, right in (("dW1", X, whole["dZ1"]), ("dW2", whole["H"], whole["dZ2"])):
        both = lo[k] + hi[k]
        mag = left.abs().t() @ right.abs()
        assert float(((whole[k] - both).abs() / mag).max()) <= 2e-5, k
        ref = (left[:, :8].double().t() @ right.double())          # eight full rows in float64
        assert float(((whole[k][:8].double() - ref).abs() / mag[:8].double()).max()) <= 1e-5, k
    # the extended builtins give the bits of the one-launch-per-builtin chain at this size too
    chain = step(slice(0, batch), False)
    for k in ("L", "dW1", "dW2", "W1", "W2"):
        assert torch.equal(whole[k].view(torch.int32), chain[k].view(torch.int32)), k
    # mean loss of an untrained 10-way sigmoid classifier with these initial weights
    assert 0.6 < float(whole["L"].mean()) < 0.9
    from polarai_framework_b200.capi import lib
    assert lib().cdll.polar_b200_device_status() == 0
