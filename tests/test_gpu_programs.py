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
