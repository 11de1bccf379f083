"""The extended (fused) builtins give the same bits as the chains of reference
builtins they stand for."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch
    import __graft_entry__ as ge
    pkg = ge.load_package()
    from polarai_framework_b200.device_builtins import DeviceBuiltins
    return torch, pkg.lib(), DeviceBuiltins()


def st(torch):
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("n", [1, 5, 1024, 1_000_003])
def test_fsigmoid_grad_equals_the_three_launch_chain(env, n):
    torch, lib, d = env
    g = torch.empty(n, device="cuda").uniform_(-2, 2)
    s = torch.empty(n, device="cuda").uniform_(1e-5, 1 - 1e-5)
    ones = torch.ones(n, device="cuda")
    t1, t2, want, got = (torch.empty(n, device="cuda") for _ in range(4))
    d.fadd(ones, 1.0, s, -1.0, t1)
    d.fmul(t1, s, t2)
    d.fmul(g, t2, want)
    lib.call("polar_b200_fsigmoid_grad", g.data_ptr(), s.data_ptr(), got.data_ptr(), n, st(torch))
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int32), want.view(torch.int32))


@pytest.mark.parametrize("n", [1, 7, 4096, 655_360])
def test_fsigmoid_logloss_grad_equals_the_seven_launch_chain(env, n):
    torch, lib, d = env
    torch.manual_seed(n)
    p = torch.empty(n, device="cuda").uniform_(1e-5, 1 - 1e-5)
    y = (torch.rand(n, device="cuda") < 0.5).float()
    # the values fsigmoid's clamp produces, and a soft label
    edge = min(n, 4)
    p[:edge] = torch.tensor([1e-5, 1 - 1e-5, 0.5, 0.25], device="cuda")[:edge]
    if n > 5:
        y[5] = 0.3
    ones = torch.ones(n, device="cuda")
    pmy, pp, den, dldp, omp, sp, want, got = (torch.empty(n, device="cuda") for _ in range(8))
    d.fadd(p, 1.0, y, -1.0, pmy)
    d.fmul(p, p, pp)
    d.fadd(p, 1.0, pp, -1.0, den)
    d.fdivide(pmy, den, dldp)
    d.fadd(ones, 1.0, p, -1.0, omp)
    d.fmul(omp, p, sp)
    d.fmul(dldp, sp, want)
    lib.call("polar_b200_fsigmoid_logloss_grad", p.data_ptr(), y.data_ptr(), got.data_ptr(), n, st(torch))
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int32), want.view(torch.int32))
    # analytically dZ = p - y; away from the clamp values (where p - p*p cancels and the
    # reference's chain itself loses digits) the seven roundings stay within 1e-5 of it
    mid = (p > 0.05) & (p < 0.95)
    assert torch.allclose(got[mid], (p - y)[mid], rtol=0, atol=1e-5)


SHAPES = [
    (0, 0, 512, 512, 256),      # tensor cores, one work unit per tile: sigmoid in the epilogue
    (0, 0, 1024, 1024, 2048),   # tensor cores, k cut into work units: sigmoid in the summing kernel
    (0, 0, 300, 10, 512),       # small n, k slabs: sigmoid applied where the row sums are stored
    (0, 0, 4100, 10, 4096),     # small n, small operand resident in shared memory: same
    (1, 0, 1028, 5, 1000),      # small n, split k: no fused form, second builtin in place
    (0, 1, 1000, 512, 10),      # small k: sigmoid_grad fused
    (1, 1, 200, 301, 7),        # small k, ragged n (scalar stores)
    (1, 0, 33, 17, 50),         # FFMA fallback
]


@pytest.mark.parametrize("tl,tr,m,n,k", SHAPES)
def test_fused_matmuls_equal_two_launches(env, tl, tr, m, n, k):
    torch, lib, d = env
    torch.manual_seed(m + n + k)
    L = torch.empty((k, m) if tl else (m, k), device="cuda").uniform_(-1, 1)
    R = torch.empty((n, k) if tr else (k, n), device="cuda").uniform_(-1, 1)
    S = torch.empty((m, n), device="cuda").uniform_(1e-5, 1 - 1e-5)
    prod, want1, want2, got1, got2 = (torch.empty((m, n), device="cuda") for _ in range(5))
    d.fmatmul(tl, tr, L, R, prod)
    d.fsigmoid(prod, want1)
    lib.call("polar_b200_fsigmoid_grad", prod.data_ptr(), S.data_ptr(), want2.data_ptr(), m * n, st(torch))
    lib.call("polar_b200_fmatmul_sigmoid", tl, tr, m, n, k, L.data_ptr(), R.data_ptr(), got1.data_ptr(), None, 0,
             st(torch))
    lib.call("polar_b200_fmatmul_sigmoid_grad", tl, tr, m, n, k, L.data_ptr(), R.data_ptr(), S.data_ptr(),
             got2.data_ptr(), None, 0, st(torch))
    torch.cuda.synchronize()
    assert torch.equal(got1.view(torch.int32), want1.view(torch.int32))
    assert torch.equal(got2.view(torch.int32), want2.view(torch.int32))
    assert d.device_status() == 0


@pytest.mark.parametrize("batch,hidden", [(1024, 4096), (200, 256)])
def test_fused_mlp_program_is_bit_identical(env, batch, hidden):
    from polarai_framework_b200.program import DeviceExecutor, fuse_program, mlp_program
    rng = np.random.default_rng(1)
    X = rng.standard_normal((batch, 784)).astype(np.float32)
    Y = np.eye(10, dtype=np.float32)[rng.integers(0, 10, batch)]
    a1, a2 = np.sqrt(6 / (784 + hidden)), np.sqrt(6 / (hidden + 10))
    W1 = rng.uniform(-a1, a1, (784, hidden)).astype(np.float32)
    W2 = rng.uniform(-a2, a2, (hidden, 10)).astype(np.float32)
    plain = mlp_program(batch, 784, hidden, 10, 0.1)
    fused = fuse_program(plain)
    assert fused.launches() == plain.launches() - 11      # 20 launches become 9
    outs = []
    for prog in (plain, fused):
        ex = DeviceExecutor(prog)
        ex.set_inputs(X=X, Y=Y, W1=W1, W2=W2)
        ex.run()
        outs.append({k: ex.output(k) for k in prog.outputs})
    for k in plain.outputs:
        assert np.array_equal(outs[0][k].view(np.uint32), outs[1][k].view(np.uint32)), k
