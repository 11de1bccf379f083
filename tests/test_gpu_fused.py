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


@pytest.mark.parametrize("rows,kh,n", [
    (8192, 4096, 10),      # the MLP's output layer on one GPU of eight
    (1000, 260, 10),       # rows not a multiple of the staging depth, ragged last split
    (640, 1024, 16), (300, 64, 1), (4096, 512, 3),
    (100, 36, 17),         # more outputs than the one-pass kernel takes: the two builtins in sequence
    (16, 64, 4),           # too few rows: likewise
])
def test_fdense_grad_equals_its_two_builtins(env, rows, kh, n):
    # dW = H^T.dZ and dIn = (dZ.W^T)*((1-H)*H) from one pass over H: the bits of fmatmul_t_f and
    # fmatmul_f_t_sigmoid_grad, with the library's own scratch and with a caller workspace
    torch, lib, d = env
    torch.manual_seed(rows + kh + n)
    H = torch.empty((rows, kh), device="cuda").uniform_(1e-5, 1 - 1e-5)
    dZ = torch.empty((rows, n), device="cuda").uniform_(-1, 1)
    W = torch.empty((kh, n), device="cuda").uniform_(-0.5, 0.5)
    want_dw, got_dw = torch.empty((kh, n), device="cuda"), torch.full((kh, n), float("nan"), device="cuda")
    want_in, got_in = torch.empty((rows, kh), device="cuda"), torch.full((rows, kh), float("nan"), device="cuda")
    d.fmatmul(1, 0, H, dZ, want_dw)
    lib.call("polar_b200_fmatmul_sigmoid_grad", 0, 1, rows, kh, n, dZ.data_ptr(), W.data_ptr(), H.data_ptr(),
             want_in.data_ptr(), None, 0, st(torch))
    lib.call("polar_b200_fdense_grad", rows, kh, n, dZ.data_ptr(), W.data_ptr(), H.data_ptr(), got_dw.data_ptr(),
             got_in.data_ptr(), None, 0, st(torch))
    torch.cuda.synchronize()
    assert torch.equal(got_dw.view(torch.int32), want_dw.view(torch.int32))
    assert torch.equal(got_in.view(torch.int32), want_in.view(torch.int32))
    need = int(lib.cdll.polar_b200_fdense_grad_workspace_bytes(rows, kh, n))
    if need:
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        got_dw.fill_(float("nan")), got_in.fill_(float("nan"))
        lib.call("polar_b200_fdense_grad", rows, kh, n, dZ.data_ptr(), W.data_ptr(), H.data_ptr(), got_dw.data_ptr(),
                 got_in.data_ptr(), ws.data_ptr(), need, st(torch))
        torch.cuda.synchronize()
        assert torch.equal(got_dw.view(torch.int32), want_dw.view(torch.int32))
        assert torch.equal(got_in.view(torch.int32), want_in.view(torch.int32))
        assert lib.cdll.polar_b200_fdense_grad(rows, kh, n, dZ.data_ptr(), W.data_ptr(), H.data_ptr(),
                                               got_dw.data_ptr(), got_in.data_ptr(), ws.data_ptr(), need - 16,
                                               st(torch)) == 5
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
    assert fused.launches() == plain.launches() - 12      # 20 launches become 8
    outs = []
    for prog in (plain, fused):
        ex = DeviceExecutor(prog)
        ex.set_inputs(X=X, Y=Y, W1=W1, W2=W2)
        ex.run()
        outs.append({k: ex.output(k) for k in prog.outputs})
    for k in plain.outputs:
        assert np.array_equal(outs[0][k].view(np.uint32), outs[1][k].view(np.uint32)), k
