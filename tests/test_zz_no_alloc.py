"""The allocation-free fmatmul entry point against the regular one.

polar_b200_fmatmul_tn_small_n_static is for hosts that cannot allocate device
memory while they run (all of it already belongs to their own allocator, or they
cannot afford cudaMalloc's device-wide synchronisation): its scratch is an array
inside the library image.  Here it is called through the C ABI twice in a row -
the second product smaller than the first, so values left in the shared scratch by
the first call would show if the kernel depended on a clean array - and each
result is compared with polar_b200_fmatmul on the same operands and, since that entry
point runs the same kernel, also with the CPU oracle's double-accumulated product.

The file name sorts last so that a run that stops at the first failure has
already run every other test."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1e-4   # |c - ref| / sum_k |a||b|, the bound the fmatmul tests use


@pytest.fixture(scope="module")
def env():
    import torch
    import __graft_entry__ as ge
    pkg = ge.load_package()
    assert torch.cuda.is_available()
    return torch, pkg.lib()


def both(torch, lib, m, n, k, tr, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    left = torch.empty((k, m), device="cuda").uniform_(-1, 1, generator=g)
    right = torch.empty((n, k) if tr else (k, n), device="cuda").uniform_(-1, 1, generator=g)
    ref = torch.full((m, n), float("nan"), device="cuda")
    got = torch.full((m, n), float("nan"), device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    lib.call("polar_b200_fmatmul", 1, tr, m, n, k, left.data_ptr(), right.data_ptr(), ref.data_ptr(), None, 0, st)
    lib.call("polar_b200_fmatmul_tn_small_n_static", tr, m, n, k, left.data_ptr(), right.data_ptr(),
             got.data_ptr(), st)
    torch.cuda.synchronize()
    mag = (left.T.double().abs() @ (right.T if tr else right).double().abs())
    err = float(((got.double() - ref.double()).abs() / mag).max())
    # against the oracle: sum over k in double on the CPU, error relative to sum_k |a||b|
    from oracle import oracle as orc
    cpu = orc.Oracle()
    cpu.set_threads(cpu.max_threads())
    exact, omag = cpu.fmatmul_f64(1, tr, left.cpu().numpy(), right.cpu().numpy())
    oerr = float(np.max(np.abs(got.cpu().numpy().astype(np.float64) - exact) / omag))
    return max(err, oerr), bool(torch.isfinite(got).all())


def test_two_calls_in_a_row_match_the_regular_entry_point(env):
    torch, lib = env
    assert lib.cdll.polar_b200_static_scratch_bytes() == 16 << 20
    # first call: the MLP's H^T dZ2 shape (12 MiB of partial sums)
    err, finite = both(torch, lib, 4096, 10, 16384, 0, seed=1)
    assert finite and err <= TOL
    # second call, straight after: smaller, other n, transposed right operand
    err, finite = both(torch, lib, 784, 3, 1000, 1, seed=2)
    assert finite and err <= TOL
    # and the first shape once more over the leftovers of the second
    err, finite = both(torch, lib, 4096, 10, 16384, 0, seed=3)
    assert finite and err <= TOL


def test_sizes_beyond_the_built_in_scratch_are_rejected(env):
    torch, lib = env
    m, n, k = 65536, 16, 8192              # 5 splits x 65536 x 16 floats = 20 MiB of partial sums
    need = lib.cdll.polar_b200_fmatmul_workspace_bytes(1, 0, m, n, k)
    assert need > lib.cdll.polar_b200_static_scratch_bytes()
    x = torch.zeros(16, device="cuda")
    rc = lib.cdll.polar_b200_fmatmul_tn_small_n_static(0, m, n, k, x.data_ptr(), x.data_ptr(), x.data_ptr(), None)
    assert rc == 5 and "16 MiB" in lib.last_error()
    # shapes the kernel does not serve are refused, not mis-computed
    rc = lib.cdll.polar_b200_fmatmul_tn_small_n_static(0, 4096, 64, 4096, x.data_ptr(), x.data_ptr(), x.data_ptr(), None)
    assert rc == 3
