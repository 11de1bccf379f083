"""polar_b200_allreduce_fadd: the gradient sum over ranks fused with the weight update, over
NVLink peer memory.  One rank (always): same bits as the all-reduce-free program.  Two ranks
(when the box has two GPUs; one process per GPU, never two waiting kernels on one GPU):
replicas identical, and identical to NCCL all-reduce + fadd (a sum of two terms has one order)."""
import ctypes
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _inputs(batch, hidden, seed=0):
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((batch, 784)).astype(np.float32)
    Y = np.eye(10, dtype=np.float32)[rng.integers(0, 10, batch)]
    W1 = rng.uniform(-0.05, 0.05, (784, hidden)).astype(np.float32)
    W2 = rng.uniform(-0.2, 0.2, (hidden, 10)).astype(np.float32)
    return X, Y, W1, W2


def test_one_rank_equals_the_plain_program_over_several_steps():
    import torch
    import __graft_entry__ as ge
    pkg = ge.load_package()
    from polarai_framework_b200.peer_gradients import PeerGradients
    from polarai_framework_b200.program import DeviceExecutor, fuse_gradient_exchange, fuse_program, mlp_program
    lib = pkg.lib()
    lib.cdll.polar_b200_device_status_clear()
    batch, hidden = 512, 1024
    X, Y, W1, W2 = _inputs(batch, hidden)
    fused = fuse_program(mlp_program(batch, 784, hidden, 10, 0.1))
    xprog = fuse_gradient_exchange(fused)
    peers = PeerGradients({g: xprog.tensors[g] for g in xprog.exchanged()}, 0, 1, "cuda:0")
    from polarai_framework_b200.program import overlap_gradient_exchange
    oprog = overlap_gradient_exchange(xprog)
    opeers = PeerGradients({g: oprog.tensors[g] for g in oprog.exchanged()}, 0, 1, "cuda:0")
    a = DeviceExecutor(fused, "cuda:0")
    b = DeviceExecutor(xprog, "cuda:0", peers=peers)
    c = DeviceExecutor(oprog, "cuda:0", peers=opeers)
    for ex in (a, b, c):
        ex.set_inputs(X=X, Y=Y, W1=W1, W2=W2)
    for step in range(4):
        a.run(), b.run(), c.run()
        for k in ("L", "W1", "W2", "dW1", "dW2"):
            assert np.array_equal(a.output(k).view(np.uint32), b.output(k).view(np.uint32)), (step, k)
        # dW1 in two blocks of rows on two streams: the same sums up to how the tensor-core path
        # runs a block (tile orientation, cuts of k), so W1 agrees to rounding and, from the second
        # step on, so does everything computed from it
        for k in ("L", "dW2"):
            if step == 0:
                assert np.array_equal(a.output(k).view(np.uint32), c.output(k).view(np.uint32)), (step, k)
        # (a rounding difference in W1 grows from step to step: lr = 0.1 on gradients of size 70)
        for k in ("L", "dW1", "dW2", "W1", "W2"):
            assert np.max(np.abs(a.output(k) - c.output(k))) <= 1e-5 * 10 ** step * np.abs(a.output(k)).max(), (step, k)
    assert lib.cdll.polar_b200_device_status() == 0
    del b, c
    peers.close()
    opeers.close()


def test_bad_arguments_are_statuses():
    import torch
    import __graft_entry__ as ge
    pkg = ge.load_package()
    from polarai_framework_b200.peer_gradients import PeerGradients, UpdateSegment
    lib = pkg.lib()
    peers = PeerGradients({"g": (64,)}, 0, 1, "cuda:0")
    w = torch.zeros(64, device="cuda")
    fn = lib.cdll.polar_b200_allreduce_fadd
    s = torch.cuda.current_stream().cuda_stream
    seg = peers.segments([(w, "g")])
    assert fn(peers.buffers, 1, 1, peers.n, seg, 1, 1.0, -0.1, s) != 0          # rank outside the group
    assert fn(peers.buffers, 0, 17, peers.n, seg, 1, 1.0, -0.1, s) != 0         # more ranks than the control block holds
    bad = (UpdateSegment * 1)()
    bad[0].weights, bad[0].offset, bad[0].count = w.data_ptr(), 32, 64            # runs past the payload
    assert fn(peers.buffers, 0, 1, peers.n, bad, 1, 1.0, -0.1, s) != 0
    bad[0].offset, bad[0].count = 2, 8                                            # gradient not 16-byte aligned
    assert fn(peers.buffers, 0, 1, peers.n, bad, 1, 1.0, -0.1, s) != 0
    assert "allreduce_fadd" in lib.last_error()
    null = (ctypes.c_void_p * 1)()
    assert fn(null, 0, 1, peers.n, seg, 1, 1.0, -0.1, s) != 0
    # and a good call still works afterwards: g = 3, w = 1  ->  w = 1*1 + 3*(-0.5) = -0.5
    peers.tensors["g"].fill_(3.0)
    w.fill_(1.0)
    assert fn(peers.buffers, 0, 1, peers.n, seg, 1, 1.0, -0.5, s) == 0
    torch.cuda.synchronize()
    assert torch.all(w == -0.5) and lib.cdll.polar_b200_device_status() == 0
    peers.close()


def test_a_peer_that_never_arrives_is_a_timeout_status_and_leaves_the_weights_alone():
    # One GPU, one launch: this rank is told it has a peer (a second buffer on the same GPU that
    # nothing ever signals).  With the wait limit set to 50 ms the kernel gives up on "ready",
    # skips the sum, never publishes "done", gives up on that too, and ends without touching W.
    # The status word says 301, the status check returns POLAR_B200_ERR_TIMEOUT, and after
    # a clear the library works as before.  Nothing here traps, faults or waits without a bound.
    import time
    import torch
    import __graft_entry__ as ge
    pkg = ge.load_package()
    from polarai_framework_b200.capi import PolarB200Error
    from polarai_framework_b200.peer_gradients import CONTROL_BYTES, PeerGradients
    lib = pkg.lib()
    c = lib.cdll
    c.polar_b200_device_status_clear()
    assert c.polar_b200_wait_limit_ns() == 0
    mine = PeerGradients({"g": (1 << 16,)}, 0, 1, "cuda:0")
    silent = ctypes.c_void_p()
    lib.check(c.polar_b200_peer_alloc(mine.n * 4, ctypes.byref(silent)))
    try:
        w = torch.full((1 << 16,), 1.0, device="cuda")
        mine.tensors["g"].fill_(3.0)
        seg = mine.segments([(w, "g")])
        buffers = (ctypes.c_void_p * 2)(mine.own, silent.value)
        st = torch.cuda.current_stream().cuda_stream
        c.polar_b200_set_wait_limit_ns(50_000_000)
        t0 = time.perf_counter()
        assert c.polar_b200_allreduce_fadd(buffers, 0, 2, mine.n, seg, 1, 1.0, -0.5, st) == 0   # the launch itself is fine
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t0
        assert 0.09 <= elapsed < 2.0, elapsed                       # two waits of 50 ms, not the 4 s default
        assert c.polar_b200_device_status() == 301 and c.polar_b200_device_status_of(0) == 301
        assert c.polar_b200_check_device_status() == 4                 # POLAR_B200_ERR_TIMEOUT
        assert "301" in lib.last_error()
        with pytest.raises(PolarB200Error) as err:
            lib.call("polar_b200_check_device_status")
        assert err.value.status == 4
        assert bool(torch.all(w == 1.0))                               # no update from a sum that never completed
        assert bool(torch.all(mine.tensors["g"] == 3.0))               # and the gradient is as it was
    finally:
        c.polar_b200_set_wait_limit_ns(0)
        c.polar_b200_device_status_clear()
    assert c.polar_b200_check_device_status() == 0
    # the context is intact: a one-rank step on the same buffer works (its step counter moved on)
    assert c.polar_b200_allreduce_fadd(buffers, 0, 1, mine.n, seg, 1, 1.0, -0.5, st) == 0
    torch.cuda.synchronize()
    assert bool(torch.all(w == -0.5)) and c.polar_b200_device_status() == 0
    c.polar_b200_peer_free(silent)
    mine.close()


def _rank_main(rank, world, port, out_dir, transport):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch
    import torch.distributed as dist
    import __graft_entry__ as ge
    pkg = ge.load_package()
    from polarai_framework_b200.data_parallel import init_from_env, make_allreduce, shard_rows
    from polarai_framework_b200.peer_gradients import PeerGradients
    from polarai_framework_b200.program import (DeviceExecutor, fuse_gradient_exchange, fuse_program, mlp_program,
                                                overlap_gradient_exchange)
    r, w, local = init_from_env("nccl")
    dev = f"cuda:{local}"
    batch, hidden = 1024, 1024
    lo, hi = shard_rows(batch, r, w)
    X, Y, W1, W2 = _inputs(batch, hidden)
    fused = fuse_program(mlp_program(hi - lo, 784, hidden, 10, 0.1))
    xprog = fuse_gradient_exchange(fused)
    try:
        peers = PeerGradients({g: xprog.tensors[g] for g in xprog.exchanged()}, r, w, dev, transport=transport)
    except RuntimeError as exc:
        # asked for "multicast" and the ranks agreed that there is none (the vote makes every rank land here)
        if r == 0:
            with open(os.path.join(out_dir, "no_multicast"), "w") as f:
                f.write(str(exc))
        dist.barrier()
        dist.destroy_process_group()
        return
    # the same exchange cut in two: the first block of dW1's rows travels on a second stream while
    # the second block is computed
    oprog = overlap_gradient_exchange(xprog)
    assert oprog.ops[-1][0] == "ALLREDUCE_FADD_PART"
    opeers = PeerGradients({g: oprog.tensors[g] for g in oprog.exchanged()}, r, w, dev, transport=transport)
    a = DeviceExecutor(fused, dev, make_allreduce(w))
    b = DeviceExecutor(xprog, dev, peers=peers)
    c = DeviceExecutor(oprog, dev, peers=opeers)
    for ex in (a, b, c):
        ex.set_inputs(X=X[lo:hi], Y=Y[lo:hi], W1=W1, W2=W2)
    res = {}
    for step in range(3):
        a.run(), b.run(), c.run()
    torch.cuda.synchronize()
    # and once more as a CUDA graph (fork and join of the second stream are captured)
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            c.run()
    torch.cuda.synchronize()
    dist.barrier()
    a.run(), b.run(), g.replay()
    torch.cuda.synchronize()
    for k in ("W1", "W2", "dW1", "dW2"):
        res[f"nccl_{k}"], res[f"peer_{k}"], res[f"over_{k}"] = a.output(k), b.output(k), c.output(k)
    res["status"] = np.array([pkg.lib().cdll.polar_b200_device_status()])
    res["multicast"] = np.array([1 if peers.transport == "multicast" else 0])
    np.savez(os.path.join(out_dir, f"rank{r}.npz"), **res)
    dist.barrier()
    torch.cuda.synchronize()
    del b, c, g
    peers.close()
    opeers.close()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("transport", ["ipc", "multicast"])
def test_two_ranks_on_two_gpus(tmp_path, transport):
    # "ipc": plain peer loads and stores.  "multicast": the sum inside the NVLink switch, on
    # symmetric memory with a multicast address (skipped where the machine offers none).  With
    # two ranks a sum has one rounding whatever its order, so both must give NCCL's bits.
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs: one process per GPU")
    port = 29700 + os.getpid() % 200 + (0 if transport == "ipc" else 1)
    mp.spawn(_rank_main, args=(2, port, str(tmp_path), transport), nprocs=2, join=True)
    if (tmp_path / "no_multicast").exists():
        pytest.skip("no NVLink multicast for symmetric memory here: " + (tmp_path / "no_multicast").read_text())
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    assert int(r0["status"][0]) == 0 and int(r1["status"][0]) == 0
    assert int(r0["multicast"][0]) == int(r1["multicast"][0]) == (1 if transport == "multicast" else 0)
    for k in ("W1", "W2", "dW1", "dW2"):
        assert np.array_equal(r0[f"peer_{k}"], r1[f"peer_{k}"]), k            # replicas identical
        assert np.array_equal(r0[f"peer_{k}"], r0[f"nccl_{k}"]), k            # a + b has one rounding
        assert np.array_equal(r0[f"over_{k}"], r1[f"over_{k}"]), k            # overlapped form: replicas identical too
        # the overlapped form computes dW1 in two blocks of rows, which the tensor-core path may
        # run in another tile orientation: equal to rounding in the first step, and after five
        # steps at lr = 0.1 to what that rounding has grown into
        scale = np.abs(r0[f"peer_{k}"]).max()
        assert np.max(np.abs(r0[f"over_{k}"] - r0[f"peer_{k}"])) <= 1e-3 * scale, k
