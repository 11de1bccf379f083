"""world_size-2 gloo test of the data-parallel host logic on CPU: two ranks each
run the MLP program on their half of the batch with the oracle as the compute
engine and all-reduce the weight gradients; the result must equal one rank running
the whole batch (up to summation order)."""
import os
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _inputs(batch, hidden):
    rng = np.random.default_rng(0)
    X = rng.standard_normal((batch, 784)).astype(np.float32)
    Y = np.eye(10, dtype=np.float32)[rng.integers(0, 10, batch)]
    W1 = rng.uniform(-0.05, 0.05, (784, hidden)).astype(np.float32)
    W2 = rng.uniform(-0.2, 0.2, (hidden, 10)).astype(np.float32)
    return X, Y, W1, W2


def _worker(rank, world, port, batch, hidden, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch
    import torch.distributed as dist
    import __graft_entry__ as ge
    ge.load_package()
    from polarai_framework_b200.data_parallel import init_from_env, shard_rows
    from polarai_framework_b200.program import mlp_program
    from oracle import oracle as orc
    from oracle.program_executor import OracleExecutor
    r, w, _ = init_from_env("gloo")
    lo, hi = shard_rows(batch, r, w)
    X, Y, W1, W2 = _inputs(batch, hidden)

    def allreduce(a):
        t = torch.from_numpy(a.copy())
        dist.all_reduce(t)
        return t.numpy()

    ex = OracleExecutor(mlp_program(hi - lo, 784, hidden, 10, 0.1), orc.Oracle(2), allreduce)
    ex.set_inputs(X=X[lo:hi], Y=Y[lo:hi], W1=W1, W2=W2)
    ex.run()
    np.savez(os.path.join(out_dir, f"rank{r}.npz"), W1=ex.output("W1"), W2=ex.output("W2"),
             dW1=ex.output("dW1"), L=ex.output("L"))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_equal_one(tmp_path):
    sys.path.insert(0, ROOT)
    import __graft_entry__ as ge
    ge.load_package()
    from polarai_framework_b200.program import mlp_program
    from oracle import oracle as orc
    from oracle.program_executor import OracleExecutor
    batch, hidden = 64, 96
    port = 29600 + os.getpid() % 300
    mp.spawn(_worker, args=(2, port, batch, hidden, str(tmp_path)), nprocs=2, join=True)
    X, Y, W1, W2 = _inputs(batch, hidden)
    one = OracleExecutor(mlp_program(batch, 784, hidden, 10, 0.1), orc.Oracle(2))
    one.set_inputs(X=X, Y=Y, W1=W1, W2=W2)
    one.run()
    r0 = np.load(tmp_path / "rank0.npz")
    r1 = np.load(tmp_path / "rank1.npz")
    # replicas stay bit-identical to each other
    assert np.array_equal(r0["W1"], r1["W1"]) and np.array_equal(r0["W2"], r1["W2"])
    # and equal the single-rank step up to the order of the batch sum
    for k in ("W1", "W2", "dW1"):
        want = one.output(k)
        assert np.max(np.abs(r0[k] - want)) / np.abs(want).max() <= 1e-5, k
    # per-row losses are shard-local and exact
    assert np.array_equal(np.concatenate([r0["L"], r1["L"]]), one.output("L"))


def test_shard_rows_rejects_uneven_batches():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as ge
    ge.load_package()
    from polarai_framework_b200.data_parallel import shard_rows
    assert shard_rows(65536, 3, 8) == (24576, 32768)
    with pytest.raises(ValueError):
        shard_rows(10, 0, 3)


def _late_worker(rank, world, port, out_dir):
    # Two steps.  Rank 1 takes part in the first exchange and then stays away from the second
    # (it waits, alive, then leaves between steps with nothing in flight).  Rank 0's second
    # exchange has a one-second limit: it must come back with POLAR_B200_ERR_TIMEOUT, not block.
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import time
    import torch
    import torch.distributed as dist
    import __graft_entry__ as ge
    ge.load_package()
    from polarai_framework_b200.capi import PolarB200Error
    from polarai_framework_b200.data_parallel import ERR_TIMEOUT, init_from_env, make_allreduce
    r, w, _ = init_from_env("gloo", timeout_s=30)
    allreduce = make_allreduce(w, timeout_s=1.0)
    g = torch.full((1024,), float(r + 1))
    allreduce(g)                                           # step 1: both ranks
    ok_first = bool(torch.all(g == 3.0))
    result = "no error"
    if r == 0:
        t0 = time.perf_counter()
        try:
            allreduce(torch.ones(1024))                    # step 2: the peer never joins
        except PolarB200Error as exc:
            result = f"status {exc.status} after {time.perf_counter() - t0:.2f}s"
            assert exc.status == ERR_TIMEOUT
    else:
        time.sleep(3.0)                                    # alive, not participating
    with open(os.path.join(out_dir, f"late{r}.txt"), "w") as fh:
        fh.write(f"{ok_first} {result}")
    # no further collective: the group is broken by design; leave without the usual barrier
    os._exit(0)


def test_a_rank_that_stays_away_is_a_timeout_status_on_the_host(tmp_path):
    port = 29900 + os.getpid() % 90
    mp.spawn(_late_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0 = open(tmp_path / "late0.txt").read()
    r1 = open(tmp_path / "late1.txt").read()
    assert r0.startswith("True status 4 after"), r0
    assert float(r0.split("after ")[1][:-1]) < 2.9                 # the limit, not the peer's sleep
    assert r1 == "True no error"
