"""Host logic of the peer-memory gradient exchange, on CPU: the program rewrite, the payload
layout and slice split the kernel uses, and the rewritten program on the oracle (one rank and
two gloo ranks) against the plain program."""
import os
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as ge  # noqa: E402

ge.load_package()
from polarai_framework_b200.peer_gradients import payload_layout, slice_bounds  # noqa: E402
from polarai_framework_b200.program import (Program, exchange_pieces, fuse_gradient_exchange, fuse_program,  # noqa: E402
                                            logreg_program, mlp_program, overlap_gradient_exchange)


def test_rewrite_of_the_mlp_tail():
    p = fuse_gradient_exchange(fuse_program(mlp_program(64, 784, 96, 10, 0.1)))
    kinds = [k for k, _ in p.ops]
    assert "ALLREDUCE" not in kinds and kinds.count("ALLREDUCE_FADD") == 1 and kinds[-1] == "ALLREDUCE_FADD"
    k, a = p.ops[-1]
    assert a[:2] == [1.0, -0.1] and a[2:] == ["W2", "dW2", "W1", "dW1"]
    assert p.exchanged() == ["dW2", "dW1"]
    assert not any(k == "fadd" and a[0] in ("W1", "W2") for k, a in p.ops)
    # the unfused chain is rewritten the same way
    q = fuse_gradient_exchange(mlp_program(64, 784, 96, 10, 0.1))
    assert q.ops[-1][0] == "ALLREDUCE_FADD" and q.launches() == mlp_program(64, 784, 96, 10, 0.1).launches() - 1
    assert fuse_gradient_exchange(logreg_program()).ops[-1] == ("ALLREDUCE_FADD", [1.0, -0.1, "W", "dW"])


def test_rewrite_declines_what_it_cannot_prove():
    # different learning rates per tensor
    p = mlp_program(8, 16, 12, 4, 0.1)
    p.ops[-1] = ("fadd", ["W1", 1.0, "dW1", -0.2, "W1"])
    assert fuse_gradient_exchange(p) is p
    # a gradient with no update
    p = mlp_program(8, 16, 12, 4, 0.1)
    del p.ops[-1]
    assert fuse_gradient_exchange(p) is p
    # something reads a weight after the first update
    p = mlp_program(8, 16, 12, 4, 0.1)
    p.tensor("peek", 16, 12)
    p.ops.insert(len(p.ops) - 1, ("fmul", ["W2", "W2", "dW2"]))
    assert fuse_gradient_exchange(p) is p
    # no collective at all
    q = Program("plain")
    q.tensor("a", 4), q.tensor("b", 4)
    q.op("fmul", "a", "a", "b")
    assert fuse_gradient_exchange(q) is q


def test_payload_layout_and_slices_cover_the_vector_once():
    offsets, n = payload_layout({"dW2": (4096, 10), "odd": (7,), "dW1": (784, 4096)})
    assert offsets["dW2"] == (0, 40960) and offsets["odd"] == (40960, 7) and offsets["dW1"][0] == 40968
    assert n == 40968 + 784 * 4096 and all(off % 4 == 0 for off, _ in offsets.values())
    for n_floats in (1, 5, 4096, 3252224, 3252231):
        for world in (1, 2, 3, 4, 8, 16):
            n4 = (n_floats + 3) // 4
            at = 0
            for r in range(world):
                lo, hi = slice_bounds(n_floats, r, world)
                assert lo == min(at, n4) and lo <= hi <= n4
                at = hi if hi > lo else at
            assert at == n4


def _inputs(batch, hidden):
    rng = np.random.default_rng(0)
    X = rng.standard_normal((batch, 784)).astype(np.float32)
    Y = np.eye(10, dtype=np.float32)[rng.integers(0, 10, batch)]
    W1 = rng.uniform(-0.05, 0.05, (784, hidden)).astype(np.float32)
    W2 = rng.uniform(-0.2, 0.2, (hidden, 10)).astype(np.float32)
    return X, Y, W1, W2


def test_rewritten_program_equals_the_plain_one_on_the_oracle():
    from oracle import oracle as orc
    from oracle.program_executor import OracleExecutor
    X, Y, W1, W2 = _inputs(32, 48)
    plain = mlp_program(32, 784, 48, 10, 0.1)
    outs = []
    for prog in (plain, fuse_gradient_exchange(fuse_program(plain))):
        ex = OracleExecutor(prog, orc.Oracle(2))
        ex.set_inputs(X=X, Y=Y, W1=W1, W2=W2)
        ex.run()
        outs.append({k: ex.output(k).copy() for k in prog.outputs})
    for k in plain.outputs:
        assert np.array_equal(outs[0][k], outs[1][k]), k


def test_overlap_rewrite_cuts_the_last_gradient_by_rows():
    base = fuse_gradient_exchange(fuse_program(mlp_program(64, 784, 96, 10, 0.1)))
    p = overlap_gradient_exchange(base)
    kinds = [k for k, _ in p.ops]
    assert kinds[-4:] == ["fmatmul_t_f_rows", "ALLREDUCE_FADD_PART", "fmatmul_t_f_rows", "ALLREDUCE_FADD_PART"]
    (_, a1), (_, x1), (_, a2), (_, x2) = p.ops[-4:]
    assert a1 == ["X", "dZ1", 0.0, 512.0, "dW1"] and a2 == ["X", "dZ1", 512.0, 272.0, "dW1"]   # 784 = 512 + 272
    assert x1[2:4] == [1.0, 1.0] and exchange_pieces(x1) == [("W1", "dW1", 0, 512)]               # channel 1, overlapped
    assert x2[2:4] == [0.0, 0.0] and exchange_pieces(x2) == [("W1", "dW1", 512, 272), ("W2", "dW2", 0, -1)]
    assert p.exchanged() == ["dW1", "dW2"]          # payload order: the rest of dW1 and dW2 are adjacent
    # the pieces of the second exchange are adjacent in the payload, the first one starts it
    offsets, n = payload_layout({g: p.tensors[g] for g in p.exchanged()})
    assert offsets["dW1"] == (0, 784 * 96) and offsets["dW2"][0] == 784 * 96
    # too few rows to cut, or no exchange at the end: unchanged
    small = fuse_gradient_exchange(fuse_program(mlp_program(64, 300, 96, 10, 0.1)))
    assert overlap_gradient_exchange(small) is small
    plain = mlp_program(64, 784, 96, 10, 0.1)
    assert overlap_gradient_exchange(plain) is plain


def _worker(rank, world, port, batch, hidden, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch
    import torch.distributed as dist
    ge.load_package()
    from polarai_framework_b200.data_parallel import init_from_env, shard_rows
    from oracle import oracle as orc
    from oracle.program_executor import OracleExecutor
    r, w, _ = init_from_env("gloo")
    lo, hi = shard_rows(batch, r, w)
    X, Y, W1, W2 = _inputs(batch, hidden)

    def allreduce(a):
        t = torch.from_numpy(a.copy())
        dist.all_reduce(t)
        return t.numpy()

    res = {}
    for tag, rewrite in (("plain", 0), ("xchg", 1), ("over", 2)):
        prog = mlp_program(hi - lo, 784, hidden, 10, 0.1)
        if rewrite:
            prog = fuse_gradient_exchange(fuse_program(prog))
        if rewrite == 2:
            prog = overlap_gradient_exchange(prog)
            assert prog.ops[-1][0] == "ALLREDUCE_FADD_PART"
        ex = OracleExecutor(prog, orc.Oracle(2), allreduce)
        ex.set_inputs(X=X[lo:hi], Y=Y[lo:hi], W1=W1, W2=W2)
        ex.run()
        for k in ("W1", "W2", "dW1", "dW2"):
            res[f"{tag}_{k}"] = ex.output(k)
    np.savez(os.path.join(out_dir, f"rank{r}.npz"), **res)
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_rewritten_equals_plain(tmp_path):
    port = 29900 + os.getpid() % 90
    mp.spawn(_worker, args=(2, port, 32, 48, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    for k in ("W1", "W2", "dW1", "dW2"):
        assert np.array_equal(r0[f"xchg_{k}"], r0[f"plain_{k}"]), k      # same sums, same update arithmetic
        assert np.array_equal(r0[f"xchg_{k}"], r1[f"xchg_{k}"]), k       # replicas identical
        assert np.array_equal(r0[f"over_{k}"], r0[f"plain_{k}"]), k      # cut by rows and exchanged in two parts: same bits
        assert np.array_equal(r0[f"over_{k}"], r1[f"over_{k}"]), k
