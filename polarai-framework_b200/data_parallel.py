"""Batch-sharded (data-parallel) execution of a builtin program.

The reference runs every node on devices.front() (ExecutorImpl.cpp:71-75;
ath_device_select, routines.cpp:73-79) and has no collective.  Here each rank
owns one GPU and the rows [rank*B/n, (rank+1)*B/n) of every batch-shaped tensor;
weights are replicated; the only exchange per step is the sum of the weight
gradients over ranks, after which every rank applies the identical update, so the
replicas stay bit-identical.  torch.distributed provides the process group.

`DataParallelExecutor` is the whole of it for a caller: build the per-rank program,
choose the exchange (one kernel per rank over NVLink peer memory, or NCCL all-reduces
followed by fadd updates - every rank takes the NCCL form if mapping peer memory fails
on any rank), place replicated and sharded inputs, step, optionally as a CUDA graph.
"""
import datetime
import hashlib
import os

import torch
import torch.distributed as dist

from .capi import PolarB200Error

ERR_TIMEOUT = 4   # POLAR_B200_ERR_TIMEOUT


def shard_rows(global_batch, rank, world):
    """Row range of this rank; the global batch must divide evenly so that every
    rank launches identical shapes."""
    if global_batch % world:
        raise ValueError(f"global batch {global_batch} is not divisible by {world} ranks")
    per = global_batch // world
    return rank * per, (rank + 1) * per


def init_from_env(backend=None, timeout_s=None):
    """Joins the process group described by RANK/WORLD_SIZE/MASTER_ADDR/MASTER_PORT
    (as torchrun sets them).  Returns (rank, world, local_rank).  `timeout_s` bounds every
    collective of the group (NCCL: enforced by its watchdog; gloo: by the call itself)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kw = {}
        if timeout_s is not None:
            kw["timeout"] = datetime.timedelta(seconds=float(timeout_s))
        if backend == "nccl":
            torch.cuda.set_device(local)
            dist.init_process_group(backend, rank=rank, world_size=world,
                                    device_id=torch.device(f"cuda:{local}"), **kw)
        else:
            dist.init_process_group(backend, rank=rank, world_size=world, **kw)
    return rank, world, local


def make_allreduce(world, timeout_s=None):
    """Sum over ranks, in place, in the current stream's order.

    With `timeout_s` the call is bounded on the host: a rank that never joins (or a lost
    connection) raises PolarB200Error with status POLAR_B200_ERR_TIMEOUT instead of blocking
    the caller for ever.  On a CPU process group (gloo) the wait itself carries the limit; on
    NCCL the collective is stream-ordered and the limit is the process group's (init_from_env
    passes it on), whose watchdog aborts the communicator - the error then surfaces at the next
    synchronisation and is mapped to the same status."""
    if world <= 1:
        return None
    limit = None if timeout_s is None else datetime.timedelta(seconds=float(timeout_s))

    def allreduce(t):
        try:
            if limit is not None and not t.is_cuda:
                work = dist.all_reduce(t, op=dist.ReduceOp.SUM, async_op=True)
                if not work.wait(limit):
                    raise RuntimeError("all-reduce did not complete")
            else:
                dist.all_reduce(t, op=dist.ReduceOp.SUM)
        except (RuntimeError, dist.DistBackendError) as exc:
            raise PolarB200Error(ERR_TIMEOUT, f"gradient all-reduce over {world} ranks failed or ran out of "
                                              f"time: {exc}") from exc
        return t
    return allreduce


def tensor_digest(*tensors):
    """SHA-256 of the tensors' bytes (through the host): equal digests = bit-identical replicas."""
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.detach().contiguous().cpu().numpy().tobytes())
    return h.hexdigest()


class DataParallelExecutor:
    """One rank of a batch-sharded program.

    make_program(rows) builds the builtin program for `rows` rows (program.mlp_program,
    program.logreg_program); `sharded` names the inputs whose first dimension is the batch.
    builtins = "extended" applies program.fuse_program (outputs bit-identical to the chain);
    collective = "peer" asks for the single-kernel exchange over NVLink peer memory ("peer-ipc": plain
    peer loads and stores only, the form to use where a rank may leave in mid-run; "peer-multicast":
    the sum done inside the switch where symmetric memory has a multicast address, else plain); with
    overlap=True the last weight gradient is computed in two blocks of rows and the first block's
    exchange runs on a second stream while the second block is computed
    (program.overlap_gradient_exchange).  Off by default: on B200 the two-block matmul costs
    34-40 us more than the one-launch form at the per-GPU shapes of the 784-4096-10 step, which is
    what the overlap hides of the exchange - measured 0.805 vs 0.779 ms per step at 8 GPUs.
    """

    def __init__(self, make_program, global_batch, sharded=("X", "Y"), rank=0, world=1, device="cuda:0",
                 builtins="extended", collective="peer", timeout_s=None, overlap=False):
        from .peer_gradients import PeerGradients
        from .program import DeviceExecutor, fuse_gradient_exchange, fuse_program, overlap_gradient_exchange
        self.rank, self.world = rank, world
        self.device = torch.device(device)
        self.global_batch = global_batch
        self.lo, self.hi = shard_rows(global_batch, rank, world)
        self.rows = self.hi - self.lo
        self.sharded = tuple(sharded)
        self.chain = make_program(self.rows)
        fused = builtins == "extended"
        program = fuse_program(self.chain) if fused else self.chain
        self.peers = None
        self.collective = "none (one rank)"
        if world > 1:
            self.collective = "nccl all-reduce, then fadd updates"
            if fused and collective in ("peer", "peer-ipc", "peer-multicast"):
                xprog = fuse_gradient_exchange(program)
                if overlap:
                    xprog = overlap_gradient_exchange(xprog)
                why = ""
                peers = None
                if xprog.exchanged():
                    try:
                        shapes = {g: xprog.tensors[g] for g in xprog.exchanged()}
                        want = {"peer-ipc": "ipc", "peer-multicast": "multicast"}.get(collective, "auto")
                        try:
                            peers = PeerGradients(shapes, rank, world, self.device, transport=want)
                        except RuntimeError:
                            if want != "multicast":
                                raise
                            # no multicast address here (every rank lands here together: the ranks vote)
                            peers = PeerGradients(shapes, rank, world, self.device, transport="ipc")
                    except Exception as exc:               # noqa: BLE001 - any failure means "not available here"
                        why = f"{type(exc).__name__}: {exc}"
                # every rank must take the same form: a vote
                ok = torch.tensor([0 if peers is None else 1], device=self.device)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN)
                if int(ok.item()) == 1:
                    program, self.peers = xprog, peers
                    self.collective = ("peer memory over NVLink: sum over ranks and weight update in one kernel "
                                       "per rank" + (", the sum done inside the switch (multimem)"
                                                     if peers.transport == "multicast" else ""))
                    if any(k == "ALLREDUCE_FADD_PART" for k, _ in xprog.ops):
                        self.collective += ("; the last weight gradient in two blocks of rows, the first block's "
                                            "exchange overlapping the second block's matmul")
                else:
                    if peers is not None:
                        peers.close()
                    self.collective += f" (peer memory unavailable on some rank{': ' + why if why else ''})"
        self.program = program
        with torch.cuda.device(self.device):
            self.ex = DeviceExecutor(program, self.device, make_allreduce(world, timeout_s), peers=self.peers)
        self.t = self.ex.t
        self.graph = None
        self.capture_error = ""

    # ---- data placement
    def set_replicated(self, **arrays):
        self.ex.set_inputs(**arrays)

    def set_sharded(self, **global_arrays):
        """Takes the GLOBAL batch; this rank keeps its rows."""
        self.ex.set_inputs(**{k: v[self.lo:self.hi] for k, v in global_arrays.items()})

    # ---- execution
    def step(self):
        """One pass of the program on torch's current stream (eager, or the captured graph)."""
        if self.graph is not None:
            self.graph.replay()
        else:
            self.ex.run()

    def capture(self, warmup=1):
        """Captures one step into a CUDA graph (after `warmup` eager steps on the capture stream);
        step() replays it from then on.  Returns False, and stays eager, if capture fails."""
        try:
            with torch.cuda.device(self.device):
                side = torch.cuda.Stream(self.device)
                side.wait_stream(torch.cuda.current_stream(self.device))
                with torch.cuda.stream(side):
                    for _ in range(max(1, warmup)):
                        self.ex.run()
                    torch.cuda.synchronize(self.device)
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=side):
                        self.ex.run()
                torch.cuda.synchronize(self.device)
            self.graph = graph
            return True
        except Exception as exc:                           # noqa: BLE001 - capture is an optimisation
            self.graph = None
            self.capture_error = f"{type(exc).__name__}: {exc}"
            torch.cuda.synchronize(self.device)
            return False

    def output(self, name):
        return self.ex.output(name)

    def replicas_identical(self, *names):
        """True when every rank holds the same bits in the named (replicated) tensors."""
        torch.cuda.synchronize(self.device)
        mine = tensor_digest(*[self.t[n] for n in names])
        if self.world <= 1:
            return True
        all_digests = [None] * self.world
        dist.all_gather_object(all_digests, mine)
        return all(d == all_digests[0] for d in all_digests)

    def device_status(self):
        return int(self.ex.lib.cdll.polar_b200_device_status_of(self.device.index or 0))

    def close(self):
        """Drops the graph and unmaps peer memory.  Every rank must have finished its last step
        (a barrier on the host) before any rank calls this."""
        self.graph = None
        torch.cuda.synchronize(self.device)
        if self.peers is not None:
            self.ex.t = {}
            self.t = {}
            self.peers.close()
            self.peers = None
