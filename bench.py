#!/usr/bin/env python
"""Benchmark of the PolarAI B200 runtime's hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--workload mlp|gemm|elementwise] [--builtins extended|reference]
                    [--collective peer|nccl] [--batch B] [--no-graph] [--no-extras]
                    [--no-parity] [--no-plugin]

Default workload (the one that shards over 1/2/4/8 GPUs): one training step of the
2-layer MLP 784-4096-10 (Sigmoid hidden layer, LogLoss on one-hot targets, fp32,
global batch 65536 batch-sharded over the ranks, sum of the weight gradients over
the ranks, SGD update at lr = 0.1), expressed as the reference's builtins
(polarai-framework_b200/program.py) - by default with the extended (fused)
builtins, whose outputs are bit-identical to the one-launch-per-builtin chain, and
at N > 1 with the gradient sum and the update as one kernel over NVLink peer memory
(--collective nccl: NCCL all-reduces followed by fadd).  Data is synthetic:
X ~ N(0,1), uniform labels, Xavier-uniform weights, seed 0.

One JSON line is printed by rank 0.  `value` is samples/s with the inputs already
in HBM; `e2e` is samples/s through the reference-facing runtime plugin (Device::launch
per builtin) when every step writes its X and Y shard from host arrays and reads the
loss back (`e2e_direct`: the same through direct C-ABI calls and a CUDA graph).  At N > 1
`parity` compares one step with the same step on one GPU; the run fails above 1e-4.  `roofline` describes the
dominant kernel (the tcgen05 fmatmul), `cpu_baseline` the same builtin program
timed on host cores on a bounded sample (rank 0, N=1 only).  With --workload gemm
or elementwise the line reports fp32 MatMul TFLOP/s at 8192^3 or HBM GB/s of the
elementwise builtins at 2^28 elements instead (single GPU).

--impl reference times the reference's own CPU statement of the builtins (its
OpenCL C kernels compiled as C when oracle/_ref was built, else the C restatement)
on all host cores, on a bounded sample of the same workload per step.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_IN, N_HIDDEN, N_OUT, GLOBAL_BATCH, LR = 784, 4096, 10, 65536, 0.1
FLOP_PER_SAMPLE = 2 * (2 * N_IN * N_HIDDEN + 3 * N_HIDDEN * N_OUT)   # 13,090,816
CPU_SAMPLE_ROWS = 512   # rows per step of every CPU timing (baseline leg and reference arm alike)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])), mx.append(float(f[2])), power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def mlp_inputs(rng, batch):
    import numpy as np
    X = rng.standard_normal((batch, N_IN), dtype=np.float32)
    labels = rng.integers(0, N_OUT, batch)
    Y = np.zeros((batch, N_OUT), np.float32)
    Y[np.arange(batch), labels] = 1.0
    return X, Y


def mlp_weights(rng):
    import numpy as np
    a1, a2 = np.sqrt(6.0 / (N_IN + N_HIDDEN)), np.sqrt(6.0 / (N_HIDDEN + N_OUT))
    W1 = rng.uniform(-a1, a1, (N_IN, N_HIDDEN)).astype(np.float32)
    W2 = rng.uniform(-a2, a2, (N_HIDDEN, N_OUT)).astype(np.float32)
    return W1, W2


def cpu_impl():
    """The CPU engine for baselines: the reference's kernels compiled as C when
    oracle/_ref exists, else the C restatement; all host threads."""
    from oracle import oracle as orc
    if orc.RefOcl.available():
        impl = orc.RefOcl()
    else:
        impl = orc.Oracle()
    impl.set_threads(impl.max_threads())
    return impl


def cpu_mlp_baseline(sample_batch, steps=1, warmup=0):
    """The MLP builtin program on host cores over `sample_batch` rows per step."""
    import numpy as np
    import __graft_entry__ as ge
    ge.load_package()
    from polarai_framework_b200.program import mlp_program
    from oracle.program_executor import OracleExecutor
    impl = cpu_impl()
    rng = np.random.default_rng(0)
    X, Y = mlp_inputs(rng, sample_batch)
    W1, W2 = mlp_weights(rng)
    ex = OracleExecutor(mlp_program(sample_batch, N_IN, N_HIDDEN, N_OUT, LR), impl)
    ex.set_inputs(X=X, Y=Y, W1=W1, W2=W2)
    for _ in range(warmup):
        ex.run()
    t0 = time.perf_counter()
    for _ in range(steps):
        ex.run()
    dt = (time.perf_counter() - t0) / steps
    return {"value": sample_batch / dt, "unit": "samples/s", "cores": impl.threads, "kind": impl.kind,
            "sample": f"{steps} step(s) of the same MLP builtin program on {sample_batch} of the "
                      f"{GLOBAL_BATCH} rows, {dt:.2f} s per step"}, dt


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = CPU_SAMPLE_ROWS
    base, dt = cpu_mlp_baseline(sample, steps=max(1, args.steps), warmup=min(args.warmup, 1))
    line = {"impl": "reference", "metric": "mlp_fwd_bwd_samples_per_s", "value": base["value"],
            "unit": "samples/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": "mlp_784_4096_10_fwd_bwd_sgd", "global_batch": GLOBAL_BATCH,
                       "sample_batch_per_step": sample, "parallelism": "host threads"},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "samples/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def time_region(torch, fn, steps, dist, world):
    """barrier + sync, `steps` calls of fn, sync + barrier; device time by CUDA
    events on the launching stream; max over ranks."""
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        fn()
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e)
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    return ms


def per_op_times(torch, ex, reps):
    """Replays the program with an event pair around every launch."""
    prog = ex.program
    acc = [0.0] * len(prog.ops)
    s = torch.cuda.current_stream().cuda_stream
    for _ in range(reps):
        evs = []
        for i, (kernel, arr, n) in enumerate(ex._compiled):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            if kernel is None:
                if ex.allreduce is not None:
                    ex.allreduce(ex.t[arr])
            elif kernel == "peers":
                ex.peers.launch(arr[0], arr[1], arr[2], s)
            elif kernel == "peers_part":     # timed in order here; in the step the first part overlaps a matmul
                seg, first, count, channel, _, sw, sg = arr
                ex.peers.launch_range(channel, first, count, seg, sw, sg, s)
            else:
                ex.lib.check(ex._fn(kernel, arr, n, ex._ws_ptr, ex._ws_bytes, s))
            b.record()
            evs.append((a, b))
        torch.cuda.synchronize()
        for i, (a, b) in enumerate(evs):
            acc[i] += a.elapsed_time(b)
    return [x / reps for x in acc]


def measure_tf32_peak(torch, dev, seconds=1.5):
    """Dense TF32 rate of the library GEMM on this GPU, measured the way the driver measured
    bf16: torch.matmul at 8192^3 with TF32 allowed, best of 10 (burst) and back to back for
    `seconds` (sustained, under the power cap).  TFLOP/s."""
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        n = 8192
        a = torch.empty((n, n), device=dev).uniform_(-1, 1)
        b = torch.empty((n, n), device=dev).uniform_(-1, 1)
        c = torch.empty((n, n), device=dev)
        flop = 2.0 * n ** 3
        for _ in range(3):
            torch.matmul(a, b, out=c)
        best = 1e9
        for _ in range(10):
            best = min(best, event_time(torch, lambda: torch.matmul(a, b, out=c), 1, warmup=0))
        per = max(best, 0.05)
        reps = max(10, int(seconds * 1e3 / per))
        sustained = event_time(torch, lambda: torch.matmul(a, b, out=c), reps, warmup=0)
        del a, b, c
        return {"burst": flop / best / 1e9, "sustained": flop / sustained / 1e9,
                "how": f"torch.matmul fp32 inputs with allow_tf32, {n}^3: best of 10, and {reps} back to back"}
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


def cross_n_parity(torch, dist, dp, X, Y, W1, W2, rank, world, dev):
    """One step at N ranks against the same step on ONE GPU (rank 0 runs the full batch alone):
    max |difference| of dW1, dW2 and of the updated W1, W2, relative to sum_k |a||b| of the
    contraction over the batch (the metric of the matmul tests); bit-identity of the replicas;
    mean loss of that step.  Every rank takes part; rank 0 returns the record."""
    from polarai_framework_b200.program import DeviceExecutor, fuse_program, mlp_program
    dp.set_replicated(W1=W1, W2=W2)
    dp.ex.run()                                            # eager: one step with the exchange
    torch.cuda.synchronize()
    identical = dp.replicas_identical("W1", "W2", "dW1", "dW2")
    loss_sum = dp.t["L"].double().sum().reshape(1)
    if world > 1:
        dist.all_reduce(loss_sum)
    rec = None
    if rank == 0:
        one = DeviceExecutor(fuse_program(mlp_program(GLOBAL_BATCH, N_IN, N_HIDDEN, N_OUT, LR)), dev)
        one.set_inputs(X=X, Y=Y, W1=W1, W2=W2)
        one.run()
        torch.cuda.synchronize()
        old = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        mag1 = torch.matmul(one.t["X"].abs().t(), one.t["dZ1"].abs())      # sum over the batch of |x||dz1|
        mag2 = torch.matmul(one.t["H"].abs().t(), one.t["dZ2"].abs())
        torch.backends.cuda.matmul.allow_tf32 = old
        tiny = 1e-30
        err = {}
        for g, w, mag in (("dW1", "W1", mag1), ("dW2", "W2", mag2)):
            err[g] = float(((dp.t[g] - one.t[g]).abs() / (mag + tiny)).max())
            # W = fl(W0 + fl(-lr dW)): the difference is lr x the gradient's, plus one rounding of W
            err[w] = float(((dp.t[w] - one.t[w]).abs() / (LR * mag + one.t[w].abs() * 2.0 ** -22 + tiny)).max())
        loss_one = float(one.t["L"].double().sum()) / (GLOBAL_BATCH * N_OUT)
        loss_n = float(loss_sum.item()) / (GLOBAL_BATCH * N_OUT)
        rec = {"vs": "the same step on one GPU (full batch), same seeded data", "metric": "max |delta| / sum_k |a||b|",
               **err, "tolerance": 1e-4, "replicas_identical": bool(identical),
               "first_step_mean_loss": loss_n, "first_step_mean_loss_one_gpu": loss_one,
               "loss_rel_diff": abs(loss_n - loss_one) / abs(loss_one)}
        rec["ok"] = bool(identical and max(err.values()) <= 1e-4 and rec["loss_rel_diff"] <= 1e-4)
        del one, mag1, mag2
        torch.cuda.empty_cache()
    if world > 1:
        dist.barrier()
    return rec


def plugin_e2e(torch, dist, program, Xs, Ys, W1, W2, rank, world, local, steps, in_place):
    """The step driven end to end through the device-runtime plugin (libpolar_rt_cuda.so) the way
    the reference's executor drives a runtime: every step, this rank's X and Y shard is written
    from pageable host arrays into the records (ath_load's role: host copy into pinned memory,
    upload on the device's upload stream into a fresh block while the previous step still
    computes), one Device::launch per builtin by native name (the exchange through
    polar_b200_rt_allreduce_fadd), `fsum` of the loss tensor into one of two scalar records, and
    the 4-byte loss of the PREVIOUS step read back (the read waits for that scalar's writer
    only).  in_place: the batch is produced in the records' pinned buffers (a loader writing
    where AbstractLoaderInternal::load is told to), so the step's host-to-device copy reads
    pinned memory directly, as in the direct loop; otherwise polar_b200_rt_write copies it there
    from pageable arrays first (MemcpyLoader's way).  Wall clock between device barriers,
    maximum over ranks."""
    import numpy as np
    from polarai_framework_b200.peer_gradients import PeerGradients
    from polarai_framework_b200.runtime import Runtime, RuntimeProgramExecutor
    dev = f"cuda:{local}"
    peers = None
    if program.exchanged():
        peers = PeerGradients({g: program.tensors[g] for g in program.exchanged()}, rank, world, dev)
    rt = Runtime()
    ex = RuntimeProgramExecutor(program, rt, device=local, peers=peers)
    ex.set_inputs(W1=W1, W2=W2)
    scal = [rt.tensor((1,), local), rt.tensor((1,), local)]
    sums = [rt.command("fsum", [ex.t["L"], s]) for s in scal]
    got = np.zeros(1, np.float32)
    losses = []
    count = [0]

    tx, ty = ex.t["X"], ex.t["Y"]
    filled = {}

    def produce_in_place(t, data):
        # A loader that produces its data in the record's own pinned buffer.  The synthetic batch
        # never changes, so each of the record's two alternating buffers is filled once; every
        # step still publishes a new version, which uploads the buffer from pinned memory.
        buf = rt.host_buffer(t)
        key = (t.virt_addr, buf.ctypes.data)
        if key not in filled:
            np.copyto(buf, data)
            filled[key] = True
        rt.publish(t)

    def step():
        i = count[0]
        count[0] += 1
        if in_place:
            produce_in_place(tx, Xs), produce_in_place(ty, Ys)
        else:
            ex.set_inputs(X=Xs, Y=Ys)
        ex.run()
        rt.launch_command(sums[i % 2][0], local)
        if i > 0:
            rt.read(scal[(i - 1) % 2], got)
            losses.append(float(got[0]))

    def region(k):
        rt.barrier(local)
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(k):
            step()
        rt.barrier(local)
        dt = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([dt], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        return dt

    region(3)                                              # warm-up: pools, pinned buffers, both scalars
    dt = region(steps) / steps
    rt.read(scal[(count[0] - 1) % 2], got)
    losses.append(float(got[0]))
    rows = Xs.shape[0]
    status = int(rt.cdll.polar_b200_rt_barrier(rt.h, local))
    if world > 1:
        dist.barrier()
    ex.close()
    for s in scal:
        rt.free(s)
    rt.close()
    if peers is not None:
        peers.close()
    return {"value": GLOBAL_BATCH / dt, "unit": "samples/s", "ms_per_step": dt * 1e3, "steps": steps,
            "h2d_bytes_per_step": int(Xs.nbytes + Ys.nbytes) * world, "d2h_bytes_per_step": 4 * world,
            "losses_read": len(losses), "last_mean_loss": losses[-1] / (rows * N_OUT), "rt_status": status,
            "timing": "host wall clock between device barriers, max over ranks",
            "path": ("X,Y shard produced in the records' pinned host buffers (polar_b200_rt_host_begin/end_write) -> "
                     "upload started on the upload stream into a fresh block" if in_place else
                     "numpy X,Y shard -> polar_b200_rt_write (host copy into the record's pinned buffer, upload "
                     "started on the upload stream into a fresh block)") + " -> Device::launch per builtin"
                    + (" + polar_b200_rt_allreduce_fadd" if peers is not None else "")
                    + " -> fsum -> 4-byte loss read back one step later"}


def run_mlp(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    import __graft_entry__ as ge
    pkg = ge.load_package()
    from polarai_framework_b200.data_parallel import DataParallelExecutor, init_from_env
    from polarai_framework_b200.program import DeviceExecutor, mlp_program

    rank, world, local = init_from_env()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    # The same seeded global batch at every N: X, labels, W1, W2 drawn in that order from
    # default_rng(0); rank r keeps rows [r B/N, (r+1) B/N).
    rng = np.random.default_rng(0)
    X, Y = mlp_inputs(rng, GLOBAL_BATCH)
    W1, W2 = mlp_weights(rng)
    fused = args.builtins == "extended"
    dp = DataParallelExecutor(lambda rows: mlp_program(rows, N_IN, N_HIDDEN, N_OUT, LR), GLOBAL_BATCH, ("X", "Y"),
                              rank, world, dev, builtins=args.builtins, collective=args.collective,
                              overlap=args.overlap_exchange)
    ex, program, chain, peers, per = dp.ex, dp.program, dp.chain, dp.peers, dp.rows
    Xs, Ys = np.ascontiguousarray(X[dp.lo:dp.hi]), np.ascontiguousarray(Y[dp.lo:dp.hi])
    x_host = torch.from_numpy(Xs).pin_memory()
    y_host = torch.from_numpy(Ys).pin_memory()
    w1, w2 = torch.from_numpy(W1).to(dev), torch.from_numpy(W2).to(dev)
    dp.set_sharded(X=X, Y=Y)
    loss_acc = torch.zeros(1, dtype=torch.float64, device=dev)
    lib = pkg.lib()

    def reset_weights():
        ex.t["W1"].copy_(w1), ex.t["W2"].copy_(w2)

    # ---- one step at N ranks against one GPU, before anything is timed ----
    parity = None
    if world > 1 and not args.no_parity:
        parity = cross_n_parity(torch, dist, dp, torch.from_numpy(X), torch.from_numpy(Y), W1, W2, rank, world, dev)
    del X, Y

    reset_weights()
    for _ in range(max(3, args.warmup)):                    # warm-up, eager (also primes NCCL)
        dp.step()
    torch.cuda.synchronize()
    if not args.no_graph and not dp.capture():
        if rank == 0:
            print(f"[bench] CUDA graph capture failed ({dp.capture_error}); running eagerly", file=sys.stderr)
    graph = dp.graph
    if graph is not None:
        for _ in range(2):
            dp.step()
        torch.cuda.synchronize()
    launches_per_step = program.launches()
    timed_step = dp.step

    # ---- device-resident throughput ----
    reset_weights()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    n0 = lib.launch_count()
    ms = time_region(torch, timed_step, args.steps, dist, world)
    launched = lib.launch_count() - n0
    ms_per_step = ms / args.steps
    value = GLOBAL_BATCH / (ms_per_step / 1e3)

    # ---- end to end, direct C ABI: host batch in, mean loss out, every step ----
    # Each step consumes a batch that was copied from pinned host memory into a
    # staging buffer on a copy stream while the previous step computed, moves it
    # into the program's X and Y (device to device), starts the copy of the next
    # batch, runs the program and reads the mean loss back.  One host-to-device
    # copy of a full X,Y shard and one 8-byte device-to-host read per step.
    copy_stream = torch.cuda.Stream()
    stage_x, stage_y = torch.empty_like(ex.t["X"]), torch.empty_like(ex.t["Y"])
    ev_staged, ev_consumed = torch.cuda.Event(), torch.cuda.Event()

    def prefetch():
        with torch.cuda.stream(copy_stream):
            stage_x.copy_(x_host, non_blocking=True)
            stage_y.copy_(y_host, non_blocking=True)
            ev_staged.record(copy_stream)

    # The loss of step i is read on the host while step i+1 is already queued: the read-back
    # goes to one of two pinned slots and the host waits for the PREVIOUS step's slot, so the
    # GPU is never idle while the host issues the next step.  Every step's loss is read; the
    # last one after the region's closing synchronize.
    loss_slots = torch.zeros(2, dtype=torch.float64).pin_memory()
    ev_loss = [torch.cuda.Event(), torch.cuda.Event()]
    losses_read = []
    e2e_count = [0]

    def e2e_step():
        cur = torch.cuda.current_stream()
        i = e2e_count[0]
        e2e_count[0] += 1
        cur.wait_event(ev_staged)
        ex.t["X"].copy_(stage_x, non_blocking=True)
        ex.t["Y"].copy_(stage_y, non_blocking=True)
        ev_consumed.record(cur)
        copy_stream.wait_event(ev_consumed)
        prefetch()
        timed_step()
        loss_acc.zero_()
        ex.lib.call("polar_b200_fsum", ex.t["L"].data_ptr(), loss_acc.data_ptr(), ex.t["L"].numel(),
                    cur.cuda_stream)
        loss_slots[i % 2:i % 2 + 1].copy_(loss_acc, non_blocking=True)
        ev_loss[i % 2].record(cur)
        if i > 0:
            ev_loss[(i - 1) % 2].synchronize()
            losses_read.append(float(loss_slots[(i - 1) % 2]))

    reset_weights()
    prefetch()
    e2e_step()
    e2e_ms = time_region(torch, e2e_step, args.steps, dist, world) / args.steps
    losses_read.append(float(loss_slots[(e2e_count[0] - 1) % 2]))
    # the same host-to-device copy with the GPU otherwise idle: the floor PCIe sets for a step
    h2d_ms = event_time(torch, lambda: (stage_x.copy_(x_host, non_blocking=True),
                                        stage_y.copy_(y_host, non_blocking=True)), 3, warmup=1)
    copy_stream.synchronize()
    e2e_direct = {"value": GLOBAL_BATCH / (e2e_ms / 1e3), "unit": "samples/s",
                  "h2d_bytes_per_step": int(x_host.numel() * 4 + y_host.numel() * 4) * world,
                  "d2h_bytes_per_step": 8 * world, "ms_per_step": e2e_ms,
                  "path": "pinned host X,Y shard -> cudaMemcpyAsync on a copy stream (overlaps the previous step) -> "
                          "device-to-device into the program's inputs -> builtin program by direct C-ABI calls "
                          "(CUDA graph) -> fsum -> 8-byte loss readback (the host reads step i's loss after "
                          "queuing step i+1)",
                  "losses_read": len(losses_read), "h2d_copy_alone_ms": h2d_ms,
                  "h2d_copy_alone_gbs": (x_host.numel() + y_host.numel()) * 4 / (h2d_ms / 1e3) / 1e9}
    del stage_x, stage_y

    # ---- end to end through the reference-facing plugin (Device::launch with host buffers) ----
    e2e = None
    if not args.no_plugin:
        try:
            e2e = plugin_e2e(torch, dist, program, Xs, Ys, W1, W2, rank, world, local, args.steps, True)
            e2e_memcpy = plugin_e2e(torch, dist, program, Xs, Ys, W1, W2, rank, world, local, args.steps, False)
        except Exception as exc:                            # noqa: BLE001 - reported in the line, never hidden
            e2e = None
            plugin_error = f"{type(exc).__name__}: {exc}"
            if world > 1:
                raise
        torch.cuda.set_device(local)
    # Clocks are sampled over the timed regions.  At 8 GPUs one region lasts about 25 ms,
    # shorter than nvidia-smi's period, so every rank runs the same number of further steps
    # (the count derives from the max-reduced step time, identical on all ranks) until about
    # 1 s is covered.
    covered_ms = (ms_per_step + e2e_ms) * args.steps + (e2e["ms_per_step"] * args.steps if e2e else 0.0)
    if covered_ms < 1000.0:
        for _ in range(int((1000.0 - covered_ms) / ms_per_step) + 1):
            timed_step()
        torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None

    # ---- first-step loss, for the record ----
    reset_weights()
    dp.ex.run()
    loss_acc.zero_()
    ex.lib.call("polar_b200_fsum", ex.t["L"].data_ptr(), loss_acc.data_ptr(), ex.t["L"].numel(),
                torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.all_reduce(loss_acc)
    first_loss = float(loss_acc.item()) / (GLOBAL_BATCH * N_OUT)

    # ---- roofline of the dominant kernel, measured live with events per launch ----
    reset_weights()
    times = per_op_times(torch, ex, reps=min(5, args.steps))
    total_ops_ms = sum(times)
    by_kernel = {}
    seen_part = 0
    for (kernel, a), t in zip(program.ops, times):
        key = kernel if not kernel.startswith("fmatmul") else f"{kernel}:{a[-1]}"
        if kernel == "ALLREDUCE_FADD_PART":
            seen_part += 1
            key = f"ALLREDUCE_FADD_PART:{seen_part}" + (" (overlapped in the step)" if a[3] else "")
        d = by_kernel.setdefault(key, {"launches": 0, "ms": 0.0})
        d["launches"] += 1
        d["ms"] += t
    peaks = load_peaks()
    tf32 = measure_tf32_peak(torch, dev) if (rank == 0 and world == 1 and not args.no_extras) else None
    if tf32 is not None:
        tf32_peak, peak_source = tf32["sustained"], ("dense TF32 measured in this run: " + tf32["how"] +
                                                     " (the sustained figure: the kernel is timed inside a long step)")
    else:
        tf32_peak = peaks["bf16_tflops_sustained"] / 2.0
        peak_source = f"MEASURED_PEAKS.json bf16_tflops_sustained / 2 ({peaks['source']})"
    tc_ops = [(i, k, a) for i, (k, a) in enumerate(program.ops)
              if k.startswith("fmatmul") and lib.cdll.polar_b200_fmatmul_path(
                  int(k[8] == "t"), int(k[10] == "t"), *mm_dims(program, k, a)) == 0]
    tc_ms = sum(times[i] for i, _, _ in tc_ops)
    tc_flops = sum(2.0 * np.prod(mm_dims(program, k, a)) for _, k, a in tc_ops)
    achieved = tc_flops / (tc_ms / 1e3) / 1e12 if tc_ms > 0 else 0.0
    sm_mhz = (clocks or {}).get("sm_mhz") or 0.0
    hw_rate = 4096.0 * sm_count_of(torch, local) * sm_mhz * 1e6 / 1e12 if sm_mhz else None   # TF32 flop/s at that clock
    roofline = {"kernel": "fmatmul_tc_kernel (tcgen05, 3xTF32)", "bound": "tensor",
                "achieved": achieved, "peak": tf32_peak, "unit": "TFLOP/s", "frac": achieved / tf32_peak,
                "frac_bound": "an fp32-accurate product issues three TF32 MMAs: algorithmic = issued / 3.  The "
                              "denominator is a library GEMM (cuBLAS TF32 through torch), not the hardware limit, so "
                              "issued_frac can read above 1.0 - this kernel then issues TF32 MMAs faster than that "
                              "GEMM runs; tensor_pipe_util is the fraction of the hardware rate",
                "issued_tflops": 3.0 * achieved, "issued_frac": 3.0 * achieved / tf32_peak,
                "tensor_pipe_util": (3.0 * achieved / hw_rate) if hw_rate else None,
                "tensor_pipe_util_note": "issued TF32 flops / (4096 flop/clk/SM x SMs x the median SM clock sampled "
                                         "during this run): comparable with ncu's sm__pipe_tensor_cycles_active",
                "peak_source": peak_source,
                "tf32_peak_measured": tf32,
                "launches_per_step": len(tc_ops), "avg_launch_ms": tc_ms / max(1, len(tc_ops)),
                "share_of_step": tc_ms / total_ops_ms if total_ops_ms else None,
                **tc_traffic(program, tc_ops, per)}

    line = {"metric": "mlp_fwd_bwd_samples_per_s", "value": value, "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": "mlp_784_4096_10_fwd_bwd_sgd", "global_batch": GLOBAL_BATCH,
                       "per_gpu_batch": per, "lr": LR, "parallelism": f"dp{world}",
                       "cuda_graph": graph is not None,
                       "builtins": "extended (fused launches, every output bit-identical to the builtin chain)"
                       if fused else "the reference's builtin chain, one launch per builtin",
                       "collective": dp.collective,
                       "data_seed": "numpy default_rng(0): X, labels, W1, W2 in that order; the same global batch "
                                    "at every N, sharded by rows",
                       "l2": "per-step working set (X 205 MB/GPU-share, seven Bx4096 activations) "
                             "exceeds the 126 MB L2 at every N"},
            "flop_per_sample": FLOP_PER_SAMPLE, "tflops": value * FLOP_PER_SAMPLE / 1e12,
            "first_step_mean_loss": first_loss,
            "gpu_launches": int(launched) if graph is None else launches_per_step * args.steps,
            "launches_per_step": launches_per_step,
            "clocks": clocks, "e2e": e2e if e2e is not None else e2e_direct, "e2e_direct": e2e_direct,
            "roofline": roofline,
            "breakdown_ms": {k: round(v["ms"], 4) for k, v in sorted(by_kernel.items(), key=lambda kv: -kv[1]["ms"])}}
    if e2e is None and not args.no_plugin:
        line["e2e_plugin_error"] = plugin_error
    elif e2e is not None:
        line["e2e_memcpy_loader"] = e2e_memcpy
    if parity is not None:
        line["parity"] = parity
    if peers is not None:
        line["exchange_phases_us"] = {k: round(v, 1) for k, v in peers.phase_times_us().items()}
        if any(k == "ALLREDUCE_FADD_PART" for k, _ in program.ops):
            line["exchange_phases_us_overlapped_part"] = {k: round(v, 1) for k, v in peers.phase_times_us(1).items()}
    line["device_status"] = dp.device_status()             # 0: no bounded device-side wait gave up
    if fused and not args.no_extras:
        # The same step as the reference's own builtin chain, one launch per builtin (20 launches
        # instead of 8-9) with NCCL all-reduces: same outputs bit for bit at one rank.  Every
        # rank runs it (its all-reduces are collective).
        cdp = DataParallelExecutor(lambda rows: mlp_program(rows, N_IN, N_HIDDEN, N_OUT, LR), GLOBAL_BATCH,
                                   ("X", "Y"), rank, world, dev, builtins="reference", collective="nccl")
        cex = cdp.ex
        cex.t["X"].copy_(ex.t["X"]), cex.t["Y"].copy_(ex.t["Y"])
        cex.t["W1"].copy_(w1), cex.t["W2"].copy_(w2)
        for _ in range(3):
            cex.run()
        cms = time_region(torch, cex.run, args.steps, dist, world) / args.steps
        line["builtin_chain"] = {"value": GLOBAL_BATCH / (cms / 1e3), "unit": "samples/s", "ms_per_step": cms,
                                 "launches_per_step": chain.launches(), "cuda_graph": False,
                                 "note": "the unfused program: one launch per reference builtin, NCCL "
                                         "all-reduce of dW2 and dW1, fadd updates"}
        cdp.close()
        del cex, cdp
    if rank == 0 and world == 1 and not args.no_extras:
        line["cpu_baseline"] = cpu_mlp_baseline(CPU_SAMPLE_ROWS, steps=5, warmup=1)[0]
        torch.cuda.empty_cache()
        # the bandwidth numbers first: the GEMM loop leaves the GPU at its power cap
        line["extras"] = {"elementwise_sweep": elementwise_sweep(torch, lib, dev, peaks),
                          "gemm_sweep": gemm_sweep(torch, lib, dev, tf32),
                          "latency_bound_programs": small_program_latencies(torch, dev)}
    ok = parity is None or parity["ok"]
    if rank == 0:
        print(json.dumps(line), flush=True)
        if not ok:
            print("[bench] cross-N parity FAILED: see `parity` in the line", file=sys.stderr)
    shutdown(torch, dist, world, dp, 0 if ok else 1)


def sm_count_of(torch, index):
    return torch.cuda.get_device_properties(index).multi_processor_count


def tc_traffic(program, tc_ops, rows):
    """DRAM bytes per launch of the tensor-core matmuls from the ncu capture summarised in
    profiles/fmatmul_tc_256row_tiles_mlp_batch16384_full.md (dram__bytes_read.sum +
    dram__bytes_write.sum of the step's two launches at batch 16384: 280.8 MB and 425.6 MB),
    scaled by rows - X, H and dZ1 grow with the batch, the 12.8 MB weight-shaped operands do
    not - next to the algorithmic bytes 4(mk + kn + mn)."""
    alg = [4.0 * (m * k + k * n + m * n) for m, n, k in (mm_dims(program, k_, a) for _, k_, a in tc_ops)]
    measured_at_16384 = (280.8e6 + 425.6e6) / 2.0
    return {"traffic": rows * measured_at_16384 / 16384.0,
            "algorithmic_bytes": sum(alg) / max(1, len(alg)),
            "traffic_note": "average of the step's two tensor-core launches; ncu capture of the same kernel "
                            "configuration at batch 16384, scaled by rows"}


def shutdown(torch, dist, world, dp, code=0):
    """One rank: an ordinary exit, so that interpreter-exit hooks run.  Several ranks: tearing
    down an NCCL communicator while a captured CUDA graph still references its kernels was seen
    to block for minutes after the result had been printed, so: drop the graph and the peer
    mappings, drain the device, meet the other ranks once, give destroy_process_group a few
    seconds on a helper thread, then leave without running further teardown."""
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    dp.close()
    torch.cuda.synchronize()
    if world == 1:
        if code:
            raise SystemExit(code)
        return
    dist.barrier()
    torch.cuda.synchronize()
    t = threading.Thread(target=dist.destroy_process_group, daemon=True)
    t.start()
    t.join(timeout=10.0)
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(code)


def mm_dims(program, kernel, args):
    tl, tr = kernel[8] == "t", kernel[10] == "t"
    ls, rs = program.tensors[args[0]], program.tensors[args[1]]
    m = ls[1] if tl else ls[0]
    k = ls[0] if tl else ls[1]
    n = rs[0] if tr else rs[1]
    if kernel == "fmatmul_t_f_rows":
        m = int(args[3])                                    # a block of rows of the product
    return int(m), int(n), int(k)


def event_time(torch, fn, reps, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(reps):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / reps


def gemm_shape_numbers(torch, lib, dev, m, n, k, reps):
    """TFLOP/s (algorithmic, 2mnk) of the four transpose forms of one shape on `dev`."""
    st = torch.cuda.current_stream(dev).cuda_stream
    out = {}
    for tl in (0, 1):
        for tr in (0, 1):
            a = torch.empty((k, m) if tl else (m, k), device=dev).uniform_(-1, 1)
            b = torch.empty((n, k) if tr else (k, n), device=dev).uniform_(-1, 1)
            c = torch.empty((m, n), device=dev)
            need = int(lib.cdll.polar_b200_fmatmul_workspace_bytes(tl, tr, m, n, k))
            ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
            ms = event_time(torch, lambda: lib.call("polar_b200_fmatmul", tl, tr, m, n, k, a.data_ptr(), b.data_ptr(),
                                                    c.data_ptr(), ws.data_ptr() if need else None, need, st), reps)
            out[f"fmatmul_{'t' if tl else 'f'}_{'t' if tr else 'f'}"] = {"ms": ms, "tflops": 2.0 * m * n * k / ms / 1e9}
            del a, b, c, ws
    return out


def gemm_numbers(torch, lib, n, reps, dev="cuda:0"):
    return gemm_shape_numbers(torch, lib, dev, n, n, n, reps)


def gemm_sweep(torch, lib, dev, tf32):
    """The matmul part of the metric: square 1024..8192 and the skinny 65536 x 784 x 1024 case
    (batch x in x out: m = 65536, k = 784, n = 1024), all four transpose forms.  `frac` is
    algorithmic TFLOP/s over the dense TF32 rate measured in this run (burst: these kernels
    are timed alone); three TF32 products per fp32 product bound it at 1/3."""
    peak = tf32["burst"] if tf32 else load_peaks()["bf16_tflops"] / 2.0
    out = {"peak_tflops": peak, "peak_source": "torch.matmul TF32 8192^3 burst, this run" if tf32 else
           "MEASURED_PEAKS.json bf16_tflops / 2", "frac_bound": 1.0 / 3.0, "shapes": {}}
    for (m, n, k) in ((1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192),
                      (65536, 1024, 784)):
        res = gemm_shape_numbers(torch, lib, dev, m, n, k, reps=5 if m * n * k < 2 ** 37 else 3)
        for v in res.values():
            v["frac"] = v["tflops"] / peak
        out["shapes"][f"{m}x{n}x{k}"] = res
    torch.cuda.empty_cache()
    return out


EW_BYTES = {"ffill": 4, "fcopy": 8, "fsigmoid": 8, "fmulconcat": 8, "fadd": 12, "fmul": 12, "fdivide": 12,
            "flogloss": 12}


def elementwise_numbers(torch, lib, n, peaks, reps, dev="cuda:0", rotate_bytes=512 << 20):
    """GB/s (algorithmic bytes per element x n / time) of the eight elementwise builtins at n
    elements.  Below L2 size the operands would stay cached from launch to launch, so each
    stream lives in a pool of at least `rotate_bytes` and every launch takes the next slice."""
    st = torch.cuda.current_stream(dev).cuda_stream
    slices = max(1, min(64, rotate_bytes // (4 * n)))
    total = n * slices
    a = torch.empty(total, device=dev).uniform_(-1, 1)
    b = torch.empty(total, device=dev).uniform_(0.5, 2)
    p = torch.empty(total, device=dev).uniform_(0.01, 0.99)
    y = (torch.rand(total, device=dev) < 0.5).float()
    o = torch.empty(total, device=dev)
    A, B, P, Y, O = (t.data_ptr() for t in (a, b, p, y, o))
    turn = [0]

    def off():
        turn[0] = (turn[0] + 1) % slices
        return 4 * n * turn[0]

    def op(name):
        d = off()
        if name == "ffill":
            lib.call("polar_b200_ffill", 1.234, O + d, n, st)
        elif name == "fcopy":
            lib.call("polar_b200_fcopy", A + d, O + d, n, st)
        elif name == "fsigmoid":
            lib.call("polar_b200_fsigmoid", A + d, O + d, n, st)
        elif name == "fmulconcat":
            lib.call("polar_b200_fmulconcat", B, A + d, O + d, n, st)
        elif name == "fadd":
            lib.call("polar_b200_fadd", A + d, 1.0, B + d, 1.0, O + d, n, st)
        elif name == "fmul":
            lib.call("polar_b200_fmul", A + d, B + d, O + d, n, st)
        elif name == "fdivide":
            lib.call("polar_b200_fdivide", A + d, B + d, O + d, n, st)
        else:
            lib.call("polar_b200_flogloss", P + d, Y + d, O + d, n, st)

    out = {}
    for name, bpe in EW_BYTES.items():
        ms = event_time(torch, lambda: op(name), reps)
        gbs = bpe * n / ms / 1e6
        out[name] = {"ms": ms, "gbs": gbs, "frac_of_measured_copy": gbs / peaks["hbm_gbs"], "frac_of_8tbs": gbs / 8000.0}
    del a, b, p, y, o
    return out


def elementwise_sweep(torch, lib, dev, peaks):
    """The bandwidth part of the metric: 2^16 .. 2^30 elements in powers of 4, eight builtins.
    Sizes below 2^26 are launch- or L2-bound and are reported for the curve, not as roofline
    points."""
    out = {"peak_gbs": peaks["hbm_gbs"], "peak_source": f"MEASURED_PEAKS.json hbm_gbs ({peaks['source']})",
           "buffers": "each stream is a pool of >= 512 MB; consecutive launches take consecutive slices", "sizes": {}}
    for log2n in range(16, 31, 2):
        n = 1 << log2n
        out["sizes"][f"2^{log2n}"] = elementwise_numbers(torch, lib, n, peaks, reps=20 if log2n < 30 else 5, dev=dev)
        torch.cuda.empty_cache()
    return out


def small_program_latencies(torch, dev="cuda:0", reps=200):
    """The two latency-bound configurations: microseconds per evaluation of the four-builtin
    elementwise chain on 2^20 elements and of the logistic-regression step on 256 x 784, launched
    builtin by builtin and replayed as a CUDA graph; inputs resident (both fit in L2)."""
    import numpy as np
    from polarai_framework_b200.program import DeviceExecutor, elementwise_chain_program, fuse_program, logreg_program
    rng = np.random.default_rng(0)
    n = 1 << 20
    chain_in = {k: rng.uniform(-1, 1, n).astype(np.float32) for k in "abc"}
    chain_in["d"] = rng.uniform(0.5, 2, n).astype(np.float32)
    lr_in = {"X": rng.standard_normal((256, 784)).astype(np.float32),
             "W": (0.01 * rng.standard_normal((784, 1))).astype(np.float32),
             "Y": (rng.random((256, 1)) < 0.5).astype(np.float32)}
    out = {}
    for name, prog, inputs in (("elementwise_chain_2pow20", elementwise_chain_program(n), chain_in),
                               ("logreg_step_256x784", logreg_program(256, 784, 0.1), lr_in),
                               ("logreg_step_256x784_extended", fuse_program(logreg_program(256, 784, 0.1)), lr_in)):
        ex = DeviceExecutor(prog, dev)
        ex.set_inputs(**inputs)
        eager_us = event_time(torch, ex.run, reps, warmup=10) * 1e3
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            ex.run()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                ex.run()
        torch.cuda.synchronize()
        graph_us = event_time(torch, g.replay, reps, warmup=10) * 1e3
        out[name] = {"launches": prog.launches(), "us_per_eval": eager_us, "us_per_eval_cuda_graph": graph_us}
        del g, ex
    return out


def run_single_kernel_workload(args):
    """--workload gemm | elementwise: single-GPU lines for the other two parts of the metric."""
    import torch
    import __graft_entry__ as ge
    pkg = ge.load_package()
    lib = pkg.lib()
    peaks = load_peaks()
    torch.cuda.set_device(0)
    sampler = ClockSampler(0)
    sampler.start()
    n0 = lib.launch_count()
    if args.workload == "gemm":
        n = args.size or 8192
        res = gemm_numbers(torch, lib, n, reps=max(1, args.steps))
        ms = res["fmatmul_f_f"]["ms"]
        tf = res["fmatmul_f_f"]["tflops"]
        if args.no_extras:    # profiling runs: no library GEMM loop around the kernel of interest
            tf32 = {"burst": peaks["bf16_tflops"] / 2.0, "sustained": peaks["bf16_tflops_sustained"] / 2.0,
                    "how": f"not measured (--no-extras): MEASURED_PEAKS.json bf16 / 2 ({peaks['source']})"}
        else:
            tf32 = measure_tf32_peak(torch, "cuda:0")
        peak = tf32["burst"]
        line = {"metric": "fp32_matmul_tflops", "value": tf, "unit": "TFLOP/s", "ms_per_step": ms, "dtype": "f32",
                "config": {"workload": f"fmatmul_f_f_{n}x{n}x{n}",
                           "l2": f"operands and result {12 * n * n / 1e6:.0f} MB vs 126 MB L2"},
                "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak,
                             "issued_tflops": 3 * tf, "traffic": None, "tf32_peak_measured": tf32,
                             "frac_bound": "1/3: three TF32 products per fp32 product",
                             "peak_source": "dense TF32 measured in this run (burst): " + tf32["how"]},
                "variants": res}
    else:
        n = 1 << (args.size or 28)
        res = elementwise_numbers(torch, lib, n, peaks, reps=max(3, args.steps))
        gbs = res["fadd"]["gbs"]
        line = {"metric": "elementwise_hbm_gbs", "value": gbs, "unit": "GB/s", "ms_per_step": res["fadd"]["ms"],
                "dtype": "f32",
                "config": {"workload": f"fadd_{n}_elements", "l2": f"three {4 * n / 2**20:.0f} MiB streams vs 126 MB L2"},
                "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": gbs / peaks["hbm_gbs"], "traffic": None,
                             "peak_source": f"MEASURED_PEAKS.json hbm_gbs ({peaks['source']})"},
                "builtins": res}
    line.update({"n_gpus": 1, "steps": args.steps, "warmup": 3, "higher_is_better": True, "scaling": "weak",
                 "vs_baseline": None, "data": "synthetic", "gpu_launches": int(lib.launch_count() - n0),
                 "clocks": sampler.stop()})
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="mlp", choices=["mlp", "gemm", "elementwise"])
    ap.add_argument("--size", type=int, default=0,
                    help="gemm: m=n=k (default 8192); elementwise: log2 of the element count (default 28)")
    ap.add_argument("--batch", type=int, default=0,
                    help="mlp: global batch override for profiling small cases (default 65536, the metric's)")
    ap.add_argument("--builtins", default="extended", choices=["extended", "reference"],
                    help="mlp: 'extended' runs the fused launches (every output bit-identical to the chain), "
                         "'reference' one launch per reference builtin")
    ap.add_argument("--collective", default="peer", choices=["peer", "peer-ipc", "peer-multicast", "nccl"],
                    help="mlp at N>1 with extended builtins: gradient sum + update as one peer-memory kernel, "
                         "or NCCL all-reduces followed by fadd")
    ap.add_argument("--overlap-exchange", action="store_true",
                    help="mlp at N>1: compute the last weight gradient in two blocks of rows and exchange the first "
                         "block on a second stream meanwhile (measured slower at these shapes; off by default)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--no-parity", action="store_true",
                    help="mlp at N>1: skip the one-step comparison with the full batch on one GPU")
    ap.add_argument("--no-plugin", action="store_true",
                    help="mlp: skip the end-to-end loop through the runtime plugin (e2e is then the direct C-ABI loop)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the runtime has no CPU path (use --impl reference "
                         "for the CPU arm)")
    if args.workload == "mlp":
        if args.batch:
            global GLOBAL_BATCH
            GLOBAL_BATCH = args.batch
        run_mlp(args)
    else:
        run_single_kernel_workload(args)


if __name__ == "__main__":
    main()
