#!/usr/bin/env python
"""Benchmark of the PolarAI B200 runtime's hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--workload mlp|gemm|elementwise] [--builtins extended|reference]
                    [--collective peer|nccl] [--batch B] [--no-graph] [--no-extras]

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
in HBM; `e2e` is samples/s when every step also copies its X and Y shard from
pinned host memory and reads the mean loss back.  `roofline` describes the
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
    sample = 512
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
            else:
                ex.lib.check(ex._fn(kernel, arr, n, ex._ws_ptr, ex._ws_bytes, s))
            b.record()
            evs.append((a, b))
        torch.cuda.synchronize()
        for i, (a, b) in enumerate(evs):
            acc[i] += a.elapsed_time(b)
    return [x / reps for x in acc]


def run_mlp(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    import __graft_entry__ as ge
    pkg = ge.load_package()
    from polarai_framework_b200.data_parallel import init_from_env, make_allreduce, shard_rows
    from polarai_framework_b200.peer_gradients import PeerGradients
    from polarai_framework_b200.program import (DeviceExecutor, fuse_gradient_exchange, fuse_program,
                                                mlp_program)

    rank, world, local = init_from_env()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    lo, hi = shard_rows(GLOBAL_BATCH, rank, world)
    per = hi - lo
    rng = np.random.default_rng(0)
    W1, W2 = mlp_weights(rng)                               # identical on every rank
    Xs, Ys = mlp_inputs(np.random.default_rng(1000 + rank), per)   # this rank's rows
    chain = mlp_program(per, N_IN, N_HIDDEN, N_OUT, LR)
    fused = args.builtins == "extended"
    program = fuse_program(chain) if fused else chain
    # Gradient exchange: one kernel per rank over NVLink peer memory (sum over ranks + weight
    # update), or NCCL all-reduces followed by the fadd updates.  Mapping the peers' buffers can
    # fail (no peer access, IPC closed in the container): every rank then takes the NCCL form.
    peers, collective = None, "none (one rank)"
    if world > 1:
        collective = "nccl all-reduce, then fadd updates"
        if fused and args.collective == "peer":
            xprog = fuse_gradient_exchange(program)
            why = ""
            try:
                peers = PeerGradients({g: xprog.tensors[g] for g in xprog.exchanged()}, rank, world, dev)
            except Exception as exc:                        # noqa: BLE001 - any failure means "not available"
                why = f"{type(exc).__name__}: {exc}"
            ok = torch.tensor([0 if peers is None else 1], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 1:
                program = xprog
                collective = "peer memory over NVLink: sum over ranks and weight update in one kernel per rank"
            else:
                peers = None
                collective += f" (peer memory unavailable on some rank{': ' + why if why else ''})"
    ex = DeviceExecutor(program, dev, make_allreduce(world), peers=peers)
    x_host = torch.from_numpy(Xs).pin_memory()
    y_host = torch.from_numpy(Ys).pin_memory()
    w1, w2 = torch.from_numpy(W1).to(dev), torch.from_numpy(W2).to(dev)
    ex.t["X"].copy_(x_host), ex.t["Y"].copy_(y_host)
    loss_acc = torch.zeros(1, dtype=torch.float64, device=dev)
    lib = pkg.lib()

    def reset_weights():
        ex.t["W1"].copy_(w1), ex.t["W2"].copy_(w2)

    def step():
        ex.run()

    use_graph = not args.no_graph
    graph = None
    reset_weights()
    for _ in range(max(3, args.warmup)):                    # warm-up, eager (also primes NCCL)
        step()
    torch.cuda.synchronize()
    if use_graph:
        try:
            cap_stream = torch.cuda.Stream()
            cap_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(cap_stream):
                step()
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=cap_stream):
                    step()
            torch.cuda.synchronize()
            for _ in range(2):
                graph.replay()
            torch.cuda.synchronize()
        except Exception as exc:                            # capture is an optimisation, not a requirement
            if rank == 0:
                print(f"[bench] CUDA graph capture failed ({exc}); running eagerly", file=sys.stderr)
            graph = None
    launches_per_step = program.launches()

    def timed_step():
        if graph is not None:
            graph.replay()
        else:
            step()

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

    # ---- end to end: host batch in, mean loss out, every step ----
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
    # Clocks are sampled over both timed regions (device-resident and end to end).
    # At 8 GPUs one region lasts about 25 ms, shorter than nvidia-smi's period, so
    # every rank runs the same number of further steps (the count derives from the
    # max-reduced step time, identical on all ranks) until about 1 s is covered.
    covered_ms = (ms_per_step + e2e_ms) * args.steps
    if covered_ms < 1000.0:
        for _ in range(int((1000.0 - covered_ms) / ms_per_step) + 1):
            timed_step()
        torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None
    e2e = {"value": GLOBAL_BATCH / (e2e_ms / 1e3), "unit": "samples/s",
           "h2d_bytes_per_step": int(x_host.numel() * 4 + y_host.numel() * 4) * world,
           "d2h_bytes_per_step": 8 * world, "ms_per_step": e2e_ms,
           "path": "pinned host X,Y shard -> cudaMemcpyAsync on a copy stream (overlaps the previous step) -> "
                   "device-to-device into the program's inputs -> builtin program -> fsum -> 8-byte loss readback "
                   "(the host reads step i's loss after queuing step i+1)",
           "losses_read": len(losses_read), "h2d_copy_alone_ms": h2d_ms,
           "h2d_copy_alone_gbs": (x_host.numel() + y_host.numel()) * 4 / (h2d_ms / 1e3) / 1e9}

    # ---- first-step loss, for the record ----
    reset_weights()
    step()
    loss_acc.zero_()
    ex.lib.call("polar_b200_fsum", ex.t["L"].data_ptr(), loss_acc.data_ptr(), ex.t["L"].numel(),
                torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    first_loss = float(loss_acc.item()) / (per * N_OUT)

    # ---- roofline of the dominant kernel, measured live with events per launch ----
    reset_weights()
    times = per_op_times(torch, ex, reps=min(5, args.steps))
    total_ops_ms = sum(times)
    by_kernel = {}
    for (kernel, a), t in zip(program.ops, times):
        key = kernel if not kernel.startswith("fmatmul") else f"{kernel}:{a[-1]}"
        d = by_kernel.setdefault(key, {"launches": 0, "ms": 0.0})
        d["launches"] += 1
        d["ms"] += t
    peaks = load_peaks()
    tf32_peak = peaks["bf16_tflops_sustained"] / 2.0        # dense TF32 = half the dense bf16 rate
    tc_ops = [(i, k, a) for i, (k, a) in enumerate(program.ops)
              if k.startswith("fmatmul") and lib.cdll.polar_b200_fmatmul_path(
                  int(k[8] == "t"), int(k[10] == "t"), *mm_dims(program, k, a)) == 0]
    tc_ms = sum(times[i] for i, _, _ in tc_ops)
    tc_flops = sum(2.0 * np.prod(mm_dims(program, k, a)) for _, k, a in tc_ops)
    achieved = tc_flops / (tc_ms / 1e3) / 1e12 if tc_ms > 0 else 0.0
    roofline = {"kernel": "fmatmul_tc_kernel (tcgen05, 3xTF32)", "bound": "tensor",
                "achieved": achieved, "peak": tf32_peak, "unit": "TFLOP/s", "frac": achieved / tf32_peak,
                "pipe_frac": 3.0 * achieved / tf32_peak,
                "peak_source": f"MEASURED_PEAKS.json bf16_tflops_sustained / 2 ({peaks['source']}); "
                               "fp32-accurate products issue 3 TF32 MMAs each, so frac <= 1/3 and "
                               "pipe_frac = 3 x frac is the tensor-pipe utilisation",
                "launches_per_step": len(tc_ops), "avg_launch_ms": tc_ms / max(1, len(tc_ops)),
                "share_of_step": tc_ms / total_ops_ms if total_ops_ms else None,
                # dram__bytes_read + write per launch from the ncu capture at batch 8192
                # (summarised under profiles/: 118.4 MB and 174.3 MB for the two launches),
                # scaled by rows: traffic grows in proportion with the batch.
                "traffic": per * (118.4e6 + 174.3e6) / 2.0 / 8192.0,
                "traffic_note": "ncu capture at batch 8192 scaled by rows; algorithmic 4(mk+kn+mn) is "
                                f"{4.0 * (per * N_IN + N_IN * N_HIDDEN + per * N_HIDDEN):.3e} bytes per launch"}

    line = {"metric": "mlp_fwd_bwd_samples_per_s", "value": value, "unit": "samples/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": "mlp_784_4096_10_fwd_bwd_sgd", "global_batch": GLOBAL_BATCH,
                       "per_gpu_batch": per, "lr": LR, "parallelism": f"dp{world}",
                       "cuda_graph": graph is not None,
                       "builtins": "extended (fused launches, every output bit-identical to the builtin chain)"
                       if fused else "the reference's builtin chain, one launch per builtin",
                       "collective": collective,
                       "l2": "per-step working set (X 205 MB/GPU-share, seven Bx4096 activations) "
                             "exceeds the 126 MB L2 at every N"},
            "flop_per_sample": FLOP_PER_SAMPLE, "tflops": value * FLOP_PER_SAMPLE / 1e12,
            "first_step_mean_loss": first_loss,
            "gpu_launches": int(launched) if graph is None else launches_per_step * args.steps,
            "launches_per_step": launches_per_step,
            "clocks": clocks, "e2e": e2e, "roofline": roofline,
            "breakdown_ms": {k: round(v["ms"], 4) for k, v in sorted(by_kernel.items(), key=lambda kv: -kv[1]["ms"])}}
    if peers is not None:
        line["exchange_phases_us"] = {k: round(v, 1) for k, v in peers.phase_times_us().items()}
    status = int(lib.cdll.polar_b200_device_status())
    line["device_status"] = status                          # 0: no bounded device-side wait gave up
    if fused and not args.no_extras:
        # The same step as the reference's own builtin chain, one launch per builtin (20 launches
        # instead of 8-9) with NCCL all-reduces: same outputs bit for bit at one rank.  Every
        # rank runs it (its all-reduces are collective).
        cex = DeviceExecutor(chain, dev, make_allreduce(world))
        cex.t["X"].copy_(ex.t["X"]), cex.t["Y"].copy_(ex.t["Y"])
        cex.t["W1"].copy_(w1), cex.t["W2"].copy_(w2)
        for _ in range(3):
            cex.run()
        cms = time_region(torch, cex.run, args.steps, dist, world) / args.steps
        line["builtin_chain"] = {"value": GLOBAL_BATCH / (cms / 1e3), "unit": "samples/s", "ms_per_step": cms,
                                 "launches_per_step": chain.launches(), "cuda_graph": False,
                                 "note": "the unfused program: one launch per reference builtin, NCCL "
                                         "all-reduce of dW2 and dW1, fadd updates"}
        del cex
    if rank == 0 and world == 1 and not args.no_extras:
        line["e2e_plugin"] = plugin_e2e(program, Xs, Ys, W1, W2, per)
        line["cpu_baseline"] = cpu_mlp_baseline(2048, steps=1)[0]
        # the bandwidth numbers first: the GEMM loop leaves the GPU at its power cap
        ew = elementwise_numbers(torch, lib, 1 << 28, peaks, reps=10)
        line["extras"] = {"elementwise_2pow28": ew, "gemm_8192": gemm_numbers(torch, lib, 8192, reps=3),
                          "latency_bound_programs": small_program_latencies(torch)}
    if rank == 0:
        print(json.dumps(line), flush=True)
    shutdown(torch, dist, world, graph)


def plugin_e2e(program, X, Y, W1, W2, rows, steps=5):
    """The same step driven through the device-runtime plugin (libpolar_rt_cuda.so) the way
    the reference's executor drives a runtime: X and Y written from pageable host arrays into
    the records' host copies (ath_load's role), uploaded when the first launch locks them on
    the device, one Device::launch per builtin, the loss tensor read back to the host.  Wall
    clock around whole steps; everything in it is synchronous with the host."""
    import numpy as np
    from polarai_framework_b200.runtime import RuntimeProgramExecutor
    ex = RuntimeProgramExecutor(program)
    ex.set_inputs(W1=W1, W2=W2)
    loss = np.empty(program.tensors["L"], np.float32)

    def step():
        ex.set_inputs(X=X, Y=Y)
        ex.run()
        ex.output("L", loss)
        return float(loss.mean(dtype=np.float64))

    step()
    t0 = time.perf_counter()
    for _ in range(steps):
        mean_loss = step()
    dt = (time.perf_counter() - t0) / steps
    ex.close()
    ex.rt.close()
    return {"value": rows / dt, "unit": "samples/s", "ms_per_step": dt * 1e3, "steps": steps,
            "h2d_bytes_per_step": int(X.nbytes + Y.nbytes), "d2h_bytes_per_step": int(loss.nbytes),
            "last_mean_loss": mean_loss,
            "path": "numpy X,Y -> polar_b200_rt_write (host copy of the record) -> upload on first device lock -> "
                    "Device::launch per builtin -> polar_b200_rt_read of the loss tensor"}


def shutdown(torch, dist, world, graph):
    """Leaves the process promptly.  Tearing down an NCCL communicator while a
    captured CUDA graph still references its kernels was seen to block for
    minutes after the result had been printed, so: drop the graph, drain the
    device, meet the other ranks once, give destroy_process_group a few seconds
    on a helper thread, then exit without running further teardown."""
    del graph
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        t = threading.Thread(target=dist.destroy_process_group, daemon=True)
        t.start()
        t.join(timeout=10.0)
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def mm_dims(program, kernel, args):
    tl, tr = kernel[8] == "t", kernel[10] == "t"
    ls, rs = program.tensors[args[0]], program.tensors[args[1]]
    m = ls[1] if tl else ls[0]
    k = ls[0] if tl else ls[1]
    n = rs[0] if tr else rs[1]
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


def gemm_numbers(torch, lib, n, reps):
    st = torch.cuda.current_stream().cuda_stream
    a = torch.empty((n, n), device="cuda").uniform_(-1, 1)
    b = torch.empty((n, n), device="cuda").uniform_(-1, 1)
    c = torch.empty((n, n), device="cuda")
    out = {}
    for tl in (0, 1):
        for tr in (0, 1):
            ms = event_time(torch, lambda: lib.call("polar_b200_fmatmul", tl, tr, n, n, n, a.data_ptr(),
                                                    b.data_ptr(), c.data_ptr(), None, 0, st), reps)
            out[f"fmatmul_{'t' if tl else 'f'}_{'t' if tr else 'f'}"] = {"ms": ms, "tflops": 2.0 * n ** 3 / ms / 1e9}
    return out


def elementwise_numbers(torch, lib, n, peaks, reps):
    st = torch.cuda.current_stream().cuda_stream
    a = torch.empty(n, device="cuda").uniform_(-1, 1)
    b = torch.empty(n, device="cuda").uniform_(0.5, 2)
    p = torch.empty(n, device="cuda").uniform_(0.01, 0.99)
    y = (torch.rand(n, device="cuda") < 0.5).float()
    o = torch.empty(n, device="cuda")
    A, B, P, Y, O = (t.data_ptr() for t in (a, b, p, y, o))
    ops = {
        "ffill": (4, lambda: lib.call("polar_b200_ffill", 1.234, O, n, st)),
        "fcopy": (8, lambda: lib.call("polar_b200_fcopy", A, O, n, st)),
        "fsigmoid": (8, lambda: lib.call("polar_b200_fsigmoid", A, O, n, st)),
        "fadd": (12, lambda: lib.call("polar_b200_fadd", A, 1.0, B, 1.0, O, n, st)),
        "fmul": (12, lambda: lib.call("polar_b200_fmul", A, B, O, n, st)),
        "fdivide": (12, lambda: lib.call("polar_b200_fdivide", A, B, O, n, st)),
        "flogloss": (12, lambda: lib.call("polar_b200_flogloss", P, Y, O, n, st)),
    }
    out = {}
    for name, (bpe, fn) in ops.items():
        ms = event_time(torch, fn, reps)
        gbs = bpe * n / ms / 1e6
        out[name] = {"ms": ms, "gbs": gbs, "frac_of_measured_copy": gbs / peaks["hbm_gbs"], "frac_of_8tbs": gbs / 8000.0}
    return out


def small_program_latencies(torch, reps=200):
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
        ex = DeviceExecutor(prog)
        ex.set_inputs(**inputs)
        eager_us = event_time(torch, ex.run, reps, warmup=10) * 1e3
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
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
        peak = peaks["bf16_tflops"] / 2.0
        line = {"metric": "fp32_matmul_tflops", "value": tf, "unit": "TFLOP/s", "ms_per_step": ms, "dtype": "f32",
                "config": {"workload": f"fmatmul_f_f_{n}x{n}x{n}",
                           "l2": f"operands and result {12 * n * n / 1e6:.0f} MB vs 126 MB L2"},
                "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak,
                             "pipe_frac": 3 * tf / peak, "traffic": None,
                             "peak_source": f"MEASURED_PEAKS.json bf16_tflops / 2 ({peaks['source']})"},
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
    ap.add_argument("--collective", default="peer", choices=["peer", "nccl"],
                    help="mlp at N>1 with extended builtins: gradient sum + update as one peer-memory kernel, "
                         "or NCCL all-reduces followed by fadd")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-extras", action="store_true")
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
