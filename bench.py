#!/usr/bin/env python
"""Benchmark of the data-parallel MLP training step and of the kernels behind it.

    python bench.py [--gpus N] [--steps K] [--warmup W]         one JSON line on rank 0
    python bench.py --impl reference ...                        Knet's CPU path (the oracle port), full batch
    python bench.py --sweep [--sweep-out FILE]                  per-kernel GB/s over the sweeps

Workload ("mlp_dp"): 4096 -> [8192 x4 hidden] -> 1000, relu + dropout(0.5) after each hidden
layer, logsoftmax + nll, Adam, Float32, per-GPU batch 8192, x ~ N(0,1), labels uniform in
1..1000, gradients all-reduced with NCCL before update!.  Synthetic data, random-init weights.
A step = forward + backward + all-reduce + update on one batch.  `value` times steps whose
inputs are already in HBM; `e2e` includes the pinned-host -> device copy of every batch and
the device -> host read of the loss.  Inputs (134 MB per batch, rotating over several
batches) and the 3.9 GB parameter/optimizer set exceed the 126 MB L2, so no flush is needed.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "knet.jl_b200"))

SIZES = [4096, 8192, 8192, 8192, 8192, 1000]
BATCH = 8192
PDROP = 0.5
NPARAMS = sum(SIZES[i] * SIZES[i + 1] + SIZES[i + 1] for i in range(len(SIZES) - 1))
ADAM_BYTES_PER_PARAM = 28            # read w,g,m,v + write w,m,v, Float32
# dram__bytes_read.sum + dram__bytes_write.sum of one opt_kernel<float, AdamF> launch: ncu measured
# 1359.80 MB for 50 356 224 parameters, i.e. 27.0 B per parameter; traffic is proportional to the
# parameter count, so it is scaled to this parameter set
ADAM_NCU_TRAFFIC_BYTES = int(round(1359.80e6 / 50356224 * NPARAMS))
WORKLOAD = "mlp_dp 4096-[8192x4]-1000 relu+dropout(0.5) nll Adam, per-GPU batch 8192"


def workload_config(world, sharded=False):
    """The `config` object, identical in the GPU arm and the reference arm for the same N."""
    return {"workload": WORKLOAD, "global_batch": BATCH * world, "params": NPARAMS,
            "parallelism": f"dp{world}" + ("+sharded-update" if sharded else ""),
            "l2": "inputs and parameter set larger than L2, batches rotate"}


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


class LaunchProbe:
    """CUDA events around every library launch of a step (MLP.probe): per-kernel time and
    algorithmic bytes of the hand-written kernels, with the cache state the GEMMs leave."""

    def __init__(self, torch):
        self.torch, self.recs, self.cur = torch, [], None

    def begin(self, label, nbytes):
        e = self.torch.cuda.Event(enable_timing=True)
        e.record()
        self.cur = (label, nbytes, e)

    def end(self):
        e = self.torch.cuda.Event(enable_timing=True)
        e.record()
        self.recs.append(self.cur + (e,))

    def summary(self, steps, peak, step_ms):
        per = {}
        for label, nbytes, a, b in self.recs:
            d = per.setdefault(label, {"launches": 0, "ms": 0.0, "bytes": 0})
            d["launches"] += 1
            d["ms"] += a.elapsed_time(b)
            d["bytes"] += nbytes
        tot_ms = sum(d["ms"] for d in per.values())
        tot_b = sum(d["bytes"] for d in per.values())
        for d in per.values():
            d["gbs"] = round(d["bytes"] / (d["ms"] * 1e-3) / 1e9, 1)
            d["frac"] = round(d["gbs"] / peak, 3)
            d["launches"], d["ms"], d["bytes"] = d["launches"] / steps, round(d["ms"] / steps, 4), d["bytes"] // steps
        gbs = tot_b / (tot_ms * 1e-3) / 1e9
        return {"what": "every launch of this library inside a step (all but the cuBLAS products and NCCL), "
                        "CUDA events around each launch, mean over the probed steps",
                "probed_steps": steps, "ms_per_step": tot_ms / steps, "algorithmic_bytes_per_step": tot_b // steps,
                "gbs": gbs, "frac": gbs / peak, "frac_of_8000": gbs / 8000.0,
                "share_of_step": tot_ms / steps / step_ms, "per_kernel": per}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [t.strip() for t in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------
def run_gpu(args):
    import torch
    import torch.distributed as dist
    import knet_sm100 as K
    from knet_sm100 import dp

    torch.backends.cuda.matmul.allow_tf32 = False          # Knet calls cublasSgemm: true Float32
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    os.environ.setdefault("NCCL_DEBUG", "WARN")     # the caller's setting wins
    # NCCL writes its log to stdout unless NCCL_DEBUG_FILE names a file.  So that stdout carries the one
    # JSON line and nothing else at any log level, file descriptor 1 is pointed at stderr for the rest of
    # the run and the JSON line goes to a private copy of the original stdout.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    rank, world = dp.init_from_env("nccl")
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but world size is {world}", file=sys.stderr)
    pg = dist.group.WORLD if world > 1 else None
    comm_note = "torch.distributed NCCL"
    gemm_note = "cuBLAS fp32 via torch.mm"
    if K.ops.GEMM_MODE != "torch":
        g = K.ops.gemm_handle()
        if K.ops.GEMM_MODE == "emulated" and not g.emulation:
            raise SystemExit(f"--gemm emulated: cuBLAS {g.version} in this process does not offer the FP32 emulation")
        gemm_note = (f"cuBLAS {g.version} via knet_gemm_32_S, " +
                     ("fp32 emulated on bf16 tensor cores (bf16x9)" if K.ops.GEMM_MODE == "emulated" else "plain fp32"))
    if world > 1 and args.comm in ("knet", "auto"):   # gradients travel through the library's knet_dp_* entry points
        comm, err = None, ""
        try:
            comm = dp.KnetComm(rank, world)
        except Exception as e:                         # noqa: BLE001 - any failure means "use torch.distributed"
            err = str(e)[:120]
        ok = torch.tensor([1.0 if comm is not None else 0.0], device=torch.device("cuda", local))
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)      # every rank must have it, or none uses it
        if ok.item() == 1.0:
            pg, comm_note = comm, "knet_dp_* (NCCL via the C ABI)"
        else:
            comm_note = f"torch.distributed NCCL (knet_dp_* not available: {err})" if err else comm_note + " (a peer could not create a knet_dp communicator)"
    dev = torch.device("cuda", local)

    model = K.MLP(SIZES, BATCH, pdrop=PDROP, seed=1, optimizer=K.Adam(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8),
                  device=dev, process_group=pg, dropout_seed=1000 + rank, shard_update=args.shard_update)
    nbatches = 3
    g = torch.Generator(device="cpu").manual_seed(100 + rank)
    host_x = [torch.randn(BATCH, SIZES[0], generator=g).pin_memory() for _ in range(nbatches)]
    host_y = [torch.randint(1, SIZES[-1] + 1, (BATCH,), generator=g, dtype=torch.int32).pin_memory()
              for _ in range(nbatches)]
    dev_x = [K.KnetArray(h.to(dev).view(-1), (SIZES[0], BATCH)) for h in host_x]
    dev_y = [h.to(dev) for h in host_y]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        model.step(dev_x[i % nbatches], dev_y[i % nbatches])
    barrier()

    # ---- device-resident timing -----------------------------------------------------------------
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = model.launches
    upd = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        x, y = dev_x[i % nbatches], dev_y[i % nbatches]
        scores = model.forward(x)
        model.loss(scores, y)
        model.backward(x, y)
        upd[i][0].record()
        model.update()
        upd[i][1].record()
        model.step_no += 1
    model.sync_weights()                     # sharded update: the last weight all-gathers belong to the step
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    launches = model.launches - launches0
    adam_ms = statistics.mean(a.elapsed_time(b) for a, b in upd)
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    loss_total, loss_count = float(model.total.item()), int(model.count.item())

    # ---- end to end: host batches in, loss out, every step ---------------------------------------
    # Two staging buffers: the copy of batch i+1 runs on a side stream under step i, and the loss
    # of step i is read from pinned memory while step i+1 runs.  Every batch still crosses from
    # pinned host memory inside the timed region and every step's loss reaches the host.
    copy_stream = torch.cuda.Stream()
    stage = [(K.KnetArray(torch.empty(BATCH * SIZES[0], device=dev), (SIZES[0], BATCH)),
              torch.empty(BATCH, dtype=torch.int32, device=dev)) for _ in range(2)]
    pin_tot = [torch.zeros(1, dtype=model.total.dtype).pin_memory() for _ in range(2)]
    pin_cnt = [torch.zeros(1, dtype=torch.int32).pin_memory() for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    freed = [None, None]
    done = [torch.cuda.Event() for _ in range(2)]
    losses = []

    def upload(i, k):
        with torch.cuda.stream(copy_stream):
            if freed[k] is not None:
                copy_stream.wait_event(freed[k])           # the step that last used this buffer is over
            stage[k][0].data.copy_(host_x[i % nbatches].view(-1), non_blocking=True)
            stage[k][1].copy_(host_y[i % nbatches], non_blocking=True)
            ready[k].record(copy_stream)

    barrier()
    t0 = time.perf_counter()
    upload(0, 0)
    for i in range(args.steps):
        k = i & 1
        if i + 1 < args.steps:
            upload(i + 1, k ^ 1)
        torch.cuda.current_stream().wait_event(ready[k])
        tot, cnt = model.step(stage[k][0], stage[k][1])
        freed[k] = torch.cuda.Event()
        freed[k].record()
        pin_tot[k].copy_(tot, non_blocking=True)
        pin_cnt[k].copy_(cnt, non_blocking=True)
        done[k].record()
        if i > 0:
            done[k ^ 1].synchronize()
            losses.append(float(pin_tot[k ^ 1].item()) / max(int(pin_cnt[k ^ 1].item()), 1))
    done[(args.steps - 1) & 1].synchronize()
    k = (args.steps - 1) & 1
    losses.append(float(pin_tot[k].item()) / max(int(pin_cnt[k].item()), 1))
    barrier()
    e2e_s = time.perf_counter() - t0
    t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_s = float(t.item())

    # ---- the library's own launches, one by one (a few extra steps, outside both timed regions) ----
    peak, peak_kind = peaks()
    probe = LaunchProbe(torch)
    nprobe = min(args.steps, 5)
    model.sync_weights()
    model.probe = probe
    for i in range(nprobe):
        model.step(dev_x[i % nbatches], dev_y[i % nbatches])
    model.probe = None
    barrier()
    kernels_step = probe.summary(nprobe, peak, ms / args.steps)

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    adam_bytes = (int(model.offsets[-1]) // world if model.sharded else NPARAMS) * ADAM_BYTES_PER_PARAM
    adam_kernel = "opt_kernel<float,AdamF> (multi-tensor update!, 10 arrays)"
    if model.sharded:      # one launch per layer, interleaved with the backward pass: take them from the per-launch probe
        pk = kernels_step["per_kernel"]["update! (own shard of one layer)"]
        adam_ms, adam_kernel = pk["ms"], f"opt_kernel<float,AdamF> ({len(SIZES) - 1} launches, this rank's 1/{world} of every layer)"
    achieved = adam_bytes / (adam_ms * 1e-3) / 1e9
    out = {
        "metric": "mlp_train_samples_per_s", "value": BATCH * world * args.steps / (ms * 1e-3),
        "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": workload_config(world, model.sharded),
        "notes": {"collectives": comm_note if world > 1 else None, "gemm": gemm_note},
        "e2e": {"value": BATCH * world * args.steps / e2e_s, "unit": "samples/s",
                "h2d_bytes_per_step": BATCH * SIZES[0] * 4 + BATCH * 4, "d2h_bytes_per_step": 8},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {"kernel": adam_kernel, "bound": "hbm",
                     "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                     "frac": achieved / peak, "frac_of_8000": achieved / 8000.0,
                     "traffic": int(ADAM_NCU_TRAFFIC_BYTES * adam_bytes / (NPARAMS * ADAM_BYTES_PER_PARAM)),
                     "algorithmic_bytes": adam_bytes, "ms": adam_ms},
        "kernels_step": kernels_step,
        "loss": loss_total / max(loss_count, 1),
    }
    if world == 1 and not args.no_cpu:
        out["cpu_baseline"] = cpu_baseline(steps=1, warm_full=False)
    if world == 1 and not args.no_kernels:
        out["kernels"] = headline_kernels(K, torch, peak)
    if world == 1 and args.gemm == "torch" and args.emulated:
        out["emulated_fp32_gemm"] = emulated_leg(args)
    os.write(json_fd, (json.dumps(out) + "\n").encode())
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
def emulated_leg(args):
    """The same step with the matrix products in cuBLAS's FP32 emulation (bench.py --gemm
    emulated), measured in a child process because the cuBLAS copy that offers it has to be
    loaded before PyTorch's.  Reported beside the headline, which stays on plain FP32."""
    cmd = [sys.executable, os.path.abspath(__file__), "--gemm", "emulated", "--steps", str(args.steps),
           "--warmup", str(args.warmup), "--no-cpu", "--no-kernels"]
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
        if r.returncode != 0 or not lines:
            return {"unavailable": (r.stderr.strip().splitlines() or ["no output"])[-1][:200]}
        d = json.loads(lines[-1])
        return {"value": d["value"], "unit": d["unit"], "ms_per_step": d["ms_per_step"], "e2e": d["e2e"]["value"],
                "gemm": d["notes"]["gemm"], "clocks": d["clocks"], "loss": d["loss"],
                "accuracy": "per-entry error of the emulated product <= plain FP32's on the same inputs (tests/test_gpu_gemm.py)"}
    except Exception as e:                                   # the headline must not depend on this leg
        return {"unavailable": f"{type(e).__name__}: {e}"[:200]}


def fit_steps(steps, warmup, budget_s, elapsed_s, first_s):
    """How many full CPU steps to run when the first one took `first_s` seconds and `elapsed_s`
    of the `budget_s` are gone: (warm-up steps including the one already done, timed steps).
    Timed steps are kept before warm-up steps; at least one of each is always run."""
    fit = max(1, int((budget_s - elapsed_s) / max(first_s, 1e-9)))
    if warmup - 1 + steps > fit:
        warmup = 1 + max(0, min(warmup - 1, fit - steps))
        steps = max(1, min(steps, fit - (warmup - 1)))
    return warmup, steps


def cpu_baseline(steps=1, warm_full=True, budget_s=None, warmup=1):
    """Knet's CPU path for the same step, as restated in oracle/: the full per-GPU batch of 8192
    columns on the full 243M-parameter model.  BLAS gemm (NumPy) on all host threads; the other
    ops are Knet's loops, split over all host cores with OpenMP where the box can build that
    copy (Julia itself runs them on one core).  `warm_full`: the warm-up steps are full steps too
    (otherwise one 64-column step that only allocates the Adam state and pages the code in).
    `budget_s` caps the run: warm-up and timed steps are cut (never below one timed full step)
    so that the estimate from the first full step fits."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import knet_oracle as ko
    from threadpoolctl import threadpool_limits
    ko.build()
    omp = ko.have_openmp()
    ko.use_openmp(omp)
    cores = host_threads()
    with threadpool_limits(limits=cores):             # a launcher may have pinned OMP_NUM_THREADS=1
        rng = np.random.default_rng(1)
        model = ko.MLP(SIZES, rng, pdrop=PDROP, optimizer="adam", lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8)
        x = rng.standard_normal((SIZES[0], BATCH), dtype=np.float32)
        y = rng.integers(1, SIZES[-1] + 1, BATCH)
        us = [np.asfortranarray(rng.random((SIZES[i + 1], BATCH), dtype=np.float32)) for i in range(len(SIZES) - 2)]
        t_begin = time.perf_counter()
        done_warm = 0
        if warm_full:
            t0 = time.perf_counter()
            model.step(x, y, us)
            first = time.perf_counter() - t0
            done_warm = 1
            if budget_s is not None:                  # what still fits after the first full step
                warmup, steps = fit_steps(steps, warmup, budget_s, time.perf_counter() - t_begin, first)
            for _ in range(warmup - 1):
                model.step(x, y, us)
                done_warm += 1
        else:
            model.step(x[:, :64], y[:64], [u[:, :64] for u in us])
        model.timers = {}
        t0 = time.perf_counter()
        for _ in range(steps):
            model.step(x, y, us)
        dt = (time.perf_counter() - t0) / steps
    ko.use_openmp(False)
    gemm_s, upd_s = model.timers.get("gemm", 0.0) / steps, model.timers.get("update", 0.0) / steps
    loops = "other ops OpenMP on all cores" if omp else "other ops one core as in Julia"
    return {"value": BATCH / dt, "unit": "samples/s", "cores": cores, "kind": "port",
            "sample": f"{steps} full step(s): batch {BATCH} of {BATCH} columns, full 243M-parameter model, after "
                      f"{done_warm if warm_full else 'a 64-column'} warm-up step(s); gemm on {cores} threads (NumPy BLAS), {loops}; "
                      f"{dt:.2f} s/step = {gemm_s:.2f} s gemm + {upd_s:.2f} s update! + {dt - gemm_s - upd_s:.2f} s other ops",
            "s_per_step": dt, "steps": steps, "warmup": done_warm if warm_full else 0,
            "gemm_s_per_step": gemm_s, "update_s_per_step": upd_s}


def run_reference(args):
    """The reference arm: Knet's own CPU implementation cannot run (no Julia in the image), so
    this times the oracle port of that path on the host cores, on the same configuration as
    the GPU arm (full batch).  Steps and warm-up follow --steps/--warmup as far as --ref-budget
    seconds allow; the JSON line reports what was actually run."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    cb = cpu_baseline(steps=max(1, args.steps), warm_full=True, budget_s=args.ref_budget, warmup=max(1, args.warmup))
    out = {"impl": "reference", "metric": "mlp_train_samples_per_s", "value": cb["value"], "unit": "samples/s",
           "n_gpus": world, "steps": cb["steps"], "warmup": cb["warmup"], "ms_per_step": cb["s_per_step"] * 1e3,
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
           "config": workload_config(world),
           "notes": {"what": "CPU port of Knet's path (Julia is not available) on the host cores of rank 0, one replica "
                             "of the per-GPU workload; steps/warmup are the requested ones cut to the time budget",
                     "requested_steps": args.steps, "requested_warmup": args.warmup, "budget_s": args.ref_budget},
           "cpu_baseline": cb,
           "e2e": {"value": cb["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(out), flush=True)


# ------------------------------------------------------------------------------------------------
def time_kernel(torch, fn, reps=10, warm=3, inner=8):
    """Device time of one launch of fn(i): (median, best) in ms.  `inner` consecutive launches
    are recorded into a CUDA graph and the graph is replayed `reps` times between CUDA events,
    so the time is the kernel's own even where it is shorter than the host's launch path
    (a Python call through ctypes costs 10-20 us, more than many of the kernels here).  fn gets
    the launch number and may rotate over several buffer sets; callers do that wherever one
    set would fit the 126 MB L2.  Falls back to events around eager launches if the calls
    cannot be captured."""
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    try:
        with torch.cuda.graph(graph):
            for i in range(inner):
                fn(i)
    except Exception:                                   # noqa: BLE001 - not capturable: time eagerly
        graph, inner = None, 1
        torch.cuda.synchronize()
    if graph is not None:
        graph.replay()
        torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    for i, (a, b) in enumerate(evs):
        a.record()
        if graph is not None:
            graph.replay()
        else:
            fn(i)
        b.record()
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) / inner for a, b in evs)
    return ts[len(ts) // 2], ts[0]


def headline_kernels(K, torch, peak):
    """A few kernels of the sweeps at their largest shapes (median of 10, buffers > L2)."""
    from knet_sm100.lib import knet, knet8, ptr
    res = {}
    n = 1 << 28
    x = torch.randn(n, device="cuda")
    y = torch.empty_like(x)
    z = torch.empty_like(x)

    def rec(name, nbytes, fn, reps=10):
        med, best = time_kernel(torch, fn, reps)
        gbs = nbytes / (med * 1e-3) / 1e9
        res[name] = {"ms": round(med, 4), "gbs": round(gbs, 1), "frac": round(gbs / peak, 3)}

    rec("relu_32 2^28", 8 * n, lambda i: knet8("relu_32", n, ptr(x), ptr(y)))
    rec("sigm_32 2^28", 8 * n, lambda i: knet8("sigm_32", n, ptr(x), ptr(y)))
    rec("tanh_32 2^28", 8 * n, lambda i: knet8("tanh_32", n, ptr(x), ptr(y)))
    rec("reluback_32_11 2^28", 12 * n, lambda i: knet8("reluback_32_11", n, ptr(x), ptr(y), ptr(z)))
    rec("tanhback_32_11 2^28", 12 * n, lambda i: knet8("tanhback_32_11", n, ptr(x), ptr(y), ptr(z)))
    C_, B_ = 50257, 4096
    nl = C_ * B_
    s = torch.empty(max(C_, B_), device="cuda")
    rec("sum_32_21 dims=1 50257x4096", 4 * nl, lambda i: knet8("sum_32_21", nl, ptr(x), C_, B_, ptr(s)))
    rec("sum_32_21 dims=2 50257x4096", 4 * nl, lambda i: knet8("sum_32_21", nl, ptr(x), 1, C_, ptr(s)))
    rec("logsoftmax_fwd 50257x4096", 8 * nl, lambda i: knet("knet_logsoftmax_fwd_32", ptr(x), ptr(y), 1, C_, B_))
    rec("logsoftmax_bwd 50257x4096", 12 * nl,
        lambda i: knet("knet_logsoftmax_bwd_32", ptr(y), ptr(x), ptr(z), 1, C_, B_))
    return res


def _timed(fn):
    t0 = time.perf_counter()
    fn()
    return time.perf_counter() - t0


def run_sweep(args):
    """Per-kernel achieved GB/s over the elementwise, broadcast, reduction/softmax and
    optimizer sweeps; one JSON line per case."""
    import torch
    import knet_sm100 as K
    from knet_sm100.lib import knet, knet8, ptr
    torch.cuda.set_device(0)
    peak, kind = peaks()
    rows = []

    def emit(group, name, nbytes, med, best):
        gbs = nbytes / (med * 1e-3) / 1e9
        row = {"group": group, "case": name, "bytes": nbytes, "ms_median": med, "ms_best": best, "gbs": gbs,
               "frac_of_peak": gbs / peak, "frac_of_8000": gbs / 8000, "peak_kind": kind}
        rows.append(row)
        print(json.dumps(row), flush=True)

    # elementwise forward / backward, Float32 and Float64, 2^20 .. 2^28
    for S, dt, sz in (("32", torch.float32, 4), ("64", torch.float64, 8)):
        nmax = 1 << 28
        x = torch.randn(nmax, device="cuda", dtype=dt)
        y = torch.empty_like(x)
        dx = torch.empty_like(x)
        for k in (20, 24, 26, 28):
            n = 1 << k
            R = max(1, min(8, nmax // n))                  # windows of the big buffers, so that L2 does not help
            w = lambda t, i: ptr(t[(i % R) * n:(i % R) * n + n])
            for op in ("relu", "sigm", "tanh", "elu"):
                med, best = time_kernel(torch, lambda i: knet8(f"{op}_{S}", n, w(x, i), w(y, i)))
                emit("unary", f"{op}_{S} n=2^{k}", 2 * n * sz, med, best)
                med, best = time_kernel(torch, lambda i: knet8(f"{op}back_{S}_11", n, w(x, i), w(y, i), w(dx, i)))
                emit("actback", f"{op}back_{S}_11 n=2^{k}", 3 * n * sz, med, best)
        del x, y, dx
    # broadcast (N,1)+(N,M) and (1,M)+(N,M)
    for N in (64, 1024, 8192):
        for M in (128, 4096, 65536):
            nset = 1 if N * M * 4 > 400e6 else 4
            bigs = [K.KnetArray(torch.randn(N * M, device="cuda"), (N, M)) for _ in range(nset)]
            col = K.KnetArray(torch.randn(N, device="cuda") + 3, (N, 1))
            row = K.KnetArray(torch.randn(M, device="cuda") + 3, (1, M))
            for op in ("add", "mul", "div"):
                for nm, v in (("(N,1)", col), ("(1,M)", row)):
                    med, best = time_kernel(torch, lambda i: K.ops.broadcast(op, v, bigs[i % nset]), reps=7)
                    emit("broadcast", f"{op} {nm}+({N},{M})", (2 * N * M + len(v)) * 4, med, best)
            del bigs
    # reductions, softmax family, nll on C x B logits
    # the last three: short runs (one group of lanes per instance) at sizes beyond L2
    for C_, B_ in [(c, b) for c in (10, 1000, 50257) for b in (64, 512, 4096)] + [(64, 524288), (128, 262144), (1000, 32768)]:
        n = C_ * B_
        nset = 1 if n * 4 > 400e6 else 4            # rotate where one set would stay in L2
        xs = [K.KnetArray(torch.randn(n, device="cuda") * 3, (C_, B_)) for _ in range(nset)]
        dys = [K.KnetArray(torch.randn(n, device="cuda"), (C_, B_)) for _ in range(nset)]
        ys = [x.similar() for x in xs]
        lab = torch.randint(1, C_ + 1, (B_,), device="cuda", dtype=torch.int32)
        for d in (1, 2):
            for op in ("sum", "maximum"):
                med, best = time_kernel(torch, lambda i: K.ops.reduce(op, xs[i % nset], d), reps=7)
                emit("reduce", f"{op} dims={d} {C_}x{B_}", (n + (B_ if d == 1 else C_)) * 4, med, best)
            if d == 2 and B_ > 4096:
                continue        # the short-run shapes: a softmax along 2^15..2^19 strided columns is no workload
            med, best = time_kernel(torch, lambda i: K.logsumexp(xs[i % nset], d), reps=7)
            emit("reduce", f"logsumexp dims={d} {C_}x{B_}", (n + (B_ if d == 1 else C_)) * 4, med, best)
        for f in ("softmax", "logsoftmax"):
            med, best = time_kernel(torch, lambda i: knet(f"knet_{f}_fwd_32", ptr(xs[i % nset].data), ptr(ys[i % nset].data), 1, C_, B_), reps=7)
            emit("softmax", f"{f}_fwd {C_}x{B_}", 2 * n * 4, med, best)
            med, best = time_kernel(torch, lambda i: knet(f"knet_{f}_bwd_32", ptr(ys[i % nset].data), ptr(dys[i % nset].data), ptr(xs[i % nset].data), 1, C_, B_), reps=7)
            emit("softmax", f"{f}_bwd {C_}x{B_}", 3 * n * 4, med, best)
        tot = torch.empty(1, device="cuda")
        cnt = torch.empty(1, device="cuda", dtype=torch.int32)
        per = torch.empty(B_, device="cuda")
        med, best = time_kernel(torch, lambda i: knet("knet_nll_fwd_32", ptr(xs[i % nset].data), ptr(lab), C_, B_, 1, ptr(tot), ptr(cnt), ptr(per)), reps=7)
        emit("nll", f"nll_fwd {C_}x{B_}", n * 4 + B_ * 4, med, best)
        med, best = time_kernel(torch, lambda i: knet("knet_nll_bwd_32", ptr(xs[i % nset].data), ptr(lab), C_, B_, 1, 1, K.ops._CT[torch.float32](1.0), ptr(cnt), ptr(ys[i % nset].data)), reps=7)
        emit("nll", f"nll_bwd {C_}x{B_}", 2 * n * 4, med, best)
        res = torch.empty(2, device="cuda", dtype=torch.int32)
        med, best = time_kernel(torch, lambda i: knet("knet_accuracy_32", ptr(xs[i % nset].data), ptr(lab), C_, B_, 1, ptr(res)), reps=7)
        emit("nll", f"accuracy {C_}x{B_}", n * 4 + B_ * 4, med, best)
        del xs, dys, ys
    # the same family along dims=2: instances are rows (B x C scores), classes strided
    for R_, C_ in ((32768, 1000), (131072, 256)):
        n = R_ * C_
        xs = [torch.randn(n, device="cuda") * 3 for _ in range(4)]
        dys = [torch.randn(n, device="cuda") for _ in range(4)]
        ys = [torch.empty_like(x) for x in xs]
        lab = torch.randint(1, C_ + 1, (R_,), device="cuda", dtype=torch.int32)
        for f in ("softmax", "logsoftmax"):
            med, best = time_kernel(torch, lambda i: knet(f"knet_{f}_fwd_32", ptr(xs[i % 4]), ptr(ys[i % 4]), R_, C_, 1), reps=7)
            emit("softmax", f"{f}_fwd dims=2 {R_}x{C_}", 2 * n * 4, med, best)
            med, best = time_kernel(torch, lambda i: knet(f"knet_{f}_bwd_32", ptr(ys[i % 4]), ptr(dys[i % 4]), ptr(xs[i % 4]), R_, C_, 1), reps=7)
            emit("softmax", f"{f}_bwd dims=2 {R_}x{C_}", 3 * n * 4, med, best)
        tot = torch.empty(1, device="cuda")
        cnt = torch.empty(1, device="cuda", dtype=torch.int32)
        per = torch.empty(R_, device="cuda")
        med, best = time_kernel(torch, lambda i: knet("knet_nll_fwd_32", ptr(xs[i % 4]), ptr(lab), R_, C_, 2, ptr(tot), ptr(cnt), ptr(per)), reps=7)
        emit("nll", f"nll_fwd dims=2 {R_}x{C_}", n * 4 + R_ * 4, med, best)
        med, best = time_kernel(torch, lambda i: knet("knet_nll_bwd_32", ptr(xs[i % 4]), ptr(lab), R_, C_, 2, 1, K.ops._CT[torch.float32](1.0), ptr(cnt), ptr(ys[i % 4])), reps=7)
        emit("nll", f"nll_bwd dims=2 {R_}x{C_}", 2 * n * 4, med, best)
        res = torch.empty(2, device="cuda", dtype=torch.int32)
        med, best = time_kernel(torch, lambda i: knet("knet_accuracy_32", ptr(xs[i % 4]), ptr(lab), R_, C_, 2, ptr(res)), reps=7)
        emit("nll", f"accuracy dims=2 {R_}x{C_}", n * 4 + R_ * 4, med, best)
        del xs, dys, ys
    # optimizer step over 24 x (4096,4096) + 24 x (4096,)
    sizes = [4096 * 4096, 4096] * 24
    total = sum(sizes)
    w = torch.randn(total, device="cuda") * 0.02
    g = torch.randn(total, device="cuda") * 1e-3
    m = torch.zeros(total, device="cuda")
    v = torch.zeros(total, device="cuda")
    arrays, o = [], 0
    for nsz in sizes:
        arrays.append((w[o:o + nsz], g[o:o + nsz], m[o:o + nsz], v[o:o + nsz]))
        o += nsz
    plan = K.MultiTensorPlan(arrays)
    for name, opt, bpp in (("sgd", K.SGD(lr=0.1), 12), ("momentum", K.Momentum(lr=0.05, gamma=0.9), 20), ("adam", K.Adam(), 28)):
        med, best = time_kernel(torch, lambda i: K.update_multi_(plan, opt), reps=7)
        emit("update", f"{name} multi-tensor 48 arrays {total} params", total * bpp, med, best)
    # the same Adam step with per-array gradient clipping: norms and factors on the device (one more
    # read of the gradients), then the update with the factors applied on load
    clipped = K.Adam(gclip=1.0)
    med, best = time_kernel(torch, lambda i: K.update_multi_(plan, clipped), reps=7)
    emit("update", f"adam + gclip multi-tensor 48 arrays {total} params", total * (28 + 4), med, best)
    del w, g, m, v, plan
    # hidden-layer pieces of the MLP workload: 8192 x 8192, p = 0.5
    N = B_ = 8192
    nl = N * B_
    z = torch.randn(nl, device="cuda")
    bvec = torch.randn(N, device="cuda")
    yb, dz = torch.empty_like(z), torch.empty_like(z)
    half = K.ops._CT[torch.float32](0.5)
    med, best = time_kernel(torch, lambda i: knet("knet_bias_relu_dropout_fwd_32", ptr(z), ptr(bvec), ptr(yb), N, B_, half, 1, 0), reps=7)
    emit("layer", "bias+relu+dropout(philox) fwd 8192x8192", 2 * nl * 4, med, best)
    med, best = time_kernel(torch, lambda i: knet("knet_relu_dropout_bwd_32", ptr(yb), ptr(z), ptr(dz), nl, half), reps=7)
    emit("layer", "dropback+reluback bwd 8192x8192", 3 * nl * 4, med, best)
    dbv = torch.empty(N, device="cuda")
    med, best = time_kernel(torch, lambda i: knet("knet_relu_dropout_bias_bwd_32", ptr(yb), ptr(z), ptr(dz), ptr(dbv), N, B_, half), reps=7)
    emit("layer", "dropback+reluback+bias gradient bwd 8192x8192", (3 * nl + N) * 4, med, best)
    med, best = time_kernel(torch, lambda i: knet("knet_dropout_philox_32", nl, half, 1, 0, ptr(z), ptr(yb)), reps=7)
    emit("layer", "dropout(philox) 8192x8192", 2 * nl * 4, med, best)
    med, best = time_kernel(torch, lambda i: knet8("dropout_32", nl, half, ptr(z), ptr(yb)), reps=7)
    emit("layer", "dropout_32 (supplied uniforms) 8192x8192", 3 * nl * 4, med, best)
    med, best = time_kernel(torch, lambda i: knet8("sum_32_21", nl, ptr(z), 1, N, ptr(bvec)), reps=7)
    emit("layer", "bias gradient sum dims=2 8192x8192", (nl + N) * 4, med, best)
    del z, yb, dz
    # embedding lookup w[:, tokens] and its scatter-add gradient: E x V table, n tokens
    for E, V, cnt in ((1024, 50257, 262144), (256, 50257, 1048576), (4096, 32000, 65536)):
        wtab = torch.randn(E * V, device="cuda")
        tok = torch.randint(1, V + 1, (cnt,), device="cuda", dtype=torch.int32)
        emb = torch.empty(E * cnt, device="cuda")
        med, best = time_kernel(torch, lambda i: knet8("getcols_32", E, V, cnt, ptr(tok), ptr(wtab), ptr(emb)), reps=7)
        emit("index", f"getcols (embedding lookup) {E}x{V}, {cnt} tokens", 2 * E * cnt * 4 + 4 * cnt, med, best)
        med, best = time_kernel(torch, lambda i: knet8("addcols_32", E, V, cnt, ptr(tok), ptr(wtab), ptr(emb)), reps=7)
        emit("index", f"addcols (embedding gradient) {E}x{V}, {cnt} tokens", 3 * E * cnt * 4 + 4 * cnt, med, best)
        del wtab, emb
    xm = torch.randn(8192 * 8192, device="cuda")
    rsel = torch.randint(1, 8193, (4096,), device="cuda", dtype=torch.int32)
    ysel = torch.empty(4096 * 8192, device="cuda")
    med, best = time_kernel(torch, lambda i: knet8("getrows_32", 8192, 8192, 4096, ptr(rsel), ptr(xm), ptr(ysel)), reps=7)
    emit("index", "getrows 4096 of 8192x8192", 2 * 4096 * 8192 * 4, med, best)
    blk = torch.empty(4096 * 8192, device="cuda")
    med, best = time_kernel(torch, lambda i: knet8("xcopy", 4096 * 4, 8192, ptr(xm), 8192 * 4, ptr(blk), 4096 * 4), reps=7)
    emit("index", "xcopy A[1:4096, :] of 8192x8192", 2 * 4096 * 8192 * 4, med, best)
    del xm, ysel, blk
    # MLP 784-64-10, batch 100, Adam: launch-latency-bound, reported as time per step
    small = K.MLP([784, 64, 10], 100, optimizer=K.Adam(lr=1e-3))
    xs = K.KnetArray(torch.rand(784 * 100, device="cuda"), (784, 100))
    ys = torch.randint(1, 11, (100,), device="cuda", dtype=torch.int32)
    for _ in range(20):
        small.step(xs, ys)
    torch.cuda.synchronize()
    l0, t0 = small.launches, time.perf_counter()
    for _ in range(100):
        small.step(xs, ys)
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / 100
    row = {"group": "mlp_small", "case": "MLP 784-64-10 batch 100 Adam, one step (host-launch bound)",
           "ms_per_step": dt * 1e3, "samples_per_s": 100 / dt, "library_launches_per_step": (small.launches - l0) / 100}
    rows.append(row)
    print(json.dumps(row), flush=True)
    small.capture()                                  # the same step as one CUDA graph launch
    for _ in range(20):
        small.step_graph(xs, ys)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(200):
        small.step_graph(xs, ys)
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / 200
    row = {"group": "mlp_small", "case": "MLP 784-64-10 batch 100 Adam, one step as a captured CUDA graph",
           "ms_per_step": dt * 1e3, "samples_per_s": 100 / dt, "library_launches_per_step": small.launches_per_replay}
    rows.append(row)
    print(json.dumps(row), flush=True)
    # Knet's CPU path (oracle port, one host core like Julia's broadcast/reduction loops) on a
    # bounded sample of the same kernels: 2^24 elements, best of 3
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import knet_oracle as ko
    ko.build()
    rng = np.random.default_rng(0)
    nc = 1 << 24
    xc = rng.standard_normal(nc).astype(np.float32)
    yc = ko.unary("relu", xc)
    lg = np.asfortranarray(xc.reshape(4096, 4096))

    def cpu(name, nbytes, fn):
        for omp in ((False, True) if ko.have_openmp() else (False,)):     # one core as in Julia, then all cores
            ko.use_openmp(omp)
            best = min(_timed(fn) for _ in range(3))
            r = {"group": "cpu_oracle", "case": name, "bytes": nbytes, "ms_best": best * 1e3, "gbs": nbytes / best / 1e9,
                 "cores": os.cpu_count() if omp else 1, "host_cores": os.cpu_count(), "kind": "port",
                 "sample": "2^24 Float32 elements"}
            rows.append(r)
            print(json.dumps(r), flush=True)
        ko.use_openmp(False)

    cpu("relu_32", 2 * nc * 4, lambda: ko.unary("relu", xc))
    cpu("sigm_32", 2 * nc * 4, lambda: ko.unary("sigm", xc))
    cpu("tanh_32", 2 * nc * 4, lambda: ko.unary("tanh", xc))
    cpu("reluback_32", 3 * nc * 4, lambda: ko.actback("reluback", xc, yc))
    cpu("add (N,1)+(4096,4096)", 2 * nc * 4, lambda: ko.binary("add", lg, lg[:, :1]))
    cpu("sum dims=1 4096x4096", nc * 4, lambda: ko.reduce_dim("sum", lg, 1))
    cpu("sum dims=2 4096x4096", nc * 4, lambda: ko.reduce_dim("sum", lg, 2))
    cpu("logsoftmax_fwd 4096x4096", 2 * nc * 4, lambda: ko.logsoftmax(lg, 1))
    cpu("logsoftmax_bwd 4096x4096", 3 * nc * 4, lambda: ko.logsoftmax_bwd(lg, lg, 1))
    wc, mc, vc = xc.copy(), np.zeros_like(xc), np.zeros_like(xc)
    cpu("adam 2^24 params", 28 * nc, lambda: ko.adam(wc, yc, mc, vc, 1))
    cpu("sgd 2^24 params", 12 * nc, lambda: ko.sgd(wc, yc, 0.1))
    if args.sweep_out:
        os.makedirs(os.path.dirname(os.path.abspath(args.sweep_out)), exist_ok=True)
        with open(args.sweep_out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")


def run_case(args):
    """One kernel at a reduced size, launched a few times: the command that ncu captures.
    Cases: unary:<op>_<S>, back:<op>_<S>, scalar:<op>_<S>, softmax:<fn>:<C>x<B>, softmax2:<fn>:<R>x<C> (dims=2),
    accuracy:<dims>:<R>x<K>, reduce:<op>:<dims>:<C>x<B>, bcast16:<op>, xcopy,
    bcast:<op>:<col|row>:<N>x<M>, update:<sgd|momentum|adam>, layer:<fwd|bwd|bwdb>,
    index:<getcols|setcols|addcols|getrows|addrows>:<E>x<V>x<n>, gemm:<mode>:<m>x<n>x<k>."""
    import torch
    import knet_sm100 as K
    from knet_sm100.lib import knet, knet8, ptr
    torch.cuda.set_device(0)
    kind, *rest = args.case.split(":")
    n = args.n
    if kind in ("unary", "back"):
        name = rest[0]
        dt = torch.float32 if name.endswith("32") else torch.float64
        x = torch.randn(n, device="cuda", dtype=dt)
        y, z = torch.empty_like(x), torch.empty_like(x)
        if kind == "unary":
            fn = lambda: knet8(name, n, ptr(x), ptr(y))
        else:
            fn = lambda: knet8(name + "_11", n, ptr(x), ptr(y), ptr(z))
    elif kind == "scalar":
        # scalar:<op>_<S>  (s op array, the _01 entry points)
        name = rest[0]
        dt = torch.float32 if name.endswith("32") else torch.float64
        x = torch.randn(n, device="cuda", dtype=dt) + 3
        y = torch.empty_like(x)
        sc = K.ops._CT[dt](1.7)
        fn = lambda: knet8(name + "_01", n, sc, ptr(x), ptr(y))
    elif kind == "softmax":
        f, shape = rest
        C_, B_ = (int(v) for v in shape.split("x"))
        x = torch.randn(C_ * B_, device="cuda") * 3
        y, z = torch.empty_like(x), torch.empty_like(x)
        if f.endswith("bwd"):
            fn = lambda: knet(f"knet_{f}_32", ptr(x), ptr(y), ptr(z), 1, C_, B_)
        else:
            fn = lambda: knet(f"knet_{f}_32", ptr(x), ptr(y), 1, C_, B_)
    elif kind == "softmax2":
        # softmax2:<f>:<R>x<C>  the same family along dims=2 (instances are rows)
        f, shape = rest
        R_, C_ = (int(v) for v in shape.split("x"))
        x = torch.randn(R_ * C_, device="cuda") * 3
        y, z = torch.empty_like(x), torch.empty_like(x)
        if f.endswith("bwd"):
            fn = lambda: knet(f"knet_{f}_32", ptr(x), ptr(y), ptr(z), R_, C_, 1)
        else:
            fn = lambda: knet(f"knet_{f}_32", ptr(x), ptr(y), R_, C_, 1)
    elif kind == "accuracy":
        # accuracy:<dims>:<R>x<K>
        d, shape = rest
        R_, K_ = (int(v) for v in shape.split("x"))
        ninst, ncls = (K_, R_) if int(d) == 1 else (R_, K_)
        x = torch.randn(R_ * K_, device="cuda")
        lab = torch.randint(1, ncls + 1, (ninst,), device="cuda", dtype=torch.int32)
        res = torch.empty(2, device="cuda", dtype=torch.int32)
        fn = lambda: knet("knet_accuracy_32", ptr(x), ptr(lab), R_, K_, int(d), ptr(res))
    elif kind == "reduce":
        op, d, shape = rest
        C_, B_ = (int(v) for v in shape.split("x"))
        x = K.KnetArray(torch.randn(C_ * B_, device="cuda"), (C_, B_))
        fn = lambda: (K.logsumexp(x, int(d)) if op == "logsumexp" else K.ops.reduce(op, x, int(d)))
    elif kind == "bcast":
        op, which, shape = rest
        N, M = (int(v) for v in shape.split("x"))
        big = K.KnetArray(torch.randn(N * M, device="cuda"), (N, M))
        v = K.KnetArray(torch.randn(N if which == "col" else M, device="cuda") + 3, (N, 1) if which == "col" else (1, M))
        fn = lambda: K.ops.broadcast(op, v, big)
    elif kind == "bcast16":
        # bcast16:<op>  (256,1,256,1) (+) (256,64,256,8): the general strided broadcast, 134 MB result
        a = K.KnetArray(torch.randn(256 * 256, device="cuda") + 3, (256, 1, 256, 1))
        b = K.KnetArray(torch.randn(256 * 64 * 256 * 8, device="cuda") + 3, (256, 64, 256, 8))
        fn = lambda: K.ops.broadcast(rest[0], a, b)
    elif kind == "xcopy":
        # xcopy: A[1:4096, :] of an 8192 x 8192 Float32 matrix (2-d strided copy)
        xm = torch.randn(8192 * 8192, device="cuda")
        blk = torch.empty(4096 * 8192, device="cuda")
        fn = lambda: knet8("xcopy", 4096 * 4, 8192, ptr(xm), 8192 * 4, ptr(blk), 4096 * 4)
    elif kind == "update":
        sizes = [2048 * 4096, 4096] * 6                       # a slice of the 48-array parameter set
        total = sum(sizes)
        bufs = [torch.randn(total, device="cuda") * 1e-3 for _ in range(2)] + [torch.zeros(total, device="cuda") for _ in range(2)]
        arrays, o = [], 0
        for s in sizes:
            arrays.append(tuple(b[o:o + s] for b in bufs))
            o += s
        plan = K.MultiTensorPlan(arrays)
        opt = {"sgd": K.SGD(lr=0.1), "momentum": K.Momentum(lr=0.05, gamma=0.9), "adam": K.Adam()}[rest[0]]
        fn = lambda: K.update_multi_(plan, opt)
    elif kind == "layer":
        N, B_ = 8192, 2048
        z = torch.randn(N * B_, device="cuda")
        b = torch.randn(N, device="cuda")
        y, dz = torch.empty_like(z), torch.empty_like(z)
        if rest[0] == "fwd":
            fn = lambda: knet("knet_bias_relu_dropout_fwd_32", ptr(z), ptr(b), ptr(y), N, B_, K.ops._CT[torch.float32](0.5), 1, 0)
        elif rest[0] == "bwdb":
            fn = lambda: knet("knet_relu_dropout_bias_bwd_32", ptr(z), ptr(y), ptr(dz), ptr(b), N, B_, K.ops._CT[torch.float32](0.5))
        else:
            fn = lambda: knet("knet_relu_dropout_bwd_32", ptr(z), ptr(y), ptr(dz), N * B_, K.ops._CT[torch.float32](0.5))
    elif kind == "index":
        # index:<getcols|setcols|addcols|getrows|addrows>:<E>x<V>x<n>  (x is E x V, n picked columns / rows)
        f, shape = rest
        E, V, cnt = (int(v) for v in shape.split("x"))
        x = torch.randn(E * V, device="cuda")
        cols = f.endswith("cols")
        hi = V if cols else E
        idx = (torch.randperm(hi, device="cuda")[:cnt] if f.startswith("set") else torch.randint(0, hi, (cnt,), device="cuda")).to(torch.int32) + 1
        y = torch.randn(E * cnt if cols else cnt * V, device="cuda")
        fn = lambda: knet8(f"{f}_32", E, V, idx.numel(), ptr(idx), ptr(x), ptr(y))
    elif kind == "gemm":
        # gemm:<mode 0|1|2>:<m>x<n>x<k>  (knet_gemm_32_S; modes 1 and 2 need --gemm emulated)
        mode, shape = rest
        m_, n_, k_ = (int(v) for v in shape.split("x"))
        a = torch.randn(m_ * k_, device="cuda")
        b = torch.randn(k_ * n_, device="cuda")
        c = torch.empty(m_ * n_, device="cuda")
        fn = lambda: K.ops.gemm_(0, 0, m_, n_, k_, a, m_, b, k_, c, m_, mode=int(mode))
        flops = 2.0 * m_ * n_ * k_
    else:
        raise SystemExit(f"unknown case {args.case}")
    for _ in range(args.reps):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    rep = {"case": args.case, "n": n, "reps": args.reps, "ms_per_launch": e0.elapsed_time(e1) / args.reps}
    if kind == "gemm":
        g = K.ops.gemm_handle()
        rep.update(tflops=flops / (rep["ms_per_launch"] * 1e-3) / 1e12, cublas=g.version, emulation=g.emulation)
    print(json.dumps(rep))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default=None, help="run one kernel case (see run_case)")
    ap.add_argument("--n", type=int, default=1 << 26)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--sweep-out", default=None)
    ap.add_argument("--comm", default="auto", choices=["auto", "torch", "knet"],
                    help="N>1: who issues the NCCL collectives (torch.distributed, or the library's knet_dp_* entry points)")
    ap.add_argument("--shard-update", action="store_true",
                    help="N>1: reduce-scatter, update 1/N of every layer per GPU, all-gather the weights")
    ap.add_argument("--gemm", default="torch", choices=["torch", "native", "emulated"],
                    help="who makes the cuBLAS call of the matrix products: torch.mm; knet_gemm_32_S in plain "
                         "FP32; knet_gemm_32_S with cuBLAS's FP32 emulation on the BF16 tensor cores")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--emulated", action="store_true",
                    help="also run the step with emulated-FP32 matrix products in a child process (opt-in)")
    ap.add_argument("--ref-budget", type=float, default=240.0,
                    help="--impl reference: seconds the CPU steps may take in total")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel leg")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" and not args.sweep else args.warmup
    if args.gemm != "torch" and args.impl == "ours":
        os.environ["KNET_SM100_GEMM"] = args.gemm
        if args.gemm == "emulated":
            # the emulation needs cuBLAS >= 12.9; the toolkit's copy is loaded ahead of the one
            # PyTorch bundles, which only works while torch has not been imported yet
            os.environ.setdefault("KNET_SM100_CUBLAS_DIR", "/usr/local/cuda/lib64")
        import knet_sm100  # noqa: F401
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.sweep:
        run_sweep(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
