#!/usr/bin/env python
"""Benchmark of the Seera training hot path (forward + loss + backward + optimizer) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c3|c4|c5] [--impl reference] [--scaling weak|strong]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Prints ONE JSON line (rank 0).  `value` is whole-job training samples/s with the batches already resident in HBM
(a captured step graph replayed on four rotating device batches); `e2e` is the same through the public Python API
with every batch copied from pinned host memory and every loss read back.  Both are the median over `--repeats`
timed regions of K steps each; the spread is printed beside them.  `roofline` covers the contraction kernels
(Dense / convolution forward, dX, dW, each with its own sub-record) and lists the bandwidth-bound passes with their
algorithmic bytes against the HBM peak; all of it is timed live with CUDA events in a separate profiled pass.
`cpu_baseline` is the reference's own CPU engine on this box's host cores on a bounded sample.

With N > 1 the batch is sharded: every rank trains `batch` samples per step (weak scaling; `--scaling strong` splits
the configuration's batch over the ranks instead), the gradient arena is summed over the ranks by the engine's own
NCCL data plane in buckets that overlap the rest of backward - inside the captured step graph - and the optimizer
divides by the world size.  After the timed steps the ranks' weights are compared (`dp_check`).
`--impl reference` times the reference CPU engine (oracle/_ref, else the C restatement) driven op for op as the
reference's CPU path runs, with the thread layout stated in its line.
"""
import os

# The reference's CPU engine calls a pthread OpenBLAS inside `omp parallel for` loops (engine/src/conv_ops.cpp:109-175):
# with both pools at the core count, cores^2 threads fight.  Pin one level before either library loads (a launcher that
# presets OMP_NUM_THREADS=1 must not change the CPU arm); `cpu_threads` below switches layouts at run time.
_CORES = os.cpu_count() or 1
os.environ["OMP_NUM_THREADS"] = str(_CORES)
os.environ["OPENBLAS_NUM_THREADS"] = "1"

import argparse
import ctypes
import json
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from ml_framework_b200 import workloads as wl  # noqa: E402

METRIC = "train samples/s (fwd+bwd+optimizer)"


def _peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm": p["hbm_gbs"], "tensor_burst": p["bf16_tflops"], "tensor": p["bf16_tflops_sustained"], "src": "measured"}
    except Exception:
        return {"hbm": 6650.0, "tensor_burst": 1590.0, "tensor": 1400.0, "src": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()          # the exact child started above
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        return False

    def summary(self):
        sm, mx, reasons = [], 0, set()
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx = max(mx, float(r[2]))
            except Exception:
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7), ("sw_power_cap", 8)):
                if len(r) > col and r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# reference arm: the reference's CPU engine on the host cores
# ------------------------------------------------------------------------------------------------
def cpu_engine():
    from oracle import ref_engine, cpu_oracle
    E = ref_engine.load()
    if E is not None:
        return E, "reference", "seera_cpp compiled from the reference's engine/src, sgemm: " + ref_engine.sgemm_kind()
    return cpu_oracle, "port", "C restatement of the reference CPU engine (oracle/seera_oracle.c)"


def cpu_threads(omp, blas):
    """Sets the OpenMP and OpenBLAS thread counts of the libraries already loaded in this process."""
    done = []
    try:
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(int(omp))
        done.append("omp=%d" % omp)
    except OSError:
        pass
    try:
        with open("/proc/self/maps") as f:
            libs = sorted({line.split()[-1] for line in f if "openblas" in line.split()[-1]})
        for path in libs:
            if "opencv" not in path:            # the engine links the OpenBLAS inside the opencv wheel; NumPy's own copy is not on this path
                continue
            lib = ctypes.CDLL(path)
            for name in ("openblas_set_num_threads", "openblas_set_num_threads64_"):
                if hasattr(lib, name):
                    getattr(lib, name)(int(blas))
                    done.append("blas=%d" % blas)
                    break
    except OSError:
        pass
    return " ".join(done)


def cpu_time_steps(net, X, Y, steps, warmup):
    for _ in range(warmup):
        net.step(X, Y)
    t0 = time.perf_counter()
    for _ in range(steps):
        net.step(X, Y)
    return (time.perf_counter() - t0) / max(steps, 1)


def cpu_steps(work, sample, steps, warmup):
    """Times training steps of `sample` samples on the CPU engine under both thread layouts (all cores to the OpenMP loops
    with one BLAS thread each, and all cores to BLAS with one OpenMP thread), keeps the faster for the `steps` timed steps.
    Returns (samples/s, ms/step, kind, description)."""
    from oracle.train_oracle import RefNet
    E, kind, how = cpu_engine()
    net = RefNet(work.layers, work.params(0), work.loss, work.opt, E)
    X, Y = work.batch(sample, 0)
    trial = {}
    for name, (omp, blas) in (("omp%d_blas1" % _CORES, (_CORES, 1)), ("omp1_blas%d" % _CORES, (1, _CORES))):
        set_to = cpu_threads(omp, blas)
        trial[name] = (cpu_time_steps(net, X, Y, 2, 1), omp, blas, set_to)
    best = min(trial, key=lambda k: trial[k][0])
    cpu_threads(trial[best][1], trial[best][2])
    dt = cpu_time_steps(net, X, Y, steps, warmup)
    layout = "threads %s (chosen from %s)" % (best, ", ".join("%s %.0f ms/step" % (k, v[0] * 1e3) for k, v in trial.items()))
    return sample / dt, dt * 1e3, kind, how + "; " + layout


CPU_SAMPLE = {"c1": 64, "c2": 512, "c3": 32, "c4": 16}


def run_reference(args, work):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = CPU_SAMPLE[args.workload]
    v, ms, kind, how = cpu_steps(work, sample, args.steps, args.warmup)
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "samples/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": "f32", "data": "synthetic (seeded, shapes and value ranges of the configuration)",
            "config": {"workload": work.name, "per_gpu_batch": work.batch_size, "global_batch": work.batch_size * args.gpus, "optimizer": work.opt["kind"],
                       "step_sample": sample, "note": "each step is a %d-sample slice of the workload" % sample},
            "cpu_baseline": {"value": v, "unit": "samples/s", "cores": _CORES, "kind": kind,
                             "sample": "%d steps of %d samples; %s" % (args.steps, sample, how)},
            "e2e": {"value": v, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def _apply_options(sc, args):
    for item in args.option:
        name, _, value = item.partition("=")
        sc.set_option(name, int(value))


def _median(v):
    return float(np.median(np.asarray(v, np.float64)))


def _traffic_from_profile(workload, precision):
    """DRAM bytes per contraction launch, from the committed ncu launch list of this workload if it carries the line
    `roofline.traffic_bytes_per_launch: <number> (precision <mode>)`; None otherwise (never a typed-in constant)."""
    path = os.path.join(ROOT, "profiles", "bench_%s_launch_list.txt" % workload)
    try:
        with open(path) as f:
            for line in f:
                if line.startswith("roofline.traffic_bytes_per_launch:"):
                    rest = line.split(":", 1)[1].split()
                    if "(precision" in line and precision not in line:
                        return None, None
                    return float(rest[0]), os.path.relpath(path, ROOT)
    except OSError:
        pass
    return None, None


def _dp_step_equals_joined_batch(work, rank, world, buckets, per_rank=16):
    """One sharded step against the single-process step on the joined batch, in exact-fp32 mode: every rank computes the
    gradients of its shard, the engine sums them over the ranks, and the mean is compared with the gradient arena of the same
    model run on all `world * per_rank` samples by this rank alone."""
    from ml_framework_b200 import train, dp, seera_cuda as sc
    X, Y = work.batch(per_rank * world, seed=4242)
    joined = train.Trainer(work, seed=7, precision=(0, 0))
    joined.forward_backward(X, Y)
    joined.model.gather_grads()
    want = joined.model.grads.to_host_f32().astype(np.float64)[:joined.model.n_arena]
    sharded = train.Trainer(work, seed=7, precision=(0, 0))
    dp.attach_nccl(sharded.model, buckets)
    sl = slice(rank * per_rank, (rank + 1) * per_rank)
    sharded.forward_backward(X[sl], Y[sl])
    sharded.model.gather_grads()
    sharded.model._allreduce(sharded.model.grads)
    got = sharded.model.grads.to_host_f32().astype(np.float64)[:sharded.model.n_arena] / world
    den = np.linalg.norm(want)
    return {"sharded_vs_joined_batch_grad_rel_l2": float(np.linalg.norm(got - want) / den) if den > 0 else 0.0,
            "sharded_vs_joined_batch_samples": per_rank * world}


def run_gpu(args, work):
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    from ml_framework_b200 import seera_cuda as sc, seera as S, train, dp
    sc.init(local)
    _apply_options(sc, args)
    prec = tuple(int(v) for v in args.precision.split("/"))
    prec = prec if len(prec) == 2 else (prec[0], prec[0])
    multi = world > 1 or bool(os.environ.get("SEERA_BENCH_FORCE_DP"))     # the variable exercises the collective path on one rank
    if multi:
        dp.init_from_env()
    tr = train.Trainer(work, seed=0, precision=prec)
    buckets = dp.attach_nccl(tr.model, args.buckets, optimizer=None if args.whole_arena_update else tr.opt) if multi else []
    n = work.batch_size if args.scaling == "weak" else max(1, work.batch_size // world)     # per-rank batch
    NB = 4                                                # distinct batches rotated through the step's input buffers
    host = [work.batch(n, seed=100 + 17 * rank + i) for i in range(NB)]
    dev = [(S.Tensor(x, is_leaf=True), S.Tensor(y, is_leaf=True)) for x, y in host]
    X, Y = host[0]
    Xd, Yd = S.Tensor(X.copy(), is_leaf=True), S.Tensor(Y.copy(), is_leaf=True)   # the buffers the captured step reads
    scratch = S.cuten(np.zeros(4, np.float32)) if multi else None

    def barrier():
        sc.stream_synchronize()
        if multi:
            sc.dp_allreduce(scratch.main_ptr, 1, 0)
            sc.stream_synchronize()

    def reduce_max(ms):
        if not multi:
            return ms
        sc.upload_f32(scratch.main_ptr, np.array([ms, 0, 0, 0], np.float32))
        sc.dp_allreduce(scratch.main_ptr, 1, 1)
        return float(scratch.to_host_f32()[0])

    def load_batch(i):                                    # device-to-device: the batch is already resident in HBM
        xb, yb = dev[i % NB]
        sc.cuda_memcopy_devicetodevice(Xd.value.main_ptr, xb.value.main_ptr, xb.value.size)
        sc.cuda_memcopy_devicetodevice(Yd.value.main_ptr, yb.value.main_ptr, yb.value.size)

    # ---- warm-up: eager steps until the memory pool has stopped growing, then capture the step.  With several ranks
    # every rank runs the SAME number of steps (each step holds collectives; NCCL sets its channels up lazily).
    reserved = -1
    for i in range(max(args.warmup, 3) + (9 if multi else 8)):
        load_batch(i)
        tr.step(Xd, Yd)
        sc.stream_synchronize()
        r = sc.pool_bytes_reserved()
        if not multi and i + 1 >= max(args.warmup, 3) and r == reserved:
            break
        reserved = r
    use_graph = not args.no_graph
    eager_ms = None
    if use_graph:
        e0, e1 = sc.event_create(), sc.event_create()
        sc.event_record(e0)
        for i in range(5):
            load_batch(i)
            tr.step(Xd, Yd)
        sc.event_record(e1)
        eager_ms = sc.event_elapsed_ms(e0, e1) / 5
        tr.capture(Xd, Yd)
        step_fn = tr.replay
    else:
        step_fn = lambda: tr.step(Xd, Yd)

    def run_step(i):
        load_batch(i)
        return step_fn()
    for i in range(args.warmup):
        run_step(i)

    # ---- kernel-path throughput: batches resident in HBM; `repeats` timed regions of exactly K steps --------------
    e0, e1 = sc.event_create(), sc.event_create()
    times, launches = [], 0
    with ClockSampler(local) as clk:
        for rep in range(args.repeats):
            barrier()
            l0 = sc.launch_count()
            sc.event_record(e0)
            for i in range(args.steps):
                run_step(i)
            sc.event_record(e1)
            barrier()
            launches = sc.launch_count() - l0
            times.append(reduce_max(sc.event_elapsed_ms(e0, e1)))
        ms = _median(times)
        # keep the device busy for about a second so the 200 ms clock sampler sees it under load; the count is
        # derived from the rank-reduced time, so every rank runs the same number of extra steps
        extra = 0 if args.no_clock_fill else int(min(5000, max(0.0, 1000.0 - sum(times)) / max(ms / args.steps, 1e-3)))
        for i in range(extra):
            run_step(i)
        sc.stream_synchronize()
    value = n * world * args.steps / (ms / 1e3)
    clocks = clk.summary()

    # ---- end to end: a pinned host batch -> device every step, the loss read back every step --------------------
    pinned = []
    for x, y in host:
        hx, hy = sc.host_alloc_pinned(x.nbytes), sc.host_alloc_pinned(y.nbytes)
        ctypes.memmove(hx, x.ctypes.data, x.nbytes)
        ctypes.memmove(hy, y.ctypes.data, y.nbytes)
        pinned.append((hx, hy))

    # Graph mode streams the batches (Trainer.fit_stream: upload of batch i+1 and read-back of loss i-1 on the copy
    # stream while step i runs); eager mode uploads, steps and reads the loss in turn.
    def e2e_run(k):
        if use_graph:
            return tr.fit_stream((pinned[i % NB] for i in range(k)))[-1]
        last = 0.0
        for i in range(k):
            hx, hy = pinned[i % NB]
            sc.upload_from_host_ptr(Xd.value.main_ptr, hx, X.nbytes)
            sc.upload_from_host_ptr(Yd.value.main_ptr, hy, Y.nbytes)
            last = float(step_fn().value.to_host_f32()[0])
        return last
    e2e_run(3)
    e2e_times, last, e2e_launches = [], 0.0, 0
    for rep in range(max(3, args.repeats // 2 + 1)):
        barrier()
        l1 = sc.launch_count()
        sc.event_record(e0)
        last = e2e_run(args.steps)
        sc.event_record(e1)
        barrier()
        e2e_launches = sc.launch_count() - l1
        e2e_times.append(reduce_max(sc.event_elapsed_ms(e0, e1)))
    ms_e2e = _median(e2e_times)
    e2e = n * world * args.steps / (ms_e2e / 1e3)
    if use_graph:
        tr.release_graph()

    # ---- data parallel: the ranks must hold the same weights after all those steps ---------------------------------
    dp_check = None
    if multi:
        dp_check = {"weights_max_abs_diff_across_ranks": dp.replicas_differ_by(tr.model)}
        dp_check.update(_dp_step_equals_joined_batch(work, rank, world, args.buckets))

    # ---- roofline: a separate profiled pass (events around each launch), eager so that every launch is bracketed ----
    roof = None
    peaks = _peaks()
    psteps = min(args.steps, 5)
    sc.profile_enable(1 if rank == 0 else 0)
    for i in range(psteps):                         # every rank steps (collectives), rank 0 records
        load_batch(i)
        # hold the stream for about two steps first: the step's launches then queue up and run back to back, so the
        # events around each launch time the kernel and not the host's gaps between eager launches
        sc.stream_delay(int(min(100000, max(2000, 2000 * ms / args.steps))))
        tr.step(Xd, Yd)
        sc.stream_synchronize()
    kinds = sc.profile_read_kinds()
    table = sc.profile_report()
    sc.profile_enable(0)
    if rank == 0 and sum(k[0] for k in kinds) and sum(k[1] for k in kinds) > 0:
        cnt, pms, pfl = (sum(k[j] for k in kinds) for j in range(3))
        ach = pfl / (pms / 1e3) / 1e12
        traffic, traffic_src = _traffic_from_profile(args.workload, args.precision)
        sub = {}
        for name, (kn, kms, kfl) in zip(("forward", "dX", "dW"), kinds):
            if kn and kms > 0:
                t = kfl / (kms / 1e3) / 1e12
                sub[name] = {"launches_per_step": kn / psteps, "ms_per_step": kms / psteps, "gflop_per_step": kfl / psteps / 1e9,
                             "achieved": t, "frac": t / peaks["tensor"]}
        hbm = []
        for tag, kind, kn, kms, work_bytes in table:
            if kind == 3 and kms > 0:
                g = work_bytes / (kms / 1e3) / 1e9
                hbm.append({"pass": tag, "launches_per_step": kn / psteps, "ms_per_step": kms / psteps,
                            "algorithmic_mb_per_step": work_bytes / psteps / 1e6, "achieved": g, "frac": g / peaks["hbm"]})
        hbm.sort(key=lambda r: -r["ms_per_step"])
        roof = {"bound": "tensor", "achieved": ach, "peak": peaks["tensor"], "unit": "TFLOP/s", "frac": ach / peaks["tensor"],
                "traffic": traffic, "traffic_source": traffic_src, "kernel": "contraction (Dense/Conv forward, dX, dW)",
                "launches_per_step": cnt / psteps, "ms_per_step_in_kernel": pms / psteps, "peak_source": peaks["src"] + " sustained bf16",
                "share_of_step": (pms / psteps) / (ms / args.steps), "by_kind": sub,
                "backward": None, "hbm_bound_passes": {"peak": peaks["hbm"], "unit": "GB/s", "peak_source": peaks["src"], "passes": hbm}}
        bkn, bms, bfl = (kinds[1][j] + kinds[2][j] for j in range(3))
        if bkn and bms > 0:
            t = bfl / (bms / 1e3) / 1e12
            roof["backward"] = {"achieved": t, "frac": t / peaks["tensor"], "ms_per_step": bms / psteps}

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu:
            sample = CPU_SAMPLE[args.workload]
            v, cms, kind, how = cpu_steps(work, sample, {"c3": 40, "c4": 30, "c2": 20}.get(args.workload, 50), 1)   # 10-30 s of CPU work
            cpu = {"value": v, "unit": "samples/s", "cores": _CORES, "kind": kind,
                   "sample": "%d-sample steps, %.0f ms each; %s" % (sample, cms, how)}
        dtype = {"0": "f32", "1": "bf16 (f32 accumulate)", "2": "bf16x3 (f32 accumulate)", "3": "bf16x6 (f32 accumulate)",
                 "4": "fp16x3 split products (two fp16 copies per operand, three products), f32 accumulate",
                 "4/1": "forward fp16x3 split products, backward one bf16 pass; f32 accumulate",
                 "4/5": "forward fp16x3 split products (two fp16 copies, three products), backward one fp16 pass; f32 accumulate",
                 "3/2": "bf16 split products, f32 accumulate (forward 6-term, backward 3-term)"}.get(args.precision, args.precision)
        line = {"metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
                "dtype": dtype, "data": "synthetic (seeded, shapes and value ranges of the configuration)",
                "config": {"workload": work.name, "per_gpu_batch": n, "global_batch": n * world,
                           "parallelism": "dp%d" % world if world > 1 else "single",
                           "optimizer": work.opt["kind"], "precision_mode": args.precision, "distinct_batches": NB,
                           "l2": "activations per step exceed the 126 MB L2; no explicit flush" if args.workload in ("c2", "c3", "c4")
                                 else "working set fits L2 (latency-bound configuration)"},
                "repeats": {"n": len(times), "ms_per_step_median": ms / args.steps, "ms_per_step_min": min(times) / args.steps,
                            "ms_per_step_max": max(times) / args.steps},
                "clocks": clocks,
                "e2e": {"value": e2e, "unit": "samples/s", "h2d_bytes_per_step": int(X.nbytes + Y.nbytes) * world,
                        "d2h_bytes_per_step": 4 * world, "ms_per_step": ms_e2e / args.steps,
                        "ms_per_step_min": min(e2e_times) / args.steps, "ms_per_step_max": max(e2e_times) / args.steps,
                        "repeats": len(e2e_times)},
                "gpu_launches": int(e2e_launches), "launches_per_step": launches / args.steps, "final_loss": last,
                "step_mode": ("eager launches" if not use_graph else "CUDA graph replay of the captured step") +
                             (", gradient buckets summed by NCCL on the engine's communication stream inside the step, overlapping "
                              "the rest of backward (%d buckets)%s" % (len(buckets), "" if args.whole_arena_update else
                                                                       ", each bucket's optimizer update enqueued behind its sum")
                              if multi else ""),
                "eager_ms_per_step": eager_ms,
                "algorithmic_gflop_per_step": work.flops_per_sample() * n * world / 1e9,
                "dp_check": dp_check, "roofline": roof, "cpu_baseline": cpu}
        print(json.dumps(line), flush=True)
    if multi:
        barrier()
        dp.finalize()


def run_c5(args):
    """Conv2D-backward microbenchmark (configuration 5): dX and dW of a 3x3 s1 p1 convolution with C = K, bf16
    operands (precision mode 1), operands resident in HBM, timed with CUDA events; TFLOP/s against the measured
    bf16 peak.  One JSON line with the per-shape table; `value` is the geometric mean over the shapes run."""
    from ml_framework_b200 import seera_cuda as sc
    from ml_framework_b200.cuTen import cuten
    sc.init(int(os.environ.get("LOCAL_RANK", "0")))
    _apply_options(sc, args)
    mode = int(args.precision or "1")
    sc.set_precision(mode)
    peaks = _peaks()
    shapes = [tuple(int(v) for v in args.c5_shape.split(","))] if args.c5_shape else wl.C5_SHAPES
    nb = args.c5_batch
    rows, l0 = [], sc.launch_count()
    for ck, hw in shapes:
        X, W, dY = wl.c5_conv_bwd(ck, hw, n=nb)
        x, w, dy = cuten(X), cuten(W), cuten(dY)
        dx, dw = cuten(np.zeros_like(X)), cuten(np.zeros_like(W))
        fl = 2.0 * nb * hw * hw * ck * ck * 9
        res = {"C=K": ck, "H=W": hw, "N": nb, "gflop_each": fl / 1e9}
        for name, pdx, pdw in (("dX", dx.main_ptr, 0), ("dW", 0, dw.main_ptr), ("both", dx.main_ptr, dw.main_ptr)):
            call = lambda: sc.cuda_conv2d_bwd(w.main_ptr, x.main_ptr, dy.main_ptr, pdx, pdw, nb, ck, hw, hw, ck, 3, 3, 1, 1, 1, 1)
            for _ in range(max(args.warmup, 3)):
                call()
            sc.stream_synchronize()
            e0, e1 = sc.event_create(), sc.event_create()
            sc.event_record(e0)
            for _ in range(args.steps):
                call()
            sc.event_record(e1)
            ms = sc.event_elapsed_ms(e0, e1) / args.steps
            sc.profile_enable(1)
            for _ in range(args.steps):
                call()
            sc.stream_synchronize()
            cnt, kms, kfl = sc.profile_read()
            sc.profile_enable(0)
            nfl = fl * (2 if name == "both" else 1)
            res[name] = {"ms_call": ms, "tflops_call": nfl / ms / 1e9, "ms_kernel": kms / args.steps,
                         "tflops_kernel": kfl / (kms / 1e3) / 1e12 if kms > 0 else None}
        rows.append(res)
    assert sc.tc_device_status() == 0
    gm = float(np.exp(np.mean([np.log(r["both"]["tflops_call"]) for r in rows])))
    best = max(r["both"]["tflops_kernel"] or 0 for r in rows)
    print(json.dumps({"metric": "Conv2D backward (dX + dW) TFLOP/s, call including operand conversion", "value": gm, "unit": "TFLOP/s",
                      "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "vs_baseline": None,
                      "dtype": {1: "bf16 (f32 accumulate)", 2: "bf16x3", 3: "bf16x6", 0: "f32"}[mode], "data": "synthetic (seeded)",
                      "config": {"workload": "C5 Conv2D backward sweep 3x3 s1 p1, N=%d" % nb, "shapes": rows},
                      "roofline": {"bound": "tensor", "achieved": best, "peak": peaks["tensor"], "unit": "TFLOP/s",
                                   "frac": best / peaks["tensor"], "traffic": None, "kernel": "tma_gemm_kernel (best shape, kernel only)"},
                      "gpu_launches": int(sc.launch_count() - l0)}), flush=True)


def run_adjacent(args):
    """The device passes of the rows next to the training step - BatchNorm forward / backward, Concatenate forward / backward,
    one-hot labels - each timed alone with CUDA events on operands resident in HBM: algorithmic bytes / time against the
    measured HBM peak, and the same call on the CPU engine (a bounded sample of the rows) beside it.  One JSON line."""
    import time
    from ml_framework_b200 import seera_cuda as sc
    from oracle import cpu_oracle as co
    sc.init(int(os.environ.get("LOCAL_RANK", "0")))
    _apply_options(sc, args)
    peaks = _peaks()
    rs = np.random.RandomState(7)
    l0 = sc.launch_count()

    def dev(a):
        return sc.to_device_f32(np.ascontiguousarray(a, np.float32).ravel())

    def timed(call):
        for _ in range(max(args.warmup, 3)):
            call()
        sc.stream_synchronize()
        e0, e1 = sc.event_create(), sc.event_create()
        sc.event_record(e0)
        for _ in range(args.steps):
            call()
        sc.event_record(e1)
        ms = sc.event_elapsed_ms(e0, e1) / args.steps
        sc.event_destroy(e0), sc.event_destroy(e1)
        return ms

    def cpu_timed(call, reps=3):
        call()
        t0 = time.perf_counter()
        for _ in range(reps):
            call()
        return (time.perf_counter() - t0) / reps * 1e3

    passes = []

    def add(name, shape, nbytes, ms, cpu_ms, cpu_bytes, note):
        g = nbytes / (ms / 1e3) / 1e9
        passes.append({"pass": name, "shape": shape, "algorithmic_mb": nbytes / 1e6, "ms": ms, "achieved": g, "frac": g / peaks["hbm"],
                       "cpu_gbs": cpu_bytes / (cpu_ms / 1e3) / 1e9, "cpu_sample": note})

    # BatchNorm2d (512, 64, 32, 32) and BatchNorm1d (4096, 1024): read x + write y; backward read dy, x + write dx
    for tag, (N, C, S) in (("batchnorm2d", (512, 64, 1024)), ("batchnorm1d", (4096, 1024, 1))):
        x = rs.standard_normal((N, C, S)).astype(np.float32)
        gam, bet = rs.uniform(0.5, 1.5, C).astype(np.float32), rs.standard_normal(C).astype(np.float32)
        xd, gd, bd, yd, dxd = dev(x), dev(gam), dev(bet), sc.cuda_malloc_f32(x.size), sc.cuda_malloc_f32(x.size)
        rm, rv, mean, si, dg, db = (dev(np.zeros(C)), dev(np.ones(C)), sc.cuda_malloc_f32(C), sc.cuda_malloc_f32(C),
                                    sc.cuda_malloc_f32(C), sc.cuda_malloc_f32(C))
        ms_f = timed(lambda: sc.batchnorm_fwd(xd, gd, bd, rm, rv, yd, mean, si, N, C, S, 0.1, 1e-5, 1))
        ms_b = timed(lambda: sc.batchnorm_bwd(yd, xd, mean, si, gd, dxd, dg, db, N, C, S))
        ns = max(1, N // 16)                                    # CPU: a sixteenth of the rows
        xs = x[:ns].reshape((ns, C, S) if S > 1 else (ns, C))
        r0, r1 = np.zeros(C, np.float32), np.ones(C, np.float32)
        c_f = cpu_timed(lambda: co.batchnorm_forward(xs, gam, bet, r0, r1, 0.1, 1e-5, True))
        _, xh, _, sinv = co.batchnorm_forward(xs, gam, bet, r0, r1, 0.1, 1e-5, True)
        c_b = cpu_timed(lambda: co.batchnorm_backward(xs, xh, sinv, gam))
        add(tag + "_fwd", [N, C, S], 8.0 * x.size, ms_f, c_f, 8.0 * xs.size, "%d of %d rows" % (ns, N))
        add(tag + "_bwd", [N, C, S], 12.0 * x.size, ms_b, c_b, 12.0 * xs.size, "%d of %d rows" % (ns, N))
        for p in (xd, gd, bd, yd, dxd, rm, rv, mean, si, dg, db):
            sc.cuda_free(p)
    # Concatenate two (512, 64*32*32) tensors along axis 1 and split the joined gradient
    N, n1, n2 = 512, 65536, 65536
    a, b = rs.standard_normal((N, n1)).astype(np.float32), rs.standard_normal((N, n2)).astype(np.float32)
    ad, bd, od = dev(a), dev(b), sc.cuda_malloc_f32(N * (n1 + n2))
    ms_f = timed(lambda: sc.concat_fwd(ad, bd, od, N, n1, n2))
    ms_b = timed(lambda: sc.concat_bwd(od, ad, bd, N, n1, n2))
    ns = N // 16
    c_f = cpu_timed(lambda: np.concatenate([a[:ns], b[:ns]], axis=1))
    joined = np.concatenate([a[:ns], b[:ns]], axis=1)
    c_b = cpu_timed(lambda: (np.ascontiguousarray(joined[:, :n1]), np.ascontiguousarray(joined[:, n1:])))
    add("concat_fwd", [N, n1, n2], 8.0 * N * (n1 + n2), ms_f, c_f, 8.0 * ns * (n1 + n2), "%d of %d rows, numpy" % (ns, N))
    add("concat_bwd", [N, n1, n2], 8.0 * N * (n1 + n2), ms_b, c_b, 8.0 * ns * (n1 + n2), "%d of %d rows, numpy" % (ns, N))
    for p in (ad, bd, od):
        sc.cuda_free(p)
    # one-hot rows from integer labels
    n, classes = 1 << 20, 10
    labels = rs.randint(0, classes, n).astype(np.int32)
    ld, oh = sc.to_device_i32(labels), sc.cuda_malloc_f32(n * classes)
    ms_o = timed(lambda: sc.onehot_f32(ld, oh, n, classes))
    c_o = cpu_timed(lambda: np.eye(classes, dtype=np.float32)[labels[: n // 16]])
    add("onehot", [n, classes], 4.0 * n * (1 + classes), ms_o, c_o, 4.0 * (n // 16) * (1 + classes), "%d of %d labels, numpy" % (n // 16, n))
    sc.cuda_free(ld), sc.cuda_free(oh)

    gm = float(np.exp(np.mean([np.log(p["achieved"]) for p in passes])))
    top = max(passes, key=lambda p: p["ms"])
    print(json.dumps({"metric": "adjacent device passes (BatchNorm, Concatenate, one-hot): algorithmic GB/s, geometric mean", "value": gm,
                      "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "higher_is_better": True,
                      "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded)",
                      "config": {"workload": "rows next to the training step, each pass timed alone on operands in HBM", "passes": passes,
                                 "l2": "operands of 134-268 MB exceed the 126 MB L2 except batchnorm1d (17 MB) and one-hot (46 MB)"},
                      "roofline": {"bound": "hbm", "achieved": top["achieved"], "peak": peaks["hbm"], "unit": "GB/s", "frac": top["frac"],
                                   "traffic": None, "kernel": top["pass"], "peak_source": peaks["src"]},
                      "gpu_launches": int(sc.launch_count() - l0)}), flush=True)



def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c3", choices=sorted(wl.WORKLOADS) + ["c5", "adjacent"])
    ap.add_argument("--c5-shape", default=None, help="C,HW of one point of the C5 sweep (default: the four diagonal shapes)")
    ap.add_argument("--c5-batch", type=int, default=256)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--precision", default=None,
                    help="0 fp32 CUDA cores | 1 bf16 | 2 bf16x3 | 3 bf16x6 | F/B per phase; default: 1 for c2 (a bf16 configuration), "
                         "3/2 for the fp32 configurations")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE",
                    help="engine option for seera_set_option (repeatable), e.g. tile_n_cap3=128")
    ap.add_argument("--buckets", type=int, default=5, help="data parallel: target number of gradient buckets (all-reduces) per step")
    ap.add_argument("--whole-arena-update", action="store_true",
                    help="data parallel: one optimizer launch over the whole arena after the last sum, instead of each bucket's update "
                         "on the communication stream right behind its sum")
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of --steps steps each; the median is reported")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="N > 1: weak = the configuration's batch on every GPU; strong = that batch split over the GPUs")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--no-clock-fill", action="store_true",
                    help="do not keep the device busy for a second after the timed regions (the clock sampler then sees few samples); "
                         "for runs under a profiler")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel eagerly instead of replaying a captured step")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.workload == "c5":
        if int(os.environ.get("RANK", "0")) == 0:
            run_c5(args)
        return
    if args.workload == "adjacent":
        if int(os.environ.get("RANK", "0")) == 0:
            run_adjacent(args)
        return
    work = wl.WORKLOADS[args.workload]()
    if args.precision is None:
        from ml_framework_b200.train import POLICY          # the policy the parity gates are checked at
        f, b = POLICY[work.precision]
        args.precision = str(f) if f == b else "%d/%d" % (f, b)
    if args.impl == "reference":
        run_reference(args, work)
    else:
        run_gpu(args, work)


if __name__ == "__main__":
    main()
