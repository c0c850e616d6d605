#!/usr/bin/env python
"""Benchmark of the Seera training hot path (forward + loss + backward + optimizer) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c3|c4] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Prints ONE JSON line (rank 0).  `value` is whole-job training samples/s with the batch already
resident in HBM; `e2e` is the same through the public Python API with the batch copied from pinned
host memory every step and the loss read back every step.  `roofline` covers the contraction
kernels (Dense / convolution forward, dX, dW), timed live with CUDA events in a separate profiled
pass; `cpu_baseline` is the reference's own CPU engine on this box's host cores on a bounded sample.

With N > 1 the batch is sharded: every rank trains `batch` samples per step (weak scaling), the
gradient arena is all-reduced with NCCL in buckets that overlap the rest of backward, and the
optimizer divides by the world size.  `--impl reference` times the reference CPU engine
(oracle/_ref, else the C restatement) driven op for op as the reference's CPU path runs.
"""
import argparse
import json
import os
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


def cpu_steps(work, sample, steps, warmup):
    """Times `steps` training steps of `sample` samples on the CPU engine; returns (samples/s, ms/step)."""
    from oracle.train_oracle import RefNet
    E, kind, how = cpu_engine()
    net = RefNet(work.layers, work.params(0), work.loss, work.opt, E)
    X, Y = work.batch(sample, 0)
    for _ in range(warmup):
        net.step(X, Y)
    t0 = time.perf_counter()
    for _ in range(steps):
        net.step(X, Y)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return sample / dt, dt * 1e3, kind, how


CPU_SAMPLE = {"c1": 64, "c2": 512, "c3": 32, "c4": 16}


def run_reference(args, work):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count()
    os.environ.setdefault("OMP_NUM_THREADS", str(cores))
    os.environ.setdefault("OPENBLAS_NUM_THREADS", str(cores))
    sample = CPU_SAMPLE[args.workload]
    v, ms, kind, how = cpu_steps(work, sample, args.steps, args.warmup)
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "samples/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic (seeded, shapes and value ranges of the configuration)",
            "config": {"workload": work.name, "per_gpu_batch": work.batch_size, "global_batch": work.batch_size * args.gpus, "optimizer": work.opt["kind"],
                       "step_sample": sample, "note": "each step is a %d-sample slice of the workload" % sample},
            "cpu_baseline": {"value": v, "unit": "samples/s", "cores": cores, "kind": kind,
                             "sample": "%d steps of %d samples; %s" % (args.steps, sample, how)},
            "e2e": {"value": v, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
class _ArenaView:
    """Exposes a device range to torch (for NCCL) without copying."""

    def __init__(self, ptr, n):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 2}


def setup_data_parallel(model, world, local_rank):
    """Bucketed, overlapped all-reduce of the gradient arena through torch.distributed (NCCL)."""
    import torch
    import torch.distributed as dist
    from ml_framework_b200 import seera_cuda as sc, seera as S
    import datetime
    torch.cuda.set_device(local_rank)
    opts = None
    if os.environ.get("SEERA_NCCL_HIGH_PRIORITY", "1") != "0":
        # the bucket sums run beside persistent kernels that fill every SM: let the collective's blocks go first
        opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=120),
                            pg_options=opts)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    sc.stream_synchronize()                         # uploads enqueued so far ran on the engine's own stream
    sc.set_stream(stream.cuda_stream)               # the engine enqueues on the stream NCCL orders against
    full = torch.as_tensor(_ArenaView(model.grads.main_ptr, model.n_arena), device="cuda")
    from ml_framework_b200 import dp
    model._arena_allreduce = lambda: dist.all_reduce(full, op=dist.ReduceOp.SUM)     # whole arena, stream-ordered
    model._reduce_range = lambda b, e: dist.all_reduce(full[b:e], op=dist.ReduceOp.SUM, async_op=True)
    model._reduce_wait = lambda w: w.wait()
    dp.attach(model, world, reduce_range=model._reduce_range, wait=model._reduce_wait)
    return dist, torch


def _apply_options(sc, args):
    for item in args.option:
        name, _, value = item.partition("=")
        sc.set_option(name, int(value))


def run_gpu(args, work):
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    from ml_framework_b200 import seera_cuda as sc, seera as S, train
    sc.init(local)
    _apply_options(sc, args)
    prec = tuple(int(v) for v in args.precision.split("/"))
    prec = prec if len(prec) == 2 else (prec[0], prec[0])
    tr = train.Trainer(work, seed=0, precision=prec)
    dist = torch = None
    if world > 1 or os.environ.get("SEERA_BENCH_FORCE_DP"):      # the variable exercises the collective path on one rank
        dist, torch = setup_data_parallel(tr.model, world, local)
        # ("--option sm_reserve=R" leaves R SMs to the overlapped all-reduce; measured at 2 GPUs it only costs: 1.122 ms per step
        # with R = 0, 1.157 / 1.170 / 1.185 with R = 4 / 8 / 16)
    n = work.batch_size                                  # per-rank batch: weak scaling
    X, Y = work.batch(n, seed=100 + rank)
    Xd, Yd = S.Tensor(X, is_leaf=True), S.Tensor(Y, is_leaf=True)

    def barrier():
        sc.stream_synchronize()
        if dist is not None:
            dist.barrier()
            sc.stream_synchronize()

    def reduce_max(ms):
        if dist is None:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- warm-up: eager steps until the memory pool has stopped growing, then (single process) capture the step
    # (with several ranks every rank must run the SAME number of steps: each step holds collectives)
    reserved = -1
    for i in range(max(args.warmup, 3) + (17 if dist is not None else 8)):      # NCCL sets its channels up lazily
        tr.step(Xd, Yd)
        sc.stream_synchronize()
        r = sc.pool_bytes_reserved()
        if dist is None and i + 1 >= max(args.warmup, 3) and r == reserved:
            break
        reserved = r
    use_graph = not args.no_graph
    eager_ms = None
    if use_graph and dist is not None:
        from ml_framework_b200 import dp
        loss_t = tr.capture_data_parallel(Xd, Yd, tr.model._arena_allreduce, buckets=dp.plan_buckets(tr.model, args.buckets),
                                          reduce_range=tr.model._reduce_range, wait=tr.model._reduce_wait)
        for _ in range(args.warmup):
            tr.replay_data_parallel()
        run_step = tr.replay_data_parallel
    elif use_graph:
        e0, e1 = sc.event_create(), sc.event_create()
        sc.event_record(e0)
        for _ in range(5):
            tr.step(Xd, Yd)
        sc.event_record(e1)
        eager_ms = sc.event_elapsed_ms(e0, e1) / 5
        loss_t = tr.capture(Xd, Yd)
        for _ in range(args.warmup):
            tr.replay()
        run_step = tr.replay
    else:
        run_step = lambda: tr.step(Xd, Yd)

    # ---- kernel-path throughput: inputs resident in HBM ------------------------------------------
    barrier()
    e0, e1 = sc.event_create(), sc.event_create()
    l0 = sc.launch_count()
    with ClockSampler(local) as clk:
        t_wall = time.perf_counter()
        sc.event_record(e0)
        for _ in range(args.steps):
            loss = run_step()
        sc.event_record(e1)
        barrier()
        ms = reduce_max(sc.event_elapsed_ms(e0, e1))
        # keep the device busy for about a second so the 200 ms clock sampler sees it under load; the count is
        # derived from the rank-reduced time, so every rank runs the same number of extra steps
        extra = int(min(5000, max(0.0, 1000.0 - ms) / max(ms / args.steps, 1e-3)))
        for _ in range(extra):
            run_step()
        sc.stream_synchronize()
    launches = (sc.launch_count() - l0)
    value = n * world * args.steps / (ms / 1e3)
    clocks = clk.summary()
    launches_per_step = None

    # ---- end to end: pinned host batch -> device every step, loss read back every step ---------------
    import ctypes
    hx, hy = sc.host_alloc_pinned(X.nbytes), sc.host_alloc_pinned(Y.nbytes)
    ctypes.memmove(hx, X.ctypes.data, X.nbytes)
    ctypes.memmove(hy, Y.ctypes.data, Y.nbytes)

    # Graph mode streams the batches (Trainer.fit_stream: upload of batch i+1 and read-back of loss i-1 on the copy
    # stream while step i runs); eager mode uploads, steps and reads the loss in turn.
    def e2e_run(k):
        if use_graph:
            return tr.fit_stream(((hx, hy) for _ in range(k)), data_parallel=dist is not None)[-1]
        last = 0.0
        for _ in range(k):
            sc.upload_from_host_ptr(Xd.value.main_ptr, hx, X.nbytes)
            sc.upload_from_host_ptr(Yd.value.main_ptr, hy, Y.nbytes)
            last = float(run_step().value.to_host_f32()[0])
        return last
    e2e_run(3)
    barrier()
    l1 = sc.launch_count()
    sc.event_record(e0)
    last = e2e_run(args.steps)
    sc.event_record(e1)
    barrier()
    launches_per_step = (sc.launch_count() - l1) / args.steps
    ms_e2e = reduce_max(sc.event_elapsed_ms(e0, e1))
    e2e = n * world * args.steps / (ms_e2e / 1e3)
    if use_graph:
        tr.release_graph()

    # ---- roofline of the contraction kernels: a separate profiled pass (events around each launch) -----
    roof = None
    peaks = _peaks()
    sc.profile_enable(1 if rank == 0 else 0)
    for _ in range(min(args.steps, 5)):             # every rank steps (collectives), rank 0 records
        # hold the stream for about two steps first: the step's launches then queue up and run back to back, so the
        # events around each contraction time the kernel and not the host's gaps between eager launches
        sc.stream_delay(int(min(100000, max(2000, 2000 * ms / args.steps))))
        tr.step(Xd, Yd)
        sc.stream_synchronize()
    sc.stream_synchronize()
    cnt, pms, pfl = sc.profile_read()
    sc.profile_enable(0)
    if rank == 0:
        if cnt and pms > 0:
            ach = pfl / (pms / 1e3) / 1e12
            # DRAM bytes per contraction launch from the ncu launch list of this workload (profiles/bench_c3_launch_list.txt:
            # dram__bytes_read.sum + dram__bytes_write.sum of the 17 contraction launches of a C3 step = 620.9 MB)
            traffic = 35.4e6 if (args.workload == "c3" and args.precision == "3/2") else None
            roof = {"bound": "tensor", "achieved": ach, "peak": peaks["tensor"], "unit": "TFLOP/s", "frac": ach / peaks["tensor"],
                    "traffic": traffic, "kernel": "contraction (Dense/Conv fwd, dX, dW)", "launches_per_step": cnt / min(args.steps, 5),
                    "ms_per_step_in_kernel": pms / min(args.steps, 5), "peak_source": peaks["src"] + " sustained bf16",
                    "share_of_step": (pms / min(args.steps, 5)) / (ms / args.steps)}

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu:
            cores = os.cpu_count()
            sample = CPU_SAMPLE[args.workload]
            v, cms, kind, how = cpu_steps(work, sample, {"c3": 8, "c4": 12}.get(args.workload, 10), 1)      # about 10 s of CPU work
            cpu = {"value": v, "unit": "samples/s", "cores": cores, "kind": kind,
                   "sample": "%d-sample steps, %.0f ms each; %s" % (sample, cms, how)}
        line = {"metric": METRIC, "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": {"0": "f32", "1": "bf16 (f32 accumulate)", "2": "bf16x3 (f32 accumulate)", "3": "bf16x6 (f32 accumulate)",
                          "3/2": "bf16 split products, f32 accumulate (forward 6-term, backward 3-term)"}.get(args.precision, args.precision),
                "data": "synthetic (seeded, shapes and value ranges of the configuration)",
                "config": {"workload": work.name, "per_gpu_batch": n, "global_batch": n * world,
                           "parallelism": "dp%d" % world if world > 1 else "single",
                           "optimizer": work.opt["kind"], "precision_mode": args.precision,
                           "l2": "activations per step exceed the 126 MB L2; no explicit flush" if args.workload in ("c2", "c3", "c4")
                                 else "working set fits L2 (latency-bound configuration)"},
                "clocks": clocks,
                "e2e": {"value": e2e, "unit": "samples/s", "h2d_bytes_per_step": int(X.nbytes + Y.nbytes) * world,
                        "d2h_bytes_per_step": 4 * world, "ms_per_step": ms_e2e / args.steps},
                "gpu_launches": int(launches_per_step * args.steps), "launches_per_step": launches_per_step, "final_loss": last,
                "step_mode": ("eager launches, bucketed all-reduce overlapping backward" if not use_graph else
                              "CUDA graphs of forward+backward cut at the gradient buckets, each bucket's NCCL all-reduce overlapping the next graph, fused optimizer"
                              if dist is not None else "CUDA graph replay of the captured step"),
                "eager_ms_per_step": eager_ms,
                "algorithmic_gflop_per_step": work.flops_per_sample() * n * world / 1e9,
                "roofline": roof, "cpu_baseline": cpu}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c3", choices=sorted(wl.WORKLOADS) + ["c5"])
    ap.add_argument("--c5-shape", default=None, help="C,HW of one point of the C5 sweep (default: the four diagonal shapes)")
    ap.add_argument("--c5-batch", type=int, default=256)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--precision", default=None,
                    help="0 fp32 CUDA cores | 1 bf16 | 2 bf16x3 | 3 bf16x6 | F/B per phase; default: 1 for c2 (a bf16 configuration), "
                         "3/2 for the fp32 configurations")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE",
                    help="engine option for seera_set_option (repeatable), e.g. tile_n_cap3=128")
    ap.add_argument("--buckets", type=int, default=4, help="data parallel: gradient buckets (all-reduces) per step")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel eagerly instead of replaying a captured step")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.workload == "c5":
        if int(os.environ.get("RANK", "0")) == 0:
            run_c5(args)
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
