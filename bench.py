#!/usr/bin/env python
"""Benchmark of the one hot path: deformable convolution forward + backward (dX, dOffset, dW).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config 1|2|3|4] [--precision auto|exact|bf16]
    python bench.py --impl reference ...      # the reference algorithm on the host cores (CPU oracle port)

One "step" is one forward + backward-data + backward-weight pass of the configured workload over a batch of
seeded synthetic tensors.  Prints ONE JSON line (rank 0).  Under torchrun every rank runs the same per-GPU
batch (weak scaling) and the weight gradient -- the only quantity that sums over the batch -- is all-reduced
with NCCL inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _host_threads() -> int:
    """Host threads for the CPU legs (the reference arm and cpu_baseline): every core this process may run on.
    torchrun exports OMP_NUM_THREADS=1 to its workers, which would silently turn a "16 cores" baseline into a
    one-thread run; the count is therefore set explicitly, before numpy / torch load their OpenMP and BLAS
    runtimes, on the one rank that runs a CPU leg (rank 0; with several ranks only the reference arm has one)."""
    return len(os.sched_getaffinity(0))


if int(os.environ.get("RANK", "0")) == 0 and ("reference" in sys.argv or int(os.environ.get("WORLD_SIZE", "1")) == 1):
    for _v in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[_v] = str(_host_threads())

import torch  # noqa: E402

from deform_conv3d_pytorch_op_b200 import workloads  # noqa: E402

METRIC = "deform_conv_fwd_bwd_tflops"
UNIT = "TFLOP/s"

# (config, pass) -> (dram__bytes_read.sum + dram__bytes_write.sum of the pass's main kernel in one ncu capture,
# output positions of the captured launch).  Figures and commands: profiles/tc_bwd2d_kernel_cfg2.md and
# profiles/tc_forward_wgrad_kernels_cfg2_batch16.md (batch 16: a working set larger than L2).
NCU_DRAM_BYTES = {
    (2, "forward"): (41422336 + 3489280, 50176),
    (2, "backward_data"): (96318976 + 25689344, 50176),
    (2, "backward_weight"): (68251392 + 1722112, 50176),
}


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi sampling of SM clocks and throttle reasons during the timed region (read-only)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [a.strip() for a in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for nm, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_port_run(wl, n_samples: int, repeats: int = 1):
    """Times the CPU oracle (the reference algorithm restated) on `n_samples` samples of the workload."""
    import numpy as np
    from oracle import oracle as orc
    from deform_conv3d_pytorch_op_b200 import workloads
    x, w, off, dy = [t.numpy() for t in workloads.make_inputs(wl, n=n_samples)]
    p = orc.Problem(wl.ndim, n_samples, wl.C, wl.O, wl.in_size, wl.kernel, wl.stride, wl.pad, wl.dil, wl.G, wl.cpg)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        orc.fwd_bwd(p, x, off, w, dy)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best


def _omp_threads() -> int:
    """Threads the OpenMP runtime of the oracle library will actually use."""
    import ctypes
    for name in ("libgomp.so.1", "libomp.so", "libiomp5.so"):
        try:
            return int(ctypes.CDLL(name).omp_get_max_threads())
        except OSError:
            continue
    return int(os.environ.get("OMP_NUM_THREADS", "1"))


def our_config(wl, prec: str, world: int, flush: bool, working_set: float) -> dict:
    """The `config` object of the JSON line; both arms print the same one for the same workload."""
    return {"workload": wl.name, "per_gpu_batch": wl.N, "precision": prec, "io_dtype": "f32",
            "l2": "flushed between steps" if flush else "working set %.0f MB > 126 MB L2" % (working_set / 1e6),
            "parallelism": "batch-sharded x%d, dW all-reduce" % world if world > 1 else "single GPU"}


def workload_l2(wl):
    """(working set in bytes, whether the bench flushes L2 between steps)."""
    x = wl.N * wl.C * wl.iv
    off = wl.N * wl.offset_channels * wl.ov
    dy = wl.N * wl.O * wl.ov
    ws = (x + off + dy) * 4 * 2 + x * 4
    return ws, ws < 512 * 1024 * 1024


def reference_kernels_run(wl, dev):
    """The reference's own device kernels (its lib/*_kernel.cu compiled unmodified for sm_100a into oracle/_ref)
    driven by the reference's host loop (serial over the batch, one GEMM per group through torch.mm where the
    reference calls cuBLAS SGEMM): forward + both backward passes of the whole batch on this GPU.  Part of the
    baseline leg, outside every timed region of the operator.  None where oracle/_ref is not built or the
    reference has no fp32 package for the shape (2-D with dilation or groups)."""
    from oracle import ref_gpu, oracle as orc
    if not ref_gpu.available():
        return None
    if wl.ndim == 2 and (tuple(wl.dil) != (1, 1) or wl.G != 1):
        return None
    from deform_conv3d_pytorch_op_b200 import workloads
    variant = "deform3d" if wl.ndim == 3 else "deform2d"
    p = orc.Problem(wl.ndim, wl.N, wl.C, wl.O, wl.in_size, wl.kernel, wl.stride, wl.pad, wl.dil, wl.G, wl.cpg)
    x, w, off, dy = [t.to(dev) for t in workloads.make_inputs(wl)]
    op = ref_gpu.RefOp(variant, p)

    def once():
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        op.forward(x, off, w)
        op.backward_data(x, off, w, dy)
        op.backward_weight(x, off, dy)
        torch.cuda.synchronize()
        return time.perf_counter() - t0
    once()
    dt = min(once(), once())
    return {"value": wl.flops() / dt / 1e12, "unit": UNIT, "ms_per_step": dt * 1e3,
            "what": "reference %s kernels (unmodified, sm_100a build) + torch.mm fp32 GEMMs, per-sample host loop "
                    "with a device synchronisation around every kernel launch, whole batch" % variant}


def run_reference(args, wl):
    """--impl reference: the reference algorithm on the host cores.  The reference ships CUDA kernels only
    and no CPU path, so this is the oracle port (kind "port"), with all host threads (OpenMP + BLAS).  One step
    is the whole per-GPU batch unless --ref-samples bounds it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = _host_threads()
    torch.set_num_threads(cores)
    n = wl.N if args.ref_samples <= 0 else max(1, min(wl.N, args.ref_samples))
    from oracle import oracle as orc
    orc.build()
    for _ in range(args.warmup):
        cpu_port_run(wl, n)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_port_run(wl, n)
    dt = (time.perf_counter() - t0) / args.steps
    val = wl.flops(n) / dt / 1e12
    sample = "%d of %d samples per step, forward + backward (dX, dOffset, dW), fp32" % (n, wl.N)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    ws, flush = workload_l2(wl)
    prec = "exact" if (args.precision == "exact" or (args.precision == "auto" and args.config == 1)) else "bf16"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": our_config(wl, prec, world, flush, ws),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "omp_threads": _omp_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def model_bench(args, world, rank, local, dev, steps, warm):
    """Config 5: SGD training steps of the R3D-18-style network with deformable stages 3-4 on N = 64 clips of
    3x16x112x112, the batch split over the ranks (strong scaling), parameter gradients all-reduced over NCCL in flat
    buckets.  Returns the fields of the `model` object (rank 0; None elsewhere).  The process group is the
    caller's."""
    from deform_conv3d_pytorch_op_b200 import r3d, _lib
    if world > 1:
        import torch.distributed as dist
    total = args.model_batch if args.model_batch > 0 else 64
    g = torch.Generator().manual_seed(0)
    labels_all = torch.randint(0, 400, (total,), generator=g)
    per = total // world
    gs = torch.Generator().manual_seed(100 + rank)
    x_h = torch.randn((per, 3, 16, 112, 112), generator=gs).pin_memory()
    y_h = labels_all[rank * per:(rank + 1) * per].contiguous().pin_memory()
    torch.manual_seed(0)
    prec = "auto" if args.precision == "auto" else args.precision
    model = r3d.R3D18Deform(400, 64, precision=prec).to(dev)
    torch.backends.cudnn.benchmark = True
    chl = not args.no_channels_last
    if chl:
        # cuDNN's convolutions and batch-norms run natively in channels-last, and the deformable operator takes and
        # returns channels-last activations as they are (only the offset tensors are converted)
        model = model.to(memory_format=torch.channels_last_3d)
    use_graph = not args.no_graph
    use_ddp = world > 1 and not args.no_ddp and not use_graph     # the graphed step all-reduces flat buckets itself
    net = model
    if use_ddp:
        net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local], gradient_as_bucket_view=True)
    opt = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9, fused=True)
    x_d, y_d = x_h.to(dev), y_h.to(dev)
    if chl:
        x_d = x_d.contiguous(memory_format=torch.channels_last_3d)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def rank_max(v):
        if world > 1:
            t = torch.tensor([v], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return v

    ev = lambda: torch.cuda.Event(enable_timing=True)
    graphed = r3d.GraphedTrainStep(model, opt, x_d, y_d, world) if use_graph else None

    def one_step(xd=None, yd=None, timed=False):
        if graphed is not None:
            return graphed(xd, yd, timed=timed)
        return r3d.train_step(net, opt, x_d if xd is None else xd, y_d if yd is None else yd, world, ddp=use_ddp)

    for _ in range(warm):
        one_step()
    sync_all()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    a, b = ev(), ev()
    sync_all()
    a.record()
    for _ in range(steps):
        one_step()
    b.record()
    sync_all()
    clocks = sampler.stop() if rank == 0 else None
    ms = rank_max(a.elapsed_time(b) / steps)
    # phases, in a separate short loop (the events between the phases do not serialise anything that was not
    # already serial: replay, all-reduce and optimizer step are stream-ordered)
    phases = None
    if graphed is not None:
        acc = [0.0, 0.0, 0.0]
        n_ph = max(3, min(steps, 10))
        for _ in range(n_ph):
            one_step(timed=True)
            torch.cuda.synchronize()
            e = graphed.phase_events
            for k in range(3):
                acc[k] += e[k].elapsed_time(e[k + 1])
        phases = {"compute_graph_replay": rank_max(acc[0] / n_ph), "grad_all_reduce": rank_max(acc[1] / n_ph),
                  "optimizer": rank_max(acc[2] / n_ph)}
    _lib.check(_lib.lib().dcn_check_status(_lib.current_stream(dev)), "device status after the timed region")

    # end to end: the shard comes from pinned host memory every step and the loss goes back to the host
    e2e = None
    if not args.no_e2e:
        def e2e_step():
            if graphed is not None:
                return float(one_step(x_h, y_h))          # pinned host -> static device buffers -> replay
            xd = x_h.to(dev, non_blocking=True)
            yd = y_h.to(dev, non_blocking=True)
            return float(one_step(xd, yd))
        for _ in range(2):
            e2e_step()
        sync_all()
        n_e2e = max(3, min(steps, 10))
        a.record()
        for _ in range(n_e2e):
            e2e_step()
        b.record()
        sync_all()
        e_ms = rank_max(a.elapsed_time(b) / n_e2e)
        e2e = {"value": total / (e_ms * 1e-3), "unit": "clips/s", "ms_per_step": e_ms,
               "h2d_bytes_per_step": (x_h.numel() * 4 + y_h.numel() * 8) * world, "d2h_bytes_per_step": 4 * world}
    n_deform = sum(1 for m_ in model.modules() if isinstance(m_, r3d.DeformUnit))
    n_param = sum(p.numel() for p in model.parameters())
    del graphed, model, opt, net, x_d, y_d
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    return {"workload": "cfg5_r3d18_deform_stage3_4", "clips_per_s": total / (ms * 1e-3), "ms_per_step": ms,
            "steps": steps, "warmup": warm, "global_batch": total, "per_gpu_batch": per, "n_gpus": world,
            "scaling": "strong", "phases_ms": phases, "e2e": e2e, "clocks": clocks,
            "clip": [3, 16, 112, 112], "classes": 400, "parameters": n_param, "optimizer": "SGD momentum 0.9, fused",
            "parallelism": ("ddp x%d" % world) if use_ddp else ("flat-bucket all-reduce (mean) x%d" % world if world > 1 else "single GPU"),
            "launch": "CUDA graph replay (forward + backward); all-reduce and optimizer eager" if use_graph else "eager",
            "stock_layers": "channels_last_3d" if chl else "NCDHW", "deformable_layers": n_deform}


def run_model(args):
    """--config 5: the model-level workload alone, as its own JSON line."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the reference ships no model and no CPU path; "
                              "config 5 has no reference arm (operator-level arm: --config 1..4)"}), flush=True)
        return
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU implementation)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    args.model_batch = args.batch if args.batch > 0 else args.model_batch
    warm = max(args.warmup, 3)
    m = model_bench(args, world, rank, local, dev, args.steps, warm)
    if rank == 0:
        line = {
            "metric": "r3d18_deform_train_clips_per_s", "value": m["clips_per_s"], "unit": "clips/s",
            "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": m["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 (deformable layers, fp32 I/O) + tf32/fp32 (cuDNN layers)", "data": "synthetic",
            "config": {"workload": m["workload"], "global_batch": m["global_batch"], "per_gpu_batch": m["per_gpu_batch"],
                       "clip": m["clip"], "classes": 400, "optimizer": m["optimizer"], "parallelism": m["parallelism"],
                       "launch": m["launch"], "stock_layers": m["stock_layers"],
                       "l2": "activations of one step exceed the 126 MB L2"},
            "roofline": None, "cpu_baseline": None, "e2e": m["e2e"], "clocks": m["clocks"], "model": m,
            # per deformable layer and step: 4 forward + 8 fused backward library launches (the other layers are
            # cuDNN / torch)
            "gpu_launches": m["deformable_layers"] * 12 * args.steps,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_small(args, wl):
    """Configuration 1 (1.4 MB of tensors, 57 MFLOP per step): the roofline time is 0.2 us, far below the latency of
    a kernel launch, so the step is measured the way such a layer would run in practice -- replayed from a CUDA
    graph -- and set against the launch floor (a graph of the same number of empty nodes).  L2 hygiene: the graph
    walks 128 independent input sets (180 MB, more than the 126 MB L2), one step each."""
    import deform_conv3d_pytorch_op_b200 as dcn
    from deform_conv3d_pytorch_op_b200 import _lib
    import ctypes
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU implementation)"
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    sets = 128
    x_h, w_h, off_h, dy_h = workloads.make_inputs(wl, seed=0, pin=True)
    xs = [x_h.to(dev) + 0.0 * i for i in range(sets)]
    offs = [off_h.to(dev).clone() for _ in range(sets)]
    dys = [dy_h.to(dev).clone() for _ in range(sets)]
    w = w_h.to(dev)
    op = dcn.Op(xs[0], w, wl.stride, wl.pad, wl.dil, wl.cpg, wl.G, precision=args.precision)
    prec = "bf16" if op.p.precision == _lib.PREC_BF16 else "exact"
    launches_per_step = sum(_lib.lib().dcn_launch_count(ctypes.byref(op.p), ps) for ps in (0, 3))

    def one(i):
        y, fws = op.forward(xs[i], offs[i], w, None, keep_workspace=True)
        return (y,) + tuple(op.backward(xs[i], offs[i], w, dys[i], True, True, True, False, fws)[:3])

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(3):
            one(i)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        keep = [one(i) for i in range(sets)]
    # the launch floor: as many trivial nodes as a step has kernels and zero fills
    zero_fills = 0 if prec == "exact" else 2            # the exact small-problem path zero-fills in a kernel of its own
    tiny = [torch.zeros(1, device=dev) for _ in range(launches_per_step + zero_fills)]
    floor_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(floor_graph):
        for _ in range(sets):
            for t in tiny:
                t.zero_()
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def timed(gr, reps):
        for _ in range(3):
            gr.replay()
        torch.cuda.synchronize()
        a, b = ev(), ev()
        a.record()
        for _ in range(reps):
            gr.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / (reps * sets)
    sampler = ClockSampler(0)
    sampler.start()
    reps = max(1, (args.steps + sets - 1) // sets) * 4
    ms_per_step = timed(graph, reps)
    clocks = sampler.stop()
    floor_ms = timed(floor_graph, reps)
    # the same step launched eagerly through the Python binding (what a caller without a graph sees)
    for i in range(8):
        one(i)
    torch.cuda.synchronize()
    a, b = ev(), ev()
    a.record()
    for i in range(sets):
        one(i)
    b.record()
    torch.cuda.synchronize()
    eager_ms = a.elapsed_time(b) / sets
    _lib.check(_lib.lib().dcn_check_status(_lib.current_stream(dev)), "device status after the timed region")
    value = wl.flops() / (ms_per_step * 1e-3) / 1e12

    # end to end: pinned host tensors in, all results back, through the public autograd Function, one step at a time
    e2e = None
    if not args.no_e2e:
        fn = dcn.ConvOffset3dFunction if wl.ndim == 3 else dcn.ConvOffset2dFunction
        outs_h = None

        def e2e_step():
            nonlocal outs_h
            xd = x_h.to(dev, non_blocking=True).requires_grad_(True)
            od = off_h.to(dev, non_blocking=True).requires_grad_(True)
            wd = w_h.to(dev, non_blocking=True).requires_grad_(True)
            dyd = dy_h.to(dev, non_blocking=True)
            yd = fn.apply(xd, od, wd, None, wl.stride, wl.pad, wl.dil, wl.cpg, wl.G, prec)
            yd.backward(dyd)
            res = (yd.detach(), xd.grad, od.grad, wd.grad)
            if outs_h is None:
                outs_h = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in res]
            for h, t in zip(outs_h, res):
                h.copy_(t, non_blocking=True)
        for _ in range(3):
            e2e_step()
        torch.cuda.synchronize()
        n_e2e = 50
        a.record()
        for _ in range(n_e2e):
            e2e_step()
        b.record()
        torch.cuda.synchronize()
        e_ms = a.elapsed_time(b) / n_e2e
        e2e = {"value": wl.flops() / (e_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e_ms,
               "h2d_bytes_per_step": sum(t.numel() * 4 for t in (x_h, off_h, w_h, dy_h)),
               "d2h_bytes_per_step": sum(t.numel() * 4 for t in outs_h)}
    peaks = _peaks()
    fwd_b, bwd_b = wl.bytes_alg()
    t_roof = max(wl.flops() / (peaks["bf16_tflops"] * 1e12), (fwd_b + bwd_b) / (peaks["hbm_gbs"] * 1e9))
    ach = (fwd_b + bwd_b) / (ms_per_step * 1e-3) / 1e9
    roof = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
            "traffic": None, "peak_source": peaks["source"], "kernel": "whole step (%d kernels + %d zero fills)" % (launches_per_step, zero_fills),
            "t_roof_us": t_roof * 1e6, "launch_floor_us": floor_ms * 1e3,
            "frac_of_launch_floor": floor_ms / ms_per_step, "eager_step_us": eager_ms * 1e3,
            "note": "launch-latency bound: the roofline time is below one kernel launch; the floor is a CUDA graph of "
                    "the same number of empty nodes"}
    cpu = None
    if not args.no_cpu_baseline:
        from oracle import oracle as orc
        orc.build()
        cpu_port_run(wl, wl.N)
        dt = cpu_port_run(wl, wl.N, repeats=5)
        cpu = {"value": wl.flops() / dt / 1e12, "unit": UNIT, "cores": _host_threads(), "omp_threads": _omp_threads(),
               "kind": "port", "seconds": dt,
               "sample": "%d of %d samples, forward + backward (dX, dOffset, dW), fp32 oracle port" % (wl.N, wl.N)}
        cpu["reference_kernels_b200"] = reference_kernels_run(wl, dev)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": reps * sets, "warmup": 3 * sets,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if prec == "bf16" else "f32", "data": "synthetic",
        "config": dict(our_config(wl, prec, 1, False, 0.0), l2="128 input sets (180 MB > 126 MB L2), one per step",
                       launch="CUDA graph replay"),
        "roofline": roof, "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks, "model": None,
        "gpu_launches": launches_per_step * reps * sets,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=2, choices=[1, 2, 3, 4, 5])
    ap.add_argument("--no-ddp", action="store_true", help="config 5: bucketed all-reduce after backward instead of DDP")
    ap.add_argument("--no-graph", action="store_true", help="config 5: launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-channels-last", action="store_true",
                    help="config 5: keep the stock layers in NCDHW instead of channels_last_3d")
    ap.add_argument("--precision", default="auto", choices=["auto", "exact", "bf16"])
    ap.add_argument("--batch", type=int, default=0, help="override the per-GPU batch (0: the configuration's)")
    ap.add_argument("--model-batch", type=int, default=64, help="global batch (clips) of the model-level workload")
    ap.add_argument("--no-model", action="store_true",
                    help="leave the model-level workload (config 5, the `model` object) out of the operator line")
    ap.add_argument("--ref-samples", type=int, default=0,
                    help="samples per step of the --impl reference arm (0: the whole per-GPU batch)")
    ap.add_argument("--cpu-baseline-samples", type=int, default=16)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()

    if args.config == 5:
        run_model(args)
        return

    from deform_conv3d_pytorch_op_b200 import workloads
    wl = workloads.CONFIGS[args.config]
    if args.batch > 0:
        import dataclasses
        wl = dataclasses.replace(wl, N=args.batch)

    if args.impl == "reference":
        run_reference(args, wl)
        return
    if args.config == 1 and int(os.environ.get("WORLD_SIZE", "1")) == 1:
        run_small(args, wl)
        return

    import deform_conv3d_pytorch_op_b200 as dcn
    from deform_conv3d_pytorch_op_b200 import _lib
    import ctypes

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU implementation)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    # every rank draws its own batch (seed = rank): weak scaling, no data-path collective but the dW all-reduce
    x_h, w_h, off_h, dy_h = workloads.make_inputs(wl, seed=rank, pin=True)
    w_h0 = workloads.make_inputs(wl, seed=0, n=1)[1]
    w_h.copy_(w_h0)                                   # the weight is replicated
    x, w, off, dy = [t.to(dev) for t in (x_h, w_h, off_h, dy_h)]

    op = dcn.Op(x, w, wl.stride, wl.pad, wl.dil, wl.cpg, wl.G, precision=args.precision)
    prec = "bf16" if op.p.precision == _lib.PREC_BF16 else "exact"
    launches_per_step = sum(_lib.lib().dcn_launch_count(ctypes.byref(op.p), ps) for ps in (0, 3))

    # L2 hygiene: the working set of configs 2-4 is several times the 126 MB L2; for small ones flush.
    working_set, flush = workload_l2(wl)
    flush_buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev) if flush else None

    ev = lambda: torch.cuda.Event(enable_timing=True)
    pass_ms = {"forward": 0.0, "backward_data": 0.0, "backward_weight": 0.0}

    def step(timed: bool):
        """The measured step: forward, then all gradients through the fused backward entry point (which takes
        over the forward's channels-last input copy), then the dW all-reduce when there are several ranks."""
        if flush:
            flush_buf.zero_()
        y, fws = op.forward(x, off, w, None, keep_workspace=True)
        dx, doff, dw, _ = op.backward(x, off, w, dy, True, True, True, False, fws)
        if world > 1:
            dist.all_reduce(dw)
        return None, (y, dx, doff, dw)

    def breakdown_step():
        """Same work through the three separate entry points, for the per-pass timings of the roofline object."""
        e = [ev() for _ in range(4)]
        e[0].record()
        op.forward(x, off, w, None)
        e[1].record()
        op.backward_data(x, off, w, dy)
        e[2].record()
        op.backward_weight(x, off, dy)
        e[3].record()
        return e

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step(False)
    sync_all()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t_begin, t_end = ev(), ev()
    evs = []
    flush_ms = 0.0
    sync_all()
    t_begin.record()
    for _ in range(args.steps):
        e, _ = step(True)
        evs.append(e)
    t_end.record()
    sync_all()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = t_begin.elapsed_time(t_end)
    n_bd = max(3, min(args.steps, 10))
    for _ in range(2):                      # let the allocator see the separate passes' buffer sizes first
        breakdown_step()
    torch.cuda.synchronize()
    evs = [breakdown_step() for _ in range(n_bd)]
    torch.cuda.synchronize()
    for e in evs:
        pass_ms["forward"] += e[0].elapsed_time(e[1])
        pass_ms["backward_data"] += e[1].elapsed_time(e[2])
        pass_ms["backward_weight"] += e[2].elapsed_time(e[3])
    for k in pass_ms:
        pass_ms[k] /= n_bd
    if flush:
        # the flush memset sits inside the bracket; measure it alone and take it out
        torch.cuda.synchronize()
        a, b = ev(), ev()
        a.record()
        for _ in range(args.steps):
            flush_buf.zero_()
        b.record()
        torch.cuda.synchronize()
        flush_ms = a.elapsed_time(b)
    ms_per_step = (total_ms - flush_ms) / args.steps
    if world > 1:
        t = torch.tensor([ms_per_step], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_per_step = float(t.item())
    st = _lib.lib().dcn_check_status(_lib.current_stream(dev))
    _lib.check(st, "device status after the timed region")
    value = wl.flops() * world / (ms_per_step * 1e-3) / 1e12

    # ---- end to end: pinned host tensors in, results back to the host, through the public autograd API ----
    e2e = None
    if not args.no_e2e:
        fn = dcn.ConvOffset3dFunction if wl.ndim == 3 else dcn.ConvOffset2dFunction
        # Three streams, the way a prefetching loader drives the operator: the inputs of step i+1 cross PCIe while
        # step i computes and the results of step i-1 go back, with two sets of device input buffers.  Every step
        # still copies all of its inputs in and all of its results out inside the timed region.
        hosts = (x_h, off_h, w_h, dy_h)
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        main = torch.cuda.current_stream(dev)
        bufs = [[torch.empty(h.shape, dtype=h.dtype, device=dev) for h in hosts] for _ in range(2)]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_free = [torch.cuda.Event() for _ in range(2)]      # the buffer set's last consumer has finished
        ev_done = torch.cuda.Event()
        outs_h = None

        def copy_in(k):
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_free[k % 2])
                for d, h in zip(bufs[k % 2], hosts):
                    d.copy_(h, non_blocking=True)
                ev_in[k % 2].record(s_in)

        def e2e_run(n):
            nonlocal outs_h
            for e in ev_free:
                e.record(main)
            copy_in(0)
            for i in range(n):
                if i + 1 < n:
                    copy_in(i + 1)
                main.wait_event(ev_in[i % 2])
                xb, ob, wb, dyb = bufs[i % 2]
                xd = xb.detach().requires_grad_(True)
                od = ob.detach().requires_grad_(True)
                wd = wb.detach().requires_grad_(True)
                yd = fn.apply(xd, od, wd, None, wl.stride, wl.pad, wl.dil, wl.cpg, wl.G, prec)
                yd.backward(dyb)
                if world > 1:
                    dist.all_reduce(wd.grad)
                ev_free[i % 2].record(main)
                res = (yd.detach(), xd.grad, od.grad, wd.grad)
                if outs_h is None:
                    outs_h = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in res]
                ev_done.record(main)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done)
                    for h, t in zip(outs_h, res):
                        t.record_stream(s_out)
                        h.copy_(t, non_blocking=True)
            main.wait_stream(s_out)

        n_e2e = max(3, min(args.steps, 10))
        e2e_run(2)
        sync_all()
        a, b = ev(), ev()
        a.record()
        e2e_run(n_e2e)
        b.record()
        sync_all()
        e2e_ms = a.elapsed_time(b) / n_e2e
        if world > 1:
            t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        h2d = sum(t.numel() * t.element_size() for t in (x_h, off_h, w_h, dy_h))
        d2h = sum(t.numel() * t.element_size() for t in outs_h)
        e2e = {"value": wl.flops() * world / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}

    # ---- the same workload as a LAYER (offset-producing convolution + deformable convolution in one library call,
    # the caller pattern of deform3d/test_model.py:18-30): times only, outside the timed region of `value`.  A failure
    # here must not cost the bench line, so it is reported as null.
    layer_obj = None
    if rank == 0 and not args.no_model:
        try:
            g = torch.Generator(device="cpu").manual_seed(1)
            ow = (torch.randn(op.offset_weight_shape(), generator=g) * 0.02).to(dev)
            ob = torch.zeros(op.offset_channels, device=dev)
            yl, offl, wsl = op.layer_forward(x, ow, ob, w, None, keep_workspace=True)

            def _t(fn, reps=10):
                for _ in range(2):
                    fn()
                torch.cuda.synchronize(dev)
                a, b = ev(), ev()
                a.record()
                for _ in range(reps):
                    fn()
                b.record()
                torch.cuda.synchronize(dev)
                return a.elapsed_time(b) / reps
            layer_obj = {
                "forward_ms": _t(lambda: op.layer_forward(x, ow, ob, w, None)),
                "backward_ms": _t(lambda: op.layer_backward(x, offl, ow, w, dy, True, True, True, True, False, wsl)),
                "launches": [int(_lib.lib().dcn_layer_launch_count(ctypes.byref(op.p), ps)) for ps in (0, 3)],
                "offset_channels": int(op.offset_channels), "offset_weight_std": 0.02,
            }
            del yl, offl, wsl, ow, ob
        except Exception as exc:                                  # pragma: no cover
            layer_obj = {"error": str(exc)[:200]}

    # ---- the model-level workload (config 5) of the same metric, on the same ranks, as the `model` object ----
    model_obj = None
    if not args.no_model:
        del x, off, dy, op
        if flush_buf is not None:
            flush_buf = None
        torch.cuda.empty_cache()
        model_obj = model_bench(args, world, rank, local, dev, max(3, min(args.steps, 10)), 3)

    if rank == 0:
        peaks = _peaks()
        dom = max(pass_ms, key=pass_ms.get)
        per_pass_flops = wl.flops() / 3.0
        fwd_b, bwd_b = wl.bytes_alg()
        t_tc = per_pass_flops / (peaks["bf16_tflops"] * 1e12)
        pass_bytes = wl.bytes_per_pass()[dom]
        t_hbm = pass_bytes / (peaks["hbm_gbs"] * 1e9)
        if t_tc >= t_hbm:
            ach = per_pass_flops / (pass_ms[dom] * 1e-3) / 1e12
            roof = {"bound": "tensor", "achieved": ach, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": ach / peaks["bf16_tflops"]}
        else:
            ach = pass_bytes / (pass_ms[dom] * 1e-3) / 1e9
            roof = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": ach / peaks["hbm_gbs"]}
        # second reading of the target: three gather / scatter passes (forward gather, weight-gradient gather,
        # input-gradient scatter) of 2^D fp32 corners per sample at HBM bandwidth
        t_gs = 3.0 * wl.bytes_gather_scatter() / (peaks["hbm_gbs"] * 1e9)
        roof.update({"gather_scatter": {"bytes_per_pass": wl.bytes_gather_scatter(), "passes": 3,
                                        "t_roof_ms": t_gs * 1e3, "frac": t_gs / (ms_per_step * 1e-3)}})
        # DRAM bytes per launch of the dominant pass's main kernel, from one ncu capture (profiles/: the summary
        # named for that kernel gives the capture's command, batch and byte counts), scaled by positions
        traffic = None
        if prec == "bf16" and (args.config, dom) in NCU_DRAM_BYTES:
            cap_bytes, cap_positions = NCU_DRAM_BYTES[(args.config, dom)]
            traffic = cap_bytes * (wl.N * wl.ov) / float(cap_positions)
        roof.update({"kernel": dom, "kernel_ms": pass_ms[dom], "traffic": traffic, "peak_source": peaks["source"],
                     "pass_ms": pass_ms,
                     "whole_step_frac": max(wl.flops() / (peaks["bf16_tflops"] * 1e12),
                                            (fwd_b + bwd_b) / (peaks["hbm_gbs"] * 1e9)) / (ms_per_step * 1e-3)})
        cpu = None
        if not args.no_cpu_baseline and world == 1:       # a CPU leg only at N = 1 (rank 0)
            from oracle import oracle as orc
            orc.build()
            n = max(1, min(wl.N, args.cpu_baseline_samples))
            cpu_port_run(wl, 1)
            dt = cpu_port_run(wl, n)
            cpu = {"value": wl.flops(n) / dt / 1e12, "unit": UNIT, "cores": _host_threads(),
                   "omp_threads": _omp_threads(), "kind": "port", "seconds": dt,
                   "sample": "%d of %d samples, forward + backward (dX, dOffset, dW), fp32 oracle port" % (n, wl.N)}
            torch.cuda.empty_cache()
            cpu["reference_kernels_b200"] = reference_kernels_run(wl, dev)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16" if prec == "bf16" else "f32", "data": "synthetic",
            "config": our_config(wl, prec, world, flush, working_set),
            "roofline": roof, "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks, "model": model_obj, "layer": layer_obj,
            "gpu_launches": launches_per_step * args.steps,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
