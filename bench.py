#!/usr/bin/env python
"""Benchmark of the fused BEV pooling forward (and forward+backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg2]

One "step" is one operator call over one batch of synthetic input of the headline
configuration (cfg2, Z = 8: 6 cameras, 16x44x80 bfloat16 features, 118 depth bins,
200x200 BEV grid, categorical depth, sum pooling).  With N > 1 every rank runs its own
sample(s) of the batch (weak scaling, no collective on the data path).  Rank 0 prints one
JSON line:

  value        BEV cells/s over all ranks, inputs resident in HBM: the K steps queued back to back between one
               pair of CUDA events, every step on its own copy of the inputs and its own output (64 copies
               in rotation, 0.5 GB, so nothing a step touches is in the L2); extra holds the figure with one
               launch between its own events after an L2 flush as well
  e2e          the same through the public Python call with pinned host inputs and a host read-back
               of the result inside the timed region
  roofline     algorithmic HBM bytes / kernel time against the measured copy bandwidth, plus the
               same for the gather traffic against a measured L2-resident read bandwidth
  cpu_baseline the CPU oracle (a port of the reference arithmetic) on the host cores, N = 1 only
  extra        forward+backward time and other context

`--impl reference` times the CPU implementation alone (the reference publishes no CPU build that
can travel; the port in oracle/ is used, all host threads).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from flashbev_b200 import synth  # noqa: E402



def ncu_counters(workload):
    """Counters of the forward kernel taken with ncu (never in a timed run): DRAM bytes and executed warp
    instructions per launch, with the commit and command of the capture.  Kept in a small tracked file so that
    the line printed here says which build they belong to."""
    try:
        with open(os.path.join(ROOT, "profiles", "ncu_counters.json")) as fh:
            return json.load(fh).get("fwd_kernel", {}).get(workload)
    except Exception:
        return None

METRIC = "bev_pool_forward_cells_per_s"
UNIT = "BEV cells/s"


def workload_description(w, B_local, mode):
    return (f"{w.name}: B={B_local}/GPU, {w.N} cams, {w.H}x{w.W}x{w.C} {w.dtype} features, D={w.D}, "
            f"BEV {w.X}x{w.Y}x{w.Z}, {mode} depth, forward")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and clock-event reasons of one GPU through NVML while the benchmark runs."""
    BITS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz, self.ok = [], set(), None, False
        self._stop = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.ok = False
        self.t = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(int(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM)))
                try:
                    r = int(self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    r = int(self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for bit, name in self.BITS.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.01)

    def __enter__(self):
        if self.ok:
            self.t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self.ok:
            self.t.join(timeout=1.0)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


def host_thread_count():
    """Threads for the CPU runs: the cores this process may use.  (torchrun exports OMP_NUM_THREADS=1, which
    would otherwise pin the OpenMP oracle to one thread; the count is passed to it explicitly.)"""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_forward_rate(w, mode, threads, min_seconds, min_reps=2):
    """Times the CPU oracle's forward on the same workload (one sample); returns cells/s and the run's facts."""
    from oracle import oracle as O
    inp = synth.make_inputs(w, mode, batch_slice=(0, 1))
    p = O.Problem(
        feats=inp["image_feats"].float().numpy(), depth=inp["depth_params"].float().numpy(),
        proj=inp["projection_matrices"].numpy(), image_size=w.image_size, roi=w.roi, grid=w.grid,
        mode=O.MODE_CATEGORICAL if mode == "categorical" else O.MODE_LAPLACE, threshold=0.0, d0=w.d0, delta=w.delta)
    O.forward(p, threads=threads)  # warm-up
    times = []
    t_end = time.perf_counter() + min_seconds
    while len(times) < min_reps or time.perf_counter() < t_end:
        t0 = time.perf_counter()
        O.forward(p, threads=threads)
        times.append(time.perf_counter() - t0)
    return times


def reference_cuda_kernel_us(w):
    """Device time of the reference's own forward kernel (flash_bevpool_cuda.cu:6, launched through
    flash_bevpool(), :757) on this box, when a GPU is present and oracle/_ref was built from a reference checkout.
    Float32, parametric laplace depth, mean pooling: the only mode the reference has.  Informational."""
    path = os.path.join(ROOT, "oracle", "_ref", "libflashbev_ref.so")
    if not (os.path.exists(path) and torch.cuda.is_available()):
        return {"available": False, "why": "no GPU or oracle/_ref not built"}
    import numpy as np
    ref = ctypes.CDLL(path)
    vp, i32, f32c = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    ref.flashbev_ref_forward.argtypes = [i32] * 7 + [f32c, f32c] + [vp] * 5 + [i32] * 3 + [f32c] * 6 + [vp]
    dev = torch.device("cuda", 0)
    wp = synth.workload(w.name, dtype="fp32")
    inp = {k: v.to(dev) for k, v in synth.make_inputs(wp, "parametric", batch_slice=(0, 1)).items()}
    roi = [float(v) for v in inp["roi_range"].tolist()]
    vs = [float((np.float32(roi[2 * i + 1]) - np.float32(roi[2 * i])) / np.float32(g)) for i, g in enumerate(wp.grid)]
    out = torch.zeros(1, wp.Y, wp.X, wp.C, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def call():  # launches on the legacy default stream, as the reference does
        rc = ref.flashbev_ref_forward(out.numel(), wp.C, wp.N, 1, 1, 0, 0, 1e-6, 1e-6, inp["depth_params"].data_ptr(),
                                      inp["image_feats"].data_ptr(), inp["projection_matrices"].data_ptr(),
                                      inp["feature_size"].data_ptr(), inp["image_size"].data_ptr(), wp.X, wp.Y, wp.Z,
                                      vs[0], vs[1], vs[2], roi[0], roi[2], roi[4], out.data_ptr())
        if rc:
            raise RuntimeError(f"reference launch failed: {rc}")

    null = torch.cuda.default_stream(dev)
    with torch.cuda.stream(null):
        for _ in range(5):
            call()
        torch.cuda.synchronize()
        times = []
        for _ in range(50):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(null)
            call()
            e.record(null)
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e) * 1e3)
    return {"available": True, "forward_us_median": statistics.median(times), "forward_us_min": min(times),
            "mode": "float32, laplace, mean pooling, optimize_z_precompute=False, L2 flushed between launches"}


def reference_pytorch_cpu(w, threads):
    """The reference's own dense PyTorch path on the host cores (project_coords + sampling_vt_pytorch,
    flashbev/flashbevpool/sampling_vt.py:449-466, 36-123), float32, parametric laplace depth, mean pooling, on the
    same workload with (mean, sigma) taken from the same seeded distribution.  Needs a reference checkout
    (FBEV_REFERENCE, else a directory "reference" beside this repository); reported as absent otherwise.  A second,
    labelled CPU figure: the arm's own value stays the OpenMP port."""
    import types
    root = os.environ.get("FBEV_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
    if not os.path.exists(os.path.join(root, "flashbev", "flashbevpool", "sampling_vt.py")):
        return {"available": False, "why": "no reference checkout on this machine"}
    try:
        for n in ("flashbevpool.flashbevpool_ext", "flashbevpool.sampling_vt_ext", "flashbevpool_ext", "sampling_vt_ext"):
            sys.modules.setdefault(n, types.ModuleType(n))  # the package imports its compiled extensions; unused here
        saved = list(sys.path)
        mine = {k: sys.modules.pop(k) for k in list(sys.modules) if k == "flashbevpool" or k.startswith("flashbevpool.")
                and not k.endswith("_ext")}
        sys.path.insert(0, os.path.join(root, "flashbev"))
        try:
            import flashbevpool.sampling_vt as R
        finally:
            sys.path[:] = saved
            for k in [k for k in sys.modules if k == "flashbevpool" or k.startswith("flashbevpool.")]:
                del sys.modules[k]
            sys.modules.update(mine)
        torch.set_num_threads(threads)
        wp = synth.workload(w.name, dtype="fp32")
        inp = synth.make_inputs(wp, "parametric", batch_slice=(0, 1))
        roi = torch.tensor(wp.roi, dtype=torch.float32).view(3, 2)
        axes = [torch.linspace(float(roi[i, 0]), float(roi[i, 1]), g + 1)[:-1] + (roi[i, 1] - roi[i, 0]) / g / 2.0
                for i, g in enumerate(wp.grid)]
        coords = torch.stack(torch.meshgrid(*axes, indexing="ij"), dim=-1)[None, None].expand(1, wp.N, -1, -1, -1, -1)
        feats = inp["image_feats"].flatten(0, 1).movedim(-1, 1).contiguous()
        depth = inp["depth_params"].flatten(0, 1).movedim(-1, 1).contiguous()

        def run():
            with torch.no_grad():
                uvd = R.project_coords(coords_xyz=coords, projection_matrices=inp["projection_matrices"])
                return R.sampling_vt_pytorch(image_uvd=uvd, features_pv=feats, depths=depth, B=1, N=wp.N,
                                             image_size=wp.image_size, depth_weight_threshold=0.0,
                                             depth_distribution="laplace", epsilon=1e-6)

        run()
        times = []
        for _ in range(3):
            t0 = time.perf_counter()
            run()
            times.append(time.perf_counter() - t0)
        t = statistics.median(times)
        return {"available": True, "ms_per_forward": t * 1e3, "cells_per_s": wp.X * wp.Y / t, "threads": threads,
                "torch": torch.__version__,
                "what": "project_coords + sampling_vt_pytorch of the reference, float32, laplace, mean pooling, one sample"}
    except Exception as exc:  # noqa: BLE001
        return {"available": False, "why": f"{type(exc).__name__}: {str(exc)[:160]}"}


def reference_arm(args, rank):
    """CPU implementation of the path on the host cores (the oracle port, OpenMP over BEV rows)."""
    if rank != 0:
        return
    from oracle import oracle as O
    w = synth.workload(args.workload)
    threads = host_thread_count()
    inp = synth.make_inputs(w, args.mode, batch_slice=(0, 1))
    p = O.Problem(
        feats=inp["image_feats"].float().numpy(), depth=inp["depth_params"].float().numpy(),
        proj=inp["projection_matrices"].numpy(), image_size=w.image_size, roi=w.roi, grid=w.grid,
        mode=O.MODE_CATEGORICAL if args.mode == "categorical" else O.MODE_LAPLACE, threshold=0.0, d0=w.d0,
        delta=w.delta)
    for _ in range(args.warmup):
        O.forward(p, threads=threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.forward(p, threads=threads)
    dt = (time.perf_counter() - t0) / args.steps
    cells = w.X * w.Y
    value = cells / dt
    ref_gpu = reference_cuda_kernel_us(w)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_description(w, 1, args.mode), "l2": "n/a (CPU)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"one whole forward of one sample per step, {args.steps} steps, "
                                   f"float32 oracle, OpenMP over BEV rows; host has {os.cpu_count()} logical CPUs"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "extra": {"reference_cuda_kernel": ref_gpu, "reference_pytorch_cpu": reference_pytorch_cpu(w, threads)},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2")
    ap.add_argument("--mode", default="categorical", choices=["categorical", "parametric"])
    ap.add_argument("--batch-per-gpu", type=int, default=1)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip backward / e2e / L2 probe (for profiler runs)")
    ap.add_argument("--quick", action="store_true", help="skip the extras on other workloads (cfg3, cfg4, cfg5)")
    ap.add_argument("--only-backward", type=int, default=0, metavar="FLAGS",
                    help="profiler helper: launch only fbev_backward with these flags (1 features, 2 depth, 3 both) "
                         "--steps times on the default workload, print the mean device time and exit")
    ap.add_argument("--train-step", action="store_true",
                    help="profiler helper: launch only forward + backward of a training step (forward keeps its lists) "
                         "--steps times on the default workload, print the mean device time and exit")
    ap.add_argument("--tune", default=None, help="tile_x,tile_y,chunks_per_lane,warps,min_blocks (0 = automatic)")
    ap.add_argument("--exp", type=int, default=0, help="experiment bits of fbev_debug.h for every forward launch (profiler runs)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        args.steps = args.steps if args.steps is not None else 20
        args.warmup = args.warmup if args.warmup is not None else 3
        reference_arm(args, rank)
        return
    args.steps = args.steps if args.steps is not None else 500
    args.warmup = max(args.warmup if args.warmup is not None else 20, 3)

    import torch.distributed as dist
    from flashbev_b200 import _lib, flash_bevpool
    from flashbev_b200.flash_bevpool import DepthSpec, forward_with_count, make_problem

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path for the product arm")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    lib = _lib.load()
    if args.tune:
        lib.fbev_set_tuning(*[int(v) for v in args.tune.split(",")])
    if args.exp:
        lib.fbev_set_experiment(args.exp)

    w = synth.workload(args.workload)
    Bl = args.batch_per_gpu
    w_all = synth.workload(args.workload, B=Bl * world)
    inp_cpu = synth.make_inputs(w_all, args.mode, batch_slice=(rank * Bl, (rank + 1) * Bl))
    inp = {k: v.to(device) for k, v in inp_cpu.items()}
    mode_int = 2 if args.mode == "categorical" else 1
    extra_kw = {"depth_bin_range": (w.d0, w.delta)} if args.mode == "categorical" else {}
    spec = DepthSpec(mode_int, **extra_kw)
    prob, keep = make_problem(inp["depth_params"], inp["image_feats"], inp["projection_matrices"],
                              inp["feature_size"], inp["image_size"], inp["roi_range"], inp["grid_size"], spec,
                              1e-6, 0.0)
    out = torch.empty(Bl, w.Y, w.X, w.C, dtype=inp["image_feats"].dtype, device=device)
    stream = torch.cuda.current_stream().cuda_stream
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device)  # larger than the 126 MB L2

    def flush():
        flush_buf.zero_()

    def fwd_raw():
        rc = lib.fbev_forward(ctypes.byref(prob), out.data_ptr(), None, stream)
        if rc:
            raise RuntimeError(_lib.strerror(rc))

    def timed(fn, steps, warmup):
        """Device time of `steps` calls of fn, each bracketed by its own events, L2 flushed before each."""
        for _ in range(warmup):
            flush()
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        for i in range(steps):
            flush()
            starts[i].record()
            fn()
            ends[i].record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = [s.elapsed_time(e) for s, e in zip(starts, ends)]
        return sum(ms) / steps, ms

    if args.train_step:
        go = synth.upstream_grad(w, B=Bl).to(device=device, dtype=inp["image_feats"].dtype)
        g_feats, g_depth = torch.empty_like(keep[0]), torch.empty_like(keep[1])
        nsaved = lib.fbev_saved_state_bytes(ctypes.byref(prob))
        saved = torch.empty(max(nsaved, 16), dtype=torch.uint8, device=device)
        prob.saved_state, prob.saved_state_bytes = saved.data_ptr(), nsaved
        nbytes = lib.fbev_backward_scratch_bytes(ctypes.byref(prob), 3)
        scratch = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=device)

        def train_step():
            rc = lib.fbev_forward(ctypes.byref(prob), out.data_ptr(), None, stream)
            rc = rc or lib.fbev_backward(ctypes.byref(prob), go.data_ptr(), g_feats.data_ptr(), g_depth.data_ptr(),
                                         scratch.data_ptr() if nbytes else None, nbytes, 3, stream)
            if rc:
                raise RuntimeError(_lib.strerror(rc))

        ms, _ = timed(train_step, args.steps, args.warmup)
        if rank == 0:
            print(json.dumps({"train_step_us": ms * 1e3, "workload": workload_description(w, Bl, args.mode)}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    if args.only_backward:
        go = synth.upstream_grad(w, B=Bl).to(device=device, dtype=inp["image_feats"].dtype)
        g_feats, g_depth = torch.empty_like(keep[0]), torch.empty_like(keep[1])
        nbytes = lib.fbev_backward_scratch_bytes(ctypes.byref(prob), args.only_backward)
        scratch = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=device)

        def bwd_only():
            rc = lib.fbev_backward(ctypes.byref(prob), go.data_ptr(), g_feats.data_ptr(), g_depth.data_ptr(),
                                   scratch.data_ptr() if nbytes else None, nbytes, args.only_backward, stream)
            if rc:
                raise RuntimeError(_lib.strerror(rc))

        ms, _ = timed(bwd_only, args.steps, args.warmup)
        if rank == 0:
            print(json.dumps({"only_backward_flags": args.only_backward, "us_per_call": ms * 1e3,
                              "workload": workload_description(w, Bl, args.mode)}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # The timed region: K steps queued back to back between one pair of events.  Every step reads its OWN copy of the
    # inputs and writes its own output; ROTATE copies are used in turn, together far larger than the L2 (126 MB), so no
    # step finds its inputs, or an output written earlier, in the L2.
    ROTATE = 64
    step_bytes = sum(inp[k].numel() * inp[k].element_size() for k in ("image_feats", "depth_params", "projection_matrices")) \
        + out.numel() * out.element_size()
    rot = []
    for i in range(ROTATE):
        ci = {k: (v.clone() if k in ("image_feats", "depth_params", "projection_matrices") else v) for k, v in inp.items()}
        pi, ki = make_problem(ci["depth_params"], ci["image_feats"], ci["projection_matrices"], ci["feature_size"],
                              ci["image_size"], ci["roi_range"], ci["grid_size"], spec, 1e-6, 0.0)
        rot.append((pi, ki, torch.empty_like(out)))

    def timed_rotating(steps, warmup):
        for i in range(warmup):
            pr, _, o = rot[i % ROTATE]
            lib.fbev_forward(ctypes.byref(pr), o.data_ptr(), None, stream)
        flush()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for i in range(steps):
            pr, _, o = rot[(warmup + i) % ROTATE]
            rc = lib.fbev_forward(ctypes.byref(pr), o.data_ptr(), None, stream)
            if rc:
                raise RuntimeError(_lib.strerror(rc))
        e0.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        return s0.elapsed_time(e0) / steps

    with ClockSampler(physical_gpu_index(local_rank)) as clocks:
        ms_fwd = timed_rotating(args.steps, args.warmup)
        ms_flushed, ms_list = timed(fwd_raw, max(50, args.steps // 5), 5)
        extra = {"fwd_us_one_launch_between_events_l2_flushed": ms_flushed * 1e3,
                 "fwd_us_one_launch_between_events_median": statistics.median(ms_list) * 1e3,
                 "fwd_us_one_launch_between_events_min": min(ms_list) * 1e3,
                 "timing_note": ("ms_per_step: the steps queued back to back between one pair of events, every step on its own "
                                 f"copy of the inputs and its own output ({ROTATE} copies, {ROTATE * step_bytes / 1e6:.0f} MB in rotation); "
                                 "the one-launch figures bracket each launch with its own events after a 256 MiB L2 flush and so "
                                 "include the launch and drain of a single kernel")}
        e2e = None
        l2_gbs = None
        if not args.no_extras:
            # forward + backward through the C ABI, upstream gradient and gradient buffers resident
            go = synth.upstream_grad(w, B=Bl).to(device=device, dtype=inp["image_feats"].dtype)
            kw = dict(depth_distribution=mode_int, depth_weight_threshold=0.0, **extra_kw)
            g_feats = torch.empty_like(keep[0])
            g_depth = torch.empty_like(keep[1])
            flags = _lib.BWD_FEATS | _lib.BWD_DEPTH
            nbytes = lib.fbev_backward_scratch_bytes(ctypes.byref(prob), flags)
            scratch = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=device)

            # a training step keeps the forward's lists for the backward (FbevProblem.saved_state), as the autograd
            # wrapper does; the variant without them rebuilds the lists in the backward
            prob_t = type(prob).from_buffer_copy(prob)
            nsaved = lib.fbev_saved_state_bytes(ctypes.byref(prob_t))
            saved = torch.empty(max(nsaved, 16), dtype=torch.uint8, device=device)
            prob_t.saved_state, prob_t.saved_state_bytes = saved.data_ptr(), nsaved

            def make_step(pr):
                def step():
                    rc = lib.fbev_forward(ctypes.byref(pr), out.data_ptr(), None, stream)
                    rc = rc or lib.fbev_backward(ctypes.byref(pr), go.data_ptr(), g_feats.data_ptr(), g_depth.data_ptr(),
                                                 scratch.data_ptr() if nbytes else None, nbytes, flags, stream)
                    if rc:
                        raise RuntimeError(_lib.strerror(rc))
                return step

            def fwd_train():
                rc = lib.fbev_forward(ctypes.byref(prob_t), out.data_ptr(), None, stream)
                if rc:
                    raise RuntimeError(_lib.strerror(rc))

            fwd_bwd = make_step(prob)
            nb = max(10, args.steps // 5)
            ms_fb, _ = timed(fwd_bwd, nb, 5)
            extra["fwd_bwd_us"] = ms_fb * 1e3
            extra["fwd_bwd_note"] = "forward + backward (gradients for features and depth), device time, L2 flushed"
            # the optional variant in which the forward keeps its lists for the backward (FbevProblem.saved_state)
            extra["fwd_bwd_us_lists_saved_by_forward"] = timed(make_step(prob_t), nb, 5)[0] * 1e3
            extra["fwd_us_forward_that_saves_lists"] = timed(fwd_train, nb, 5)[0] * 1e3
            extra["saved_lists_mb"] = nsaved / 2 ** 20

            # the same step through the Python autograd function, by the host's clock (steps issued back to back, one
            # synchronisation): what a training loop without CUDA graphs sees, with autograd's device thread and without
            if Bl == 1:
                leaf = {k: inp[k].detach().clone().requires_grad_(True) for k in ("image_feats", "depth_params")}
                rest = {k: inp[k] for k in ("projection_matrices", "feature_size", "image_size", "roi_range", "grid_size")}

                def autograd_step():
                    leaf["image_feats"].grad = None
                    leaf["depth_params"].grad = None
                    flash_bevpool(**leaf, **rest, **kw).backward(go)

                def host_clock(n):
                    for _ in range(10):
                        autograd_step()
                    torch.cuda.synchronize()
                    t0 = time.perf_counter()
                    for _ in range(n):
                        autograd_step()
                    torch.cuda.synchronize()
                    return (time.perf_counter() - t0) / n * 1e6

                extra["fwd_bwd_us_python_autograd_host_clock"] = host_clock(4 * nb)
                with torch.autograd.set_multithreading_enabled(False):
                    extra["fwd_bwd_us_python_autograd_host_clock_single_thread"] = host_clock(4 * nb)
                del leaf

            # bitwise reproducible gradients (FBEV_BWD_DETERMINISTIC: fixed-point sums, a measuring launch first)
            flags_det = flags | _lib.BWD_DETERMINISTIC
            nbytes_det = lib.fbev_backward_scratch_bytes(ctypes.byref(prob), flags_det)
            scratch_det = torch.empty(max(nbytes_det, 1), dtype=torch.uint8, device=device)

            def fwd_bwd_det():
                rc = lib.fbev_forward(ctypes.byref(prob), out.data_ptr(), None, stream)
                rc = rc or lib.fbev_backward(ctypes.byref(prob), go.data_ptr(), g_feats.data_ptr(), g_depth.data_ptr(),
                                             scratch_det.data_ptr(), nbytes_det, flags_det, stream)
                if rc:
                    raise RuntimeError(_lib.strerror(rc))

            extra["fwd_bwd_us_deterministic"] = timed(fwd_bwd_det, nb, 3)[0] * 1e3
            del scratch_det

            # the same launches replayed from a CUDA graph (what a training loop with static shapes does)
            side = torch.cuda.Stream(device=device)
            with torch.cuda.stream(side):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    cs = torch.cuda.current_stream().cuda_stream
                    rc = lib.fbev_forward(ctypes.byref(prob), out.data_ptr(), None, cs)
                    rc = rc or lib.fbev_backward(ctypes.byref(prob), go.data_ptr(), g_feats.data_ptr(), g_depth.data_ptr(),
                                                 scratch.data_ptr() if nbytes else None, nbytes, flags, cs)
                if rc:
                    raise RuntimeError(_lib.strerror(rc))
            torch.cuda.synchronize()
            ms_g, _ = timed(graph.replay, nb, 5)
            extra["fwd_bwd_us_cuda_graph"] = ms_g * 1e3

            # forward kernel with each experiment switch of fbev_debug.h (kept as a record of what each buys)
            if Bl == 1:
                exp_us = {}
                for bits in (0, 1, 2, 4, 8):
                    lib.fbev_set_experiment(bits)
                    exp_us[str(bits)] = timed(fwd_raw, max(20, args.steps // 5), 5)[0] * 1e3
                lib.fbev_set_experiment(0)
                extra["fwd_us_by_experiment_bits"] = exp_us
                extra["fwd_experiment_bits"] = ("0 none (the shipped kernel), 1 L2 prefetch at start, 2 camera cull per group of "
                                                "cells, 4 second round of units drawn from a counter, 8 gathers served from "
                                                "shared memory (ceiling of any staging scheme; result invalid)")
                if not args.tune:
                    # smaller tiles with three warps per block
                    lib.fbev_set_tuning(6, 3, 0, 3, 0)
                    extra["fwd_us_tiles_6x3_3warps"] = timed(fwd_raw, max(20, args.steps // 5), 5)[0] * 1e3
                    for nw in (2, 8):  # same units and order, other block sizes (1776 / 444 blocks instead of 888)
                        lib.fbev_set_tuning(0, 0, 0, nw, 0)
                        extra[f"fwd_us_{nw}_warps_per_block"] = timed(fwd_raw, max(20, args.steps // 5), 5)[0] * 1e3
                    lib.fbev_set_tuning(0, 0, 0, 0, 3)
                    extra["fwd_us_96_registers_5_blocks"] = timed(fwd_raw, max(20, args.steps // 5), 5)[0] * 1e3
                    lib.fbev_set_tuning(6, 3, 0, 3, 3)
                    extra["fwd_us_tiles_6x3_3warps_96_registers"] = timed(fwd_raw, max(20, args.steps // 5), 5)[0] * 1e3
                    lib.fbev_set_tuning(0, 0, 0, 0, 0)

            # the training shape (cfg3: B=4, float32, 32x88 maps), forward and forward + backward
            if world == 1 and not args.quick:
                w3 = synth.workload("cfg3")
                in3 = {k: v.to(device) for k, v in synth.make_inputs(w3, args.mode).items()}
                prob3, keep3 = make_problem(in3["depth_params"], in3["image_feats"], in3["projection_matrices"],
                                            in3["feature_size"], in3["image_size"], in3["roi_range"], in3["grid_size"],
                                            DepthSpec(mode_int, **extra_kw) if args.mode == "categorical" else DepthSpec(1),
                                            1e-6, 0.0)
                out3 = torch.empty(w3.B, w3.Y, w3.X, w3.C, dtype=torch.float32, device=device)
                go3 = synth.upstream_grad(w3).to(device)
                gf3, gd3 = torch.empty_like(keep3[0]), torch.empty_like(keep3[1])
                prob3i = type(prob3).from_buffer_copy(prob3)   # inference forward: nothing saved
                ns3 = lib.fbev_saved_state_bytes(ctypes.byref(prob3))
                sv3 = torch.empty(max(ns3, 16), dtype=torch.uint8, device=device)
                prob3s = type(prob3).from_buffer_copy(prob3)
                prob3s.saved_state, prob3s.saved_state_bytes = sv3.data_ptr(), ns3
                nb3 = lib.fbev_backward_scratch_bytes(ctypes.byref(prob3), flags)
                sc3 = torch.empty(max(nb3, 1), dtype=torch.uint8, device=device)

                def fwd3():
                    rc = lib.fbev_forward(ctypes.byref(prob3i), out3.data_ptr(), None, stream)
                    if rc:
                        raise RuntimeError(_lib.strerror(rc))

                def fwd_bwd3():
                    rc = lib.fbev_forward(ctypes.byref(prob3), out3.data_ptr(), None, stream)
                    rc = rc or lib.fbev_backward(ctypes.byref(prob3), go3.data_ptr(), gf3.data_ptr(), gd3.data_ptr(),
                                           sc3.data_ptr() if nb3 else None, nb3, flags, stream)
                    if rc:
                        raise RuntimeError(_lib.strerror(rc))

                extra["cfg3_fwd_us"] = timed(fwd3, 20, 5)[0] * 1e3
                extra["cfg3_fwd_bwd_us"] = timed(fwd_bwd3, 20, 5)[0] * 1e3
                extra["cfg3_workload"] = workload_description(w3, w3.B, args.mode) + " + backward (both gradients)"
                def fwd_bwd3_saved():
                    rc = lib.fbev_forward(ctypes.byref(prob3s), out3.data_ptr(), None, stream)
                    rc = rc or lib.fbev_backward(ctypes.byref(prob3s), go3.data_ptr(), gf3.data_ptr(), gd3.data_ptr(),
                                                 sc3.data_ptr() if nb3 else None, nb3, flags, stream)
                    if rc:
                        raise RuntimeError(_lib.strerror(rc))

                extra["cfg3_fwd_bwd_us_lists_saved_by_forward"] = timed(fwd_bwd3_saved, 20, 5)[0] * 1e3
                nb3d = lib.fbev_backward_scratch_bytes(ctypes.byref(prob3), flags | _lib.BWD_DETERMINISTIC)
                sc3d = torch.empty(max(nb3d, 1), dtype=torch.uint8, device=device)

                def fwd_bwd3_det():
                    rc = lib.fbev_forward(ctypes.byref(prob3), out3.data_ptr(), None, stream)
                    rc = rc or lib.fbev_backward(ctypes.byref(prob3), go3.data_ptr(), gf3.data_ptr(), gd3.data_ptr(),
                                                 sc3d.data_ptr(), nb3d, flags | _lib.BWD_DETERMINISTIC, stream)
                    if rc:
                        raise RuntimeError(_lib.strerror(rc))

                extra["cfg3_fwd_bwd_us_deterministic"] = timed(fwd_bwd3_det, 10, 3)[0] * 1e3
                del sc3d
                extra["cfg3_saved_state_mb"] = ns3 / 2 ** 20
                del in3, out3, go3, gf3, gd3, sc3, sv3

            # the reference's own mode on the same shapes (float32, parametric laplace depth, mean pooling), for
            # comparison with the reference CUDA kernel that `--impl reference` times on the same box
            wp = synth.workload(args.workload, dtype="fp32")
            inp_p = {k: v.to(device) for k, v in synth.make_inputs(wp, "parametric", batch_slice=(0, Bl)).items()}
            prob_p, keep_p = make_problem(inp_p["depth_params"], inp_p["image_feats"], inp_p["projection_matrices"],
                                          inp_p["feature_size"], inp_p["image_size"], inp_p["roi_range"],
                                          inp_p["grid_size"], DepthSpec(1), 1e-6, 1e-6)
            out_p = torch.empty(Bl, w.Y, w.X, w.C, dtype=torch.float32, device=device)

            def fwd_param():
                rc = lib.fbev_forward(ctypes.byref(prob_p), out_p.data_ptr(), None, stream)
                if rc:
                    raise RuntimeError(_lib.strerror(rc))

            ms_p, _ = timed(fwd_param, max(10, args.steps // 5), 5)
            extra["fwd_us_reference_mode_fp32_laplace_mean"] = ms_p * 1e3

            # the same shapes on the reference's nuScenes calibration (matrices its create_projection_matrix built from
            # inputs/calib_nuscenes.json, kept in a test fixture): fewer candidates land in a camera than on the synthetic rig
            nus = os.path.join(ROOT, "tests", "golden", "nuscenes_laplace_thr0.npz")
            if Bl == 1 and w.N == 6 and os.path.exists(nus):
                import numpy as np
                proj_n = torch.from_numpy(np.load(nus)["proj"]).to(device)
                if tuple(proj_n.shape) == tuple(inp["projection_matrices"].shape):
                    inp_n = dict(inp, projection_matrices=proj_n)
                    prob_n, keep_n = make_problem(inp_n["depth_params"], inp_n["image_feats"], inp_n["projection_matrices"],
                                                  inp_n["feature_size"], inp_n["image_size"], inp_n["roi_range"],
                                                  inp_n["grid_size"], spec, 1e-6, 0.0)

                    def fwd_nus():
                        rc = lib.fbev_forward(ctypes.byref(prob_n), out.data_ptr(), None, stream)
                        if rc:
                            raise RuntimeError(_lib.strerror(rc))

                    cnt_n = forward_with_count(**{k: inp_n[k] for k in ("image_feats", "depth_params", "projection_matrices",
                                                                         "feature_size", "image_size", "roi_range", "grid_size")},
                                               **kw)[1]
                    acc = int(cnt_n.sum().item())
                    lib.fbev_set_experiment(args.exp)  # the loop over the experiment switches above left it at 0
                    extra["nuscenes_rig"] = {"fwd_us": timed(fwd_nus, max(10, args.steps // 5), 5)[0] * 1e3,
                                             "accepted_samples": acc,
                                             "of_candidates": acc / float(w.X * w.Y * w.N * w.Z),
                                             "note": "cfg2 tensors, projection matrices of the nuScenes calibration record; one launch between its own events, L2 flushed"}

            # back-to-back launches with warm L2 (what a model sees when the features were just produced)
            for _ in range(20):
                fwd_raw()
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(200):
                fwd_raw()
            e.record()
            torch.cuda.synchronize()
            extra["fwd_us_warm_l2_back_to_back"] = s.elapsed_time(e) / 200 * 1e3

            # calibration -> projection matrices: the one-kernel builder beside the chain of torch ops it replaces
            from flashbev_b200.sampling_vt import create_projection_matrix
            eye4 = torch.eye(4, device=device).expand(Bl, w.N, 4, 4).contiguous()
            eye3 = torch.eye(3, device=device).expand(Bl, w.N, 3, 3).contiguous()
            zero3 = torch.zeros(Bl, w.N, 3, device=device)

            def torch_chain():
                k4 = torch.zeros(Bl, w.N, 4, 4, device=device)
                k4[..., 3, 3] = 1.0
                k4[..., :3, :3] = eye3 @ eye3
                k4[..., :3, 2] += zero3
                return (k4 @ torch.linalg.inv(eye4))[:, :, :3, :]

            for name, fn in (("projection_matrices_us", lambda: create_projection_matrix(eye4, None, eye3, eye3, zero3, None)),
                             ("projection_matrices_torch_ops_us", torch_chain)):
                for _ in range(5):
                    fn()
                torch.cuda.synchronize()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                for _ in range(50):
                    fn()
                e.record()
                torch.cuda.synchronize()
                extra[name] = s.elapsed_time(e) / 50 * 1e3

            # end to end: pinned host inputs -> device, operator, result -> pinned host
            host = {k: inp_cpu[k].pin_memory() for k in ("image_feats", "depth_params", "projection_matrices")}
            host_out = torch.empty(out.shape, dtype=out.dtype).pin_memory()
            const = {k: inp[k] for k in ("feature_size", "image_size", "roi_range", "grid_size")}
            h2d = sum(t.numel() * t.element_size() for t in host.values())
            d2h = host_out.numel() * host_out.element_size()

            def e2e_step():
                with torch.no_grad():
                    dev_in = {k: t.to(device, non_blocking=True) for k, t in host.items()}
                    o = flash_bevpool(**dev_in, **const, **kw)
                    host_out.copy_(o, non_blocking=True)

            def e2e_step_direct():  # the kernel stores the result into the page-locked host buffer itself
                with torch.no_grad():
                    dev_in = {k: t.to(device, non_blocking=True) for k, t in host.items()}
                    flash_bevpool(**dev_in, **const, **kw, out=host_out)

            def e2e_step_bands(chunks):  # row bands: the copy of one band overlaps the computation of the next
                def step():
                    with torch.no_grad():
                        dev_in = {k: t.to(device, non_blocking=True) for k, t in host.items()}
                        flash_bevpool(**dev_in, **const, **kw, out=host_out, host_row_chunks=chunks)
                return step

            # the three inputs packed into one page-locked buffer: one host-to-device copy instead of three
            order = ("image_feats", "depth_params", "projection_matrices")
            offs, total = {}, 0
            for k in order:
                offs[k] = total
                total += (host[k].numel() * host[k].element_size() + 255) // 256 * 256
            packed = torch.empty(total, dtype=torch.uint8).pin_memory()
            for k in order:
                n = host[k].numel() * host[k].element_size()
                packed[offs[k]: offs[k] + n] = host[k].view(-1).view(torch.uint8)

            def unpack(dev_buf):
                return {k: dev_buf[offs[k]: offs[k] + host[k].numel() * host[k].element_size()].view(host[k].dtype)
                        .view(host[k].shape) for k in order}

            def e2e_step_packed():
                with torch.no_grad():
                    o = flash_bevpool(**unpack(packed.to(device, non_blocking=True)), **const, **kw)
                    host_out.copy_(o, non_blocking=True)

            def e2e_step_packed_bands():
                with torch.no_grad():
                    flash_bevpool(**unpack(packed.to(device, non_blocking=True)), **const, **kw, out=host_out,
                                  host_row_chunks=4)

            # the same step against include/fbev.h directly, every buffer allocated once (a serving loop in C would look
            # like this): one copy of the packed inputs, fbev_forward_to_host with `bands` bands of rows
            class AbiSlot:
                def __init__(self):
                    self.dev_buf = torch.empty(total, dtype=torch.uint8, device=device)
                    self.staging = torch.empty(out.shape, dtype=out.dtype, device=device)
                    self.host_out = torch.empty(out.shape, dtype=out.dtype).pin_memory()
                    t = unpack(self.dev_buf)
                    self.prob, self.keep = make_problem(t["depth_params"], t["image_feats"], t["projection_matrices"],
                                                        const["feature_size"], const["image_size"], const["roi_range"],
                                                        const["grid_size"], spec, 1e-6, 0.0)

            abi_slots = [AbiSlot(), AbiSlot()]

            def abi_step(slot, bands, cuda_stream):
                slot.dev_buf.copy_(packed, non_blocking=True)  # on torch's current stream, which is cuda_stream
                rc = lib.fbev_forward_to_host(ctypes.byref(slot.prob), slot.staging.data_ptr(), slot.host_out.data_ptr(),
                                              bands, cuda_stream)
                if rc:
                    raise RuntimeError(_lib.strerror(rc))

            ne = max(10, args.steps // 5)
            paths = {"device result + copy": e2e_step, "out=pinned host tensor (kernel stores to it)": e2e_step_direct,
                     "out=pinned host tensor, 4 row bands": e2e_step_bands(4),
                     "out=pinned host tensor, 8 row bands": e2e_step_bands(8),
                     "one packed input copy, device result + copy": e2e_step_packed,
                     "one packed input copy, 4 row bands": e2e_step_packed_bands,
                     "C ABI, buffers allocated once: one packed input copy, fbev_forward_to_host, 2 row bands":
                         lambda: abi_step(abi_slots[0], 2, stream),
                     "C ABI, buffers allocated once: one packed input copy, fbev_forward_to_host, 4 row bands":
                         lambda: abi_step(abi_slots[0], 4, stream)}
            times = {name: timed(fn, ne, 5)[0] for name, fn in paths.items()}
            extra["e2e_us_by_path"] = {name: t * 1e3 for name, t in times.items()}
            extra["e2e_path"] = min(times, key=times.get)
            e2e_ms_max = times[extra["e2e_path"]]
            # what the bus alone takes for this step's bytes: the copies by themselves, page-locked memory
            dev_buf = torch.empty(total, dtype=torch.uint8, device=device)

            def h2d_only():
                dev_buf.copy_(packed, non_blocking=True)

            def d2h_only():
                host_out.copy_(out, non_blocking=True)

            extra["bus_us"] = {"h2d_inputs_alone": timed(h2d_only, ne, 3)[0] * 1e3, "d2h_result_alone": timed(d2h_only, ne, 3)[0] * 1e3}
            extra["bus_us"]["serial_floor_with_kernel"] = (extra["bus_us"]["h2d_inputs_alone"] + extra["bus_us"]["d2h_result_alone"]
                                                           + ms_flushed * 1e3)
            if world > 1:  # every rank copies at the same moment: what the shared host links leave each of them
                tb = torch.tensor([extra["bus_us"]["h2d_inputs_alone"], extra["bus_us"]["d2h_result_alone"]],
                                  dtype=torch.float64, device=device)
                allb = [torch.zeros_like(tb) for _ in range(world)]
                dist.all_gather(allb, tb)
                extra["bus_us"]["h2d_by_rank"] = [round(float(t[0]), 1) for t in allb]
                extra["bus_us"]["d2h_by_rank"] = [round(float(t[1]), 1) for t in allb]
            extra["bus_us"]["note"] = ("one step moves its inputs in, computes, and moves the result out, each depending on the one "
                                       "before: copy times measured alone + the kernel = the floor of a step that overlaps nothing; "
                                       "the row-band path overlaps the kernel with the result copy")
            # the same best path by the host's clock: `ne` calls queued back to back, one synchronisation at the end
            best_fn = paths[extra["e2e_path"]]
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(ne):
                best_fn()
            torch.cuda.synchronize()
            extra["e2e_us_host_clock_pipelined"] = (time.perf_counter() - t0) / ne * 1e6
            extra["e2e_note"] = ("e2e is device time (CUDA events around one call, L2 flushed before it); the host-clock "
                                 "figure queues the calls back to back without a flush and synchronises once")
            # two steps in flight, as a double-buffered serving loop runs them: consecutive steps alternate between two
            # streams and two sets of buffers (C ABI path above), so that one step's result travels out while the next
            # step's inputs travel in and its kernel runs.  Every step still copies its own inputs in and its own result
            # out.  Host clock over all steps.  Not the e2e figure of the JSON line, which stays one step at a time.
            two = [torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)]

            def steps_two_in_flight(n):
                for i in range(n):
                    with torch.cuda.stream(two[i & 1]):
                        abi_step(abi_slots[i & 1], 2, two[i & 1].cuda_stream)

            steps_two_in_flight(6)
            torch.cuda.synchronize()
            n2 = 4 * ne
            t0 = time.perf_counter()
            steps_two_in_flight(n2)
            torch.cuda.synchronize()
            extra["e2e_us_two_steps_in_flight_host_clock"] = (time.perf_counter() - t0) / n2 * 1e6
            ref_out = flash_bevpool(**{k: inp[k] for k in order}, **const, **kw)
            torch.cuda.synchronize()
            if not all(torch.equal(sl.host_out, ref_out.cpu()) for sl in abi_slots):
                raise RuntimeError("C ABI end-to-end path: result differs from the operator's")
            rank_e2e = torch.tensor([times[extra["e2e_path"]]], dtype=torch.float64, device=device)
            if world > 1:
                allr = [torch.zeros_like(rank_e2e) for _ in range(world)]
                dist.all_gather(allr, rank_e2e)
                extra["e2e_us_per_rank"] = [float(t[0]) * 1e3 for t in allr]
                try:
                    extra["rank0_cpu_affinity"] = sorted(os.sched_getaffinity(0))[:4] + ["...", len(os.sched_getaffinity(0))]
                except AttributeError:
                    pass

            # the multi-GPU batch configuration (cfg4): 64 samples with their own rigs, 64 / N per GPU, forward and
            # forward + backward, no collective on the data path
            if not args.quick and 64 % world == 0:
                B4 = 64 // world
                w4 = synth.workload("cfg4")
                in4 = {k: v.to(device) for k, v in synth.make_inputs(w4, "categorical", batch_slice=(rank * B4, (rank + 1) * B4)).items()}
                prob4, keep4 = make_problem(in4["depth_params"], in4["image_feats"], in4["projection_matrices"],
                                            in4["feature_size"], in4["image_size"], in4["roi_range"], in4["grid_size"],
                                            DepthSpec(2, depth_bin_range=(w4.d0, w4.delta)), 1e-6, 0.0)
                out4 = torch.empty(B4, w4.Y, w4.X, w4.C, dtype=keep4[0].dtype, device=device)
                go4 = synth.upstream_grad(w4, B=B4).to(device=device, dtype=keep4[0].dtype)
                gf4, gd4 = torch.empty_like(keep4[0]), torch.empty_like(keep4[1])
                prob4i = type(prob4).from_buffer_copy(prob4)   # inference forward: nothing saved
                nb4 = lib.fbev_backward_scratch_bytes(ctypes.byref(prob4), flags)
                sc4 = torch.empty(max(nb4, 1), dtype=torch.uint8, device=device)

                def fwd4():
                    rc = lib.fbev_forward(ctypes.byref(prob4i), out4.data_ptr(), None, stream)
                    if rc:
                        raise RuntimeError(_lib.strerror(rc))

                def fwd_bwd4():
                    rc = lib.fbev_forward(ctypes.byref(prob4), out4.data_ptr(), None, stream)
                    rc = rc or lib.fbev_backward(ctypes.byref(prob4), go4.data_ptr(), gf4.data_ptr(), gd4.data_ptr(),
                                           sc4.data_ptr() if nb4 else None, nb4, flags, stream)
                    if rc:
                        raise RuntimeError(_lib.strerror(rc))

                t4 = torch.tensor([timed(fwd4, 10, 3)[0], timed(fwd_bwd4, 10, 3)[0]], dtype=torch.float64, device=device)
                if world > 1:
                    dist.all_reduce(t4, op=dist.ReduceOp.MAX)
                extra["cfg4"] = {"workload": f"cfg4: B=64 over {world} GPU(s), {B4} per GPU, per-sample rigs, bf16, categorical",
                                 "fwd_ms": float(t4[0]), "fwd_bwd_ms": float(t4[1]),
                                 "fwd_samples_per_s": 64 / (float(t4[0]) * 1e-3),
                                 "fwd_bwd_samples_per_s": 64 / (float(t4[1]) * 1e-3),
                                 "fwd_cells_per_s": 64 * w4.X * w4.Y / (float(t4[0]) * 1e-3),
                                 "backward_scratch_mb_per_gpu": nb4 / 2 ** 20}
                del in4, out4, go4, gf4, gd4, sc4

            if world > 1:
                # one large sample (cfg5) with its BEV rows split over the ranks: all-gather of the output
                # against the kernel storing its rows into every rank's buffer; one GPU alone beside them
                from flashbev_b200 import sharding
                w5 = synth.workload("cfg5")
                in5 = {k: v.to(device) for k, v in synth.make_inputs(w5, "categorical", batch_slice=(0, 1)).items()}
                kw5 = dict(depth_distribution=2, depth_bin_range=(w5.d0, w5.delta), depth_weight_threshold=0.0)
                go5 = synth.upstream_grad(w5).to(device=device, dtype=in5["image_feats"].dtype)
                y0, y1 = sharding.row_slice(w5.Y, world, rank)
                go5_rows = go5[:, y0:y1].contiguous()
                leaf = {k: in5[k].clone().requires_grad_(True) for k in ("image_feats", "depth_params")}
                rest5 = {k: v for k, v in in5.items() if k not in leaf}

                def train_one_gpu():
                    for t in leaf.values():
                        t.grad = None
                    with torch.enable_grad():
                        flash_bevpool(**leaf, **rest5, **kw5).backward(go5)

                def train_rows_local():  # rows stay sharded; only the input gradients are summed over the ranks
                    for t in leaf.values():
                        t.grad = None
                    with torch.enable_grad():
                        sharding.flash_bevpool_rows_local(**leaf, **rest5, **kw5).backward(go5_rows)
                    sharding.all_reduce_input_grads(*leaf.values())

                def train_rows_gathered():  # whole output on every rank (all-gather) + gradient all-reduce
                    for t in leaf.values():
                        t.grad = None
                    with torch.enable_grad():
                        sharding.flash_bevpool_rows(**leaf, **rest5, **kw5).backward(go5)

                variants = {
                    "rows_split_allgather_us": lambda: sharding.flash_bevpool_rows(**in5, **kw5),
                    "rows_split_peer_stores_us": lambda: sharding.flash_bevpool_rows_p2p(**in5, **kw5),
                    "rows_split_multicast_stores_us": lambda: sharding.flash_bevpool_rows_p2p(**in5, **kw5, multicast=True),
                    "rows_split_kept_sharded_us": lambda: sharding.flash_bevpool_rows_local(**in5, **kw5),
                    "rows_split_one_gpu_us": lambda: flash_bevpool(**in5, **kw5),
                    "rows_split_fwd_bwd_kept_sharded_grad_allreduce_us": train_rows_local,
                    "rows_split_fwd_bwd_allgather_grad_allreduce_us": train_rows_gathered,
                    "rows_split_fwd_bwd_one_gpu_us": train_one_gpu,
                }
                import torch.distributed._symmetric_memory as symm_mem  # noqa: F401
                with torch.no_grad():
                    for name, fn in variants.items():
                        # an extra must not cost the run its headline line: a failure is recorded, on all ranks alike
                        try:
                            fn()
                            failed = 0
                        except Exception as exc:  # noqa: BLE001
                            failed, extra[name + "_error"] = 1, str(exc)[:200]
                        tf = torch.tensor([failed], dtype=torch.int32, device=device)
                        dist.all_reduce(tf, op=dist.ReduceOp.MAX)
                        if int(tf[0]):
                            continue
                        ms_v, _ = timed(fn, 20, 5)
                        tv = torch.tensor([ms_v], dtype=torch.float64, device=device)
                        dist.all_reduce(tv, op=dist.ReduceOp.MAX)
                        extra[name] = float(tv[0]) * 1e3
                extra["rows_split_workload"] = "cfg5, one sample: 512x512x16 grid, 6 cams, C=256"
                try:
                    st5 = sharding._p2p_buffer((1, w5.Y, w5.X, w5.C), in5["image_feats"].dtype, device, None)
                    extra["rows_split_multicast_available"] = bool(getattr(st5["hdls"][0], "multicast_ptr", 0))
                except Exception as exc:  # noqa: BLE001
                    extra["rows_split_multicast_available"] = f"unknown: {str(exc)[:80]}"

            # L2-resident read bandwidth: 32 MiB buffer read 50 times
            buf = torch.empty(32 << 20, dtype=torch.uint8, device=device)
            sink = torch.zeros(1, dtype=torch.int32, device=device)
            lib.fbev_probe_read(buf.data_ptr(), buf.numel(), 5, sink.data_ptr(), stream)
            best = None
            for _ in range(5):
                s.record()
                lib.fbev_probe_read(buf.data_ptr(), buf.numel(), 50, sink.data_ptr(), stream)
                e.record()
                torch.cuda.synchronize()
                t = s.elapsed_time(e)
                best = t if best is None else min(best, t)
            l2_gbs = buf.numel() * 50 / (best * 1e-3) / 1e9
        # accepted samples (exact, from the kernel's per-cell counts) for the gather figure
        _, cnt = forward_with_count(**inp, depth_distribution=mode_int, depth_weight_threshold=0.0, **extra_kw)
        s_valid = int(cnt.sum().item())
    clk = clocks.summary()

    # max over ranks
    t = torch.tensor([ms_fwd, e2e_ms_max if not args.no_extras else 0.0], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_fwd_max, ms_e2e_max = float(t[0]), float(t[1])

    cells_total = Bl * w.X * w.Y * world
    value = cells_total / (ms_fwd_max * 1e-3)
    ncu = ncu_counters(args.workload) if (Bl == 1 and args.mode == "categorical") else None
    hbm_peak, peak_kind = measured_peaks()
    alg_bytes = synth.algorithmic_bytes(w, args.mode, B=Bl)
    achieved = alg_bytes / (ms_fwd * 1e-3) / 1e9
    es = 4 if w.dtype == "fp32" else 2
    gather_bytes = s_valid * (4 * w.C * es + 4 * (1 if args.mode == "categorical" else 2) * es)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_fwd_max, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": w.dtype, "data": "synthetic",
        "config": {"workload": workload_description(w, Bl, args.mode),
                   "l2": f"every step reads its own copy of the inputs and writes its own output, {ROTATE} copies in rotation "
                         f"({ROTATE * step_bytes / 1e6:.0f} MB > 126 MB L2)",
                   "timing": "one pair of CUDA events around the K steps, queued back to back on one stream",
                   "parallelism": f"batch samples sharded over {world} GPU(s), no data-path collective"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                     "frac": achieved / hbm_peak,
                     "traffic": ncu["dram_bytes_per_launch"] if ncu else None, "peak_kind": f"of {peak_kind}",
                     "algorithmic_bytes_per_launch": alg_bytes, "kernel": "fwd_kernel",
                     "note": (f"traffic from an ncu capture of commit {ncu['commit']}: {ncu['command']}" if ncu else
                              "no ncu capture on record for this workload")},
        "roofline_gather": {"bound": "l2", "achieved": gather_bytes / (ms_fwd * 1e-3) / 1e9, "peak": l2_gbs,
                            "unit": "GB/s", "frac": (gather_bytes / (ms_fwd * 1e-3) / 1e9 / l2_gbs) if l2_gbs else None,
                            "algorithmic_bytes_per_launch": gather_bytes, "accepted_samples": s_valid,
                            "peak_kind": "L2-resident 16-byte loads of a 32 MiB buffer, measured in this run"},
        "clocks": clk, "gpu_launches": args.steps, "extra": extra,
    }
    wi = ncu.get("warp_instructions_per_launch") if ncu else None
    if wi and clk.get("sm_mhz"):
        # what actually bounds the kernel: one warp instruction per scheduler and cycle, 4 schedulers on each SM
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        floor_us = wi / (sms * 4) / clk["sm_mhz"]
        line["roofline_issue"] = {"bound": "instruction issue", "warp_instructions_per_launch": wi,
                                  "floor_us": floor_us, "achieved_us": ms_fwd * 1e3, "frac": floor_us / (ms_fwd * 1e3),
                                  "note": f"instructions from the ncu capture of commit {ncu['commit']}, SM clock sampled in this run"}
    if not args.no_extras and "fwd_bwd_us" in extra:
        # backward alone = (forward + backward) - forward, both measured above on the same inputs
        t_bwd = max(extra["fwd_bwd_us"] - ms_flushed * 1e3, 1e-3) * 1e-6  # both with one flushed step between events
        k = 1 if args.mode == "categorical" else 2
        hbm_bwd = synth.algorithmic_bytes(w, args.mode, B=Bl, backward=True)
        gather_bwd = gather_bytes + s_valid * (4 * w.C * es + 4 * k * es)  # + the gradient scatter per accepted sample
        line["roofline_bwd"] = {
            "bound": "l2", "seconds": t_bwd, "achieved": gather_bwd / t_bwd / 1e9, "peak": l2_gbs, "unit": "GB/s",
            "frac": (gather_bwd / t_bwd / 1e9 / l2_gbs) if l2_gbs else None,
            "algorithmic_gather_bytes": gather_bwd, "algorithmic_hbm_bytes": hbm_bwd,
            "hbm_achieved": hbm_bwd / t_bwd / 1e9, "hbm_frac": hbm_bwd / t_bwd / 1e9 / hbm_peak,
            "kernels": "list + depth-gradient kernel, entry scatter, gather by texel, conversion",
            "note": "backward time = forward+backward minus forward; bytes: forward gathers re-read + one scatter per "
                    "accepted sample and corner (features and depth), against the L2-resident read bandwidth of this run"}
    if not args.no_extras:
        line["e2e"] = {"value": cells_total / (ms_e2e_max * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d,
                       "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e_max}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import oracle as O
        threads = host_thread_count()
        times = cpu_forward_rate(w, args.mode, threads, min_seconds=8.0)
        line["cpu_baseline"] = {
            "value": w.X * w.Y / statistics.median(times), "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{len(times)} whole forwards of one sample (median), float32 oracle, OpenMP over BEV rows",
            "reference_pytorch_path": reference_pytorch_cpu(w, threads)}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
