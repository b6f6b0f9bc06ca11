"""Benchmark of the lattice-filter hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config 2] [--impl ours|reference]

One step = one forward + one backward (reverse=True on an upstream gradient) lattice filter over the
whole batch of the configuration (forward only for configurations 0 and 4).  Default workload:
configuration 2, dense-CRF message passing, 16 x 512x512, 21 channels guided by RGB + xy
(pd 5, vd 22).  Metric: Mpixels/s.

Under torchrun the ONE batch of the configuration is sharded over the ranks (contiguous slices, each
item an independent lattice, no collective in the data path): strong scaling, `value` = pixels of the
whole batch / time of the slowest rank.  Single-item configurations are replicated instead.  Blocks of
K steps, each bracketed by barrier + synchronize, are repeated until they fill half a second of
device time; `ms_per_step` is the median block / K.

The line also carries: `roofline` for the slowest kernel (algorithmic bytes / CUDA-event time, against
the measured HBM copy bandwidth in MEASURED_PEAKS.json), `roofline_call` for the whole call,
`stages_ms` (per-call stage times from events recorded inside the last timed block), `e2e` (the same
step through the public host-buffer API, `HostPipeline.filter`, from pinned host memory: copies in
both directions inside the timed region, overlapped with the filter item by item; beside it the time of
the copies alone), `gather` (N > 1: the step with the ranks' outputs gathered on rank 0 by NCCL),
`weak_scaling` (N > 1: every rank filters a whole batch of its own) and `cpu_baseline` (the CPU
oracle on this box's host cores, bounded sample).  `--impl reference` times the reference CPU
implementation alone.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "Mpixels/s fwd+bwd (pd=5, vd=22 CRF)"
FALLBACK_HBM_GBS = 6650.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", type=int, default=2)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=8)
    ap.add_argument("--min-ms", type=float, default=500.0,
                    help="the timed blocks of --steps steps are repeated until they fill this much device time")
    ap.add_argument("--no-weak", action="store_true", help="skip the extra weak-scaling measurement at N > 1")
    ap.add_argument("--channels", type=int, default=0,
                    help="override the channel count of configuration 2 / 5 (value widths without a register-resident "
                         "instantiation run the generic splat / slice kernels)")
    ap.add_argument("--headline-only", action="store_true",
                    help="only the device-resident measurement (no end-to-end, gather, reuse, graph or weak-scaling "
                         "legs): short runs for profiler captures")
    ap.add_argument("--mode", default="atomic", choices=["atomic", "deterministic"],
                    help="accumulation mode of the splat stage (the headline is atomic)")
    ap.add_argument("--dtype", default="f32", choices=["f32", "f64"],
                    help="number type of the call (the headline is f32; f64 is the reference's other registered type)")
    ap.add_argument("--reuse-lattice", action="store_true",
                    help="the step builds one lattice and applies it forward and backward (what a training step through "
                         "lattice_filter(..., reuse_lattice=True) does) instead of two stateless calls; not the headline")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-threads", type=int, default=0)
    ap.add_argument("--batch", type=int, default=0,
                    help="override the batch size of the configuration (profiling of smaller cases)")
    ap.add_argument("--size", type=int, default=0,
                    help="override the side length of the configuration's images or volumes (smaller cases)")
    return ap.parse_args()


def metric_name(cfg, w):
    if cfg == 2:
        return METRIC
    return "Mpixels/s %s (pd=%d, vd=%d)" % ("fwd+bwd" if w.backward else "fwd", w.pd, w.vd)


def make_workload(cfg, rank, batch=0, size=0, channels=0):
    from permutohedral_lattice_b200 import workloads
    kw = {}
    if batch and cfg >= 2:
        kw["batch"] = batch
    if size:
        kw["size"] = size
    if channels and cfg in (2, 5):
        kw["channels"] = channels
    w = workloads.CONFIGS[cfg](**kw)
    if rank:   # another rank's batch: same distributions, other content
        rng = np.random.default_rng(1000 + rank)
        perm = rng.permutation(w.batch)
        w.input = np.ascontiguousarray(np.roll(w.input[perm], rank * 7, axis=1))
        if w.reference is not None:
            w.reference = np.ascontiguousarray(np.roll(w.reference[perm], rank * 7, axis=1))
        if w.positions is not None:
            w.positions = np.ascontiguousarray(w.positions[perm])
        if w.grad is not None:
            w.grad = np.ascontiguousarray(w.grad[perm])
    return w


def config_of(w, world):
    """The `config` object of the JSON line: the same for both arms of the comparison."""
    sharded = w.batch >= 2
    return {"workload": w.name, "global_batch": w.batch * (1 if sharded else max(1, world)),
            "batch_per_gpu": -(-w.batch // max(1, world)) if sharded else w.batch,
            "pixels_per_item": w.pixels_per_item, "pd": w.pd, "vd": w.vd,
            "direction": "fwd+bwd" if w.backward else "fwd",
            "l2_policy": "inputs larger than L2, no flush between iterations"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                return float(json.load(f)["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.proc = None
        self.gpu = gpu_index
        self.path = "/tmp/pl_bench_clocks_%d_%d.csv" % (os.getpid(), gpu_index)

    def start(self):
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.QUERY,
                 "--format=csv,noheader,nounits", "-lms", "20"], stdout=self.out,
                stderr=subprocess.DEVNULL)
            deadline = time.time() + 5.0      # wait for the first sample so the region is covered
            while time.time() < deadline and os.path.getsize(self.path) == 0:
                time.sleep(0.05)
                self.out.flush()
        except Exception:
            self.proc = None

    def mark_begin(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        import datetime
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    rows.append((ts, float(parts[1]), float(parts[2]), parts[5:9]))
                except ValueError:
                    continue
        # samples taken inside the timed region (one sampling period of slack); if the region was
        # shorter than a period, the nearest sample
        inside = [r for r in rows if self.t0 - 0.02 <= r[0] <= self.t1 + 0.02]
        if not inside and rows:
            mid = 0.5 * (self.t0 + self.t1)
            inside = [min(rows, key=lambda r: abs(r[0] - mid))]
        sm = [r[1] for r in inside]
        mx = [r[2] for r in inside]
        reasons = set()
        for r in inside:
            for name, val in zip(names, r[3]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.remove(self.path)
        except OSError:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def algorithmic_bytes(w, num_vertices):
    """Per call (one direction), whole batch: 4N(F + 2C) + 4M vd (2(pd+1) + 2), split per stage:
    build reads the features, splat reads the input and writes the M rows, each blur pass reads and
    writes the M rows, slice reads the M rows and writes the output."""
    npx = w.batch * w.pixels_per_item
    c = w.vd - 1
    f = w.pd if w.positions is not None else (w.reference.shape[-1] if w.bilateral else 0)
    rows = 4 * num_vertices * w.vd
    stage = {"build": 4 * npx * f, "splat": 4 * npx * c + rows, "blur": 2 * rows * (w.pd + 1),
             "slice": rows + 4 * npx * c, "index": 0}
    return stage, sum(stage.values()), 4 * npx * (f + 2 * c)


def cpu_baseline(w, threads, prefer_reference=True):
    """The CPU oracle on a bounded sample: the full batch (all items, fwd [+ bwd]) on `threads`
    host threads, one lattice per item.  Returns the cpu_baseline object."""
    from oracle import cpu_oracle as O
    if w.positions is not None:   # positions path: per-item filter calls, single thread
        items = min(w.batch, 1)
        t0 = time.perf_counter()
        for b in range(items):
            O.filter(w.input[b].reshape(w.pixels_per_item, -1), w.positions[b], structure=False)
        secs = time.perf_counter() - t0
        return {"value": items * w.pixels_per_item / secs / 1e6, "unit": "Mpixels/s", "cores": 1,
                "kind": "port", "sample": "%d item(s) of %s, forward, 1 thread" % (items, w.name)}
    kind = "port"
    kwargs = {}
    if prefer_reference and O.reference_available():
        try:
            O._load_reference()
            kind = "reference"
            kwargs = {"min_vertices": w.pixels_per_item * (w.pd + 1) // 4}
        except Exception:
            kind = "port"
    impl = "reference" if kind == "reference" else "port"
    args = (w.reference, w.bilateral, w.theta_alpha, w.theta_beta, w.theta_gamma)
    try:
        _, secs = O.filter_batch_timed(w.input, *args, reverse=False, impl=impl, threads=threads, **kwargs)
        if w.backward:
            _, s2 = O.filter_batch_timed(w.grad, *args, reverse=True, impl=impl, threads=threads, **kwargs)
            secs += s2
    except RuntimeError:
        # pre-sized reference table too small for this data: worst-case size
        kwargs = {"min_vertices": w.pixels_per_item * (w.pd + 1)} if kind == "reference" else {}
        _, secs = O.filter_batch_timed(w.input, *args, reverse=False, impl=impl, threads=threads, **kwargs)
        if w.backward:
            _, s2 = O.filter_batch_timed(w.grad, *args, reverse=True, impl=impl, threads=threads, **kwargs)
            secs += s2
    return {"value": w.batch * w.pixels_per_item / secs / 1e6, "unit": "Mpixels/s", "cores": threads,
            "kind": kind,
            "sample": "full batch of %s (%d items, %s) once, %d host threads, one lattice per item%s"
                      % (w.name, w.batch, "fwd+bwd" if w.backward else "fwd", threads,
                         ", hash table pre-sized (never grows)" if kind == "reference" else ""),
            "seconds": secs}


def host_threads(requested, batch):
    n = requested if requested > 0 else (os.cpu_count() or 1)
    return max(1, min(n, batch))


def run_reference(args, rank, world):
    """--impl reference: the reference's own CPU implementation of the path on the host cores."""
    if rank != 0:
        return
    w = make_workload(args.config, 0, args.batch, args.size, args.channels)
    threads = host_threads(args.cpu_threads, w.batch)
    times = []
    info = None
    for i in range(args.warmup + args.steps):
        info = cpu_baseline(w, threads)
        if i >= args.warmup:
            times.append(info["seconds"])
        if sum(times) > 240 and len(times) >= 1:   # keep the whole run within a few minutes
            break
    secs = sum(times) / len(times)
    value = w.batch * w.pixels_per_item / secs / 1e6
    line = {
        "impl": "reference", "metric": metric_name(args.config, w), "value": value,
        "unit": "Mpixels/s", "n_gpus": args.gpus, "steps": len(times), "warmup": args.warmup,
        "ms_per_step": secs * 1e3, "higher_is_better": True, "scaling": "strong" if w.batch >= 2 else "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_of(w, world),
        "details": {"mode": "cpu reference: the whole batch on rank 0's host cores, whatever --gpus says"},
        "cpu_baseline": {"value": value, "unit": "Mpixels/s", "cores": info["cores"],
                         "kind": info["kind"], "sample": info["sample"]},
        "e2e": {"value": value, "unit": "Mpixels/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit_line(line)


class Arm:
    """One arm of the measurement: a set of device-resident tensors (a rank's slice of the batch, or a whole
    batch) and the forward (+ backward) step over them."""

    def __init__(self, plb, capi, w, lo, hi, dev, mode="atomic", dtype="f32", reuse_lattice=False):
        import torch
        self.plb, self.capi, self.w, self.mode = plb, capi, w, mode
        self.reuse_lattice = reuse_lattice
        self.b, self.n, self.c = hi - lo, w.pixels_per_item, w.vd - 1
        self.use_positions = w.positions is not None
        tt = torch.float64 if dtype == "f64" else torch.float32
        self.x = torch.from_numpy(w.input[lo:hi]).to(dev, tt)
        self.ref = None if w.reference is None else torch.from_numpy(w.reference[lo:hi]).to(dev, tt)
        self.pos = None if not self.use_positions else torch.from_numpy(w.positions[lo:hi]).to(dev, tt)
        self.grad = None if w.grad is None else torch.from_numpy(w.grad[lo:hi]).to(dev, tt)
        self.out_f = torch.empty_like(self.x)
        self.out_b = torch.empty_like(self.x)
        self.ws = None

    def call(self, inp, out, reverse, events=None):
        w = self.w
        if self.b == 0:
            return
        if events is not None:
            arr = (ctypes.c_void_p * self.capi.NUM_STAGE_EVENTS)(*[e.cuda_event for e in events])
            self.capi.lib().pl_profile_next_call(arr)
        if self.use_positions:
            _, self.ws = self.plb.filter_positions(inp.view(self.b, self.n, self.c), self.pos, reverse=reverse,
                                                   mode=self.mode, out=out.view(self.b, self.n, self.c))
        else:
            _, self.ws, _ = self.plb.lattice_filter_raw(inp, self.ref, w.bilateral, w.theta_alpha, w.theta_beta,
                                                        w.theta_gamma, reverse, mode=self.mode, out=out)

    def step(self, events_f=None, events_b=None):
        if self.reuse_lattice:
            if self.b == 0:
                return
            w = self.w
            lat = self.plb.Lattice(self.ref, tuple(self.x.shape[:-1]), w.bilateral, w.theta_alpha, w.theta_beta,
                                   w.theta_gamma, max_channels=self.c, mode=self.mode)
            lat.apply(self.x, False, self.mode, out=self.out_f)
            if w.backward:
                lat.apply(self.grad, True, self.mode, out=self.out_b)
            self.ws = lat.workspace
            return
        self.call(self.x, self.out_f, False, events_f)
        if self.w.backward:
            self.call(self.grad, self.out_b, True, events_b)


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    import permutohedral_lattice_b200 as plb
    from permutohedral_lattice_b200 import capi
    from permutohedral_lattice_b200.sharding import OutputGather, shard_range

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(values):
        if world == 1:
            return [float(v) for v in values]
        t = torch.tensor(list(values), device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    def timed_blocks(step, steps, min_total_ms, last_block_step=None):
        """Blocks of exactly `steps` steps, each bracketed by barrier + synchronize on both sides and timed
        with CUDA events on the launching stream; as many blocks as it takes to fill min_total_ms (3 at
        least).  Returns the blocks' times, each the maximum over ranks."""
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)

        def block(fn):
            barrier()
            e0.record()
            for k in range(steps):
                fn(k)
            e1.record()
            barrier()
            return e0.elapsed_time(e1)

        first = block(step)
        (first_max,) = max_over_ranks([first])
        nblocks = int(min(max(-(-min_total_ms // max(first_max, 1e-3)), 3), 400))
        times = [first] + [block(step) for _ in range(nblocks - 2)] + [block(last_block_step or step)]
        return max_over_ranks(times)

    # ---- the workload and this rank's share of it -------------------------------------------------
    # The same seeded batch on every rank; a batch of several items is SHARDED over the ranks (strong
    # scaling: total work fixed), a single-item configuration is replicated (every rank filters it).
    full = make_workload(args.config, 0, args.batch, args.size, args.channels)
    B, n, c = full.batch, full.pixels_per_item, full.vd - 1
    sharded = B >= 2
    lo, hi = shard_range(B, world, rank) if sharded else (0, B)
    if args.reuse_lattice and (args.dtype != "f32" or full.positions is not None):
        raise SystemExit("--reuse-lattice: float calls on a reference image only")
    arm = Arm(plb, capi, full, lo, hi, dev, args.mode, args.dtype, args.reuse_lattice)
    real_bytes = 8 if args.dtype == "f64" else 4
    extras = not args.headline_only and args.dtype == "f32" and args.mode == "atomic" and not args.reuse_lattice
    calls_per_step = 2 if full.backward else 1
    total_pixels = B * n * (1 if sharded else world)

    warm = max(args.warmup, 3)
    for _ in range(warm):
        arm.step()
    torch.cuda.synchronize()
    if arm.ws is not None:
        st = plb.lattice_stats(arm.ws)
        if st.device_status != 0:
            raise SystemExit("device status %d" % st.device_status)
        counts = [int(st.num_vertices), int(st.num_entries)]
    else:
        counts = [0, 0]
    if world > 1:   # whole-batch counts: sum over the ranks' slices
        t = torch.tensor(counts, device=dev, dtype=torch.int64)
        if sharded:
            dist.all_reduce(t)
        counts = [int(v) for v in t.tolist()]
    num_vertices, num_entries = counts

    # stage events of every call of the last timed block
    ev = [[[torch.cuda.Event(enable_timing=True) for _ in range(capi.NUM_STAGE_EVENTS)]
           for _ in range(calls_per_step)] for _ in range(args.steps)]
    for s_ in ev:
        for call in s_:
            for e in call:
                e.record()

    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = capi.lib().pl_launch_count()
    sampler.mark_begin()
    staged = args.dtype == "f32" and not args.reuse_lattice   # the stage-event hook belongs to the one-call float filter
    block_ms = timed_blocks(lambda k: arm.step(), args.steps, args.min_ms,
                            (lambda k: arm.step(ev[k][0], ev[k][1] if full.backward else None)) if staged else None)
    sampler.mark_end()
    launches = capi.lib().pl_launch_count() - launches0
    clocks = sampler.stop()
    ms_per_step = statistics.median(block_ms) / args.steps
    value = total_pixels / (ms_per_step * 1e-3) / 1e6

    # per-stage times of a call, averaged over the calls of the last block (this rank's slice)
    stage_ms = {name: 0.0 for name in capi.STAGE_NAMES}
    ncalls = 0
    if arm.b and staged:
        for s_ in ev:
            for call in s_:
                for i, name in enumerate(capi.STAGE_NAMES):
                    stage_ms[name] += call[i].elapsed_time(call[i + 1])
                ncalls += 1
        stage_ms = {k: v / ncalls for k, v in stage_ms.items()}

    # roofline of the slowest kernel and of the whole call (this rank's launches: its slice of the batch)
    hbm_gbs, peak_kind = peaks()
    frac_of_batch = (arm.b / B) if sharded else 1.0
    stage_bytes, call_bytes, io_bytes = algorithmic_bytes(full, num_vertices // (1 if sharded else world))
    scale_b = frac_of_batch * real_bytes / 4
    stage_bytes = {k: v * scale_b for k, v in stage_bytes.items()}
    call_bytes *= scale_b
    io_bytes *= scale_b
    kernel_ms = dict(stage_ms)
    kernel_ms["blur"] = stage_ms["blur"] / (full.pd + 1)          # one blur_axis launch
    kernel_bytes = dict(stage_bytes)
    kernel_bytes["blur"] = stage_bytes["blur"] / (full.pd + 1)
    kernel_names = {"build": "build_tiles", "splat": "splat_tiles", "blur": "blur_axis",
                    "slice": "slice_tiles"}
    call_ms = ms_per_step / calls_per_step
    if args.reuse_lattice:   # one build serves the step's calls: the features are read once per step
        call_bytes -= stage_bytes["build"] * (calls_per_step - 1) / calls_per_step
    if staged:
        dominant = max(kernel_names, key=lambda k: stage_ms[k])
        achieved = kernel_bytes[dominant] / max(kernel_ms[dominant] * 1e-3, 1e-12) / 1e9
        traffic, traffic_source = measured_traffic(full.name, kernel_names[dominant], arm.b * n)
        roofline = {"bound": "hbm", "kernel": kernel_names[dominant], "achieved": achieved,
                    "peak": hbm_gbs, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / hbm_gbs,
                    "traffic": traffic, "traffic_source": traffic_source,
                    "algorithmic_bytes_per_launch": kernel_bytes[dominant],
                    "ms_per_launch": kernel_ms[dominant]}
    else:   # no per-stage events: the whole call stands for the kernel
        achieved = call_bytes / (call_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": "whole call", "achieved": achieved, "peak": hbm_gbs,
                    "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / hbm_gbs, "traffic": None,
                    "algorithmic_bytes_per_launch": call_bytes, "ms_per_launch": call_ms}
    call_gbs = call_bytes / (call_ms * 1e-3) / 1e9
    roofline_call = {"algorithmic_bytes_per_call": call_bytes, "io_floor_bytes_per_call": io_bytes,
                     "achieved": call_gbs, "peak": hbm_gbs, "unit": "GB/s", "frac": call_gbs / hbm_gbs,
                     "ms_per_call": call_ms}

    # ---- the same step with the ranks' output slices gathered on rank 0 (NCCL over NVLink) ---------
    gather = None
    if world > 1 and sharded and extras:
        comm = torch.cuda.Stream(dev)
        item_shape = tuple(arm.x.shape[1:])
        gather_f = OutputGather(B, item_shape, arm.x.dtype, dev, dst=0)
        gather_b = OutputGather(B, item_shape, arm.x.dtype, dev, dst=0) if full.backward else None
        main = torch.cuda.current_stream(dev)

        def gather_step(k):
            # the forward result travels while the backward call computes
            arm.call(arm.x, arm.out_f, False)
            comm.wait_stream(main)
            with torch.cuda.stream(comm):
                gather_f(arm.out_f)
            if full.backward:
                arm.call(arm.grad, arm.out_b, True)
                comm.wait_stream(main)
                with torch.cuda.stream(comm):
                    gather_b(arm.out_b)
            main.wait_stream(comm)

        for _ in range(3):
            gather_step(0)
        g_ms = statistics.median(timed_blocks(gather_step, args.steps, min(args.min_ms, 250.0))) / args.steps
        per = -(-B // world)
        gather = {"value": total_pixels / (g_ms * 1e-3) / 1e6, "unit": "Mpixels/s", "ms_per_step": g_ms,
                  "bytes_received_by_rank0_per_step": (world - 1) * per * n * c * 4 * calls_per_step,
                  "method": "torch.distributed gather (NCCL) of the ranks' output slices onto rank 0 on a side "
                            "stream, forward result in flight during the backward call"}

    # ---- end to end through the public API from pinned host buffers (this rank's slice) ------------
    hslice = slice(lo, hi)
    hx = torch.from_numpy(full.input[hslice]).pin_memory()
    href = None if full.reference is None else torch.from_numpy(full.reference[hslice]).pin_memory()
    hpos = None if not arm.use_positions else torch.from_numpy(full.positions[hslice]).pin_memory()
    hgrad = None if full.grad is None else torch.from_numpy(full.grad[hslice]).pin_memory()
    hout_f = torch.empty_like(hx).pin_memory()
    hout_b = torch.empty_like(hx).pin_memory()
    # the op is stateless: the reference image travels with the forward and again with the backward call
    h2d = hx.numel() * 4 + (href.numel() * 4 * calls_per_step if href is not None else 0) + \
        (hpos.numel() * 4 if hpos is not None else 0) + (hgrad.numel() * 4 if full.backward else 0)
    d2h = hx.numel() * 4 * calls_per_step
    (h2d, d2h) = [int(v) for v in sum_over_ranks([h2d, d2h], world, dev, dist)]   # whole job

    pipe = plb.HostPipeline(dev)

    def e2e_step(copy_only=False):
        w = full
        if arm.b == 0:
            return
        if arm.use_positions:
            dx = hx.to(dev, non_blocking=True)
            dp = hpos.to(dev, non_blocking=True)
            if copy_only:
                o = dx
            else:
                o, _ = plb.filter_positions(dx.view(arm.b, n, c), dp)
            hout_f.copy_(o.view_as(hout_f), non_blocking=True)
            torch.cuda.current_stream().synchronize()
        else:
            pipe.filter(hx, href, w.bilateral, w.theta_alpha, w.theta_beta, w.theta_gamma, reverse=False,
                        out_host=hout_f, wait=False, copy_only=copy_only)
            if w.backward:
                pipe.filter(hgrad, href, w.bilateral, w.theta_alpha, w.theta_beta, w.theta_gamma, reverse=True,
                            out_host=hout_b, wait=False, copy_only=copy_only)
            pipe.synchronize()     # both results are complete in host memory when the step ends

    def timed_host_steps(fn, steps):
        fn()
        barrier()
        t0 = time.perf_counter()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        wall = (time.perf_counter() - t0) * 1e3
        (ms, wall) = max_over_ranks([e0.elapsed_time(e1), wall])
        return ms / steps, wall / steps

    e2e_reuse = None
    if extras and full.backward and not arm.use_positions and arm.b:
        def e2e_reuse_step():
            pipe.filter_forward_backward(hx, hgrad, href, full.bilateral, full.theta_alpha, full.theta_beta,
                                         full.theta_gamma, out_host=hout_f, grad_out_host=hout_b, wait=True)
        r_ms, _ = timed_host_steps(e2e_reuse_step, args.e2e_steps)
        e2e_reuse = {"value": total_pixels / (r_ms * 1e-3) / 1e6, "unit": "Mpixels/s", "ms_per_step": r_ms,
                     "note": "forward + backward through HostPipeline.filter_forward_backward: the reference image "
                             "is sent once and one lattice serves both directions; not the headline metric"}
    if extras:
        e2e_ms, e2e_wall_ms = timed_host_steps(e2e_step, args.e2e_steps)
        copy_ms, _ = timed_host_steps(lambda: e2e_step(copy_only=True), args.e2e_steps)
        e2e_value = total_pixels / (e2e_ms * 1e-3) / 1e6
    else:
        e2e_ms = e2e_wall_ms = copy_ms = e2e_value = None

    # not the headline: the same step with the lattice built once and reused by the backward call
    # (pl_lattice_build_f32 + 2 x pl_lattice_apply_f32), as a training step through
    # lattice_filter(..., reuse_lattice=True) does
    reuse = None
    if not arm.use_positions and full.backward and arm.b and extras:
        w = full

        def reuse_step(k):
            lat = plb.Lattice(arm.ref, tuple(arm.x.shape[:-1]), w.bilateral, w.theta_alpha, w.theta_beta,
                              w.theta_gamma, max_channels=c)
            lat.apply(arm.x, False, out=arm.out_f)
            lat.apply(arm.grad, True, out=arm.out_b)
        for _ in range(3):
            reuse_step(0)
        reuse_ms = statistics.median(timed_blocks(reuse_step, args.steps, min(args.min_ms, 100.0))) / args.steps
        reuse = {"value": total_pixels / (reuse_ms * 1e-3) / 1e6, "unit": "Mpixels/s", "ms_per_step": reuse_ms,
                 "note": "lattice built once per step and applied forward and reverse; not the headline metric"}

    # also not the headline: the same stateless step replayed from CUDA graphs (one launch per call)
    graph = None
    if not arm.use_positions and arm.b and extras:
        w = full
        rshape = None if arm.ref is None else arm.ref.shape
        gf = plb.GraphedLatticeFilter(arm.x.shape, rshape, w.bilateral, w.theta_alpha, w.theta_beta, w.theta_gamma,
                                      False, device=dev)
        gb = plb.GraphedLatticeFilter(arm.x.shape, rshape, w.bilateral, w.theta_alpha, w.theta_beta, w.theta_gamma,
                                      True, device=dev) if w.backward else None
        gf.input.copy_(arm.x)
        if arm.ref is not None:
            gf.reference.copy_(arm.ref)
        if gb is not None:
            gb.input.copy_(arm.grad)
            if arm.ref is not None:
                gb.reference.copy_(arm.ref)

        def graph_step(k):
            gf.replay()
            if gb is not None:
                gb.replay()
        for _ in range(3):
            graph_step(0)
        graph_ms = statistics.median(timed_blocks(graph_step, args.steps, min(args.min_ms, 100.0))) / args.steps
        graph = {"value": total_pixels / (graph_ms * 1e-3) / 1e6, "unit": "Mpixels/s", "ms_per_step": graph_ms,
                 "note": "stateless forward + backward replayed from CUDA graphs; not the headline metric"}
        del gf, gb

    # weak scaling beside the strong-scaling headline: every rank filters a whole batch of its own
    weak = None
    if world > 1 and sharded and not args.no_weak and extras:
        del arm
        torch.cuda.empty_cache()
        own = Arm(plb, capi, make_workload(args.config, rank, args.batch, args.size, args.channels), 0, B, dev)
        for _ in range(3):
            own.step()
        weak_ms = statistics.median(timed_blocks(lambda k: own.step(), args.steps, min(args.min_ms, 250.0))) \
            / args.steps
        weak = {"value": B * n * world / (weak_ms * 1e-3) / 1e6, "unit": "Mpixels/s", "ms_per_step": weak_ms,
                "global_batch": B * world, "batch_per_gpu": B,
                "note": "every rank filters its own whole batch (per-GPU work fixed); not the headline metric"}

    line = {
        "metric": metric_name(args.config, full), "value": value, "unit": "Mpixels/s", "n_gpus": world,
        "steps": args.steps, "warmup": warm, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong" if sharded else "weak", "vs_baseline": None,
        "dtype": args.dtype,
        "data": "synthetic",
        "config": config_of(full, world),
        "details": {"parallelism": ("one batch of %d items sharded over %d GPU(s), no collective in the data path"
                                    % (B, world)) if sharded else "replicas only (single item), x%d" % world,
                    "mode": args.mode,
                    "lattice": ("built once per step, applied forward and backward" if args.reuse_lattice
                                else "rebuilt by every call (stateless op)"),
                    "bytes_read_per_call_on_this_rank": (hx.numel() + (
                        href.numel() if href is not None else 0)) * real_bytes,
                    "num_vertices": num_vertices, "num_entries": num_entries,
                    "timing": "median of %d blocks of %d steps, each block bracketed by barrier + synchronize, "
                              "max over ranks per block" % (len(block_ms), args.steps)},
        "blocks": {"count": len(block_ms), "min_ms": min(block_ms), "median_ms": statistics.median(block_ms),
                   "max_ms": max(block_ms)},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "Mpixels/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "wall_ms_per_step": e2e_wall_ms,
                "copy_only_ms_per_step": copy_ms,
                "note": "HostPipeline from pinned host buffers (two-item chunks, single items at both ends of a "
                        "call, 4 streams); copy_only = the same copies on the same streams without the filter "
                        "(what the host link allows)"},
        "gpu_launches": int(launches) * world,
        "launches_per_call": int(launches) // max(1, len(block_ms) * args.steps * calls_per_step),
        "roofline": roofline, "roofline_call": roofline_call,
        "stages_ms": stage_ms,
        "e2e_lattice_reuse": e2e_reuse,
        "gather": gather,
        "weak_scaling": weak,
        "lattice_reuse": reuse,
        "graph_replay": graph,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        info = cpu_baseline(full, host_threads(args.cpu_threads, full.batch))
        info.pop("seconds", None)
        line["cpu_baseline"] = info
    if rank == 0:
        emit_line(line)
    if world > 1:
        dist.destroy_process_group()


def sum_over_ranks(values, world, dev, dist):
    if world == 1:
        return values
    import torch
    t = torch.tensor(list(values), device=dev, dtype=torch.float64)
    dist.all_reduce(t)
    return t.tolist()


def measured_traffic(workload_name, kernel, points):
    """DRAM bytes of one launch of `kernel` over `points` points, scaled from the per-point figure of an ncu
    capture of a reduced batch of the same workload (every item is an independent lattice, so traffic is
    proportional to the number of points).  The figures live beside the captures' summaries; None if there
    is none for this workload."""
    path = os.path.join(ROOT, "profiles", "dram_bytes_per_point.json")
    try:
        with open(path) as f:
            table = json.load(f)
    except Exception:
        return None, None
    for prefix, entry in table.items():
        if workload_name.startswith(prefix) and kernel in entry.get("kernels", {}):
            return entry["kernels"][kernel] * points, entry.get("source")
    return None, None


class _StdoutToStderr:
    """While the benchmark runs, file descriptor 1 points at stderr, so that nothing a native library
    prints (NCCL announces its version on stdout) can precede the JSON line; `emit` writes to the real
    stdout."""

    def __enter__(self):
        sys.stdout.flush()
        self.saved = os.dup(1)
        os.dup2(2, 1)
        return self

    def emit(self, text):
        sys.stdout.flush()
        os.write(self.saved, (text + "\n").encode())

    def __exit__(self, *exc):
        sys.stdout.flush()
        os.dup2(self.saved, 1)
        os.close(self.saved)
        return False


_OUT = None


def emit_line(line):
    text = json.dumps(line)
    if _OUT is not None:
        _OUT.emit(text)
    else:
        print(text, flush=True)


if __name__ == "__main__":
    with _StdoutToStderr() as _OUT:
        main()
