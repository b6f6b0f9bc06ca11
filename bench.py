"""Benchmark of the lattice-filter hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config 2] [--impl ours|reference]

One step = one forward + one backward (reverse=True on an upstream gradient) lattice filter over the
whole batch of the configuration (forward only for configurations 0 and 4).  Default workload:
configuration 2, dense-CRF message passing, 16 x 512x512, 21 channels guided by RGB + xy
(pd 5, vd 22).  Metric: Mpixels/s.  Under torchrun every rank filters its own batch on its own GPU
(weak scaling, no collective in the data path); time is the maximum over ranks.

The line also carries: `roofline` for the slowest kernel (algorithmic bytes / CUDA-event time, against
the measured HBM copy bandwidth in MEASURED_PEAKS.json), `roofline_call` for the whole step,
`stages_ms` (per-call stage times from events recorded inside the timed steps), `e2e` (the same
step through the public host-buffer API, `HostPipeline.filter`, from pinned host memory: copies in
both directions inside the timed region, overlapped with the filter chunk by chunk) and `cpu_baseline` (the CPU
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
# DRAM bytes per point and launch (dram__bytes_read.sum + dram__bytes_write.sum) of the kernels of configuration 2,
# from the one-pass ncu capture of the full-size workload summarised in
# profiles/dram_traffic_c2_dense_crf_16x512.txt; traffic is proportional to the number of points.
NCU_DRAM_BYTES_PER_POINT_C2 = {"build_tiles": 49.2, "splat_tiles": 149.7, "slice_tiles": 125.4, "blur_axis": 20.4}
FALLBACK_HBM_GBS = 6650.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", type=int, default=2)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-threads", type=int, default=0)
    ap.add_argument("--batch", type=int, default=0,
                    help="override the batch size of the configuration (profiling of smaller cases)")
    return ap.parse_args()


def metric_name(cfg, w):
    if cfg == 2:
        return METRIC
    return "Mpixels/s %s (pd=%d, vd=%d)" % ("fwd+bwd" if w.backward else "fwd", w.pd, w.vd)


def make_workload(cfg, rank, batch=0):
    from permutohedral_lattice_b200 import workloads
    w = workloads.CONFIGS[cfg](batch=batch) if batch and cfg >= 2 else workloads.CONFIGS[cfg]()
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
    w = make_workload(args.config, 0, args.batch)
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
        "ms_per_step": secs * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": w.name, "batch_per_gpu": w.batch, "global_batch": w.batch * max(1, world),
                   "pixels_per_item": w.pixels_per_item, "pd": w.pd, "vd": w.vd,
                   "direction": "fwd+bwd" if w.backward else "fwd",
                   "parallelism": "batch-sharded x%d" % max(1, world), "mode": "cpu reference"},
        "cpu_baseline": {"value": value, "unit": "Mpixels/s", "cores": info["cores"],
                         "kind": info["kind"], "sample": info["sample"]},
        "e2e": {"value": value, "unit": "Mpixels/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit_line(line)


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

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    w = make_workload(args.config, rank, args.batch)
    b, n, c = w.batch, w.pixels_per_item, w.vd - 1
    use_positions = w.positions is not None

    x = torch.from_numpy(w.input).to(dev)
    ref = None if w.reference is None else torch.from_numpy(w.reference).to(dev)
    pos = None if not use_positions else torch.from_numpy(w.positions).to(dev)
    grad = None if w.grad is None else torch.from_numpy(w.grad).to(dev)
    out_f = torch.empty_like(x)
    out_b = torch.empty_like(x)
    xf = x.view(b, n, c)

    def one_call(inp, out, reverse, events=None):
        if events is not None:
            arr = (ctypes.c_void_p * capi.NUM_STAGE_EVENTS)(*[e.cuda_event for e in events])
            capi.lib().pl_profile_next_call(arr)
        if use_positions:
            o, ws = plb.filter_positions(inp.view(b, n, c), pos, reverse=reverse)
            return o, ws
        o, ws, _ = plb.lattice_filter_raw(inp, ref, w.bilateral, w.theta_alpha, w.theta_beta,
                                          w.theta_gamma, reverse, out=out)
        return o, ws

    def step(events_f=None, events_b=None):
        _, ws = one_call(x, out_f, False, events_f)
        if w.backward:
            one_call(grad, out_b, True, events_b)
        return ws

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # warm-up (also creates the workspace and every stage event before the timed region)
    for _ in range(max(args.warmup, 3)):
        ws = step()
    torch.cuda.synchronize()
    st = plb.lattice_stats(ws)
    if st.device_status != 0:
        raise SystemExit("device status %d" % st.device_status)
    calls_per_step = 2 if w.backward else 1
    ev = [[[torch.cuda.Event(enable_timing=True) for _ in range(capi.NUM_STAGE_EVENTS)]
           for _ in range(calls_per_step)] for _ in range(args.steps)]
    for s in ev:
        for call in s:
            for e in call:
                e.record()
    t_begin = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)

    sampler = ClockSampler(local_rank)
    sampler.start()
    barrier()
    sampler.mark_begin()
    t_begin.record()
    for k in range(args.steps):
        step(ev[k][0], ev[k][1] if w.backward else None)
    t_end.record()
    barrier()
    sampler.mark_end()
    clocks = sampler.stop()
    elapsed_ms = t_begin.elapsed_time(t_end)
    if world > 1:
        t = torch.tensor([elapsed_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    total_pixels = b * n * world
    value = total_pixels / (ms_per_step * 1e-3) / 1e6

    # per-stage times of a call, averaged over all timed calls
    stage_ms = {name: 0.0 for name in capi.STAGE_NAMES}
    ncalls = 0
    for s in ev:
        for call in s:
            for i, name in enumerate(capi.STAGE_NAMES):
                stage_ms[name] += call[i].elapsed_time(call[i + 1])
            ncalls += 1
    stage_ms = {k: v / ncalls for k, v in stage_ms.items()}

    # roofline
    hbm_gbs, peak_kind = peaks()
    stage_bytes, call_bytes, io_bytes = algorithmic_bytes(w, int(st.num_vertices))
    kernel_ms = dict(stage_ms)
    kernel_ms["blur"] = stage_ms["blur"] / (w.pd + 1)          # one blur_axis launch
    kernel_bytes = dict(stage_bytes)
    kernel_bytes["blur"] = stage_bytes["blur"] / (w.pd + 1)
    kernel_names = {"build": "build_tiles", "splat": "splat_tiles", "blur": "blur_axis",
                    "slice": "slice_tiles"}
    dominant = max(kernel_names, key=lambda k: stage_ms[k])
    achieved = kernel_bytes[dominant] / (kernel_ms[dominant] * 1e-3) / 1e9
    traffic = None
    if args.config == 2:
        traffic = NCU_DRAM_BYTES_PER_POINT_C2[kernel_names[dominant]] * b * n
    roofline = {"bound": "hbm", "kernel": kernel_names[dominant], "achieved": achieved,
                "peak": hbm_gbs, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / hbm_gbs,
                "traffic": traffic, "algorithmic_bytes_per_launch": kernel_bytes[dominant],
                "ms_per_launch": kernel_ms[dominant]}
    call_ms = ms_per_step / calls_per_step
    call_gbs = call_bytes / (call_ms * 1e-3) / 1e9
    roofline_call = {"algorithmic_bytes_per_call": call_bytes, "io_floor_bytes_per_call": io_bytes,
                     "achieved": call_gbs, "peak": hbm_gbs, "unit": "GB/s", "frac": call_gbs / hbm_gbs,
                     "ms_per_call": call_ms}

    # end to end through the public API from pinned host buffers
    hx = torch.from_numpy(w.input).pin_memory()
    href = None if w.reference is None else torch.from_numpy(w.reference).pin_memory()
    hpos = None if not use_positions else torch.from_numpy(w.positions).pin_memory()
    hgrad = None if w.grad is None else torch.from_numpy(w.grad).pin_memory()
    hout_f = torch.empty_like(hx).pin_memory()
    hout_b = torch.empty_like(hx).pin_memory()
    # the op is stateless: the reference image travels with the forward and again with the backward call
    h2d = hx.numel() * 4 + (href.numel() * 4 * calls_per_step if href is not None else 0) + \
        (hpos.numel() * 4 if hpos is not None else 0) + (hgrad.numel() * 4 if w.backward else 0)
    d2h = hx.numel() * 4 * calls_per_step

    pipe = plb.HostPipeline(dev, n_streams=3, chunk_items=2)

    def e2e_step():
        if use_positions:
            dx = hx.to(dev, non_blocking=True)
            dp = hpos.to(dev, non_blocking=True)
            o, _ = plb.filter_positions(dx.view(b, n, c), dp)
            hout_f.copy_(o.view_as(hout_f), non_blocking=True)
            torch.cuda.current_stream().synchronize()
        else:
            pipe.filter(hx, href, w.bilateral, w.theta_alpha, w.theta_beta, w.theta_gamma, reverse=False,
                        out_host=hout_f, wait=False)
            if w.backward:
                pipe.filter(hgrad, href, w.bilateral, w.theta_alpha, w.theta_beta, w.theta_gamma, reverse=True,
                            out_host=hout_b, wait=False)
            pipe.synchronize()     # both results are complete in host memory when the step ends

    e2e_step()
    barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = total_pixels / (e2e_ms / args.e2e_steps * 1e-3) / 1e6

    # not the headline: the same step with the lattice built once and reused by the backward call
    # (pl_lattice_build_f32 + 2 x pl_lattice_apply_f32), as a training step through
    # lattice_filter(..., reuse_lattice=True) does
    reuse = None
    if not use_positions and w.backward:
        def reuse_step():
            lat = plb.Lattice(ref, tuple(x.shape[:-1]), w.bilateral, w.theta_alpha, w.theta_beta, w.theta_gamma,
                              max_channels=c)
            lat.apply(x, False, out=out_f)
            lat.apply(grad, True, out=out_b)
        for _ in range(3):
            reuse_step()
        barrier()
        r0 = torch.cuda.Event(enable_timing=True)
        r1 = torch.cuda.Event(enable_timing=True)
        r0.record()
        for _ in range(args.steps):
            reuse_step()
        r1.record()
        barrier()
        reuse_ms = r0.elapsed_time(r1) / args.steps
        if world > 1:
            t = torch.tensor([reuse_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            reuse_ms = float(t.item())
        reuse = {"value": total_pixels / (reuse_ms * 1e-3) / 1e6, "unit": "Mpixels/s", "ms_per_step": reuse_ms,
                 "note": "lattice built once per step and applied forward and reverse; not the headline metric"}

    # also not the headline: the same stateless step replayed from CUDA graphs (one launch per call)
    graph = None
    if not use_positions:
        gf = plb.GraphedLatticeFilter(x.shape, None if ref is None else ref.shape, w.bilateral, w.theta_alpha,
                                      w.theta_beta, w.theta_gamma, False, device=dev)
        gb = plb.GraphedLatticeFilter(x.shape, None if ref is None else ref.shape, w.bilateral, w.theta_alpha,
                                      w.theta_beta, w.theta_gamma, True, device=dev) if w.backward else None
        gf.input.copy_(x)
        if ref is not None:
            gf.reference.copy_(ref)
        if gb is not None:
            gb.input.copy_(grad)
            if ref is not None:
                gb.reference.copy_(ref)
        for _ in range(3):
            gf.replay()
            if gb is not None:
                gb.replay()
        barrier()
        g0 = torch.cuda.Event(enable_timing=True)
        g1 = torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(args.steps):
            gf.replay()
            if gb is not None:
                gb.replay()
        g1.record()
        barrier()
        graph_ms = g0.elapsed_time(g1) / args.steps
        if world > 1:
            t = torch.tensor([graph_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            graph_ms = float(t.item())
        graph = {"value": total_pixels / (graph_ms * 1e-3) / 1e6, "unit": "Mpixels/s", "ms_per_step": graph_ms,
                 "note": "stateless forward + backward replayed from CUDA graphs; not the headline metric"}
        del gf, gb

    kernels_per_call = 7 + (w.pd + 1)   # build, clear, insert, link x2, splat, slice + blur passes
    line = {
        "metric": metric_name(args.config, w), "value": value, "unit": "Mpixels/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": w.name, "batch_per_gpu": b, "global_batch": b * world,
                   "pixels_per_item": n, "pd": w.pd, "vd": w.vd,
                   "direction": "fwd+bwd" if w.backward else "fwd", "parallelism": "batch-sharded x%d" % world,
                   "mode": "atomic", "l2_policy": "inputs larger than L2 (%.0f MB read per call)"
                   % ((x.numel() + (ref.numel() if ref is not None else 0)) * 4 / 1e6),
                   "num_vertices": int(st.num_vertices), "num_entries": int(st.num_entries)},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "Mpixels/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / args.e2e_steps},
        "gpu_launches": kernels_per_call * calls_per_step * args.steps,
        "roofline": roofline, "roofline_call": roofline_call,
        "stages_ms": stage_ms,
        "lattice_reuse": reuse,
        "graph_replay": graph,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        info = cpu_baseline(w, host_threads(args.cpu_threads, w.batch))
        info.pop("seconds", None)
        line["cpu_baseline"] = info
    if rank == 0:
        emit_line(line)
    if world > 1:
        dist.destroy_process_group()


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
