#!/usr/bin/env python
"""Benchmark of the fused V3 loss path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME|all] [--impl reference]

A step is one forward + backward of a loss module over one synthetic batch
(bench_workloads.py).  Rank 0 prints ONE JSON line.  Top-level fields describe the headline
workload (focal, the baseline file's second configuration); `workloads` carries the same
measurements for the other four configurations (1-GPU runs only, unless --workload says
otherwise).

  value      logit elements / s, forward+backward, inputs resident in HBM, timed with CUDA
             events over K steps (max over ranks), step captured in a CUDA graph when possible
  e2e        the same through the public module with pinned HOST inputs: H2D copy of logits
             and labels, forward, backward, D2H read of the loss, every step
  roofline   per C-ABI entry point (forward, backward): algorithmic bytes / average duration of
             K back-to-back launches of that entry point between one pair of CUDA events
             (rotating input sets, preallocated outputs); peak from MEASURED_PEAKS.json
             (hbm_gbs) or the 6650 GB/s fallback
  cpu_baseline  the CPU port (oracle/) on the host cores, bounded sample, N=1 only

`--impl reference` times the CPU port alone and prints the same line shape.
L2 hygiene: every workload rotates 3 distinct input sets (each larger than L2 together
with its gradient), so step k+1 never finds step k's lines in the 126 MB L2.
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
sys.path.insert(0, os.path.join(ROOT, "pytorch-loss_b200"))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

import bench_workloads as BW  # noqa: E402

N_SETS = 3
FALLBACK_HBM_GBS = 6650.0


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.lines, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def wait_first(self, timeout=3.0):
        """Blocks until the sampler has delivered its first line (or `timeout` seconds): the start
        of nvidia-smi (NVML initialisation over every GPU of the box, once per rank) must not fall
        into the timed region, which lasts about a millisecond."""
        t0 = time.perf_counter()
        while self.proc is not None and not self.lines and time.perf_counter() - t0 < timeout:
            time.sleep(0.01)

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
        return False

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
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
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def dist_env():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return world, rank, local


def time_cpu(fn, x, y, steps, warmup):
    for _ in range(warmup):
        fn(x, y)
    best = []
    for _ in range(steps):
        t0 = time.perf_counter()
        fn(x, y)
        best.append(time.perf_counter() - t0)
    return best


def cpu_baseline(wl, steps=3, warmup=1):
    """The CPU port on a bounded sample of the workload, all host threads."""
    from oracle import losses as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    items = min(wl.cpu_sample_items, wl.shape[0])
    x, y = wl.make(items=items)
    if wl.dtype == torch.float16:
        x = x.float()                       # the reference's V1 upcasts half inputs on the CPU
    times = time_cpu(wl.oracle(O), x, y, steps, warmup)
    elems = x.numel()
    return {"value": elems / min(times), "unit": "logit elements/s", "cores": cores, "kind": "port",
            "sample": "%d of %d batch items of %s, forward+backward, best of %d" % (items, wl.shape[0], wl.name, steps),
            "seconds_per_sample": min(times)}


def run_reference_arm(args):
    """`--impl reference`: the reference's CPU path (restated in oracle/) on the host cores."""
    world, rank, _ = dist_env()
    if rank != 0:
        return
    from oracle import losses as O
    wl = BW.WORKLOADS[BW.HEADLINE if args.workload in ("all", None) else args.workload]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    items = min(wl.cpu_sample_items, wl.shape[0])
    x, y = wl.make(items=items)
    if wl.dtype == torch.float16:
        x = x.float()
    times = time_cpu(wl.oracle(O), x, y, args.steps, args.warmup)
    ms = 1e3 * sum(times) / len(times)
    value = x.numel() / (ms / 1e3)
    sample = "%d of %d batch items per step" % (items, wl.shape[0])
    line = {
        "impl": "reference", "metric": "logit elements/s forward+backward", "value": value,
        "unit": "logit elements/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl.desc, "sample": sample},
        "cpu_baseline": {"value": value, "unit": "logit elements/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "logit elements/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def make_sets(wl, device, rank):
    """N_SETS distinct (logits, labels) pairs on the device; set 0 is the CPU-seeded one."""
    sets = []
    x0, y0 = wl.make(seed_offset=1000 * rank)
    sets.append((x0.to(device), y0.to(device)))
    for r in range(1, N_SETS):
        sets.append(wl.make(seed_offset=1000 * rank + 100 * r, device=device))
    return sets, (x0, y0)


def step_eager(crit, x, y):
    x.grad = None
    loss = crit(x, y)
    loss.backward()
    return loss


def try_capture(crit, sets):
    """One CUDA graph per input set holding forward+backward; None if capture fails."""
    graphs = []
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for x, y in sets:
                for _ in range(2):
                    step_eager(crit, x, y)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        for x, y in sets:
            x.grad = None
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                loss = crit(x, y)
                loss.backward()
            graphs.append((g, loss))
        torch.cuda.synchronize()
        return graphs
    except Exception as exc:  # capture is an optimisation, eager is always available
        sys.stderr.write("bench: CUDA graph capture unavailable (%s); timing eager steps\n" % (exc,))
        torch.cuda.synchronize()
        return None


def reduction_collective(world):
    """How the ranks' [sum, count] pairs were added in this run."""
    if world <= 1:
        return "none"
    from pytorch_loss import _p2p
    if any(ex is not None for ex in _p2p._contexts.values()):
        return "in-kernel exchange: peer stores into IPC-mapped slots, bounded local wait"
    return "16-byte NCCL all-reduce"


def direct_calls(wl, sets, device):
    """(forward, backward) callables that launch the workload's two C-ABI entry points on
    input set i with preallocated outputs: what `roofline` times."""
    from pytorch_loss import _cabi
    lib = _cabi.load_library()
    P = _cabi.ptr
    st = _cabi.stream_ptr(device)
    ws = _cabi.reduce_workspace(device)
    recs = [_cabi.new_record(device) for _ in sets]
    grads = [torch.empty_like(x) for x, _ in sets]
    one = torch.ones(1, dtype=torch.float32, device=device)
    xs = [x.detach() for x, _ in sets]
    ys = [y for _, y in sets]
    n, c = wl.shape[0], wl.shape[1]
    m = wl.elems // (n * c)
    dt = _cabi.dtype_code(xs[0])
    denoms = [_cabi._vp(r.data_ptr() + 8) for r in recs]
    if wl.name == "focal":
        e = wl.elems
        # the module's training step: fused forward+backward kernel, then the rescale kernel that
        # leaves at once for an upstream gradient of 1
        fwd = lambda i: _cabi.check(lib.b200_focal_forward_backward_reduced(
            P(xs[i]), P(ys[i]), P(grads[i]), P(recs[i]), P(ws), ws.numel(), None, 1.0 / e, e, dt, 2.0, 0.25, st))
        bwd = lambda i: _cabi.check(lib.b200_rescale_gradient(P(grads[i]), P(one), None, e, dt, st))
        return fwd, bwd
    if wl.name == "lovasz":
        nbytes = int(lib.b200_lovasz_workspace_bytes(n, c, m, 1))
        lws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        loss = torch.empty(n, c, dtype=torch.float32, device=device)
        jacc = torch.empty(n, c, m, dtype=torch.float32, device=device)
        up = torch.full((n, c), 1.0 / (n * c), dtype=torch.float32, device=device)
        fwd = lambda i: _cabi.check(lib.b200_lovasz_forward(P(xs[i]), P(ys[i]), P(loss), P(jacc), P(lws), nbytes,
                                                            n, c, m, dt, 255, 1, st))
        bwd = lambda i: _cabi.check(lib.b200_lovasz_backward(P(up), P(xs[i]), P(ys[i]), P(jacc), P(grads[i]),
                                                             n, c, m, dt, 255, 1, st))
        return fwd, bwd
    if wl.name == "ohem":
        nbytes = int(lib.b200_ohem_workspace_bytes(n, m))
        ows = torch.empty(nbytes, dtype=torch.uint8, device=device)
        new_labels = [torch.empty_like(y) for y in ys]
        n_min = (n * m) // 16

        cnts = [_cabi.new_record(device) for _ in sets]

        def fwd(i):
            _cabi.check(lib.b200_ohem_label(P(xs[i]), P(ys[i]), P(new_labels[i]), P(ows), nbytes, n, c, m, dt, 255,
                                            0.7, n_min, st))
            _cabi.check(lib.b200_count_valid(P(new_labels[i]), n * m, 255, P(cnts[i]), P(ws), ws.numel(), st))
            _cabi.check(lib.b200_lsr_forward_backward_reduced(
                P(xs[i]), P(new_labels[i]), P(grads[i]), P(recs[i]), P(ws), ws.numel(),
                _cabi._vp(cnts[i].data_ptr() + 8), n, c, m, dt, 255, 0.0, st))
        bwd = lambda i: _cabi.check(lib.b200_rescale_gradient(P(grads[i]), P(one), None, wl.elems, dt, st))
        return fwd, bwd
    stem, hyper, ign = {"lsr": ("lsr", 0.1, 255), "lsr_rows": ("lsr", 0.1, -100), "lmargin": ("lmargin", 0.3, 255)}[wl.name]
    if os.environ.get("B200_SOFTMAX_FUSED", "1") != "0":
        # the module's training step: count of valid labels, then ONE pass over the logits that sums
        # the loss and writes the final gradient; backward is the rescale kernel (upstream gradient 1)
        if not lib.b200_softmax_fused_step_path(P(xs[0]), P(ys[0]), P(grads[0]), n, c, m, dt):
            raise SystemExit("bench: workload %s has no fused step on this build" % wl.name)
        f_step = getattr(lib, "b200_%s_forward_backward_reduced" % stem)
        cnts = [_cabi.new_record(device) for _ in sets]

        def fwd(i):
            _cabi.check(lib.b200_count_valid(P(ys[i]), n * m, ign, P(cnts[i]), P(ws), ws.numel(), st))
            _cabi.check(f_step(P(xs[i]), P(ys[i]), P(grads[i]), P(recs[i]), P(ws), ws.numel(),
                               _cabi._vp(cnts[i].data_ptr() + 8), n, c, m, dt, ign, hyper, st))
        bwd = lambda i: _cabi.check(lib.b200_rescale_gradient(P(grads[i]), P(one), None, wl.elems, dt, st))
        return fwd, bwd
    if lib.b200_softmax_stats_path(P(xs[0]), P(ys[0]), P(grads[0]), n, c, m, dt):
        # many classes: the module hands per-pixel statistics from forward to backward
        f_fwd, f_bwd = getattr(lib, "b200_%s_forward_ex" % stem), getattr(lib, "b200_%s_backward_ex" % stem)
        stats = [torch.empty((n * m, 4), dtype=torch.float32, device=device) for _ in sets]
        fwd = lambda i: _cabi.check(f_fwd(P(xs[i]), P(ys[i]), None, P(recs[i]), P(ws), ws.numel(), P(stats[i]),
                                          n, c, m, dt, ign, hyper, st))
        bwd = lambda i: _cabi.check(f_bwd(P(xs[i]), P(ys[i]), P(stats[i]), P(one), 1, denoms[i], P(grads[i]),
                                          n, c, m, dt, ign, hyper, st))
        for i in range(len(sets)):
            fwd(i)                      # backward launches below read these statistics
        return fwd, bwd
    f_fwd, f_bwd = getattr(lib, "b200_%s_forward" % stem), getattr(lib, "b200_%s_backward" % stem)
    fwd = lambda i: _cabi.check(f_fwd(P(xs[i]), P(ys[i]), None, P(recs[i]), P(ws), ws.numel(), n, c, m, dt, ign, hyper, st))
    bwd = lambda i: _cabi.check(f_bwd(P(xs[i]), P(ys[i]), P(one), 1, denoms[i], P(grads[i]), n, c, m, dt, ign, hyper, st))
    return fwd, bwd


def time_entries(wl, sets, device, args, peak):
    """Per-entry-point durations: K back-to-back launches of the entry point through the C ABI
    (rotating input sets, preallocated outputs) between one pair of CUDA events, so the queue
    stays full and the figure is the kernels' own time, not the host's."""
    fwd_name, bwd_name = wl.entries()
    fwd_call, bwd_call = direct_calls(wl, sets, device)
    kernels = {}
    for name, call, nbytes in ((fwd_name, fwd_call, wl.bytes_forward()), (bwd_name, bwd_call, wl.bytes_backward())):
        for k in range(args.warmup):
            call(k % N_SETS)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for k in range(args.steps):
            call(k % N_SETS)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / args.steps
        gbs = nbytes / (ms / 1e3) / 1e9
        kernels[name] = {"calls": args.steps, "avg_ms": ms, "algorithmic_bytes": nbytes,
                         "achieved_gbs": gbs, "frac": gbs / peak}
    return kernels


def measure_workload(wl, args, device, world, rank, with_cpu, with_e2e):
    import pytorch_loss as P
    from pytorch_loss import _cabi
    lib = _cabi.load_library()
    peak, peak_kind = measured_peak()
    group = True if world > 1 else None
    crit = wl.criterion(P, process_group=group)
    sets, host0 = make_sets(wl, device, rank)
    for x, _ in sets:
        x.requires_grad_(True)
    if args.kernels_only:
        # short path for profiler captures: only the two entry points, launched back to back
        kernels = time_entries(wl, sets, device, args, peak)
        _cabi.read_status(device)
        return {"workload": wl.desc, "shape": list(wl.shape), "kernels_only": True, "kernels": kernels}

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput
    graphs = None if args.no_graph else try_capture(crit, sets)
    launches_before = lib.b200_kernel_launch_count()
    step_eager(crit, *sets[0])
    torch.cuda.synchronize()
    launches_per_step = lib.b200_kernel_launch_count() - launches_before

    def run_steps(n):
        for k in range(n):
            if graphs is not None:
                graphs[k % N_SETS][0].replay()
            else:
                step_eager(crit, *sets[k % N_SETS])

    run_steps(args.warmup)
    barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(device.index) as clocks:
        clocks.wait_first()
        run_steps(args.warmup)
        barrier()
        start.record()
        run_steps(args.steps)
        end.record()
        barrier()
        ms_total = start.elapsed_time(end)
        if world > 1:
            t = torch.tensor([ms_total], dtype=torch.float64, device=device)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            ms_total = float(t.item())
        # The K timed steps last about a millisecond, less than one nvidia-smi sample: keep the
        # same steps running (untimed) for about half a second so the clocks are sampled under
        # this load.  The count derives from the agreed time: every rank runs the same number of
        # extra steps (they may contain a cross-rank exchange).
        t_load = time.perf_counter()
        for _ in range(min(2000, max(1, int(500.0 / max(1e-3, ms_total))))):
            run_steps(args.steps)
        torch.cuda.synchronize()
        clock_window_s = time.perf_counter() - t_load
    ms_step = ms_total / args.steps
    value = world * wl.elems / (ms_step / 1e3)

    kernels = time_entries(wl, sets, device, args, peak)
    fwd_name, bwd_name = wl.entries()
    dominant = max(kernels, key=lambda k: kernels[k]["avg_ms"]) if kernels else None
    roofline = None
    if dominant:
        d = kernels[dominant]
        roofline = {"bound": "hbm", "kernel": dominant, "achieved": d["achieved_gbs"], "peak": peak,
                    "unit": "GB/s", "frac": d["frac"], "peak_source": peak_kind + " (MEASURED_PEAKS.json hbm_gbs)"
                    if peak_kind == "measured" else "fallback 6650 GB/s",
                    "traffic": wl.traffic_forward() if dominant == fwd_name else wl.traffic_backward(),
                    "step_frac": wl.bytes_step() / (ms_step / 1e3) / 1e9 / peak, "kernels": kernels}

    # ---- end to end from pinned host memory (eager, public module API)
    e2e = None
    if with_e2e:
        hx, hy = host0[0].pin_memory(), host0[1].pin_memory()
        dx = torch.empty_like(sets[0][0]).detach().requires_grad_(True)
        dy = torch.empty_like(sets[0][1])

        def e2e_step():
            with torch.no_grad():
                dx.copy_(hx, non_blocking=True)
                dy.copy_(hy, non_blocking=True)
            return float(step_eager(crit, dx, dy).item())

        for _ in range(max(1, args.warmup // 2)):
            e2e_step()
        n_e2e = max(3, min(args.steps, 10))
        barrier()
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            e2e_step()
        barrier()
        dt = (time.perf_counter() - t0) / n_e2e
        if world > 1:
            t = torch.tensor([dt], dtype=torch.float64, device=device)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            dt = float(t.item())
        e2e = {"value": world * wl.elems / dt, "unit": "logit elements/s",
               "h2d_bytes_per_step": hx.numel() * hx.element_size() + hy.numel() * hy.element_size(),
               "d2h_bytes_per_step": 4, "ms_per_step": dt * 1e3, "steps": n_e2e}

    _cabi.read_status(device)       # raises if any kernel gave up a bounded wait
    res = {
        "workload": wl.desc, "value": value, "ms_per_step": ms_step, "graph": graphs is not None,
        "launches_per_step": int(launches_per_step), "roofline": roofline, "e2e": e2e,
        "clocks": dict(clocks.summary(), window="the K timed steps + %.2f s of the same steps" % clock_window_s),
    }
    if with_cpu and rank == 0:
        res["cpu_baseline"] = cpu_baseline(wl)
    del sets, graphs
    torch.cuda.empty_cache()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=None, help="one of %s, or all" % ", ".join(BW.WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="time eager steps instead of CUDA-graph replays")
    ap.add_argument("--items", type=int, default=None,
                    help="batch items per GPU instead of the configuration's (reduced cases for profiler captures)")
    ap.add_argument("--kernels-only", action="store_true",
                    help="only launch the forward and backward entry points back to back (profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference_arm(args)
        return

    world, rank, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); "
                         "use --impl reference for the CPU port")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=device)
    which = args.workload or ("all" if world == 1 else BW.HEADLINE)
    names = list(BW.WORKLOADS) if which == "all" else [which]
    headline = BW.HEADLINE if BW.HEADLINE in names else names[0]

    results = {}
    for name in [headline] + [n for n in names if n != headline]:
        wl = BW.WORKLOADS[name]
        if args.items:
            wl = wl.with_items(args.items)
        try:
            results[name] = measure_workload(wl, args, device, world, rank, with_cpu=(world == 1),
                                             with_e2e=True)
        except Exception as exc:
            if name == headline:
                raise
            results[name] = {"workload": wl.desc, "error": repr(exc)}
            torch.cuda.synchronize()

    if rank == 0 and args.kernels_only:
        print(json.dumps({"kernels_only": True, "steps": args.steps, "warmup": args.warmup, "workloads": results}))
    elif rank == 0:
        h = results[headline]
        wl = BW.WORKLOADS[headline]
        if args.items:
            wl = wl.with_items(args.items)
        line = {
            "metric": "logit elements/s forward+backward", "value": h["value"], "unit": "logit elements/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": h["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16" if wl.dtype == torch.float16 else "f32", "data": "synthetic",
            "config": {"workload": wl.desc, "per_gpu_shape": list(wl.shape),
                       "l2": "3 rotating input sets, each larger than L2 with its gradient",
                       "cuda_graph": h["graph"], "reduction_collective": reduction_collective(world)},
            "roofline": h["roofline"], "cpu_baseline": h.get("cpu_baseline"), "e2e": h["e2e"],
            "gpu_launches": h["launches_per_step"] * args.steps, "clocks": h["clocks"],
            "workloads": {k: v for k, v in results.items() if k != headline},
        }
        print(json.dumps(line))
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
