#!/usr/bin/env python
"""Benchmark of the fused V3 loss path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME|all] [--impl reference]

A step is one forward + backward of a loss module over one synthetic batch
(bench_workloads.py).  Rank 0 prints ONE JSON line.  Top-level fields describe the headline
workload: the baseline file's third configuration (LargeMarginSoftmaxV3 fp32 [8,150,512,512]),
the largest one it shards over GPUs.  `workloads` carries the same measurements for the other
configurations and `table` (last key) repeats every workload in compact form.

  value      logit elements / s, forward+backward, inputs resident in HBM, timed with CUDA
             events over K x R steps (R = `run.replays_per_step`, chosen so that the timed
             region lasts at least 50 ms; max over ranks), step captured in a CUDA graph
  e2e        the same through the public module with pinned HOST inputs: H2D copy of logits
             and labels, forward, backward, D2H read of the loss, every step
  roofline   per C-ABI entry point (forward, backward): algorithmic bytes / average duration of
             K back-to-back launches of that entry point between one pair of CUDA events
             (rotating input sets, preallocated outputs); peak from MEASURED_PEAKS.json
             (hbm_gbs) or the 6650 GB/s fallback; traffic from profiles/dram_traffic.json
  cpu_baseline  the CPU port (oracle/) on the host cores, bounded sample, N=1 only
  reference_v3  (per workload, N=1 only) the reference project's own V3 CUDA extensions, built
             unmodified for sm_100a, timed by baseline/reference_v3.py in a process of its own

Multi-GPU (torchrun, one rank per GPU): STRONG scaling.  The configuration's one global batch is
split over the ranks along the batch axis (rank r holds N/G items), the modules add their
[sum, count] pairs over the ranks, `value` = global elements / slowest rank's time.  The focal
configuration (one 64 MB tensor) is additionally kept as a weak-scaling entry under `workloads`.

`--impl reference` times the CPU port alone and prints the same line shape.
L2 hygiene: every workload rotates 3 distinct input sets; where one set with its gradient is
smaller than L2 (multi-GPU shards) a 256 MB buffer is overwritten between timed steps.
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
MIN_TIMED_MS = 60.0
L2_BYTES = 126 << 20
# workloads the reference's own V3 CUDA build is timed on (N=1): every one of them ran to the end
# on a B200 when first tried; a workload whose reference kernels fault or hang is taken off here
REFERENCE_V3_WORKLOADS = ("lmargin", "lsr", "focal", "lsr_rows", "lovasz", "lovasz_full", "ohem", "focal_up2",
                          "lmargin_none", "lsr_none", "taylor", "taylor_c150", "pc_softmax", "lsr_nhwc", "lmargin_nhwc", "lsr_cls", "lsr_769")


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def measured_traffic(wl):
    """(forward, backward) DRAM bytes per launch from the committed extract of the ncu captures
    (profiles/dram_traffic.json: bytes per logit element on a reduced batch; traffic grows in
    proportion to the batch), or (None, None) for a workload without a capture."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as fh:
            recs = json.load(fh)["workloads"]
        # (reduction 'none' variants: the separate kernels of their kind; other layouts: own captures only)
        rec = recs.get(wl.name) or (recs[wl.kind] if (wl.layout == 'nchw' and len(wl.shape) > 2 and wl.pixels // wl.shape[0] % 4 == 0) else None)
        key = "fused" if (wl.fused_softmax() or wl.kind not in ("lsr", "lsr_rows", "lmargin")) else "separate"
        f, b = rec[key]
        return f * wl.elems, b * wl.elems
    except Exception:
        return None, None


def traffic_from_ncu(args):
    """`--traffic-from CSV --workload W --items I --launches L`: turns the ncu CSV of a
    `bench.py --workload W --items I --kernels-only` run (metrics dram__bytes_read.sum,
    dram__bytes_write.sum; L = warm-up + timed launches of each entry point) into the workload's
    entry of profiles/dram_traffic.json: DRAM bytes per logit element of the forward and of the
    backward entry point.  Kernels of the backward entry: the gradient rescale, the Lovasz
    and the Taylor backward; everything else of this library belongs to the forward entry (other kernels are skipped)."""
    import csv
    import re
    wl = BW.WORKLOADS[args.workload].with_items(args.items) if args.items else BW.WORKLOADS[args.workload]
    rows = list(csv.reader(ln for ln in open(args.traffic_from) if ln.startswith('"')))
    col = {h: i for i, h in enumerate(rows[0])}
    scale = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}
    sums = [0.0, 0.0]
    for r in rows[1:]:
        if not r[col["Metric Name"]].startswith("dram__bytes_"):
            continue
        name = r[col["Kernel Name"]]
        if "b200::" not in name:                      # torch's own kernels (input generation, fills)
            continue
        bwd = re.search(r"rescale_kernel|lovasz_pair_kernel<\(?(bool\))?1|lovasz_tile_kernel<\(?(bool\))?1|"
                        r"taylor_resident_kernel<\(?(bool\))?1|taylor_sliced_kernel<\(?(bool\))?1|"
                        r"taylor_spatial_kernel<[^,]+, [^,]+, \(?(bool\))?1|"
                        r"taylor_rows_kernel<[^,]+, \(?(bool\))?1", name) is not None
        sums[1 if bwd else 0] += float(r[col["Metric Value"]].replace(",", "")) * scale[r[col["Metric Unit"]]]
    per_elem = [round(v / args.launches / wl.elems, 3) for v in sums]
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    with open(path) as fh:
        doc = json.load(fh)
    key = "fused" if (wl.fused_softmax() or wl.kind not in ("lsr", "lsr_rows", "lmargin")) else "separate"
    entry = doc["workloads"].setdefault(args.workload, {})
    entry[key] = per_elem
    entry["capture"] = "bench.py --workload %s --items %d --kernels-only, %d launches per entry point" % (
        args.workload, wl.shape[0], args.launches)
    with open(path, "w") as fh:
        json.dump(doc, fh, indent=1)
        fh.write("\n")
    print(args.workload, key, per_elem)


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
        into the timed region."""
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


def bind_to_gpu_numa_node(index):
    """Pins this process to the CPUs next to its GPU, so the pinned host buffers of the end-to-end
    leg are allocated on that GPU's NUMA node (eight ranks pulling through one node halve each
    other's copy rate).  A property of this process only; no GPU setting is touched."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = [64 * i + b for i, w in enumerate(words) for b in range(64) if (w >> b) & 1]
        allowed = sorted(set(cpus) & set(os.sched_getaffinity(0)))
        if allowed:
            os.sched_setaffinity(0, allowed)
            return "cpus %d-%d (%d)" % (allowed[0], allowed[-1], len(allowed))
    except Exception as exc:                                   # noqa: BLE001  optional
        return "not bound (%s)" % type(exc).__name__
    return "not bound"


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


def base_config(wl):
    """The `config` both arms print: the workload only (run-specific facts go to `run`)."""
    return {"workload": wl.desc}


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
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": base_config(wl),
        "cpu_baseline": {"value": value, "unit": "logit elements/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "logit elements/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "run": {"sample": sample},
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


def step_eager(crit, x, y, up=None):
    """One forward+backward.  `up is DENSE`: the module is an activation, not a loss -- the set's
    second tensor is the upstream gradient."""
    x.grad = None
    loss = crit(x) if up is DENSE else crit(x, y)
    loss.backward(y if up is DENSE else up)
    return loss


DENSE = object()


def try_capture(crit, sets, up):
    """One CUDA graph per input set holding forward+backward; None if capture fails."""
    graphs = []
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for x, y in sets:
                for _ in range(2):
                    step_eager(crit, x, y, up)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        for x, y in sets:
            x.grad = None
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                loss = step_eager(crit, x, y, up)
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


def check_all_status(device):
    """Raises if any kernel of this process gave up a bounded wait: every reduction workspace
    (one per stream, the capture streams' included) and every exchange workspace is read."""
    from pytorch_loss import _cabi, _p2p
    lib = _cabi.load_library()
    torch.cuda.synchronize()
    spaces = list(_cabi._workspaces.values())
    for ex in _p2p._contexts.values():
        if ex is not None:
            spaces.extend(ex._workspaces.values())
    for ws in spaces:
        _cabi.check(lib.b200_read_status(_cabi.ptr(ws), _cabi.stream_ptr(device)))
    return len(spaces)


def direct_calls(wl, sets, device):
    """(forward, backward) callables that launch the workload's two C-ABI entry points on
    input set i with preallocated outputs: what `roofline` times.  Local sums only (no exchange
    attached): these are the kernels' own times."""
    from pytorch_loss import _cabi
    lib = _cabi.load_library()
    P = _cabi.ptr
    st = _cabi.stream_ptr(device)
    ws = _cabi.reduce_workspace(device)
    recs = [_cabi.new_record(device) for _ in sets]
    grads = [torch.empty_like(x) for x, _ in sets]
    up = torch.full((1,), float(wl.upstream), dtype=torch.float32, device=device)
    xs = [x.detach() for x, _ in sets]
    ys = [y for _, y in sets]
    n, c = wl.shape[0], wl.shape[1]
    m = wl.elems // (n * c)
    if wl.layout == 'nhwc':                 # every pixel is a row of C contiguous logits
        n, m = n * m, 1
    dt = _cabi.dtype_code(xs[0])
    denoms = [_cabi._vp(r.data_ptr() + 8) for r in recs]
    rescale = lambda i: _cabi.check(lib.b200_rescale_gradient(P(grads[i]), P(up), None, wl.elems, dt, st))
    if wl.kind == "focal":
        e = wl.elems
        # the module's training step: fused forward+backward kernel, then the rescale kernel that
        # leaves at once for an upstream gradient of 1
        fwd = lambda i: _cabi.check(lib.b200_focal_forward_backward_reduced(
            P(xs[i]), P(ys[i]), P(grads[i]), P(recs[i]), P(ws), ws.numel(), None, 1.0 / e, e, dt, 2.0, 0.25, 0, st))
        return fwd, rescale
    if wl.kind == "lovasz":
        nbytes = int(lib.b200_lovasz_workspace_bytes(n, c, m, 1))
        lws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        loss = torch.empty(n, c, dtype=torch.float32, device=device)
        jacc = torch.empty(n, c, m, dtype=torch.float32, device=device)
        upl = torch.full((n, c), 1.0 / (n * c), dtype=torch.float32, device=device)
        fwd = lambda i: _cabi.check(lib.b200_lovasz_forward(P(xs[i]), P(ys[i]), P(loss), P(jacc), P(lws), nbytes,
                                                            n, c, m, dt, 255, 1, st))
        bwd = lambda i: _cabi.check(lib.b200_lovasz_backward(P(upl), P(xs[i]), P(ys[i]), P(jacc), P(grads[i]),
                                                             n, c, m, dt, 255, 1, st))
        return fwd, bwd
    if wl.kind == "ohem":
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
                _cabi._vp(cnts[i].data_ptr() + 8), n, c, m, dt, 255, 0.0, _cabi.STEP_AFTER_COUNT, st))
        return fwd, rescale
    if wl.kind == "taylor":
        outs = [torch.empty_like(x) for x in xs]
        fwd = lambda i: _cabi.check(lib.b200_taylor_softmax_forward(P(xs[i]), P(outs[i]), n, c, m, dt, 2, 1, st))
        bwd = lambda i: _cabi.check(lib.b200_taylor_softmax_backward(P(ys[i]), P(xs[i]), P(grads[i]), n, c, m, dt, 2, 1, st))
        return fwd, bwd
    if wl.kind == "pc_softmax":
        w = torch.tensor(wl.proportions(), dtype=torch.float32, device=device)
        cnts = [_cabi.new_record(device) for _ in sets]
        if not lib.b200_pc_softmax_step_path(P(xs[0]), P(ys[0]), P(grads[0]), n, c, m, dt):
            raise SystemExit("bench: workload %s has no fused step on this build" % wl.name)

        def fwd(i):
            _cabi.check(lib.b200_count_valid(P(ys[i]), n * m, 255, P(cnts[i]), P(ws), ws.numel(), st))
            _cabi.check(lib.b200_pc_softmax_step(P(xs[i]), P(ys[i]), P(w), P(grads[i]), P(recs[i]), P(ws), ws.numel(),
                                                 _cabi._vp(cnts[i].data_ptr() + 8), n, c, m, dt, 255,
                                                 _cabi.STEP_AFTER_COUNT, st))
        return fwd, rescale
    stem, hyper, ign = {"lsr": ("lsr", 0.1, 255), "lsr_rows": ("lsr", 0.1, -100), "lmargin": ("lmargin", 0.3, 255)}[wl.kind]
    if wl.reduction == 'none':
        # per-pixel losses out, a per-pixel upstream gradient in: the separate kernels
        px = [torch.empty_like(y, dtype=xs[0].dtype) for y in ys]
        upx = wl.upstream_tensor(device).to(xs[0].dtype)
        if lib.b200_softmax_stats_path(P(xs[0]), P(ys[0]), P(grads[0]), n, c, m, dt):
            f_fwd, f_bwd = getattr(lib, "b200_%s_forward_ex" % stem), getattr(lib, "b200_%s_backward_ex" % stem)
            stats = [torch.empty((n * m, 4), dtype=torch.float32, device=device) for _ in sets]
            fwd = lambda i: _cabi.check(f_fwd(P(xs[i]), P(ys[i]), P(px[i]), None, None, 0, P(stats[i]),
                                              n, c, m, dt, ign, hyper, st))
            bwd = lambda i: _cabi.check(f_bwd(P(xs[i]), P(ys[i]), P(stats[i]), P(upx), 2, None, P(grads[i]),
                                              n, c, m, dt, ign, hyper, st))
            for i in range(len(sets)):
                fwd(i)
            return fwd, bwd
        f_fwd, f_bwd = getattr(lib, "b200_%s_forward" % stem), getattr(lib, "b200_%s_backward" % stem)
        fwd = lambda i: _cabi.check(f_fwd(P(xs[i]), P(ys[i]), P(px[i]), None, None, 0, n, c, m, dt, ign, hyper, st))
        bwd = lambda i: _cabi.check(f_bwd(P(xs[i]), P(ys[i]), P(upx), 2, None, P(grads[i]), n, c, m, dt, ign, hyper, st))
        return fwd, bwd
    if wl.fused_softmax():
        # the module's training step: count of valid labels, then ONE pass over the logits that sums
        # the loss and writes the final gradient; backward is the rescale kernel (upstream gradient 1)
        if not lib.b200_softmax_fused_step_path(P(xs[0]), P(ys[0]), P(grads[0]), n, c, m, dt):
            raise SystemExit("bench: workload %s has no fused step on this build" % wl.name)
        f_step = getattr(lib, "b200_%s_forward_backward_reduced" % stem)
        cnts = [_cabi.new_record(device) for _ in sets]

        def fwd(i):
            _cabi.check(lib.b200_count_valid(P(ys[i]), n * m, ign, P(cnts[i]), P(ws), ws.numel(), st))
            _cabi.check(f_step(P(xs[i]), P(ys[i]), P(grads[i]), P(recs[i]), P(ws), ws.numel(),
                               _cabi._vp(cnts[i].data_ptr() + 8), n, c, m, dt, ign, hyper, _cabi.STEP_AFTER_COUNT, st))
        return fwd, rescale
    one = torch.ones(1, dtype=torch.float32, device=device)
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


def reference_v3(name, args):
    """The reference's own V3 CUDA build on the same GPU, in a process of its own."""
    script = os.path.join(ROOT, "baseline", "reference_v3.py")
    if name not in REFERENCE_V3_WORKLOADS:
        return {"unavailable": "not run for this workload"}
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref")):
        return {"unavailable": "baseline/_ref not built (python baseline/build_reference_v3.py)"}
    cmd = [sys.executable, script, "--workload", name, "--steps", str(min(args.steps, 10)), "--warmup", "3"]
    if args.items:
        cmd += ["--items", str(args.items)]
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
        lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
        if not lines:
            return {"unavailable": "no output (rc %d): %s" % (r.returncode, r.stderr.strip().splitlines()[-1][:200]
                                                                if r.stderr.strip() else "")}
        out = json.loads(lines[-1])
        out.pop("workload", None)
        return out
    except subprocess.TimeoutExpired:
        return {"unavailable": "timed out after 240 s"}
    except Exception as exc:                                   # noqa: BLE001
        return {"unavailable": repr(exc)[:200]}


def measure_workload(wl, args, device, world, rank, with_cpu, with_e2e, with_entries, sharded):
    import pytorch_loss as P
    from pytorch_loss import _cabi
    lib = _cabi.load_library()
    peak, peak_kind = measured_peak()
    group = True if (world > 1 and wl.kind != "ohem") else None
    crit = wl.criterion(P, process_group=group)
    sets, host0 = make_sets(wl, device, rank)
    for x, _ in sets:
        x.requires_grad_(True)
    if args.kernels_only:
        # short path for profiler captures: only the two entry points, launched back to back
        kernels = time_entries(wl, sets, device, args, peak)
        check_all_status(device)
        return {"workload": wl.desc, "shape": list(wl.shape), "kernels_only": True, "kernels": kernels}
    up = DENSE if wl.kind == "taylor" else wl.upstream_tensor(device)
    scalar_loss = wl.kind != "taylor" and wl.reduction != 'none'

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput
    graphs = None if args.no_graph else try_capture(crit, sets, up)
    launches_before = lib.b200_kernel_launch_count()
    step_eager(crit, *sets[0], up)
    torch.cuda.synchronize()
    launches_per_step = lib.b200_kernel_launch_count() - launches_before

    set_bytes = sum(t.numel() * t.element_size() for t in sets[0]) + sets[0][0].numel() * sets[0][0].element_size()
    flush = None
    if N_SETS * set_bytes < 2 * L2_BYTES:
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def run_steps(n):
        for k in range(n):
            if flush is not None:
                flush.fill_(k & 1)
            if graphs is not None:
                graphs[k % N_SETS][0].replay()
            else:
                step_eager(crit, *sets[k % N_SETS], up)

    def timed(n):
        """Milliseconds of n steps on the device.  With an L2 flush between steps the flushes
        are timed on their own and subtracted."""
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        run_steps(n)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        if flush is not None:
            a.record()
            for k in range(n):
                flush.fill_(k & 1)
            b.record()
            torch.cuda.synchronize()
            ms -= a.elapsed_time(b)
        return ms

    run_steps(args.warmup)
    barrier()
    # R: replays per counted step, so that the timed region lasts MIN_TIMED_MS at least (agreed
    # over the ranks: they must all run the same number of steps)
    est = max(timed(args.steps) / args.steps, 1e-3)
    if world > 1:
        t = torch.tensor([est], dtype=torch.float64, device=device)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        est = float(t.item())
    replays = max(1, int(-(-MIN_TIMED_MS // (est * args.steps))))
    with ClockSampler(device.index) as clocks:
        clocks.wait_first()
        run_steps(args.warmup)
        barrier()
        ms_total = timed(args.steps * replays)
        barrier()
        if world > 1:
            t = torch.tensor([ms_total], dtype=torch.float64, device=device)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            ms_total = float(t.item())
        # keep the same steps running (untimed) until the sampler has seen about half a second of
        # this load; the count derives from the agreed time, so every rank runs the same number
        t_load = time.perf_counter()
        extra = max(0, int((500.0 - ms_total) / max(1e-3, ms_total / (args.steps * replays))))
        run_steps(min(extra, 20000))
        torch.cuda.synchronize()
        clock_window_s = time.perf_counter() - t_load + ms_total / 1e3
    ms_step = ms_total / (args.steps * replays)
    value = world * wl.elems / (ms_step / 1e3)      # strong: world x shard = the global batch; weak: world x batch

    roofline = None
    if with_entries:
        kernels = time_entries(wl, sets, device, args, peak)
        fwd_name, bwd_name = wl.entries()
        dominant = max(kernels, key=lambda k: kernels[k]["avg_ms"])
        d = kernels[dominant]
        tf, tb = measured_traffic(wl)
        roofline = {"bound": "hbm", "kernel": dominant, "achieved": d["achieved_gbs"], "peak": peak,
                    "unit": "GB/s", "frac": d["frac"], "peak_source": peak_kind + " (MEASURED_PEAKS.json hbm_gbs)"
                    if peak_kind == "measured" else "fallback 6650 GB/s",
                    "traffic": tf if dominant == fwd_name else tb,
                    "step_frac": wl.bytes_step() / (ms_step / 1e3) / 1e9 / peak, "kernels": kernels}
    step_frac = wl.bytes_step() / (ms_step / 1e3) / 1e9 / peak

    # ---- end to end from pinned host memory (eager, public module API)
    e2e = None
    if with_e2e and scalar_loss:
        hx, hy = host0[0].pin_memory(), host0[1].pin_memory()
        dx = torch.empty_like(sets[0][0]).detach().requires_grad_(True)
        dy = torch.empty_like(sets[0][1])

        def e2e_step():
            with torch.no_grad():
                dx.copy_(hx, non_blocking=True)
                dy.copy_(hy, non_blocking=True)
            return float(step_eager(crit, dx, dy, up).item())

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
        del hx, hy, dx, dy

    n_spaces = check_all_status(device)       # raises if any kernel gave up a bounded wait
    res = {
        "workload": wl.desc, "value": value, "ms_per_step": ms_step, "graph": graphs is not None,
        "replays_per_step": replays, "timed_region_ms": ms_total, "step_frac": step_frac,
        "launches_per_step": int(launches_per_step), "roofline": roofline, "e2e": e2e,
        "l2": "3 rotating input sets" + (" + a 256 MB buffer overwritten between steps (its time subtracted)"
                                        if flush is not None else ", each larger than L2 with its gradient"),
        "status_words_checked": n_spaces,
        "clocks": dict(clocks.summary(), window="the timed steps + the same steps again, %.2f s in all" % clock_window_s),
    }
    if with_cpu and rank == 0:
        res["cpu_baseline"] = cpu_baseline(wl)
    del sets, graphs, flush
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
    ap.add_argument("--no-reference-v3", action="store_true", help="skip the reference's CUDA build")
    ap.add_argument("--traffic-from", default=None, help="ncu CSV to turn into an entry of profiles/dram_traffic.json")
    ap.add_argument("--launches", type=int, default=0, help="with --traffic-from: launches of each entry point in the CSV")
    args = ap.parse_args()
    if args.traffic_from:
        traffic_from_ncu(args)
        return
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference_arm(args)
        return

    world, rank, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); "
                         "use --impl reference for the CPU port")
    numa = bind_to_gpu_numa_node(local)
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=device)
    which = args.workload or "all"
    if which == "all":
        names = list(BW.WORKLOADS) if world == 1 else list(BW.SHARDED) + [BW.WEAK]
    else:
        names = [which]
    headline = BW.HEADLINE if BW.HEADLINE in names else names[0]

    results, shard_of = {}, {}
    for name in [headline] + [n for n in names if n != headline]:
        wl = BW.WORKLOADS[name]
        sharded = world > 1 and name in BW.SHARDED and not args.items
        key = name
        if args.items:
            wl = wl.with_items(args.items)
        elif sharded:
            if wl.shape[0] % world:
                results[name] = {"workload": wl.desc, "error": "batch of %d does not split over %d ranks" % (wl.shape[0], world)}
                continue
            wl = wl.with_items(wl.shape[0] // world, note=" [rank shard: %d of %d items]" % (wl.shape[0] // world, wl.shape[0]))
        elif world > 1:
            key = name + "_weak"
        shard_of[key] = (wl, sharded)
        try:
            results[key] = measure_workload(wl, args, device, world, rank, with_cpu=(world == 1),
                                            with_e2e=True, with_entries=(world == 1 or name == headline),
                                            sharded=sharded)
            results[key]["scaling"] = "strong" if (sharded or world == 1) else "weak"
            if world == 1 and rank == 0 and not args.kernels_only and not args.no_reference_v3:
                ref = reference_v3(name, args)
                if "ms_per_step" in ref:
                    ref["ours_over_theirs"] = ref["ms_per_step"] / results[key]["ms_per_step"]
                results[key]["reference_v3"] = ref
        except Exception as exc:
            if name == headline:
                raise
            results[key] = {"workload": wl.desc, "error": repr(exc)[:300]}
            torch.cuda.synchronize()

    if rank == 0 and args.kernels_only:
        print(json.dumps({"kernels_only": True, "steps": args.steps, "warmup": args.warmup, "workloads": results}))
    elif rank == 0:
        h = results[headline]
        wl_full = BW.WORKLOADS[headline]
        wl, sharded = shard_of[headline]
        table = {}
        for k, v in results.items():
            if "error" in v:
                table[k] = "error"
                continue
            ref = v.get("reference_v3") or {}
            table[k] = [round(v["ms_per_step"], 4), round(v["step_frac"], 3), v["scaling"],
                        round(ref["ms_per_step"], 4) if "ms_per_step" in ref else None]
        line = {
            "metric": "logit elements/s forward+backward", "value": h["value"], "unit": "logit elements/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": h["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16" if wl.dtype == torch.float16 else "f32", "data": "synthetic",
            "config": base_config(wl_full if not args.items else wl),
            "run": {"per_gpu_shape": list(wl.shape), "global_shape": list(wl_full.shape if not args.items else wl.shape),
                    "l2": h["l2"], "cuda_graph": h["graph"], "replays_per_step": h["replays_per_step"],
                    "timed_region_ms": h["timed_region_ms"], "reduction_collective": reduction_collective(world),
                    "host_numa_binding": numa},
            "roofline": h["roofline"], "cpu_baseline": h.get("cpu_baseline"), "e2e": h["e2e"],
            "gpu_launches": h["launches_per_step"] * args.steps * h["replays_per_step"], "clocks": h["clocks"],
            "reference_v3": h.get("reference_v3"),
            "workloads": {k: v for k, v in results.items() if k != headline},
            "table_columns": ["ms_per_step", "fraction of HBM peak (algorithmic bytes of the step)", "scaling",
                              "reference V3 CUDA ms_per_step (N=1)"],
            "table": table,
        }
        print(json.dumps(line))
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
