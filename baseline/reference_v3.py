#!/usr/bin/env python
"""Times the reference project's own V3 CUDA path on this GPU: its unmodified extensions
(built for sm_100a by baseline/build_reference_v3.py into baseline/_ref/) driven through its own
Python modules, eager forward + backward on the benchmark's tensors, CUDA events.

    python baseline/reference_v3.py --workload lmargin [--steps 20] [--warmup 5] [--items N]

Prints ONE JSON line: {"workload", "ms_per_step", "elems_per_s", "loss", ...} or
{"workload", "unavailable": "<why>"}.  Runs in a process of its own: nothing of this repository's
library is imported (only bench_workloads.py for the seeded tensors), so the number cannot be
routed through this repository's kernels.

What runs, per workload (reference file:line):
  lsr, lsr_rows  LabelSmoothSoftmaxCEV3          pytorch_loss/label_smooth.py:148-171 + lsr_cpp
  focal          FocalLossV3                      focal_loss.py:174-200 + focal_cpp
  lmargin        LargeMarginSoftmaxV3 (fb=True)   large_margin_softmax.py:197-229 + large_margin_cpp
  lovasz(_full)  LovaszSoftmaxV3                  lovasz_softmax.py:94-116 + lovasz_softmax_cpp.
                 The reference sorts the whole batch as one group and has no per-image mode, so
                 the benchmark's per-image loss is a Python loop over the images (mean of the
                 per-image losses, one backward).
  ohem           OhemCELoss                       pytorch_loss/ohem_loss.py:13-28 + ohem_cpp
"""
import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF = os.path.join(HERE, "_ref")
N_SETS = 3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", required=True)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--items", type=int, default=None)
    ap.add_argument("--dump", default=None, help="write loss and gradient of input set 0 to this .pt file")
    args = ap.parse_args()
    out = {"workload": args.workload, "impl": "reference V3 CUDA extensions, unmodified, sm_100a"}
    try:
        out.update(run(args))
    except Exception as exc:                                  # noqa: BLE001  reported, not raised
        out["unavailable"] = "%s: %s" % (type(exc).__name__, str(exc).splitlines()[0][:300] if str(exc) else "")
    print(json.dumps(out))


def run(args):
    if not os.path.isdir(os.path.join(REF, "reference_py")):
        raise RuntimeError("baseline/_ref is not built (python baseline/build_reference_v3.py)")
    sys.path.insert(0, REF)
    sys.path.insert(0, ROOT)
    import warnings
    warnings.filterwarnings("ignore", category=FutureWarning)
    import torch
    import bench_workloads as BW
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device")
    dev = torch.device("cuda", 0)
    wl = BW.WORKLOADS[args.workload]
    if args.items:
        wl = wl.with_items(args.items)

    kind = wl.kind
    if kind in ("lsr", "lsr_rows"):
        from reference_py import label_smooth as M
        crit = M.LabelSmoothSoftmaxCEV3(0.1, wl.reduction, 255 if kind == "lsr" else -100)
        step = lambda x, y: crit(x, y)
    elif kind == "focal":
        from reference_py import focal_loss as M
        crit = M.FocalLossV3(0.25, 2, 'mean')
        step = lambda x, y: crit(x, y)
    elif kind == "lmargin":
        from reference_py import large_margin_softmax as M
        crit = M.LargeMarginSoftmaxV3(0.3, wl.reduction, 255)
        step = lambda x, y: crit(x, y)
    elif kind == "lovasz":
        from reference_py import lovasz_softmax as M
        crit = M.LovaszSoftmaxV3('mean', 255)
        step = lambda x, y: torch.stack([crit(x[i:i + 1], y[i:i + 1]) for i in range(x.shape[0])]).mean()
    elif kind == "ohem":
        from reference_py import ohem_loss as M
        crit = M.OhemCELoss(0.7, None, 255)
        step = lambda x, y: crit(x, y)
    elif kind == "taylor":
        from reference_py import taylor_softmax as M
        crit = M.LogTaylorSoftmaxV3(dim=1, n=2)
        step = lambda x, g: crit(x)               # the set's second tensor is the upstream gradient
    elif kind == "pc_softmax":
        # (no CUDA extension in the reference for this one: its V2 Function is made of torch ops)
        from reference_py import pc_softmax as M
        crit = M.PCSoftmaxCrossEntropyV2(wl.proportions(), 'mean', 255)
        step = lambda x, y: crit(x, y)
    else:
        raise RuntimeError("no reference V3 module for workload kind %s" % kind)

    sets = []
    x0, y0 = wl.make()
    sets.append((x0.to(dev).requires_grad_(True), y0.to(dev)))
    for r in range(1, N_SETS):
        x, y = wl.make(seed_offset=100 * r, device=dev)
        sets.append((x.requires_grad_(True), y))
    up = wl.upstream_tensor(dev)

    def one(k):
        x, y = sets[k % N_SETS]
        x.grad = None
        loss = step(x, y)
        loss.backward(y if kind == "taylor" else up)
        return loss

    loss0 = one(0)
    torch.cuda.synchronize()
    if args.dump:
        torch.save({"loss": loss0.detach().float().cpu(), "grad": sets[0][0].grad.detach().cpu()}, args.dump)
    for k in range(args.warmup):
        one(k)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for k in range(args.steps):
        one(k)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / args.steps
    return {"ms_per_step": ms, "elems_per_s": wl.elems / (ms / 1e3), "steps": args.steps, "loss": float(loss0.detach().float().sum()),
            "shape": list(wl.shape), "mode": "eager module forward+backward, %d rotating input sets" % N_SETS}


if __name__ == "__main__":
    main()
