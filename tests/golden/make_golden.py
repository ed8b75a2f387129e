#!/usr/bin/env python
"""Generates tests/golden/*.npz from the UNMODIFIED reference implementation.

Run where the reference checkout is mounted (argument or $PYTORCH_LOSS_REFERENCE):

    python tests/golden/make_golden.py /path/to/pytorch-loss

The reference's V3 classes need its CUDA extensions, so empty stand-in modules are
registered for `lsr_cpp`, `focal_cpp`, `large_margin_cpp`, `lovasz_softmax_cpp` before the
files are loaded by path; only the pure-PyTorch V1/V2 classes are then used, on CPU.
Which copy of each file is loaded: `pytorch_loss/label_smooth.py` (the root copy does not
import on current torch), root `focal_loss.py`, `pytorch_loss/large_margin_softmax.py` for
V1 (the root V1 multiplies 0 by inf) and root `large_margin_softmax.py` for V2, root
`lovasz_softmax.py`.

Each case stores its inputs, hyper-parameters, and the reference's loss and
d(loss)/d(logits) so the files are self-contained.
"""
import importlib.util
import os
import sys
import types
import warnings

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root):
    for name in ("lsr_cpp", "focal_cpp", "large_margin_cpp", "lovasz_softmax_cpp", "taylor_softmax_cpp"):
        sys.modules.setdefault(name, types.ModuleType(name))

    def load(rel, alias):
        spec = importlib.util.spec_from_file_location(alias, os.path.join(root, rel))
        mod = importlib.util.module_from_spec(spec)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            spec.loader.exec_module(mod)
        return mod

    return {
        "lsr": load("pytorch_loss/label_smooth.py", "ref_label_smooth"),
        "focal": load("focal_loss.py", "ref_focal_loss"),
        "lm_v1": load("pytorch_loss/large_margin_softmax.py", "ref_large_margin_installed"),
        "lm_v2": load("large_margin_softmax.py", "ref_large_margin_root"),
        "lovasz": load("lovasz_softmax.py", "ref_lovasz"),
        "taylor": load("pytorch_loss/taylor_softmax.py", "ref_taylor_softmax"),
        "pc": load("pc_softmax.py", "ref_pc_softmax"),
    }


def run(crit, logits, labels, take_first=False):
    x = logits.clone().requires_grad_(True)
    out = crit(x, labels)
    if take_first:
        out = out[0]
    (out.sum() if out.dim() else out).backward()
    return out.detach().numpy(), x.grad.numpy()


def labels_with_ignores(gen, shape, n_classes, ignore_index, frac):
    lb = torch.randint(0, n_classes, shape, generator=gen)
    if frac > 0:
        lb[torch.rand(shape, generator=gen) < frac] = ignore_index
    return lb


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("PYTORCH_LOSS_REFERENCE")
    if not root:
        sys.exit("usage: make_golden.py <checkout of CoinCheung/pytorch-loss>  (or set PYTORCH_LOSS_REFERENCE)")
    ref = load_reference(root)
    torch.set_num_threads(1)
    out = {}

    # ---- label smooth: (shape, smooth, ignore_index, ignore fraction, reduction)
    cases = [((2, 19, 8, 9), 0.1, 255, 0.2, 'mean'), ((3, 7, 5, 4), 0.25, -100, 0.3, 'sum'),
             ((6, 5), 0.1, -100, 0.0, 'mean'), ((2, 33, 4, 3), 0.05, 3, 0.0, 'none'),
             ((4, 150, 3, 5), 0.1, 255, 0.1, 'mean')]
    d = {}
    for i, (shape, sm, ign, frac, red) in enumerate(cases):
        g = torch.Generator().manual_seed(100 + i)
        logits = torch.randn(shape, generator=g) * 2.0
        labels = labels_with_ignores(g, (shape[0],) + shape[2:], shape[1], ign, frac)
        l1, g1 = run(ref["lsr"].LabelSmoothSoftmaxCEV1(sm, red, ign), logits, labels)
        l2, g2 = run(ref["lsr"].LabelSmoothSoftmaxCEV2(sm, red, ign), logits, labels)
        d.update({f"c{i}_logits": logits.numpy(), f"c{i}_labels": labels.numpy(),
                  f"c{i}_hyper": np.array([sm, ign], dtype=np.float64), f"c{i}_reduction": np.array(red),
                  f"c{i}_loss_v1": l1, f"c{i}_grad_v1": g1, f"c{i}_loss_v2": l2, f"c{i}_grad_v2": g2})
    d["n_cases"] = np.array(len(cases))
    out["label_smooth"] = d

    # ---- focal: (shape, alpha, gamma, soft labels?, reduction)
    cases = [((2, 3, 7, 5), 0.25, 2.0, False, 'mean'), ((2, 1, 9, 8), 0.25, 2.0, False, 'sum'),
             ((3, 4, 5), 0.4, 1.5, True, 'mean'), ((5, 6), 0.25, 3.0, True, 'none')]
    d = {}
    for i, (shape, al, ga, soft, red) in enumerate(cases):
        g = torch.Generator().manual_seed(200 + i)
        logits = torch.randn(shape, generator=g) * 3.0
        labels = torch.rand(shape, generator=g)
        labels = torch.sigmoid(4 * labels - 2) if soft else (labels < 0.3).float()
        l1, g1 = run(ref["focal"].FocalLossV1(al, ga, red), logits, labels)
        l2, g2 = run(ref["focal"].FocalLossV2(al, ga, red), logits, labels)
        d.update({f"c{i}_logits": logits.numpy(), f"c{i}_labels": labels.numpy(),
                  f"c{i}_hyper": np.array([al, ga], dtype=np.float64), f"c{i}_reduction": np.array(red),
                  f"c{i}_loss_v1": l1, f"c{i}_grad_v1": g1, f"c{i}_loss_v2": l2, f"c{i}_grad_v2": g2})
    d["n_cases"] = np.array(len(cases))
    out["focal"] = d

    # ---- large margin: V1/V2 drop ignored pixels from the unreduced output, so only
    # 'mean'/'sum' are stored (the unreduced V3 layout is covered by the oracle tests).
    cases = [((2, 7, 6, 5), 0.3, 255, 0.2, 'mean'), ((3, 19, 4, 4), 0.5, 255, 0.0, 'sum'),
             ((8, 10), 0.3, 255, 0.25, 'mean'), ((2, 150, 3, 4), 0.3, 255, 0.1, 'mean')]
    d = {}
    for i, (shape, lam, ign, frac, red) in enumerate(cases):
        g = torch.Generator().manual_seed(300 + i)
        logits = torch.randn(shape, generator=g)
        labels = labels_with_ignores(g, (shape[0],) + shape[2:], shape[1], ign, frac)
        l1, g1 = run(ref["lm_v1"].LargeMarginSoftmaxV1(lam, red, ign), logits, labels)
        l2, g2 = run(ref["lm_v2"].LargeMarginSoftmaxV2(lam, red, ign), logits, labels)
        d.update({f"c{i}_logits": logits.numpy(), f"c{i}_labels": labels.numpy(),
                  f"c{i}_hyper": np.array([lam, ign], dtype=np.float64), f"c{i}_reduction": np.array(red),
                  f"c{i}_loss_v1": l1, f"c{i}_grad_v1": g1, f"c{i}_loss_v2": l2, f"c{i}_grad_v2": g2})
    d["n_cases"] = np.array(len(cases))
    out["large_margin"] = d

    # ---- lovasz (V1 only; returns (loss, errs)); the per-image entries loop V1 over images
    cases = [((2, 5, 12, 11), 255, 0.1, 'mean'), ((1, 19, 16, 16), -100, 0.0, 'none'),
             ((3, 4, 9, 7), 255, 0.3, 'sum'), ((2, 7, 20, 10), 255, 0.05, 'none')]
    d = {}
    for i, (shape, ign, frac, red) in enumerate(cases):
        g = torch.Generator().manual_seed(400 + i)
        logits = torch.randn(shape, generator=g)
        labels = labels_with_ignores(g, (shape[0],) + shape[2:], shape[1], ign, frac)
        crit = ref["lovasz"].LovaszSoftmaxV1(red, ign)
        l1, g1 = run(crit, logits, labels, take_first=True)
        crit_none = ref["lovasz"].LovaszSoftmaxV1('none', ign)
        per_img = [run(crit_none, logits[k:k + 1], labels[k:k + 1], take_first=True) for k in range(shape[0])]
        d.update({f"c{i}_logits": logits.numpy(), f"c{i}_labels": labels.numpy(),
                  f"c{i}_hyper": np.array([ign], dtype=np.float64), f"c{i}_reduction": np.array(red),
                  f"c{i}_loss_v1": l1, f"c{i}_grad_v1": g1,
                  f"c{i}_loss_per_image": np.stack([p[0] for p in per_img]),
                  f"c{i}_grad_per_image": np.concatenate([p[1] for p in per_img])})
    d["n_cases"] = np.array(len(cases))
    out["lovasz"] = d

    # ---- taylor softmax (V1 function: activation and its autograd gradient for a random upstream
    # gradient), and the cross entropy built on it: (shape, dim, n, use_log)
    cases = [((2, 7, 5, 6), 1, 2, False), ((2, 7, 5, 6), 1, 4, True), ((3, 4, 6), 2, 6, False),
             ((5, 3, 4, 2), 0, 2, True), ((4, 19), 1, 8, True), ((2, 33, 3, 5), 1, 4, False)]
    d = {}
    for i, (shape, dim, order, use_log) in enumerate(cases):
        g = torch.Generator().manual_seed(500 + i)
        x = (torch.randn(shape, generator=g) * 1.5).requires_grad_(True)
        up = torch.randn(shape, generator=g)
        y = ref["taylor"].taylor_softmax_v1(x, dim, order, use_log)
        y.backward(up)
        d.update({f"c{i}_x": x.detach().numpy(), f"c{i}_up": up.numpy(), f"c{i}_out": y.detach().numpy(),
                  f"c{i}_grad": x.grad.numpy(), f"c{i}_hyper": np.array([dim, order, int(use_log)])})
    d["n_cases"] = np.array(len(cases))
    ce_cases = [((3, 6, 5, 4), 4, 255, 0.2, 'mean'), ((2, 19, 4, 4), 2, -1, 0.0, 'sum')]
    for i, (shape, order, ign, frac, red) in enumerate(ce_cases):
        g = torch.Generator().manual_seed(550 + i)
        logits = torch.randn(shape, generator=g)
        labels = labels_with_ignores(g, (shape[0],) + shape[2:], shape[1], ign, frac)
        crit = ref["taylor"].TaylorCrossEntropyLossV1(n=order, ignore_index=ign, reduction=red)
        l1, g1 = run(crit, logits, labels)
        d.update({f"ce{i}_logits": logits.numpy(), f"ce{i}_labels": labels.numpy(),
                  f"ce{i}_hyper": np.array([order, ign]), f"ce{i}_reduction": np.array(red),
                  f"ce{i}_loss": l1, f"ce{i}_grad": g1})
    d["n_ce_cases"] = np.array(len(ce_cases))
    out["taylor"] = d

    # ---- PC softmax cross entropy: V1 (loss and its autograd gradient) and V2 (its loss; V2's own
    # hand-written backward, which scales by the label's proportion, is stored for the record).
    # V1's constructor moves the proportions with `.cuda()`; on this CPU-only run that one call is
    # made a no-op while the object is built (the reference's code is not touched).
    cases = [((2, 5, 6, 7), 255, 0.2, 'mean'), ((3, 19, 4, 4), 255, 0.0, 'sum'), ((6, 7), -100, 0.0, 'mean'),
             ((2, 4, 5, 3), 255, 0.3, 'none')]
    d = {}
    for i, (shape, ign, frac, red) in enumerate(cases):
        g = torch.Generator().manual_seed(600 + i)
        logits = torch.randn(shape, generator=g) * 2.0
        labels = labels_with_ignores(g, (shape[0],) + shape[2:], shape[1], ign, frac)
        prop = torch.rand(shape[1], generator=g) + 0.05
        prop = (prop / prop.sum()).tolist()
        real_cuda = torch.Tensor.cuda
        torch.Tensor.cuda = lambda self, *a, **k: self
        try:
            crit1 = ref["pc"].PCSoftmaxCrossEntropyV1(prop, ignore_index=ign, reduction=red)
        finally:
            torch.Tensor.cuda = real_cuda
        l1, g1 = run(crit1, logits, labels)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            l2, g2 = run(ref["pc"].PCSoftmaxCrossEntropyV2(prop, red, ign), logits, labels)
        d.update({f"c{i}_logits": logits.numpy(), f"c{i}_labels": labels.numpy(),
                  f"c{i}_proportion": np.array(prop, dtype=np.float64),
                  f"c{i}_hyper": np.array([ign], dtype=np.float64), f"c{i}_reduction": np.array(red),
                  f"c{i}_loss_v1": l1, f"c{i}_grad_v1": g1, f"c{i}_loss_v2": l2, f"c{i}_grad_v2_as_written": g2})
    d["n_cases"] = np.array(len(cases))
    out["pc_softmax"] = d

    only = os.environ.get("GOLDEN_ONLY")               # e.g. GOLDEN_ONLY=taylor rewrites one file
    for name, d in out.items():
        if only and name != only:
            continue
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **d)
        print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
