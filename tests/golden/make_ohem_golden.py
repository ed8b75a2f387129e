#!/usr/bin/env python
"""Generates tests/golden/ohem.npz from the reference project's own CUDA extension.

The reference has its OHEM relabelling (`ohem_cpp.score_ohem_label`, csrc/ohem_label_kernel.cu)
in CUDA only, so unlike the other fixtures (make_golden.py, CPU) this one needs a GPU and the
extension built unmodified for it by baseline/build_reference_v3.py:

    python tests/golden/make_ohem_golden.py [--out tests/golden/ohem.npz]

Stored per case: seeded inputs (continuous random logits, so score ties have measure zero;
rounded to fp16-representable values and stored as fp16 to keep the file small -- the reference
and every test see the same fp32 numbers), the arguments, and the labels the reference returned.
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))

# (shape, ignore fraction, score_thresh, n_min as a fraction of the pixels (None: exact count below), dtype)
CASES = [
    ((2, 19, 20, 24), 0.10, 0.7, 1 / 16, torch.float32),     # 960 pixels: the block-per-pixel kernel at C < 32
    ((1, 5, 72, 64), 0.05, 0.7, 1 / 16, torch.float32),     # 4608 pixels: the thread-per-pixel kernel (C < 32, > 4096 px)
    ((1, 5, 72, 64), 0.05, 0.3, 1 / 2, torch.float32),
    ((2, 150, 6, 10), 0.10, 0.05, 1 / 4, torch.float32),     # block-per-pixel kernel
    ((64, 10), 0.0, 0.3, 1 / 16, torch.float32),             # no spatial dims
    ((1, 5, 16, 16), 0.20, 0.7, 0.0, torch.float32),         # n_min = 0: the threshold alone decides
    ((1, 5, 16, 16), 0.20, 0.99, 0.999, torch.float32),      # n_min = P - 1
    ((1, 5, 16, 16), 0.20, 0.7, 2.0, torch.float32),         # n_min > P: labels returned unchanged
]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(HERE, "ohem.npz"))
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    import ohem_cpp                                  # the reference's extension, not this repository's shim
    assert ohem_cpp.__file__.endswith(".so"), ohem_cpp.__file__
    out = {"n_cases": np.int64(len(CASES))}
    for i, (shape, frac, thresh, nfrac, dtype) in enumerate(CASES):
        g = torch.Generator().manual_seed(4000 + i)
        logits = (torch.randn(shape, generator=g) * 2.0).half().to(dtype)
        lshape = shape[:1] + shape[2:]
        labels = torch.randint(0, shape[1], lshape, generator=g)
        if frac > 0:
            labels[torch.rand(lshape, generator=g) < frac] = 255
        n_min = int(labels.numel() * nfrac)
        got = ohem_cpp.score_ohem_label(logits.cuda().float(), labels.cuda(), 255, thresh, n_min)
        torch.cuda.synchronize()
        out["c%d_logits" % i] = logits.half().numpy()
        out["c%d_labels" % i] = labels.numpy()
        out["c%d_args" % i] = np.array([255, thresh, n_min], dtype=np.float64)
        out["c%d_new_labels" % i] = got.cpu().numpy()
        print("case %d %s thresh %.2f n_min %d: %d of %d valid labels kept" % (
            i, shape, thresh, n_min, int((got != 255).sum()), int((labels != 255).sum())))
    np.savez_compressed(args.out, **out)
    print("wrote", args.out, os.path.getsize(args.out), "bytes")


if __name__ == "__main__":
    main()
