#!/usr/bin/env python
"""Builds the reference project's own V3 CUDA extensions for sm_100a, unmodified, from the
reference checkout, so that the benchmark can time them beside this library on the same GPU and
so that fixtures can be generated from the reference's CUDA-only OHEM step.

    python baseline/build_reference_v3.py [--ref /path/to/pytorch-loss] [--only focal_cpp,...]

Nothing of the reference is committed: every output goes to baseline/_ref/ (ignored by git, still
shipped with a GPU job): one `<name>.so` per extension (lsr_cpp, focal_cpp, large_margin_cpp,
lovasz_softmax_cpp, ohem_cpp, taylor_softmax_cpp), compiled straight from `csrc/*.cu` where they
lie, and the package `reference_py/`: the reference's Python modules that call those extensions (the same files a
`pip install --target` of the reference would place there), in the copies that match the
current extension signatures:
    focal_loss.py, large_margin_softmax.py, lovasz_softmax.py, taylor_softmax.py, pc_softmax.py
    (repository root; the last one has no extension behind it: tensor ops)
    label_smooth.py, ohem_loss.py (pytorch_loss/; the root label_smooth.py does not import on
    torch >= 2.4 because it calls torch.amp.custom_fwd without device_type).
Compilation needs nvcc only (no GPU); each extension takes 2-3 minutes.
"""
import argparse
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

EXTENSIONS = {
    "lsr_cpp": "lsr_kernel.cu",
    "focal_cpp": "focal_kernel.cu",
    "large_margin_cpp": "large_margin_kernel.cu",
    "lovasz_softmax_cpp": "lovasz_softmax.cu",
    "ohem_cpp": "ohem_label_kernel.cu",
    "taylor_softmax_cpp": "taylor_softmax.cu",
}
PY_MODULES = {
    "focal_loss.py": "focal_loss.py",
    "large_margin_softmax.py": "large_margin_softmax.py",
    "lovasz_softmax.py": "lovasz_softmax.py",
    "taylor_softmax.py": "taylor_softmax.py",
    "pc_softmax.py": "pc_softmax.py",
    "label_smooth.py": os.path.join("pytorch_loss", "label_smooth.py"),
    "ohem_loss.py": os.path.join("pytorch_loss", "ohem_loss.py"),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("PYTORCH_LOSS_REFERENCE"),
                    help="checkout of CoinCheung/pytorch-loss (or set PYTORCH_LOSS_REFERENCE)")
    ap.add_argument("--only", default=None)
    args = ap.parse_args()
    if not args.ref or not os.path.isdir(os.path.join(args.ref, "csrc")):
        sys.exit("no reference checkout at %s (pass --ref or set PYTORCH_LOSS_REFERENCE)" % args.ref)
    os.environ["TORCH_CUDA_ARCH_LIST"] = "10.0a"
    os.environ.setdefault("MAX_JOBS", str(os.cpu_count() or 4))
    from torch.utils import cpp_extension
    os.makedirs(os.path.join(OUT, "reference_py"), exist_ok=True)
    names = args.only.split(",") if args.only else list(EXTENSIONS)
    for name in names:
        target = os.path.join(OUT, name + ".so")
        if os.path.exists(target):
            print("have", target)
            continue
        bdir = os.path.join(OUT, "build_" + name)
        os.makedirs(bdir, exist_ok=True)
        cpp_extension.load(name=name, sources=[os.path.join(args.ref, "csrc", EXTENSIONS[name])],
                           extra_include_paths=[os.path.join(args.ref, "csrc")], build_directory=bdir,
                           is_python_module=False, verbose=True)
        shutil.copy(os.path.join(bdir, name + ".so"), target)
        shutil.rmtree(bdir)
        print("built", target)
    for dst, src in PY_MODULES.items():
        shutil.copy(os.path.join(args.ref, src), os.path.join(OUT, "reference_py", dst))
    open(os.path.join(OUT, "reference_py", "__init__.py"), "w").close()    # ohem_loss.py imports its sibling relatively
    print("reference V3 build complete:", sorted(os.listdir(OUT)))


if __name__ == "__main__":
    main()
