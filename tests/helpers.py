"""Shared helpers of the GPU parity tests: tolerances stated by the task
(fp32: loss 1e-5 relative, gradients 1e-5 abs + 1e-5 rel; fp16: 2e-3) and seeded inputs."""
import numpy as np
import torch

LOSS_RTOL_F32 = 1e-5
GRAD_ATOL_F32 = 1e-5
GRAD_RTOL_F32 = 1e-5
TOL_F16 = 2e-3


def assert_loss_close(got, want, rtol=LOSS_RTOL_F32, atol=1e-7, what="loss"):
    got = got.detach().double().cpu()
    want = want.detach().double().cpu()
    assert got.shape == want.shape, "%s: shape %s vs %s" % (what, tuple(got.shape), tuple(want.shape))
    both_nan = torch.isnan(got) & torch.isnan(want)
    err = (got - want).abs() - (atol + rtol * want.abs())
    err = torch.where(both_nan, torch.full_like(err, -1.0), err)
    assert bool((err <= 0).all()), "%s: max violation %g (got %s want %s)" % (
        what, float(err.max()), got.flatten()[:4].tolist(), want.flatten()[:4].tolist())


def assert_grad_close(got, want, atol=GRAD_ATOL_F32, rtol=GRAD_RTOL_F32, what="grad"):
    got = got.detach().double().cpu()
    want = want.detach().double().cpu()
    assert got.shape == want.shape, "%s: shape %s vs %s" % (what, tuple(got.shape), tuple(want.shape))
    err = (got - want).abs() - (atol + rtol * want.abs())
    assert bool((err <= 0).all()), "%s: max violation %g at %d" % (what, float(err.max()), int(err.argmax()))


def labels_with_ignores(gen, shape, n_classes, ignore_index, frac):
    lb = torch.randint(0, n_classes, shape, generator=gen)
    if frac > 0:
        lb[torch.rand(shape, generator=gen) < frac] = ignore_index
    return lb


def run_module(crit, logits, labels):
    """loss and d(loss.sum())/d(logits) of a module on the logits' device."""
    x = logits.detach().clone().requires_grad_(True)
    out = crit(x, labels)
    (out.sum() if out.dim() else out).backward()
    return out.detach(), x.grad.detach()
