"""CPU oracle of Taylor softmax and the cross entropy built on it — TEST INFRASTRUCTURE, NOT A
PRODUCT PATH.

Parity status: PINNED.  tests/golden/make_golden.py runs the reference's pure-PyTorch
`taylor_softmax_v1` and `TaylorCrossEntropyLossV1` (pytorch_loss/taylor_softmax.py:38-46,
:148-171) on seeded inputs and stores inputs and outputs in tests/golden/taylor.npz;
tests/test_oracle_golden.py checks this file's functions against them.

Only tests/, the smoke check and bench.py's CPU legs may import this module.
"""
import math

import torch
import torch.nn.functional as F


def _series(x, order):
    """sum_{i=0..order} x^i / i!   (reference pytorch_loss/taylor_softmax.py:40-44)."""
    out = torch.ones_like(x)
    for i in range(1, order + 1):
        out = out + x.pow(i) / math.factorial(i)
    return out


def taylor_softmax(x, dim=1, n=4, use_log=False, upstream=None, dtype=torch.float32):
    """(activation, gradient of sum(activation * upstream) with respect to x).

    Forward: f / sum_dim f, optionally its log (reference :38-46).  The gradient is written out
    in closed form, the one the reference's CUDA backward uses (csrc/taylor_softmax.cu:176-265):
    softmax  dx = f'/S * (g - sum_dim(g * out)),   log  dx = f' * (g / f - sum_dim(g) / S)."""
    assert n % 2 == 0 and n > 0
    x = x.detach().to(dtype)
    f = _series(x, n)
    s = f.sum(dim=dim, keepdim=True)
    out = f / s
    if use_log:
        out = out.log()
    if upstream is None:
        return out, None
    g = upstream.to(dtype)
    d = _series(x, n - 1)
    if use_log:
        grad = d * (g / f - g.sum(dim=dim, keepdim=True) / s)
    else:
        grad = d / s * (g - (g * f / s).sum(dim=dim, keepdim=True))
    return out, grad


def taylor_cross_entropy(logits, labels, n=2, ignore_index=-1, reduction='mean'):
    """TaylorCrossEntropyLoss (reference pytorch_loss/taylor_softmax.py:148-171): nll_loss of
    the log-Taylor softmax over dim 1.  Returns (loss, d loss / d logits) through autograd."""
    x = logits.detach().float().requires_grad_(True)
    f = _series(x, n)
    logp = (f / f.sum(dim=1, keepdim=True)).log()
    loss = F.nll_loss(logp, labels, reduction=reduction, ignore_index=ignore_index)
    (loss.sum() if loss.dim() else loss).backward()
    return loss.detach(), x.grad
