"""Taylor softmax, log-Taylor softmax and Taylor cross entropy on the B200 CUDA library.

Drop-in for the reference's V3 classes and functions (pytorch_loss/taylor_softmax.py:15-35,
:76-98, :122-144, :175-198; extension functions csrc/taylor_softmax.cu:391-421):
`TaylorSoftmaxFunc`, `taylor_softmax_v3`, `TaylorSoftmaxV3(dim=1, n=2)`,
`LogTaylorSoftmaxV3(dim=1, n=2)`, `TaylorCrossEntropyLossV3(n=2, ignore_index=-1,
reduction='mean')`.  `dim` may be any dimension (negative values count from the end).
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F
import torch.amp as amp

from . import _cabi


def _view(feat, dim):
    """(N, C, M) of `feat` around `dim`, and `dim` normalised."""
    if feat.dim() == 0:
        raise RuntimeError("taylor softmax needs at least one dimension")
    d = dim + feat.dim() if dim < 0 else dim
    if not 0 <= d < feat.dim():
        raise RuntimeError("dim %d out of range for a %d-dimensional tensor" % (dim, feat.dim()))
    shape = feat.shape
    return math.prod(shape[:d]), shape[d], math.prod(shape[d + 1:]), d


def taylor_softmax_forward(feat, dim, n, use_log):
    """The extension function of the reference: activation tensor like `feat`."""
    dev = _cabi.require_cuda(feat)
    feat = feat.contiguous()
    nn_, c, m, _ = _view(feat, int(dim))
    out = torch.empty_like(feat)
    lib = _cabi.load_library()
    with torch.cuda.device(dev):
        _cabi.check(lib.b200_taylor_softmax_forward(
            _cabi.ptr(feat), _cabi.ptr(out), nn_, c, m, _cabi.dtype_code(feat), int(n), int(bool(use_log)),
            _cabi.stream_ptr(dev)))
    return out


def taylor_softmax_backward(grad, feat, dim, n, use_log):
    """Gradient with respect to `feat` for the upstream gradient `grad` (same shape)."""
    dev = _cabi.require_cuda(grad, feat)
    feat = feat.contiguous()
    grad = grad.to(feat.dtype).contiguous()
    nn_, c, m, _ = _view(feat, int(dim))
    out = torch.empty_like(feat)
    lib = _cabi.load_library()
    with torch.cuda.device(dev):
        _cabi.check(lib.b200_taylor_softmax_backward(
            _cabi.ptr(grad), _cabi.ptr(feat), _cabi.ptr(out), nn_, c, m, _cabi.dtype_code(feat), int(n),
            int(bool(use_log)), _cabi.stream_ptr(dev)))
    return out


class TaylorSoftmaxFunc(torch.autograd.Function):
    """Reference pytorch_loss/taylor_softmax.py:17-34."""

    @staticmethod
    @amp.custom_fwd(cast_inputs=torch.float32, device_type='cuda')
    def forward(ctx, feat, dim=1, n=2, use_log=False):
        ctx.vars = feat, dim, n, use_log
        return taylor_softmax_forward(feat, dim, n, use_log)

    @staticmethod
    @amp.custom_bwd(device_type='cuda')
    def backward(ctx, grad_output):
        feat, dim, n, use_log = ctx.vars
        return taylor_softmax_backward(grad_output, feat, dim, n, use_log), None, None, None


def taylor_softmax_v3(inten, dim=1, n=4, use_log=False):
    assert n % 2 == 0 and n > 0
    return TaylorSoftmaxFunc.apply(inten, dim, n, use_log)


class TaylorSoftmaxV3(nn.Module):

    def __init__(self, dim=1, n=2):
        super().__init__()
        assert n % 2 == 0 and n > 0
        self.dim = dim
        self.n = n

    def forward(self, x):
        return taylor_softmax_v3(x, self.dim, self.n, use_log=False)


class LogTaylorSoftmaxV3(nn.Module):

    def __init__(self, dim=1, n=2):
        super().__init__()
        assert n % 2 == 0
        self.dim = dim
        self.n = n

    def forward(self, x):
        return taylor_softmax_v3(x, self.dim, self.n, use_log=True)


class TaylorCrossEntropyLossV3(nn.Module):
    """nll_loss of the log-Taylor softmax over dim 1 (reference :175-198)."""

    def __init__(self, n=2, ignore_index=-1, reduction='mean'):
        super().__init__()
        assert n % 2 == 0
        self.taylor_softmax = LogTaylorSoftmaxV3(dim=1, n=n)
        self.reduction = reduction
        self.ignore_index = ignore_index

    def forward(self, logits, labels):
        log_probs = self.taylor_softmax(logits)
        return F.nll_loss(log_probs, labels, reduction=self.reduction, ignore_index=self.ignore_index)
