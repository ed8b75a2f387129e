"""Stand-in for the reference's `focal_cpp` extension module (csrc/focal_kernel.cu:337-341).
Note the reference's argument order at this boundary: (logits, labels, gamma, alpha)."""
import torch

from pytorch_loss import _cabi
from pytorch_loss import focal_loss as _fl


def focalloss_forward(logits, labels, gamma, alpha):
    dev, logits, labels, dt = _fl._prep(logits, labels)
    losses = torch.empty_like(logits)
    with torch.cuda.device(dev):
        _cabi.check(_cabi.load_library().b200_focal_forward(
            _cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(losses), None, None, 0,
            logits.numel(), dt, float(gamma), float(alpha), _cabi.stream_ptr(dev)))
    return losses


def focalloss_backward(logits, labels, gamma, alpha):
    dev, logits, labels, dt = _fl._prep(logits, labels)
    return _fl._focal_backward(logits, labels, None, None, alpha, gamma)


def focalloss_forward_backward(logits, labels, gamma, alpha):
    dev, logits, labels, dt = _fl._prep(logits, labels)
    losses = torch.empty_like(logits)
    grads = torch.empty_like(logits)
    with torch.cuda.device(dev):
        _cabi.check(_cabi.load_library().b200_focal_forward_backward(
            _cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(losses), _cabi.ptr(grads),
            logits.numel(), dt, float(gamma), float(alpha), _cabi.stream_ptr(dev)))
    return losses, grads
