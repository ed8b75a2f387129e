"""Proportion-corrected softmax cross entropy on the B200 CUDA library.

Drop-in for the reference's `PCSoftmaxCrossEntropyV2(lb_proportion, reduction='mean',
ignore_index=-100)` and `PCSoftmaxCrossEntropyFunction` (pc_softmax.py:52-135), plus `PCSoftmax` /
`pc_softmax_func` (:15-32).  One kernel launch computes the per-pixel loss and its gradient.

The gradient is the derivative of the loss, i.e. what autograd gives for the reference's
`PCSoftmaxCrossEntropyV1` (:35-49).  The reference's V2 Function has a hand-written backward that
scales every channel by the proportion of the LABEL class instead of the channel's own
(:104-106); that is not reproduced.
"""
import torch
import torch.nn as nn
import torch.amp as amp

from . import _cabi


def _weights(lb_proportion, num_classes, device):
    w = torch.as_tensor(lb_proportion, dtype=torch.float32).reshape(-1)
    if w.numel() != num_classes:
        raise RuntimeError("lb_proportion has %d entries for %d classes" % (w.numel(), num_classes))
    return w.to(device)


def pc_softmax_ce(logits, labels, lb_proportion, ignore_index, want_grad=True):
    """(per-pixel losses [N, *spatial], unscaled gradient like logits or None), logits' dtype."""
    dev = _cabi.require_cuda(logits, labels)
    n, c, m = _cabi.split_shape(logits, labels)
    logits, labels = logits.contiguous(), labels.contiguous()
    w = _weights(lb_proportion, c, dev)
    losses = torch.empty(labels.shape, dtype=logits.dtype, device=dev)
    grads = torch.empty_like(logits) if want_grad else None
    with torch.cuda.device(dev):
        _cabi.check(_cabi.load_library().b200_pc_softmax_ce(
            _cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(w), _cabi.ptr(losses), _cabi.ptr(grads),
            n, c, m, _cabi.dtype_code(logits), int(ignore_index), _cabi.stream_ptr(dev)))
    return losses, grads


class PCSoftmaxCrossEntropyFunction(torch.autograd.Function):
    """forward(logits, label, lb_proportion, reduction, ignore_index)
    (reference pc_softmax.py:52-114)."""

    @staticmethod
    @amp.custom_fwd(cast_inputs=torch.float32, device_type='cuda')
    def forward(ctx, logits, label, lb_proportion, reduction, ignore_index):
        losses, grads = pc_softmax_ce(logits, label, lb_proportion, ignore_index, ctx.needs_input_grad[0])
        n_valid = (label != ignore_index).sum()
        ctx.vars = grads, reduction, n_valid
        if reduction == 'mean':               # (half inputs: the sum is taken in fp32)
            return losses.sum(dtype=torch.float32) / n_valid
        if reduction == 'sum':
            return losses.sum(dtype=torch.float32)
        return losses

    @staticmethod
    @amp.custom_bwd(device_type='cuda')
    def backward(ctx, grad_output):
        grads, reduction, n_valid = ctx.vars
        if reduction == 'mean':
            grad = grads * (grad_output / n_valid)
        elif reduction == 'sum':
            grad = grads * grad_output
        else:
            grad = grads * grad_output.unsqueeze(1)
        return grad, None, None, None, None


class PCSoftmaxCrossEntropyV2(nn.Module):
    """Same usage as nn.CrossEntropyLoss, with the class proportions of the training set:

        >>> criteria = PCSoftmaxCrossEntropyV2(lb_proportion=[0.2, 0.5, 0.3], ignore_index=255)
        >>> loss = criteria(logits, labels)       # logits [N, 3, ...] on the GPU, labels int64
    """

    def __init__(self, lb_proportion, reduction='mean', ignore_index=-100):
        super(PCSoftmaxCrossEntropyV2, self).__init__()
        self.lb_proportion = lb_proportion
        self.reduction = reduction
        self.ignore_index = ignore_index

    def forward(self, logits, label):
        return PCSoftmaxCrossEntropyFunction.apply(
            logits, label, self.lb_proportion, self.reduction, self.ignore_index)
