"""Label-smoothed softmax cross entropy on the B200 CUDA library.

Drop-in for the reference's V3 classes (label_smooth.py:126-171):
`LabelSmoothSoftmaxCEV3(lb_smooth=0.1, reduction='mean', ignore_index=-100)` and
`LSRCrossEntropyFunctionV3` keep names, arguments and shapes.  The reference runs
log_softmax + a loss kernel forward and softmax + an in-place kernel + a Python
multiply backward; here the forward is one kernel (which, for 'mean'/'sum', also
counts valid pixels and sums the losses) and the backward is one kernel.
"""
import torch
import torch.nn as nn
import torch.amp as amp

from . import _softmax_family as _sf


class LSRCrossEntropyFunctionV3(torch.autograd.Function):
    """Per-pixel losses [N, *spatial]; backward recomputes the softmax
    (reference label_smooth.py:126-145)."""

    @staticmethod
    @amp.custom_fwd(cast_inputs=torch.float32, device_type='cuda')
    def forward(ctx, logits, labels, lb_smooth, lb_ignore):
        losses, logits, labels, stats = _sf.forward_per_pixel("lsr", logits, labels, lb_ignore, lb_smooth,
                                                              want_stats=ctx.needs_input_grad[0])
        ctx.variables = logits, labels, lb_ignore, lb_smooth, stats
        return losses

    @staticmethod
    @amp.custom_bwd(device_type='cuda')
    def backward(ctx, grad_output):
        logits, labels, lb_ignore, lb_smooth, stats = ctx.variables
        grad = _sf.backward("lsr", logits, labels, grad_output, None, lb_ignore, lb_smooth, stats)
        return grad, None, None, None


class LabelSmoothSoftmaxCEV3(nn.Module):
    """Same usage as nn.CrossEntropyLoss:

        >>> criteria = LabelSmoothSoftmaxCEV3()
        >>> logits = torch.randn(8, 19, 384, 384).cuda()   # nchw, float/half
        >>> lbs = torch.randint(0, 19, (8, 384, 384)).cuda()  # nhw, int64
        >>> loss = criteria(logits, lbs)

    'mean' divides by the number of non-ignored pixels (NaN if there is none), 'sum' adds,
    anything else returns the per-pixel losses with zeros at ignored pixels.  Reduced
    losses are float32 whatever the logits' dtype.  `process_group` (keyword only, not in
    the reference): reduce over a batch sharded across ranks (True = default group).
    """

    def __init__(self, lb_smooth=0.1, reduction='mean', ignore_index=-100, *, process_group=None):
        super(LabelSmoothSoftmaxCEV3, self).__init__()
        self.lb_smooth = lb_smooth
        self.reduction = reduction
        self.lb_ignore = ignore_index
        self.process_group = process_group

    def forward(self, logits, labels):
        if self.reduction == 'mean' or self.reduction == 'sum':
            loss = _sf.ReducedLossFunc.apply(logits, labels, "lsr", self.lb_smooth, self.lb_ignore,
                                             self.reduction == 'mean', self.process_group)
            return _sf.wrap_if_deferred(loss, self.process_group, logits)
        return LSRCrossEntropyFunctionV3.apply(logits, labels, self.lb_smooth, self.lb_ignore)
