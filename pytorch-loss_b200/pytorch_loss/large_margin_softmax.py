"""Large-margin softmax cross entropy (Kobayashi, BMVC 2019) on the B200 CUDA library.

Drop-in for the reference's V3 classes (large_margin_softmax.py:146-229):
`LargeMarginSoftmaxV3(lam=0.3, reduction='mean', ignore_index=255, fb=True)`,
`LargeMarginSoftmaxFuncV3`, `LargeMarginSoftmaxFuncV3FB`.
"""
import torch
import torch.nn as nn
import torch.amp as amp

from . import _softmax_family as _sf


class LargeMarginSoftmaxFuncV3(torch.autograd.Function):
    """Per-pixel losses; backward recomputes, from 16 bytes of saved statistics per pixel where
    the layout has many classes (reference large_margin_softmax.py:146-169)."""

    @staticmethod
    @amp.custom_fwd(cast_inputs=torch.float32, device_type='cuda')
    def forward(ctx, logits, labels, lam=0.3, ignore_index=255):
        losses, logits, labels, stats = _sf.forward_per_pixel("lmargin", logits, labels, ignore_index, lam,
                                                              want_stats=ctx.needs_input_grad[0])
        ctx.variables = logits, labels, lam, ignore_index, stats
        return losses

    @staticmethod
    @amp.custom_bwd(device_type='cuda')
    def backward(ctx, grad_output):
        logits, labels, lam, ignore_index, stats = ctx.variables
        grads = _sf.backward("lmargin", logits, labels, grad_output, None, ignore_index, lam, stats)
        return grads, None, None, None


class LargeMarginSoftmaxFuncV3FB(torch.autograd.Function):
    """Returns (per-pixel losses, valid_cnt) like the reference's fused forward+backward
    Function (large_margin_softmax.py:172-193); valid_cnt is an int64 tensor of one element.
    The gradient is not stored in forward: backward recomputes it, which moves the same
    number of bytes as scaling a stored gradient and keeps no [N, C, H, W] buffer alive."""

    @staticmethod
    @amp.custom_fwd(cast_inputs=torch.float32, device_type='cuda')
    def forward(ctx, logits, labels, lam=0.3, ignore_index=255):
        rec, losses, logits, labels, stats = _sf.forward_reduced("lmargin", logits, labels, ignore_index, lam,
                                                                 want_losses=True, want_stats=True)
        valid_cnt = rec[:4].view(torch.float64)[1:2].to(torch.int64)
        ctx.variables = logits, labels, lam, ignore_index, stats
        ctx.mark_non_differentiable(valid_cnt)
        return losses, valid_cnt

    @staticmethod
    @amp.custom_bwd(device_type='cuda')
    def backward(ctx, grad_output, grad_cnt):
        logits, labels, lam, ignore_index, stats = ctx.variables
        grads = _sf.backward("lmargin", logits, labels, grad_output, None, ignore_index, lam, stats)
        return grads, None, None, None


class LargeMarginSoftmaxV3(nn.Module):
    """Same usage as nn.CrossEntropyLoss:

        >>> criteria = LargeMarginSoftmaxV3()
        >>> logits = torch.randn(8, 19, 384, 384).cuda()   # nchw, float/half
        >>> lbs = torch.randint(0, 19, (8, 384, 384)).cuda()  # nhw, int64
        >>> loss = criteria(logits, lbs)

    `fb` is kept for compatibility; both settings run the same kernels here.
    `process_group` (keyword only, not in the reference): reduce over a batch sharded
    across ranks (True = default group).
    """

    def __init__(self, lam=0.3, reduction='mean', ignore_index=255, fb=True, *, process_group=None):
        super(LargeMarginSoftmaxV3, self).__init__()
        self.reduction = reduction
        self.ignore_index = ignore_index
        self.lam = lam
        self.fb = fb
        self.process_group = process_group

    def forward(self, logits, labels):
        if self.reduction == 'mean' or self.reduction == 'sum':
            loss = _sf.ReducedLossFunc.apply(logits, labels, "lmargin", self.lam, self.ignore_index,
                                             self.reduction == 'mean', self.process_group)
            return _sf.wrap_if_deferred(loss, self.process_group, logits)
        return LargeMarginSoftmaxFuncV3.apply(logits, labels, self.lam, self.ignore_index)
