"""Sigmoid focal loss on the B200 CUDA library.

Drop-in for the reference's V3 classes (focal_loss.py:129-200): `FocalLossV3`,
`FocalSigmoidLossFuncV3`, `FocalSigmoidLossFuncV3FB` keep their names, arguments and
return shapes.  What differs is underneath: with reduction 'mean' or 'sum' the module
runs one forward kernel that reads logits and labels once and emits only the sum (no
per-element loss tensor, no separate `.mean()` pass), and one backward kernel that
recomputes the sigmoid and writes the already-scaled gradient.
"""
import os

import torch
import torch.nn as nn
import torch.amp as amp

from . import _cabi
from . import _p2p
from . import _sharding


def _prep(logits, labels):
    dev = _cabi.require_cuda(logits, labels)
    if labels.dtype != logits.dtype:
        raise RuntimeError("focal loss: labels must have the dtype of logits (%s), got %s"
                           % (logits.dtype, labels.dtype))
    if labels.shape != logits.shape:
        raise RuntimeError("focal loss: labels shape %s != logits shape %s"
                           % (tuple(labels.shape), tuple(logits.shape)))
    # elementwise: any dense layout goes as it is when both tensors share it (channels-last
    # included; outputs made with empty_like keep it); otherwise both are made contiguous
    dense = logits.is_contiguous() or (logits.dim() >= 3 and logits.movedim(1, -1).is_contiguous())
    if not (dense and labels.stride() == logits.stride()):
        logits, labels = logits.contiguous(), labels.contiguous()
    return dev, logits, labels, _cabi.dtype_code(logits, allow_f64=True)


def _focal_backward(logits, labels, grad_output, denom, alpha, gamma):
    """grad wrt logits, scaled by the upstream gradient (and 1/denom) inside the kernel."""
    dev = logits.device
    lib = _cabi.load_library()
    grads = torch.empty_like(logits)
    if grad_output is None:
        mode, g = 0, None
    else:
        mode, g = _cabi.grad_mode_of(grad_output, logits.shape)
        if mode == 2:
            g = g.to(logits.dtype)
            if not logits.is_contiguous():       # elementwise kernel: same memory layout as the logits
                g = torch.empty_like(logits).copy_(g)
    with torch.cuda.device(dev):
        _cabi.check(lib.b200_focal_backward(
            _cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(g), mode,
            None if denom is None else _cabi._vp(denom.data_ptr()),
            _cabi.ptr(grads), logits.numel(), _cabi.dtype_code(logits, allow_f64=True),
            float(gamma), float(alpha), _cabi.stream_ptr(dev)))
    return grads


class FocalSigmoidLossFuncV3(torch.autograd.Function):
    """Per-element focal loss; backward recomputes from logits and labels
    (reference focal_loss.py:129-149)."""

    @staticmethod
    @amp.custom_fwd(cast_inputs=torch.float32, device_type='cuda')
    def forward(ctx, logits, labels, alpha, gamma):
        dev, logits, labels, dt = _prep(logits, labels)
        lib = _cabi.load_library()
        losses = torch.empty_like(logits)
        with torch.cuda.device(dev):
            _cabi.check(lib.b200_focal_forward(
                _cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(losses), None, None, 0,
                logits.numel(), dt, float(gamma), float(alpha), _cabi.stream_ptr(dev)))
        ctx.variables = logits, labels, alpha, gamma
        return losses

    @staticmethod
    @amp.custom_bwd(device_type='cuda')
    def backward(ctx, grad_output):
        logits, labels, alpha, gamma = ctx.variables
        return _focal_backward(logits, labels, grad_output, None, alpha, gamma), None, None, None


class FocalSigmoidLossFuncV3FB(torch.autograd.Function):
    """Loss and unscaled gradient from one pass; the gradient is kept for backward
    (reference focal_loss.py:152-171)."""

    @staticmethod
    @amp.custom_fwd(cast_inputs=torch.float32, device_type='cuda')
    def forward(ctx, logits, labels, alpha, gamma):
        dev, logits, labels, dt = _prep(logits, labels)
        lib = _cabi.load_library()
        losses = torch.empty_like(logits)
        grads = torch.empty_like(logits)
        with torch.cuda.device(dev):
            _cabi.check(lib.b200_focal_forward_backward(
                _cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(losses), _cabi.ptr(grads),
                logits.numel(), dt, float(gamma), float(alpha), _cabi.stream_ptr(dev)))
        ctx.variables = grads
        return losses

    @staticmethod
    @amp.custom_bwd(device_type='cuda')
    def backward(ctx, grad_output):
        grads = ctx.variables
        return grads * grad_output, None, None, None


class _FocalReducedFunc(torch.autograd.Function):
    """'mean' / 'sum' focal loss.  Returns a 0-dim float32 loss.

    When the logits need a gradient, forward is the fused step: ONE kernel reads logits and
    labels once, reduces the loss and writes the final gradient (already divided by the
    element count for 'mean'); backward then only multiplies by the upstream gradient, and the
    kernel that does so leaves at once when that gradient is 1, as it is for `loss.backward()`.
    This is the reference's forward-backward fusion (FocalSigmoidLossFuncV3FB, focal_loss.py:152-171)
    without its separate `grads * grad_output` pass.  A second backward through the same graph
    (retain_graph) recomputes the gradient from the inputs.  Without a gradient to produce,
    forward is the reducing kernel alone."""

    @staticmethod
    def _fused_forward(ctx, logits, labels, alpha, gamma, mean, group, dev, dt, state):
        lib = _cabi.load_library()
        rec = _cabi.new_record(dev)
        exchange = _p2p.get_exchange(group, dev)
        ws = exchange.workspace() if exchange is not None else _cabi.reduce_workspace(dev)
        grads = torch.empty_like(logits)
        n = logits.numel()
        denom = None
        scale = 1.0
        correction = None
        st = _cabi.stream_ptr(dev)
        with torch.cuda.device(dev):
            if mean and exchange is not None:
                # The gradients need the GLOBAL element count.  A module keeps the count its
                # previous call found on the device and divides by that; the kernel checks it
                # against the count it sums over the ranks and leaves the ratio for backward
                # (1 unless a rank's shape changed).  Only the first call of a module, and calls
                # without a module to hold the state, exchange the count in a kernel of its own.
                key = (dev.index, id(exchange))
                predicted = state.get(key) if state is not None else None
                if predicted is None and torch.cuda.is_current_stream_capturing():
                    state = None             # memory allocated during a capture must not outlive the graph
                if predicted is None:
                    cnt = _cabi.new_record(dev)
                    _cabi.check(lib.b200_exchange_count(float(n), _cabi.ptr(cnt), _cabi.ptr(ws), ws.numel(), st))
                    denom = cnt[:4].view(torch.float64)[1:]
                    if state is not None:
                        state[key] = predicted = denom.clone()
                if predicted is not None:
                    correction = torch.empty(1, dtype=torch.float32, device=dev)
            elif mean:
                scale = 1.0 / max(n, 1)
            # across GPUs the kernel only posts its sums; backward's rescale kernel collects the
            # peers' (or whatever reads the loss first, see _p2p.DeferredLoss)
            defer = 1 if (exchange is not None and _p2p.defer_enabled()) else 0
            if correction is not None:
                _cabi.check(lib.b200_focal_forward_backward_predicted(
                    _cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(grads), _cabi.ptr(rec), _cabi.ptr(ws),
                    ws.numel(), _cabi.ptr(predicted), _cabi.ptr(correction), n, dt, float(gamma), float(alpha),
                    defer, st))
            else:
                _cabi.check(lib.b200_focal_forward_backward_reduced(
                    _cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(grads), _cabi.ptr(rec), _cabi.ptr(ws), ws.numel(),
                    None if denom is None else _cabi._vp(denom.data_ptr()), float(scale), n, dt, float(gamma),
                    float(alpha), defer, st))
            if defer:
                exchange.defer(rec, ws, predicted if correction is not None else None, correction)
        ctx.deferred = (exchange, rec) if defer else None
        ctx.fused = [grads, correction]      # handed out by the first backward
        ctx.variables = logits, labels, alpha, gamma, (rec[:4].view(torch.float64)[1:] if mean else None)
        return rec[4] if mean else rec[5]

    @staticmethod
    @amp.custom_fwd(cast_inputs=torch.float32, device_type='cuda')
    def forward(ctx, logits, labels, alpha, gamma, mean, group, state=None):
        dev, logits, labels, dt = _prep(logits, labels)
        lib = _cabi.load_library()
        ctx.fused = None
        ctx.deferred = None
        nccl_group = _sharding.group_is_active(group) and _p2p.get_exchange(group, dev) is None
        if ctx.needs_input_grad[0] and logits.numel() > 0 and not nccl_group and \
                logits.dtype != torch.float64 and os.environ.get("B200_FOCAL_FUSED", "1") != "0":
            return _FocalReducedFunc._fused_forward(ctx, logits, labels, alpha, gamma, mean, group, dev, dt, state)
        rec = _cabi.new_record(dev)
        exchange = _p2p.get_exchange(group, dev)      # sums over the ranks inside the kernel, if possible
        ws = exchange.workspace() if exchange is not None else _cabi.reduce_workspace(dev)
        with torch.cuda.device(dev):
            _cabi.check(lib.b200_focal_forward(
                _cabi.ptr(logits), _cabi.ptr(labels), None, _cabi.ptr(rec), _cabi.ptr(ws),
                ws.numel(), logits.numel(), dt, float(gamma), float(alpha), _cabi.stream_ptr(dev)))
        sum_count = rec[:4].view(torch.float64)
        if exchange is None and _sharding.group_is_active(group):
            _sharding.allreduce_sum_count(sum_count, group)
            loss = _sharding.combine_mean(sum_count) if mean else sum_count[0].to(torch.float32)
        else:
            loss = rec[4] if mean else rec[5]
        if logits.dtype == torch.float64:        # the record's float fields would round a double loss
            loss = sum_count[0] / sum_count[1] if mean else sum_count[0].clone()
        ctx.variables = logits, labels, alpha, gamma, (sum_count[1:] if mean else None)
        return loss

    @staticmethod
    @amp.custom_bwd(device_type='cuda')
    def backward(ctx, grad_output):
        logits, labels, alpha, gamma, denom = ctx.variables
        if ctx.fused:
            grads, correction = ctx.fused
            ctx.fused = None
            g = grad_output.to(torch.float32).reshape(-1)[:1].contiguous()
            lib = _cabi.load_library()
            pending = ctx.deferred[0].take_pending(ctx.deferred[1]) if ctx.deferred else None
            with torch.cuda.device(logits.device):
                if pending is not None:
                    rec, ws, state, _ = pending
                    _cabi.check(lib.b200_rescale_gradient_finish(
                        _cabi.ptr(grads), _cabi.ptr(g), _cabi.ptr(correction), grads.numel(), _cabi.dtype_code(grads),
                        _cabi.ptr(ws), _cabi.ptr(rec), _cabi.ptr(state), _cabi.stream_ptr(logits.device)))
                else:
                    _cabi.check(lib.b200_rescale_gradient(
                        _cabi.ptr(grads), _cabi.ptr(g), _cabi.ptr(correction), grads.numel(), _cabi.dtype_code(grads),
                        _cabi.stream_ptr(logits.device)))
            return grads, None, None, None, None, None, None
        grads = _focal_backward(logits, labels, grad_output, denom, alpha, gamma)
        return grads, None, None, None, None, None, None


class FocalLossV3(nn.Module):
    """Sigmoid focal loss, usage as nn.BCEWithLogitsLoss (reference focal_loss.py:174-200):

        >>> criteria = FocalLossV3()
        >>> logits = torch.randn(8, 19, 384, 384).cuda()
        >>> lbs = torch.randint(0, 2, (8, 19, 384, 384)).float().cuda()
        >>> loss = criteria(logits, lbs)

    `process_group` (keyword only, not in the reference): pass a torch.distributed group
    (or True for the default group) to make 'mean'/'sum' global over a batch that is
    sharded across ranks; the default None keeps the loss local to this process.
    """

    def __init__(self, alpha=0.25, gamma=2, reduction='mean', *, process_group=None):
        super(FocalLossV3, self).__init__()
        self.alpha = alpha
        self.gamma = gamma
        self.reduction = reduction
        self.process_group = process_group
        self._count_state = {}               # per device: the global element count of the last call

    def forward(self, logits, label):
        if self.reduction == 'mean' or self.reduction == 'sum':
            loss = _FocalReducedFunc.apply(logits, label, self.alpha, self.gamma,
                                           self.reduction == 'mean', self.process_group, self._count_state)
            return _p2p.wrap_if_deferred(loss, self.process_group, logits)
        return FocalSigmoidLossFuncV3.apply(logits, label, self.alpha, self.gamma)
