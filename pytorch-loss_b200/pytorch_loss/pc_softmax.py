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

from . import _cabi, _softmax_family


def _weights(lb_proportion, num_classes, device):
    if isinstance(lb_proportion, torch.Tensor) and lb_proportion.device == device and \
            lb_proportion.dtype == torch.float32 and lb_proportion.numel() == num_classes:
        return lb_proportion.reshape(-1).contiguous()         # (the module's cached copy: no transfer)
    w = torch.as_tensor(lb_proportion, dtype=torch.float32).reshape(-1)
    if w.numel() != num_classes:
        raise RuntimeError("lb_proportion has %d entries for %d classes" % (w.numel(), num_classes))
    return w.to(device)


def pc_softmax_ce(logits, labels, lb_proportion, ignore_index, want_grad=True, denom=None):
    """(per-pixel losses [N, *spatial], gradient like logits or None), logits' dtype.  `denom`: a
    device double the gradient is divided by inside the kernel (the valid-pixel count for 'mean')."""
    dev = _cabi.require_cuda(logits, labels)
    n, c, m = _cabi.split_shape(logits, labels)
    logits, labels = logits.contiguous(), labels.contiguous()
    w = _weights(lb_proportion, c, dev)
    losses = torch.empty(labels.shape, dtype=logits.dtype, device=dev)
    grads = torch.empty_like(logits) if want_grad else None
    with torch.cuda.device(dev):
        _cabi.check(_cabi.load_library().b200_pc_softmax_ce_scaled(
            _cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(w), _cabi.ptr(losses), _cabi.ptr(grads),
            None if denom is None else _cabi._vp(denom.data_ptr()),
            n, c, m, _cabi.dtype_code(logits), int(ignore_index), _cabi.stream_ptr(dev)))
    return losses, grads


def _rescale(grads, grad_output):
    """grads *= grad_output (a scalar) in place; the kernel leaves at once when it is 1."""
    g = grad_output.to(torch.float32).reshape(-1)[:1].contiguous()
    with torch.cuda.device(grads.device):
        _cabi.check(_cabi.load_library().b200_rescale_gradient(
            _cabi.ptr(grads), _cabi.ptr(g), None, grads.numel(), _cabi.dtype_code(grads),
            _cabi.stream_ptr(grads.device)))
    return grads


def pc_softmax_step(logits, labels, lb_proportion, ignore_index, mean):
    """The 'mean' / 'sum' training step in one pass over the logits (the label-smooth step's tile
    pipeline with the class weights inside the exponentials), or None when the layout has none.
    Returns (record, final gradient, valid-pixel count or None)."""
    dev = _cabi.require_cuda(logits, labels)
    n, c, m = _cabi.split_shape(logits, labels)
    if labels.dtype != torch.int64 or logits.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        return None
    logits, labels = logits.contiguous(), labels.contiguous()
    lib = _cabi.load_library()
    grads = torch.empty_like(logits)
    dt = _cabi.dtype_code(logits)
    if n * m == 0 or not lib.b200_pc_softmax_step_path(_cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(grads), n, c, m, dt):
        return None
    w = _weights(lb_proportion, c, dev)
    rec = _cabi.new_record(dev)
    ws = _cabi.reduce_workspace(dev)
    denom, flags = None, 0
    if mean:       # (directly in front of the step's launch: it starts under the count's tail)
        denom = _softmax_family.count_valid(labels, ignore_index)
        flags = _cabi.STEP_AFTER_COUNT
    with torch.cuda.device(dev):
        _cabi.check(lib.b200_pc_softmax_step(
            _cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(w), _cabi.ptr(grads), _cabi.ptr(rec), _cabi.ptr(ws),
            ws.numel(), None if denom is None else _cabi._vp(denom.data_ptr()), n, c, m, dt, int(ignore_index),
            flags, _cabi.stream_ptr(dev)))
    return rec, grads, denom


class PCSoftmaxCrossEntropyFunction(torch.autograd.Function):
    """forward(logits, label, lb_proportion, reduction, ignore_index)
    (reference pc_softmax.py:52-114)."""

    @staticmethod
    @amp.custom_fwd(cast_inputs=torch.float32, device_type='cuda')
    def forward(ctx, logits, label, lb_proportion, reduction, ignore_index):
        # 'mean': the valid pixels are counted first (labels only), so that the gradient leaves the
        # kernel already divided and backward has nothing to do for an upstream gradient of 1
        if reduction in ('mean', 'sum') and ctx.needs_input_grad[0] and logits.is_cuda:
            step = pc_softmax_step(logits, label, lb_proportion, ignore_index, reduction == 'mean')
            if step is not None:
                rec, grads, n_valid = step
                ctx.vars = logits, label, lb_proportion, ignore_index, reduction, n_valid
                ctx.grads = grads
                return rec[4] if reduction == 'mean' else rec[5]
        n_valid = None
        if reduction == 'mean':
            _cabi.require_cuda(logits, label)
            n_valid = _softmax_family.count_valid(label, ignore_index)
        losses, grads = pc_softmax_ce(logits, label, lb_proportion, ignore_index, ctx.needs_input_grad[0], n_valid)
        ctx.vars = logits, label, lb_proportion, ignore_index, reduction, n_valid
        ctx.grads = grads
        if reduction == 'mean':               # (half inputs: the sum is taken in fp32)
            return losses.sum(dtype=torch.float32) / n_valid[0].to(torch.float32)
        if reduction == 'sum':
            return losses.sum(dtype=torch.float32)
        return losses

    @staticmethod
    @amp.custom_bwd(device_type='cuda')
    def backward(ctx, grad_output):
        logits, label, lb_proportion, ignore_index, reduction, n_valid = ctx.vars
        grads, ctx.grads = ctx.grads, None
        if grads is None:                     # a second trip through the graph: the first scaled them in place
            _, grads = pc_softmax_ce(logits, label, lb_proportion, ignore_index, True, n_valid)
        if reduction in ('mean', 'sum'):
            return _rescale(grads, grad_output), None, None, None, None
        return grads * grad_output.unsqueeze(1), None, None, None, None


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
        self._on_device = {}          # device -> float32 tensor of the proportions (sent once)

    def forward(self, logits, label):
        w = self._on_device.get(logits.device)
        if w is None and logits.is_cuda:
            w = torch.as_tensor(self.lb_proportion, dtype=torch.float32).reshape(-1).to(logits.device)
            self._on_device[logits.device] = w
        return PCSoftmaxCrossEntropyFunction.apply(
            logits, label, self.lb_proportion if w is None else w, self.reduction, self.ignore_index)
