"""Host logic shared by the two softmax-family losses (label-smooth CE and large-margin
softmax): argument checks, the per-pixel forward/backward calls and the fused
'mean'/'sum' autograd Function.  `kind` selects the C-ABI entry points."""
import os

import torch
import torch.amp as amp

from . import _cabi
from . import _p2p
from . import _sharding

_ENTRY = {
    "lsr": ("b200_lsr_forward", "b200_lsr_backward"),
    "lmargin": ("b200_lmargin_forward", "b200_lmargin_backward"),
}
# the same with per-pixel statistics handed from forward to backward (many classes)
_ENTRY_EX = {
    "lsr": ("b200_lsr_forward_ex", "b200_lsr_backward_ex"),
    "lmargin": ("b200_lmargin_forward_ex", "b200_lmargin_backward_ex"),
}


def kernel_layout(logits):
    """(tensor whose memory the kernels read, N, C, M).  NCHW-contiguous logits go as they are.
    Channels-last logits (NHWC in memory, as `memory_format=torch.channels_last` gives) go as
    they are too: every pixel is a row of C contiguous logits, i.e. the kernels' M == 1 layout
    with N*H*W rows -- no copy (the reference calls `.contiguous()`, csrc/lsr_kernel.cu:222-224).
    Gradients made with `empty_like` keep the same memory format.  Anything else is copied."""
    n, c, m = _cabi.split_shape(logits)
    if logits.is_contiguous():
        return logits, n, c, m
    if logits.dim() >= 3 and logits.movedim(1, -1).is_contiguous():
        return logits, n * m, c, 1
    return logits.contiguous(), n, c, m


def _prep(logits, labels):
    dev = _cabi.require_cuda(logits, labels)
    _cabi.split_shape(logits, labels)                       # shape and dtype checks
    logits, n, c, m = kernel_layout(logits)
    return dev, logits, labels.contiguous(), n, c, m, _cabi.dtype_code(logits, allow_f64=True)


def forward_per_pixel(kind, logits, labels, ignore_index, hyper, want_stats=False):
    """Per-pixel losses [N, *spatial] in the logits' dtype, zeros at ignored pixels.  Returns
    (losses, logits, labels, statistics): the statistics (16 bytes per pixel; only when asked for
    and only for layouts with many classes, else None) let backward skip its own softmax pass."""
    dev, logits, labels, n, c, m, dt = _prep(logits, labels)
    lib = _cabi.load_library()
    losses = torch.empty(labels.shape, dtype=logits.dtype, device=dev)
    stats = None
    if want_stats and n * m > 0 and lib.b200_softmax_stats_path(_cabi.ptr(logits), _cabi.ptr(labels), None,
                                                                n, c, m, dt):
        stats = torch.empty((n * m, 4), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        if stats is not None:
            _cabi.check(getattr(lib, _ENTRY_EX[kind][0])(
                _cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(losses), None, None, 0, _cabi.ptr(stats),
                n, c, m, dt, int(ignore_index), float(hyper), _cabi.stream_ptr(dev)))
        else:
            _cabi.check(getattr(lib, _ENTRY[kind][0])(
                _cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(losses), None, None, 0,
                n, c, m, dt, int(ignore_index), float(hyper), _cabi.stream_ptr(dev)))
    return losses, logits, labels, stats


def forward_reduced(kind, logits, labels, ignore_index, hyper, want_losses=False, exchange=None,
                    want_stats=False):
    """Runs the reducing forward; returns (record, per-pixel losses or None, logits, labels
    [, statistics or None when `want_stats`]).  With an `_p2p.Exchange` the kernel adds the sums
    over the ranks itself and the record is the global one.  The statistics (16 bytes per pixel,
    only for layouts with many classes) let backward skip its own softmax pass."""
    dev, logits, labels, n, c, m, dt = _prep(logits, labels)
    lib = _cabi.load_library()
    rec = _cabi.new_record(dev)
    ws = exchange.workspace() if exchange is not None else _cabi.reduce_workspace(dev)
    losses = torch.empty(labels.shape, dtype=logits.dtype, device=dev) if want_losses else None
    stats = None
    if want_stats and n * m > 0 and lib.b200_softmax_stats_path(_cabi.ptr(logits), _cabi.ptr(labels), None,
                                                                n, c, m, dt):
        stats = torch.empty((n * m, 4), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        if stats is not None:
            _cabi.check(getattr(lib, _ENTRY_EX[kind][0])(
                _cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(losses), _cabi.ptr(rec), _cabi.ptr(ws),
                ws.numel(), _cabi.ptr(stats), n, c, m, dt, int(ignore_index), float(hyper),
                _cabi.stream_ptr(dev)))
        else:
            _cabi.check(getattr(lib, _ENTRY[kind][0])(
                _cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(losses), _cabi.ptr(rec), _cabi.ptr(ws),
                ws.numel(), n, c, m, dt, int(ignore_index), float(hyper), _cabi.stream_ptr(dev)))
    if want_stats:
        return rec, losses, logits, labels, stats
    return rec, losses, logits, labels


def backward(kind, logits, labels, grad_output, denom, ignore_index, hyper, stats=None):
    """d(loss)/d(logits); the upstream gradient (None = ones, a broadcast scalar, or one
    value per pixel) and the optional device-resident divisor are applied in the kernel.
    `stats`: what the forward of the same inputs returned, if anything."""
    dev = logits.device
    logits, n, c, m = kernel_layout(logits)
    lib = _cabi.load_library()
    grads = torch.empty_like(logits)
    if grad_output is None:
        mode, g = 0, None
    else:
        mode, g = _cabi.grad_mode_of(grad_output, labels.shape)
        if mode == 2:
            g = g.to(logits.dtype)
    dptr = None if denom is None else _cabi._vp(denom.data_ptr())
    with torch.cuda.device(dev):
        if stats is not None:
            _cabi.check(getattr(lib, _ENTRY_EX[kind][1])(
                _cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(stats), _cabi.ptr(g), mode, dptr, _cabi.ptr(grads),
                n, c, m, _cabi.dtype_code(logits, allow_f64=True), int(ignore_index), float(hyper), _cabi.stream_ptr(dev)))
        else:
            _cabi.check(getattr(lib, _ENTRY[kind][1])(
                _cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(g), mode, dptr, _cabi.ptr(grads),
                n, c, m, _cabi.dtype_code(logits, allow_f64=True), int(ignore_index), float(hyper), _cabi.stream_ptr(dev)))
    return grads


_ENTRY_FUSED = {
    "lsr": "b200_lsr_forward_backward_reduced",
    "lmargin": "b200_lmargin_forward_backward_reduced",
}


def count_valid(labels, ignore_index, exchange=None):
    """Device double: the number of labels != ignore_index, added over the ranks of an
    `_p2p.Exchange` inside the kernel when one is given."""
    dev = labels.device
    lib = _cabi.load_library()
    if labels.dtype != torch.int64:
        raise RuntimeError("labels must be int64, got %s" % labels.dtype)
    labels = labels.contiguous()
    ws = exchange.workspace() if exchange is not None else _cabi.reduce_workspace(dev)
    cnt = _cabi.new_record(dev)
    with torch.cuda.device(dev):
        _cabi.check(lib.b200_count_valid(_cabi.ptr(labels), labels.numel(), int(ignore_index), _cabi.ptr(cnt),
                                         _cabi.ptr(ws), ws.numel(), _cabi.stream_ptr(dev)))
    return cnt[:4].view(torch.float64)[1:]


def fused_step(kind, logits, labels, ignore_index, hyper, mean, exchange, denom=None):
    """The training step in one pass over the logits, or None when this layout has none.
    Returns (record, gradient, logits, labels) with the gradient already divided by the number of
    valid pixels for 'mean' (`denom`: what `count_valid` returned, or None to count here; with an
    `_p2p.Exchange` both the count and the loss sum are global)."""
    dev, logits, labels, n, c, m, dt = _prep(logits, labels)
    lib = _cabi.load_library()
    grads = torch.empty_like(logits)
    if n * m == 0 or not lib.b200_softmax_fused_step_path(_cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(grads),
                                                          n, c, m, dt):
        return None
    rec = _cabi.new_record(dev)
    ws = exchange.workspace() if exchange is not None else _cabi.reduce_workspace(dev)
    st = _cabi.stream_ptr(dev)
    # across GPUs the kernel only posts its sums; backward's rescale kernel collects the peers'
    # (or whatever reads the loss first, see _p2p.DeferredLoss)
    flags = _cabi.STEP_DEFER if (exchange is not None and _p2p.defer_enabled()) else 0
    if mean and denom is None:
        # everything the step needs is allocated by now: the label count is the operation directly
        # in front of the step's kernel, which may then start under the count's tail
        denom = count_valid(labels, ignore_index, exchange)
        flags |= _cabi.STEP_AFTER_COUNT
    with torch.cuda.device(dev):
        _cabi.check(getattr(lib, _ENTRY_FUSED[kind])(
            _cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(grads), _cabi.ptr(rec), _cabi.ptr(ws), ws.numel(),
            None if not mean else _cabi._vp(denom.data_ptr()), n, c, m, dt, int(ignore_index), float(hyper),
            flags, st))
    defer = flags & _cabi.STEP_DEFER
    if defer:
        exchange.defer(rec, ws)
    return rec, grads, logits, labels


class ReducedLossFunc(torch.autograd.Function):
    """'mean' / 'sum' over valid pixels as ONE reducing forward kernel (no per-pixel loss
    tensor, no separate count or sum pass) and ONE backward kernel that recomputes the
    softmax and applies grad_output / n_valid read from device memory.  With a process
    group the [sum, count] pair is summed over the ranks first -- inside the forward kernel
    when the ranks can map each other's memory (`_p2p`), else by a 16-byte all-reduce -- so the
    result is the loss of the concatenated batch.  Returns a 0-dim float32 loss."""

    @staticmethod
    @amp.custom_fwd(cast_inputs=torch.float32, device_type='cuda')
    def forward(ctx, logits, labels, kind, hyper, ignore_index, mean, group):
        exchange = _p2p.get_exchange(group, logits.device) if logits.is_cuda else None
        ctx.fused = None
        ctx.deferred = None
        nccl_group = exchange is None and _sharding.group_is_active(group)
        # Ranks must make the same sequence of exchanges whichever kernels each of them runs (a
        # rank may hold an empty or unaligned shard, or need no gradient): with 'mean' every rank
        # posts its label count first, then its loss sum -- inside fused_step, or right below.
        if ctx.needs_input_grad[0] and logits.is_cuda and not nccl_group and \
                os.environ.get("B200_SOFTMAX_FUSED", "1") != "0":
            # the fused step: loss sum and final gradient from one read of the logits
            step = fused_step(kind, logits, labels, ignore_index, hyper, mean, exchange)
            if step is not None:
                rec, grads, logits, labels = step
                ctx.fused = grads
                ctx.deferred = (exchange, rec) if (exchange is not None and exchange.pending is not None) else None
                ctx.variables = (logits, labels, kind, hyper, ignore_index,
                                 (rec[:4].view(torch.float64)[1:] if mean else None), None)
                return rec[4] if mean else rec[5]
        if exchange is not None and mean:
            _cabi.require_cuda(logits, labels)
            count_valid(labels, ignore_index, exchange)        # (the exchange every rank makes first)
        rec, _, logits, labels, stats = forward_reduced(kind, logits, labels, ignore_index, hyper,
                                                        exchange=exchange, want_stats=True)
        sum_count = rec[:4].view(torch.float64)
        if exchange is None and _sharding.group_is_active(group):
            _sharding.allreduce_sum_count(sum_count, group)
            loss = _sharding.combine_mean(sum_count) if mean else sum_count[0].to(torch.float32)
        else:
            loss = rec[4] if mean else rec[5]
        if logits.dtype == torch.float64:        # the record's float fields would round a double loss
            loss = sum_count[0] / sum_count[1] if mean else sum_count[0].clone()
        ctx.variables = logits, labels, kind, hyper, ignore_index, (sum_count[1:] if mean else None), stats
        return loss

    @staticmethod
    @amp.custom_bwd(device_type='cuda')
    def backward(ctx, grad_output):
        logits, labels, kind, hyper, ignore_index, denom, stats = ctx.variables
        if ctx.fused is not None:
            # first trip through the graph: the gradient is there, times the upstream gradient
            grads, ctx.fused = ctx.fused, None
            g = grad_output.to(torch.float32).reshape(-1)[:1].contiguous()
            lib = _cabi.load_library()
            pending = ctx.deferred[0].take_pending(ctx.deferred[1]) if ctx.deferred else None
            with torch.cuda.device(logits.device):
                if pending is not None:
                    rec, ws, _, _ = pending
                    _cabi.check(lib.b200_rescale_gradient_finish(
                        _cabi.ptr(grads), _cabi.ptr(g), None, grads.numel(), _cabi.dtype_code(grads),
                        _cabi.ptr(ws), _cabi.ptr(rec), None, _cabi.stream_ptr(logits.device)))
                else:
                    _cabi.check(lib.b200_rescale_gradient(
                        _cabi.ptr(grads), _cabi.ptr(g), None, grads.numel(), _cabi.dtype_code(grads),
                        _cabi.stream_ptr(logits.device)))
            return grads, None, None, None, None, None, None
        grads = backward(kind, logits, labels, grad_output, denom, ignore_index, hyper, stats)
        return grads, None, None, None, None, None, None


wrap_if_deferred = _p2p.wrap_if_deferred
