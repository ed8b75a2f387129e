"""Lovasz-softmax loss on the B200 CUDA library.

Drop-in for the reference's V3 classes (lovasz_softmax.py:75-116):
`LovaszSoftmaxV3(reduction='mean', ignore_index=-100)` and `LovaszSoftmaxFunctionV3`.
By default the loss is what the reference computes: per class, ONE sort over all
N*H*W pixels of the batch, output [C], reduced over classes.  `per_image=True`
(keyword only, not in the reference) sorts every image on its own: output [N, C],
'mean' averages all N*C entries, 'sum' adds them; images are then independent, which
is what lets a batch be sharded over GPUs (`process_group`).
"""
import torch
import torch.nn as nn
import torch.amp as amp
import torch.distributed as dist

from . import _cabi
from . import _sharding


def lovasz_forward(logits, labels, ignore_index, per_image=False):
    """Runs the forward pipeline.  Returns (loss, jacc, logits32, labels): loss is [C]
    ([N, C] per image), jacc the Jaccard gradient of every (class, pixel) in pixel order,
    shaped [C, N*M] ([N, C, M] per image); both float32."""
    dev = _cabi.require_cuda(logits, labels)
    n, c, m = _cabi.split_shape(logits, labels)
    if logits.dtype not in (torch.float32, torch.float16, torch.bfloat16, torch.float64):
        raise RuntimeError("lovasz softmax supports floating-point logits, got %s" % logits.dtype)
    x = logits.contiguous().float()          # every input dtype is computed in fp32 (half: as under autocast)
    labels = labels.contiguous()
    lib = _cabi.load_library()
    loss = torch.empty((n, c) if per_image else (c,), dtype=torch.float32, device=dev)
    jacc = torch.empty((n, c, m) if per_image else (c, n * m), dtype=torch.float32, device=dev)
    if n * m == 0:
        return loss.zero_(), jacc, x, labels
    nbytes = int(lib.b200_lovasz_workspace_bytes(n, c, m, int(per_image)))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _cabi.check(lib.b200_lovasz_forward(
            _cabi.ptr(x), _cabi.ptr(labels), _cabi.ptr(loss), _cabi.ptr(jacc), _cabi.ptr(ws), nbytes,
            n, c, m, _cabi.F32, int(ignore_index), int(per_image), _cabi.stream_ptr(dev)))
    return loss, jacc, x, labels


def lovasz_backward(grad, logits, labels, jacc, ignore_index, per_image=False):
    """d(loss . grad)/d(logits) as float32; `grad` has the shape of the forward's loss.
    `jacc` is only read (the reference overwrites it, csrc/lovasz_softmax.cu:734-738)."""
    dev = logits.device
    n, c, m = _cabi.split_shape(logits)
    lib = _cabi.load_library()
    g = grad.to(torch.float32).expand((n, c) if per_image else (c,)).contiguous()
    grads = torch.empty_like(logits, dtype=torch.float32)
    with torch.cuda.device(dev):
        _cabi.check(lib.b200_lovasz_backward(
            _cabi.ptr(g), _cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(jacc.contiguous()),
            _cabi.ptr(grads), n, c, m, _cabi.F32, int(ignore_index), int(per_image),
            _cabi.stream_ptr(dev)))
    return grads


class LovaszSoftmaxFunctionV3(torch.autograd.Function):
    """forward(logits, labels, ignore_index[, per_image]) -> per-class losses
    (reference lovasz_softmax.py:75-91)."""

    @staticmethod
    @amp.custom_fwd(cast_inputs=torch.float32, device_type='cuda')
    def forward(ctx, logits, labels, ignore_index, per_image=False):
        losses, jacc, x, labels = lovasz_forward(logits, labels, ignore_index, per_image)
        ctx.vars = x, labels, jacc, ignore_index, per_image, logits.dtype
        return losses

    @staticmethod
    @amp.custom_bwd(device_type='cuda')
    def backward(ctx, grad_output):
        x, labels, jacc, ignore_index, per_image, in_dtype = ctx.vars
        grad = lovasz_backward(grad_output, x, labels, jacc, ignore_index, per_image)
        return grad.to(in_dtype), None, None, None


class _AllReduceSumCount(torch.autograd.Function):
    """[local_sum, local_count] -> global; the gradient of the global sum with respect to
    this rank's contribution is the upstream gradient itself."""

    @staticmethod
    def forward(ctx, pair, group):
        out = pair.clone()
        dist.all_reduce(out, op=dist.ReduceOp.SUM, group=_sharding.resolve_group(group))
        return out

    @staticmethod
    def backward(ctx, grad):
        return grad, None


class LovaszSoftmaxV3(nn.Module):
    """Same usage as nn.CrossEntropyLoss:

        >>> criteria = LovaszSoftmaxV3()
        >>> logits = torch.randn(8, 19, 384, 384).cuda()   # nchw, float/half
        >>> lbs = torch.randint(0, 19, (8, 384, 384)).cuda()  # nhw, int64
        >>> loss = criteria(logits, lbs)

    `process_group` needs `per_image=True`: ranks hold different images and 'mean'/'sum'
    run over all of them (one all-reduce of two numbers).
    """

    def __init__(self, reduction='mean', ignore_index=-100, *, per_image=False, process_group=None):
        super(LovaszSoftmaxV3, self).__init__()
        self.reduction = reduction
        self.lb_ignore = ignore_index
        self.per_image = per_image
        self.process_group = process_group
        if process_group is not None and process_group is not False and not per_image:
            raise ValueError("process_group requires per_image=True: a batch-global sort does not shard")

    def forward(self, logits, label):
        losses = LovaszSoftmaxFunctionV3.apply(logits, label, self.lb_ignore, self.per_image)
        if self.reduction not in ('sum', 'mean'):
            return losses
        if _sharding.group_is_active(self.process_group):
            # (the count is made on the device: a host tensor could not be copied during graph capture)
            pair = torch.stack([losses.sum().double(),
                                torch.full((), float(losses.numel()), dtype=torch.float64, device=losses.device)])
            pair = _AllReduceSumCount.apply(pair, self.process_group)
            return (pair[0] / pair[1] if self.reduction == 'mean' else pair[0]).float()
        return losses.sum() if self.reduction == 'sum' else losses.mean()
