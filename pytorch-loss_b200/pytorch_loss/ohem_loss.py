"""Online hard example mining in front of the fused losses, on the B200 CUDA library.

Drop-in for the reference's `OhemCELoss` and `OhemLargeMarginLoss`
(pytorch_loss/ohem_loss.py:13-45) and for `ohem_cpp.score_ohem_label`
(csrc/ohem_label_kernel.cu:265-281): pixels that are already easy (softmax score of the
label above `score_thresh`) are relabelled to `ignore_index`, except that the `n_min`
hardest pixels always stay; the loss is then the mean over what is left.

`OhemCELoss.criteria` is the fused `LabelSmoothSoftmaxCEV3(lb_smooth=0)`, which computes what
the reference's `nn.CrossEntropyLoss(ignore_index, reduction='mean')` computes.
"""
import torch
import torch.nn as nn

from . import _cabi
from .label_smooth import LabelSmoothSoftmaxCEV3
from .large_margin_softmax import LargeMarginSoftmaxV3


def score_ohem_label(logits, labels, ignore_index, score_thresh, n_min):
    """New labels (int64, shape of `labels`): `ignore_index` where the pixel is dropped.
    Argument order of the reference's extension function."""
    dev = _cabi.require_cuda(logits, labels)
    n, c, m = _cabi.split_shape(logits, labels)
    if logits.dtype not in (torch.float32, torch.float16):
        raise RuntimeError("score_ohem_label supports float32 and float16 logits, got %s" % logits.dtype)
    if labels.dtype != torch.int64:
        raise RuntimeError("labels must be int64, got %s" % labels.dtype)
    n_min = int(n_min)
    if n_min >= n * m:                        # reference csrc/ohem_label_kernel.cu:193
        return labels
    x = logits.detach().contiguous()
    lb = labels.contiguous()
    out = torch.empty_like(lb)
    if n * m == 0:
        return out
    lib = _cabi.load_library()
    nbytes = int(lib.b200_ohem_workspace_bytes(n, m))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _cabi.check(lib.b200_ohem_label(
            _cabi.ptr(x), _cabi.ptr(lb), _cabi.ptr(out), _cabi.ptr(ws), nbytes, n, c, m,
            _cabi.dtype_code(x), int(ignore_index), float(score_thresh), n_min, _cabi.stream_ptr(dev)))
    return out


class _OhemBase(nn.Module):

    def __init__(self, score_thresh, n_min=None, ignore_index=255):
        super().__init__()
        self.score_thresh = score_thresh
        self.ignore_lb = ignore_index
        self.n_min = n_min

    def forward(self, logits, labels):
        n_min = labels.numel() // 16 if self.n_min is None else self.n_min
        with torch.no_grad():
            labels = score_ohem_label(logits, labels, self.ignore_lb, self.score_thresh, n_min)
        return self.criteria(logits, labels)


class OhemCELoss(_OhemBase):
    """Cross entropy over the mined pixels (reference pytorch_loss/ohem_loss.py:13-28)."""

    def __init__(self, score_thresh, n_min=None, ignore_index=255):
        super().__init__(score_thresh, n_min, ignore_index)
        self.criteria = LabelSmoothSoftmaxCEV3(lb_smooth=0.0, reduction='mean', ignore_index=ignore_index)


class OhemLargeMarginLoss(_OhemBase):
    """Large-margin softmax over the mined pixels (reference pytorch_loss/ohem_loss.py:31-46)."""

    def __init__(self, score_thresh, n_min=None, ignore_index=255):
        super().__init__(score_thresh, n_min, ignore_index)
        self.criteria = LargeMarginSoftmaxV3(ignore_index=ignore_index, reduction='mean')
