"""Stand-in for the reference's `lovasz_softmax_cpp` extension module
(csrc/lovasz_softmax.cu:799-802)."""
from pytorch_loss import lovasz_softmax as _lv


def lovasz_softmax_forward(logits, labels, ignore_index):
    """(loss [C], jacc [C, N*H*W]) — jacc is the Jaccard gradient of every pixel in
    original pixel order, which backward consumes."""
    loss, jacc, _, _ = _lv.lovasz_forward(logits, labels, ignore_index, per_image=False)
    return loss, jacc


def lovasz_softmax_backward(grad, logits, labels, jacc, ignore_index):
    return _lv.lovasz_backward(grad, logits.contiguous(), labels.contiguous(), jacc, ignore_index,
                               per_image=False)
