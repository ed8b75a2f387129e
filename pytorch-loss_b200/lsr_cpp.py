"""Stand-in for the reference's `lsr_cpp` extension module (csrc/lsr_kernel.cu:319-322):
same function names and argument order, implemented on libb200loss.so."""
from pytorch_loss import _softmax_family as _sf


def lsr_forward(logits, labels, ignore_index, smooth):
    """Per-pixel label-smooth CE losses [N, *spatial] (zeros at ignored pixels)."""
    return _sf.forward_per_pixel("lsr", logits, labels, ignore_index, smooth)[0]


def lsr_backward(logits, labels, ignore_index, smooth):
    """d(loss)/d(logits) for an upstream gradient of ones (the caller scales it)."""
    logits, labels = logits.contiguous(), labels.contiguous()
    return _sf.backward("lsr", logits, labels, None, None, ignore_index, smooth)
