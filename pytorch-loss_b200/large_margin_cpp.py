"""Stand-in for the reference's `large_margin_cpp` extension module
(csrc/large_margin_kernel.cu:834-838)."""
import torch

from pytorch_loss import _softmax_family as _sf


def l_margin_forward(logits, labels, lam, ignore_index):
    return _sf.forward_per_pixel("lmargin", logits, labels, ignore_index, lam)[0]


def l_margin_backward(logits, labels, lam, ignore_index):
    logits, labels = logits.contiguous(), labels.contiguous()
    return _sf.backward("lmargin", logits, labels, None, None, ignore_index, lam)


def l_margin_forward_backward(logits, labels, lam, ignore_index):
    """(losses [N,*spatial], grads like logits, valid_cnt int64[1])."""
    rec, losses, logits, labels = _sf.forward_reduced("lmargin", logits, labels, ignore_index, lam,
                                                      want_losses=True)
    grads = _sf.backward("lmargin", logits, labels, None, None, ignore_index, lam)
    valid_cnt = rec[:4].view(torch.float64)[1:2].to(torch.int64)
    return losses, grads, valid_cnt
