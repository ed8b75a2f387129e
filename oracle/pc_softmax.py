"""CPU oracle of the PC-softmax cross entropy — TEST INFRASTRUCTURE, NOT A PRODUCT PATH.

Parity status: PINNED by tests/golden/pc_softmax.npz, which tests/golden/make_golden.py writes
from the unmodified reference: loss and autograd gradient of `PCSoftmaxCrossEntropyV1`
(pc_softmax.py:35-49) and the loss of `PCSoftmaxCrossEntropyV2` (:52-135); tests/test_oracle_golden.py
checks this file against them.  Only tests/ may import this module.
"""
import torch


def pc_softmax_ce(logits, labels, lb_proportion, ignore_index=-100, reduction='mean', dtype=torch.float32):
    """(loss, d loss / d logits).  Follows PCSoftmaxCrossEntropyV1.forward (reference
    pc_softmax.py:43-49): subtract the channel maximum, log of the proportion-weighted sum of
    exponentials, negative log likelihood with `ignore_index`; the gradient is the derivative
    of that (what autograd returns for V1): W_j e^{x_j} / sum_k W_k e^{x_k} - one_hot."""
    x = logits.detach().to(dtype)
    c = x.size(1)
    shape = [1, c] + [1] * (x.dim() - 2)
    w = torch.as_tensor(lb_proportion, dtype=dtype).view(*shape)
    ignore = labels.eq(ignore_index)
    valid = ignore.logical_not()
    n_valid = valid.sum()
    lb = labels.masked_fill(ignore, 0)
    z = x - x.max(dim=1, keepdim=True)[0]
    wexp = torch.exp(z) * w
    wsum = wexp.sum(dim=1, keepdim=True)
    log_wsoftmax = z - torch.log(wsum)
    loss_px = -log_wsoftmax.gather(1, lb.unsqueeze(1)).squeeze(1) * valid.to(dtype)
    one_hot = torch.zeros_like(x).scatter_(1, lb.unsqueeze(1), 1.)
    grad = (wexp / wsum - one_hot) * valid.unsqueeze(1).to(dtype)
    if reduction == 'mean':
        return loss_px.sum() / n_valid, grad / n_valid
    if reduction == 'sum':
        return loss_px.sum(), grad
    return loss_px, grad
