"""CPU oracle for the fused V3 loss path — TEST INFRASTRUCTURE, NOT A PRODUCT PATH.

A restatement, in plain PyTorch CPU ops, of what the reference project
(CoinCheung/pytorch-loss) computes for its four fused losses, following the
reference's own pure-PyTorch V1/V2 classes op by op.  Only tests/, the smoke check
and bench.py's CPU-baseline / reference arm may import this package; nothing under
pytorch-loss_b200/ does.

Parity status: PINNED.  tests/golden/make_golden.py imports the unmodified reference
V1/V2 classes, runs them on seeded inputs and stores inputs + outputs under
tests/golden/; tests/test_oracle_golden.py checks every function here against those
files.  (The reference ships no golden vectors or tests of its own.)

Every function returns `(loss, grad_logits)` where `grad_logits` is d(loss)/d(logits)
for an upstream gradient of ones (for reduction 'none': of the un-reduced loss summed).
Unreduced shapes follow the V3 classes: [N, *spatial] with zeros at ignored pixels for
label-smooth and large-margin, the logits' shape for focal, [C] ([N, C] per image) for
Lovasz.
"""
import torch
import torch.nn.functional as F


def _reduce(loss_px, n_valid, reduction):
    if reduction == 'mean':
        return loss_px.sum() / n_valid
    if reduction == 'sum':
        return loss_px.sum()
    return loss_px


def label_smooth_ce(logits, labels, lb_smooth=0.1, ignore_index=-100, reduction='mean',
                    dtype=torch.float32):
    """Label-smoothed softmax cross entropy.

    Follows LabelSmoothSoftmaxCEV1.forward (reference pytorch_loss/label_smooth.py:26-54:
    upcast `:35`, smoothed one-hot `:37-45`, -sum(logp*y) `:47-48`, zero ignored `:49`,
    mean over valid pixels `:50-51`) and the hand-derived gradient of
    LSRCrossEntropyFunctionV2.backward (`:89-97`: coeff*softmax - one_hot, zero at
    ignored pixels).
    """
    x = logits.detach().to(dtype)
    num_classes = x.size(1)
    ignore = labels.eq(ignore_index)
    valid = ignore.logical_not()
    n_valid = valid.sum()
    lb = labels.masked_fill(ignore, 0)
    lb_pos, lb_neg = 1. - lb_smooth, lb_smooth / num_classes
    one_hot = torch.full_like(x, lb_neg).scatter_(1, lb.unsqueeze(1), lb_pos)
    one_hot = one_hot * valid.unsqueeze(1).to(dtype)
    loss_px = -(torch.log_softmax(x, dim=1) * one_hot).sum(dim=1)
    coeff = (num_classes - 1) * lb_neg + lb_pos
    grad = (torch.softmax(x, dim=1) * coeff - one_hot) * valid.unsqueeze(1).to(dtype)
    if reduction == 'mean':
        grad = grad / n_valid
    return _reduce(loss_px, n_valid, reduction), grad


def focal_loss(logits, labels, alpha=0.25, gamma=2., reduction='mean', dtype=torch.float32):
    """Sigmoid focal loss.

    Forward as FocalLossV1.forward / FocalSigmoidLossFuncV2.forward (reference
    focal_loss.py:22-45, 56-75: softplus-based log p and log(1-p), coeff = -|y-p|^gamma);
    gradient as FocalSigmoidLossFuncV2.backward (`:77-98`).
    """
    x = logits.detach().to(dtype)
    y = labels.detach().to(dtype)
    probs = torch.sigmoid(x)
    coeff = (y - probs).abs().pow(gamma).neg()
    log_probs = torch.where(x >= 0, F.softplus(x, -1, 50), x - F.softplus(x, 1, 50))
    log_1_probs = torch.where(x >= 0, -x + F.softplus(x, -1, 50), -F.softplus(x, 1, 50))
    ce = y * alpha * log_probs + (1. - y) * (1. - alpha) * log_1_probs
    loss_el = ce * coeff

    d_coeff = (y - probs).abs().pow(gamma - 1.) * gamma * probs * (1. - probs)
    d_coeff = torch.where(y < probs, -d_coeff, d_coeff)
    d_ce = y * alpha - probs * (1. - y - alpha + 2. * y * alpha)
    grad = d_coeff * ce + d_ce * coeff
    if reduction == 'mean':
        return loss_el.mean(), grad / loss_el.numel()
    if reduction == 'sum':
        return loss_el.sum(), grad
    return loss_el, grad


def large_margin_softmax(logits, labels, lam=0.3, ignore_index=255, reduction='mean',
                         dtype=torch.float32):
    """Large-margin softmax cross entropy (Kobayashi, BMVC 2019).

    Follows LargeMarginSoftmaxFuncV2 (reference large_margin_softmax.py:68-111): the
    target logit is masked to -inf, q = softmax of the rest, loss =
    CE + lam/2 * sum_{j != lb} (q_j - 1/(C-1)) * log q_j; gradient
    p + lam/2 * (q * (x + 1 - sum q x) - 1/(C-1)) off target, p - 1 on target.  Ignored
    pixels are handled as the module does (`:128-131`: label 0 then dropped); unreduced
    output keeps them as zeros like the V3 kernel (csrc/large_margin_kernel.cu:414-421).
    """
    x = logits.detach().to(dtype)
    num_classes = x.size(1)
    coeff = 1. / (num_classes - 1.)
    ignore = labels.eq(ignore_index)
    valid = ignore.logical_not()
    n_valid = valid.sum()
    lb = labels.masked_fill(ignore, 0)
    idx = torch.zeros_like(x).scatter_(1, lb.unsqueeze(1), 1.).bool()

    lgts = x.masked_fill(idx, float('-inf'))
    q = lgts.softmax(dim=1)
    log_q = lgts.log_softmax(dim=1)
    mg = ((q - coeff) * log_q * (lam / 2.)).masked_fill(idx, 0.)
    loss_px = mg.sum(dim=1) + F.cross_entropy(x, lb, reduction='none')
    loss_px = loss_px * valid.to(dtype)

    p = x.softmax(dim=1)
    qx = (q * lgts).masked_fill(idx, 0.)
    grad = (q * (lgts + 1. - qx.sum(dim=1, keepdim=True)) - coeff) * (lam / 2.)
    grad = grad.masked_fill(idx, -1.) + p
    grad = grad * valid.unsqueeze(1).to(dtype)
    if reduction == 'mean':
        grad = grad / n_valid
    return _reduce(loss_px, n_valid, reduction), grad


def _lovasz_group(x, labels, ignore_index, upstream=None):
    """One group (all pixels of `x` [n, C, *] sorted together): per-class loss [C] and
    its gradient for an upstream gradient of ones, or of `upstream` [C].  Follows LovaszSoftmaxV1.forward (reference lovasz_softmax.py:31-61):
    drop ignored pixels, errs = |one_hot - softmax|, sort descending per class, Jaccard
    index of the sorted prefix, adjacent difference, dot product."""
    x = x.detach().clone().requires_grad_(True)
    c = x.size(1)
    flat = x.transpose(0, 1).reshape(c, -1)
    lab = labels.reshape(-1)
    keep = lab.ne(ignore_index).nonzero(as_tuple=False).reshape(-1)
    probs = flat.softmax(dim=0)[:, keep]
    lab = lab[keep]
    one_hot = torch.zeros_like(probs).scatter_(0, lab.unsqueeze(0), 1).detach()
    errs = (one_hot - probs).abs()
    errs_sort, order = torch.sort(errs, dim=1, descending=True)
    n_samples = errs.size(1)
    with torch.no_grad():
        fg_sort = torch.gather(one_hot, 1, order)
        n_pos = fg_sort.sum(dim=1, keepdim=True)
        inter = n_pos - fg_sort.cumsum(dim=1)
        union = n_pos + (1. - fg_sort).cumsum(dim=1)
        jacc = 1. - inter / union
        if n_samples > 1:
            jacc[:, 1:] = jacc[:, 1:] - jacc[:, :-1]
    losses = torch.einsum('ab,ab->a', errs_sort, jacc)
    (losses.sum() if upstream is None else (losses * upstream.to(losses.dtype)).sum()).backward()
    return losses.detach(), x.grad


def lovasz_softmax(logits, labels, ignore_index=-100, reduction='mean', per_image=False,
                   dtype=torch.float32):
    """Lovasz-softmax loss.  `per_image=False`: the reference's behaviour, one sort per
    class over the whole batch (lovasz_softmax.py:33-34), loss [C] reduced over classes
    (`:63-66`).  `per_image=True`: the same applied to each image on its own, loss
    [N, C]; 'mean' averages over all N*C entries, 'sum' adds them."""
    x = logits.detach().to(dtype)
    if not per_image:
        losses, grad = _lovasz_group(x, labels, ignore_index)
    else:
        parts = [_lovasz_group(x[i:i + 1], labels[i:i + 1], ignore_index) for i in range(x.size(0))]
        losses = torch.stack([p[0] for p in parts], dim=0)
        grad = torch.cat([p[1] for p in parts], dim=0)
    if reduction == 'mean':
        return losses.mean(), grad / losses.numel()
    if reduction == 'sum':
        return losses.sum(), grad
    return losses, grad
