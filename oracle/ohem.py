"""CPU oracle of the OHEM relabelling step — TEST INFRASTRUCTURE, NOT A PRODUCT PATH.

Parity status: PINNED.  The reference implements `score_ohem_label` in CUDA only
(csrc/ohem_label_kernel.cu; its wrapper raises "this ohem method only supports gpu mode",
:270-272) and ships no CPU version, no golden vectors and no test for it.  This file restates
that CUDA algorithm step by step; tests/golden/ohem.npz holds the labels the reference's own
extension (built unmodified for sm_100a) returned on a B200 for seeded inputs
(tests/golden/make_ohem_golden.py), and tests/test_oracle_golden.py checks this file against
them.  The loss classes built on it use the pinned functions of oracle/losses.py.

Only tests/, the smoke check and bench.py's CPU legs may import this module.
"""
import torch

from . import losses as _losses


def ohem_scores(logits, labels, ignore_index):
    """score = softmax(logits)[label], 1 for ignored pixels
    (reference csrc/ohem_label_kernel.cu:112-150: max :134-139, sum of exponentials :141-145,
    score :146-147, ignored pixels :126-129)."""
    x = logits.detach().float()
    ignore = labels.eq(ignore_index)
    lb = labels.masked_fill(ignore, 0)
    p = torch.softmax(x, dim=1).gather(1, lb.unsqueeze(1)).squeeze(1)
    return torch.where(ignore, torch.ones_like(p), p)


def score_ohem_label(logits, labels, ignore_index, score_thresh, n_min):
    """New labels, and the scores they were decided on.

    Reference csrc/ohem_label_kernel.cu: unchanged labels when n_min >= number of pixels
    (:193); otherwise scores are sorted ascending together with their pixel index (:244-249)
    and every sorted position i >= n_min with score > score_thresh is set to the ignore label
    (:153-166).  The sort here is stable; the reference's is not, which only matters for
    pixels whose score equals the n_min-th smallest one."""
    scores = ohem_scores(logits, labels, ignore_index)
    flat = scores.reshape(-1)
    total = flat.numel()
    if n_min >= total:
        return labels, scores
    order = torch.sort(flat, stable=True).indices
    out = labels.clone().reshape(-1)
    tail = order[max(int(n_min), 0):]
    drop = tail[flat[tail] > score_thresh]
    out[drop] = ignore_index
    return out.reshape(labels.shape), scores


def ohem_ce_loss(logits, labels, score_thresh, n_min=None, ignore_index=255):
    """OhemCELoss (reference pytorch_loss/ohem_loss.py:13-28): relabel, then mean cross entropy
    over what is left.  Returns (loss, d loss / d logits)."""
    n_min = labels.numel() // 16 if n_min is None else n_min
    new_labels, _ = score_ohem_label(logits, labels, ignore_index, score_thresh, n_min)
    return _losses.label_smooth_ce(logits, new_labels, 0.0, ignore_index, 'mean')


def ohem_large_margin_loss(logits, labels, score_thresh, n_min=None, ignore_index=255):
    """OhemLargeMarginLoss (reference pytorch_loss/ohem_loss.py:31-46)."""
    n_min = labels.numel() // 16 if n_min is None else n_min
    new_labels, _ = score_ohem_label(logits, labels, ignore_index, score_thresh, n_min)
    return _losses.large_margin_softmax(logits, new_labels, 0.3, ignore_index, 'mean')
