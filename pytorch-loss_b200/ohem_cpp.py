"""Stand-in for the reference's `ohem_cpp` extension module
(csrc/ohem_label_kernel.cu:279-281)."""
from pytorch_loss import ohem_loss as _oh


def score_ohem_label(logits, labels, ignore_index, score_thresh, n_min):
    """Labels with the easy pixels set to `ignore_index` (the `n_min` hardest always stay)."""
    return _oh.score_ohem_label(logits, labels, ignore_index, score_thresh, n_min)
