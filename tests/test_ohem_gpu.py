"""OHEM relabelling and the two OHEM losses (CUDA, through the C ABI) against the CPU oracle.

The relabelling decides by comparing fp32 scores with a cut: a pixel whose score lies within
rounding distance of the cut may legitimately fall on either side (the oracle's softmax and the
kernel's differ in the last bits), so label mismatches are accepted only where the oracle's score
is within 2e-6 of the cut, and the cases keep them rare."""
import pytest
import torch

from helpers import assert_grad_close, assert_loss_close, labels_with_ignores, run_module

pytestmark = pytest.mark.gpu


def _check_labels(got, want, scores, cut):
    got, want = got.cpu(), want.cpu()
    bad = got != want
    if bool(bad.any()):
        near = (scores[bad] - cut).abs() <= 2e-6
        assert bool(near.all()), "label mismatch away from the cut: %d pixels" % int((~near).sum())
        assert int(bad.sum()) <= 3


def _cut(scores, thresh, n_min):
    flat = scores.reshape(-1).sort().values
    if n_min <= 0:
        return thresh
    return max(thresh, float(flat[n_min - 1]))


SHAPES = [(2, 19, 33, 41), (1, 5, 16, 16), (3, 7, 8, 9), (2, 150, 12, 20), (64, 10), (4, 3, 40, 52), (1, 40, 7, 5)]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("thresh", [0.05, 0.3, 0.7])
def test_labels_match_oracle(shape, thresh):
    import ohem_cpp
    from oracle import ohem as OH
    g = torch.Generator().manual_seed(sum(shape) + int(thresh * 100))
    logits = torch.randn(shape, generator=g) * 2.0
    labels = labels_with_ignores(g, shape[:1] + shape[2:], shape[1], 255, 0.1)
    total = labels.numel()
    for n_min in (0, 1, total // 16, total // 2, total - 1, total, total + 5):
        want, scores = OH.score_ohem_label(logits, labels, 255, thresh, n_min)
        got = ohem_cpp.score_ohem_label(logits.cuda(), labels.cuda(), 255, thresh, n_min)
        assert got.dtype == torch.int64 and got.shape == labels.shape
        if n_min >= total:
            assert torch.equal(got.cpu(), labels)
            continue
        _check_labels(got, want, scores, _cut(scores, thresh, n_min))
        if n_min < total:
            # the n_min hardest pixels keep their labels; nothing new appears
            kept = got.cpu() != 255
            assert bool((got.cpu()[kept] == labels[kept]).all())
            assert int(kept.sum()) >= min(n_min, int((labels != 255).sum()))


def test_fp16_logits_all_ignored_and_tiny_inputs():
    import ohem_cpp
    from oracle import ohem as OH
    g = torch.Generator().manual_seed(9)
    logits = torch.randn(2, 6, 10, 12, generator=g).half()
    labels = labels_with_ignores(g, (2, 10, 12), 6, 255, 0.2)
    want, scores = OH.score_ohem_label(logits.float(), labels, 255, 0.4, 20)
    got = ohem_cpp.score_ohem_label(logits.cuda(), labels.cuda(), 255, 0.4, 20)
    _check_labels(got, want, scores, _cut(scores, 0.4, 20))
    all_ign = torch.full((2, 10, 12), 255)
    got = ohem_cpp.score_ohem_label(logits.cuda(), all_ign.cuda(), 255, 0.4, 20)
    assert bool((got.cpu() == 255).all())
    one = ohem_cpp.score_ohem_label(torch.randn(1, 4, 1, 1).cuda(), torch.tensor([[[2]]]).cuda(), 255, 0.0, 0)
    assert one.shape == (1, 1, 1)
    with pytest.raises(RuntimeError):
        ohem_cpp.score_ohem_label(logits, labels, 255, 0.4, 20)          # CPU tensors: gpu only


def test_large_image_select_is_exact():
    """4 M pixels: the selection must land exactly on the n_min-th smallest score."""
    import ohem_cpp
    from oracle import ohem as OH
    g = torch.Generator().manual_seed(31)
    logits = torch.randn(4, 19, 512, 512, generator=g)
    labels = labels_with_ignores(g, (4, 512, 512), 19, 255, 0.05)
    n_min = labels.numel() // 16
    want, scores = OH.score_ohem_label(logits, labels, 255, 1e-4, n_min)     # threshold below t: rank decides
    got = ohem_cpp.score_ohem_label(logits.cuda(), labels.cuda(), 255, 1e-4, n_min)
    assert _cut(scores, 1e-4, n_min) > 1e-4
    _check_labels(got, want, scores, _cut(scores, 1e-4, n_min))
    kept = int((got.cpu() != 255).sum())
    assert abs(kept - n_min) <= 3


@pytest.mark.parametrize("cls", ["OhemCELoss", "OhemLargeMarginLoss"])
def test_ohem_losses_match_oracle(cls):
    import pytorch_loss as P
    from oracle import ohem as OH
    g = torch.Generator().manual_seed(77)
    logits = torch.randn(4, 19, 24, 28, generator=g) * 1.5
    labels = labels_with_ignores(g, (4, 24, 28), 19, 255, 0.05)
    n_min = labels.numel() // 16
    fn = OH.ohem_ce_loss if cls == "OhemCELoss" else OH.ohem_large_margin_loss
    want_loss, want_grad = fn(logits, labels, 0.2, n_min, 255)
    crit = getattr(P, cls)(score_thresh=0.2, n_min=n_min, ignore_index=255)
    loss, grad = run_module(crit, logits.cuda(), labels.cuda())
    assert_loss_close(loss, want_loss, rtol=2e-5)
    assert_grad_close(grad, want_grad, atol=2e-5)
    # default n_min = numel // 16 (reference pytorch_loss/ohem_loss.py:23)
    crit = getattr(P, cls)(score_thresh=0.2)
    loss2, _ = run_module(crit, logits.cuda(), labels.cuda())
    assert_loss_close(loss2, want_loss, rtol=2e-5)


def test_golden_from_reference_cuda(golden_dir):
    """The library against the labels the reference's own CUDA extension returned on the same
    inputs (tests/golden/ohem.npz): exact."""
    import os
    import numpy as np
    import ohem_cpp
    z = np.load(os.path.join(golden_dir, "ohem.npz"))
    for i in range(int(z["n_cases"])):
        logits = torch.from_numpy(z[f"c{i}_logits"]).float()
        labels = torch.from_numpy(z[f"c{i}_labels"])
        ign, thresh, n_min = z[f"c{i}_args"]
        want = torch.from_numpy(z[f"c{i}_new_labels"])
        got = ohem_cpp.score_ohem_label(logits.cuda(), labels.cuda(), int(ign), float(thresh), int(n_min))
        assert torch.equal(got.cpu(), want), "case %d: %d labels differ" % (i, int((got.cpu() != want).sum()))
