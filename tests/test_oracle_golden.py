"""The CPU oracle against the golden files produced by the unmodified reference
(tests/golden/make_golden.py).  Tolerances: the oracle restates the same fp32 op
sequences, so agreement is at rounding level (1e-6 abs + 1e-5 rel)."""
import os

import numpy as np
import pytest
import torch

from oracle import losses as O

RTOL, ATOL = 1e-5, 1e-6


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name + ".npz"))


def _close(a, b, what):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    assert a.shape == b.shape, "%s: shape %s vs %s" % (what, a.shape, b.shape)
    err = np.abs(a - b) - (ATOL + RTOL * np.abs(b))
    assert (err <= 0).all(), "%s: max violation %g" % (what, err.max())


def _cases(z):
    return range(int(z["n_cases"]))


def test_reference_v1_equals_v2(golden_dir):
    """The reference's own versions agree with each other on the stored cases."""
    for name in ("label_smooth", "focal", "large_margin"):
        z = _load(golden_dir, name)
        for i in _cases(z):
            _close(z[f"c{i}_loss_v1"], z[f"c{i}_loss_v2"], f"{name} c{i} loss")
            _close(z[f"c{i}_grad_v1"], z[f"c{i}_grad_v2"], f"{name} c{i} grad")


def test_label_smooth_oracle(golden_dir):
    z = _load(golden_dir, "label_smooth")
    for i in _cases(z):
        sm, ign = z[f"c{i}_hyper"]
        loss, grad = O.label_smooth_ce(torch.from_numpy(z[f"c{i}_logits"]), torch.from_numpy(z[f"c{i}_labels"]),
                                       float(sm), int(ign), str(z[f"c{i}_reduction"]))
        _close(loss.numpy(), z[f"c{i}_loss_v1"], f"lsr c{i} loss")
        _close(grad.numpy(), z[f"c{i}_grad_v1"], f"lsr c{i} grad")


def test_focal_oracle(golden_dir):
    z = _load(golden_dir, "focal")
    for i in _cases(z):
        al, ga = z[f"c{i}_hyper"]
        loss, grad = O.focal_loss(torch.from_numpy(z[f"c{i}_logits"]), torch.from_numpy(z[f"c{i}_labels"]),
                                  float(al), float(ga), str(z[f"c{i}_reduction"]))
        _close(loss.numpy(), z[f"c{i}_loss_v2"], f"focal c{i} loss")
        _close(grad.numpy(), z[f"c{i}_grad_v2"], f"focal c{i} grad")


def test_large_margin_oracle(golden_dir):
    z = _load(golden_dir, "large_margin")
    for i in _cases(z):
        lam, ign = z[f"c{i}_hyper"]
        loss, grad = O.large_margin_softmax(torch.from_numpy(z[f"c{i}_logits"]), torch.from_numpy(z[f"c{i}_labels"]),
                                            float(lam), int(ign), str(z[f"c{i}_reduction"]))
        _close(loss.numpy(), z[f"c{i}_loss_v2"], f"lm c{i} loss")
        _close(grad.numpy(), z[f"c{i}_grad_v2"], f"lm c{i} grad")


def test_lovasz_oracle(golden_dir):
    z = _load(golden_dir, "lovasz")
    for i in _cases(z):
        ign = int(z[f"c{i}_hyper"][0])
        logits, labels = torch.from_numpy(z[f"c{i}_logits"]), torch.from_numpy(z[f"c{i}_labels"])
        loss, grad = O.lovasz_softmax(logits, labels, ign, str(z[f"c{i}_reduction"]))
        _close(loss.numpy(), z[f"c{i}_loss_v1"], f"lovasz c{i} loss")
        _close(grad.numpy(), z[f"c{i}_grad_v1"], f"lovasz c{i} grad")
        loss, grad = O.lovasz_softmax(logits, labels, ign, 'none', per_image=True)
        _close(loss.numpy(), z[f"c{i}_loss_per_image"], f"lovasz c{i} per-image loss")
        _close(grad.numpy(), z[f"c{i}_grad_per_image"], f"lovasz c{i} per-image grad")


def test_unreduced_shapes_follow_v3():
    g = torch.Generator().manual_seed(7)
    logits = torch.randn(2, 5, 3, 4, generator=g)
    labels = torch.randint(0, 5, (2, 3, 4), generator=g)
    labels[0, 0, :2] = 255
    for fn in (O.label_smooth_ce, O.large_margin_softmax):
        loss, grad = fn(logits, labels, ignore_index=255, reduction='none')
        assert loss.shape == (2, 3, 4)
        assert (loss[0, 0, :2] == 0).all() and (grad[0, :, 0, :2] == 0).all()


def test_taylor_oracle(golden_dir):
    """oracle/taylor.py against the reference's taylor_softmax_v1 / TaylorCrossEntropyLossV1."""
    from oracle import taylor as OT
    z = np.load(os.path.join(golden_dir, "taylor.npz"))
    for i in range(int(z["n_cases"])):
        dim, order, use_log = (int(v) for v in z[f"c{i}_hyper"])
        x, up = torch.from_numpy(z[f"c{i}_x"]), torch.from_numpy(z[f"c{i}_up"])
        out, grad = OT.taylor_softmax(x, dim, order, bool(use_log), upstream=up)
        assert torch.allclose(out, torch.from_numpy(z[f"c{i}_out"]), atol=1e-6, rtol=1e-5), i
        assert torch.allclose(grad, torch.from_numpy(z[f"c{i}_grad"]), atol=1e-5, rtol=1e-4), i
    for i in range(int(z["n_ce_cases"])):
        order, ign = (int(v) for v in z[f"ce{i}_hyper"])
        logits, labels = torch.from_numpy(z[f"ce{i}_logits"]), torch.from_numpy(z[f"ce{i}_labels"])
        loss, grad = OT.taylor_cross_entropy(logits, labels, order, ign, str(z[f"ce{i}_reduction"]))
        assert torch.allclose(loss, torch.from_numpy(z[f"ce{i}_loss"]), atol=1e-6, rtol=1e-5), i
        assert torch.allclose(grad, torch.from_numpy(z[f"ce{i}_grad"]), atol=1e-6, rtol=1e-5), i


def test_ohem_oracle_matches_reference_cuda_output(golden_dir):
    """oracle/ohem.py against the labels the reference's own CUDA extension returned
    (tests/golden/ohem.npz, written by make_ohem_golden.py on a B200): exact, case by case."""
    from oracle import ohem as OH
    z = np.load(os.path.join(golden_dir, "ohem.npz"))
    assert int(z["n_cases"]) >= 8
    for i in range(int(z["n_cases"])):
        logits = torch.from_numpy(z[f"c{i}_logits"]).float()
        labels = torch.from_numpy(z[f"c{i}_labels"])
        ign, thresh, n_min = z[f"c{i}_args"]
        want = torch.from_numpy(z[f"c{i}_new_labels"])
        got, _ = OH.score_ohem_label(logits, labels, int(ign), float(thresh), int(n_min))
        assert torch.equal(got, want), "case %d: %d labels differ" % (i, int((got != want).sum()))


def test_pc_softmax_oracle_matches_reference(golden_dir):
    """oracle/pc_softmax.py against PCSoftmaxCrossEntropyV1 (loss, autograd gradient) and the
    loss of PCSoftmaxCrossEntropyV2, as make_golden.py recorded them from the reference."""
    from oracle import pc_softmax as PC
    z = np.load(os.path.join(golden_dir, "pc_softmax.npz"))
    for i in range(int(z["n_cases"])):
        x, y = torch.from_numpy(z[f"c{i}_logits"]), torch.from_numpy(z[f"c{i}_labels"])
        red, ign = str(z[f"c{i}_reduction"]), int(z[f"c{i}_hyper"][0])
        loss, grad = PC.pc_softmax_ce(x, y, z[f"c{i}_proportion"], ign, red)
        for ref in (z[f"c{i}_loss_v1"], z[f"c{i}_loss_v2"]):
            np.testing.assert_allclose(loss.numpy(), ref, rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(grad.numpy(), z[f"c{i}_grad_v1"], rtol=RTOL, atol=ATOL)
