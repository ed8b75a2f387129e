"""LovaszSoftmaxV3 (CUDA, through the C ABI) against the CPU oracle and the golden files.
Inputs are continuous random logits, so error ties have measure zero."""
import os

import numpy as np
import pytest
import torch

from helpers import assert_grad_close, assert_loss_close, labels_with_ignores, run_module

pytestmark = pytest.mark.gpu


def _blocky_labels(gen, n, c, h, w, cell, ignore, frac):
    cells = torch.randint(0, c, (n, (h + cell - 1) // cell, (w + cell - 1) // cell), generator=gen)
    lb = cells.repeat_interleave(cell, 1).repeat_interleave(cell, 2)[:, :h, :w].contiguous()
    if frac > 0:
        lb[torch.rand(lb.shape, generator=gen) < frac] = ignore
    return lb


SHAPES = [(2, 5, 12, 11), (1, 19, 16, 16), (3, 4, 9, 7), (2, 7, 40, 52), (1, 3, 130, 127),
          (2, 19, 96, 96), (1, 2, 8, 8), (2, 40, 33, 20), (1, 300, 12, 12),
          # 512-pixel pipelined tiles: ragged second box, widest backward / forward class counts
          (2, 19, 26, 30), (1, 26, 24, 37), (1, 40, 30, 28),
          # odd pixel counts (no 16-byte aligned channel rows): a pixel's channels in one thread's registers
          # up to 40 classes (several 256-pixel groups per image), the tile kernel without TMA beyond
          (2, 19, 37, 41), (1, 33, 9, 31), (1, 41, 9, 31)]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("per_image", [False, True])
@pytest.mark.parametrize("reduction", ["mean", "none"])
def test_matches_oracle(shape, per_image, reduction):
    import pytorch_loss as P
    from oracle import losses as O
    n, c, h, w = shape
    g = torch.Generator().manual_seed(sum(shape))
    logits = torch.randn(shape, generator=g)
    labels = labels_with_ignores(g, (n, h, w), c, 255, 0.1)
    want_loss, want_grad = O.lovasz_softmax(logits, labels, 255, reduction, per_image, dtype=torch.float64)
    loss, grad = run_module(P.LovaszSoftmaxV3(reduction, 255, per_image=per_image), logits.cuda(), labels.cuda())
    assert_loss_close(loss, want_loss.float(), atol=1e-6)
    assert_grad_close(grad, want_grad.float())
    ign = labels == 255
    assert bool((grad.cpu().transpose(0, 1)[:, ign] == 0).all())


def test_golden(golden_dir):
    import pytorch_loss as P
    z = np.load(os.path.join(golden_dir, "lovasz.npz"))
    for i in range(int(z["n_cases"])):
        ign = int(z[f"c{i}_hyper"][0])
        red = str(z[f"c{i}_reduction"])
        logits, labels = torch.from_numpy(z[f"c{i}_logits"]), torch.from_numpy(z[f"c{i}_labels"])
        loss, grad = run_module(P.LovaszSoftmaxV3(red, ign), logits.cuda(), labels.cuda())
        assert_loss_close(loss, torch.from_numpy(z[f"c{i}_loss_v1"]), atol=1e-6, what=f"c{i} loss")
        assert_grad_close(grad, torch.from_numpy(z[f"c{i}_grad_v1"]), what=f"c{i} grad")
        loss, grad = run_module(P.LovaszSoftmaxV3('none', ign, per_image=True), logits.cuda(), labels.cuda())
        assert_loss_close(loss, torch.from_numpy(z[f"c{i}_loss_per_image"]), atol=1e-6, what=f"c{i} per-image loss")
        assert_grad_close(grad, torch.from_numpy(z[f"c{i}_grad_per_image"]), what=f"c{i} per-image grad")


def test_multi_tile_segments_and_blocky_labels(monkeypatch):
    """Segments longer than one sort tile (8192 pixels), realistic label maps, absent classes; the
    pruned sort against the sort of every element."""
    import pytorch_loss as P
    from oracle import losses as O
    g = torch.Generator().manual_seed(77)
    logits = torch.randn(2, 19, 160, 200, generator=g)
    labels = _blocky_labels(g, 2, 17, 160, 200, 32, 255, 0.03)      # classes 17, 18 never occur
    for per_image in (False, True):
        want_loss, want_grad = O.lovasz_softmax(logits, labels, 255, 'none', per_image, dtype=torch.float64)
        crit = P.LovaszSoftmaxV3('none', 255, per_image=per_image)
        loss, grad = run_module(crit, logits.cuda(), labels.cuda())
        assert_loss_close(loss, want_loss.float(), atol=1e-6)
        assert_grad_close(grad, want_grad.float())
        monkeypatch.setenv("B200_LOVASZ_NO_PRUNE", "1")
        loss_full, grad_full = run_module(crit, logits.cuda(), labels.cuda())
        assert_loss_close(loss_full, loss, atol=1e-6)
        assert_grad_close(grad_full, grad, atol=1e-7)       # (a segment may take the 20-bit sort in one run only)
        # with every segment on the 30-bit sort the two runs rank identically: same bits
        monkeypatch.setenv("B200_LOVASZ_EXACT", "1")
        loss_full, grad_full = run_module(crit, logits.cuda(), labels.cuda())
        monkeypatch.delenv("B200_LOVASZ_NO_PRUNE")
        loss_pruned, grad_pruned = run_module(crit, logits.cuda(), labels.cuda())
        monkeypatch.delenv("B200_LOVASZ_EXACT")
        assert_loss_close(loss_full, loss_pruned, atol=1e-6)
        assert torch.equal(grad_full, grad_pruned)


def test_pruned_sort_cases(monkeypatch):
    """The sort drops elements past the last foreground element of their class (their dJ is exactly
    zero).  Cases that move that bound around: classes absent from some or all images, a saturated
    foreground pixel (error 0: nothing can be dropped), an image that is ignored entirely, and the
    unpruned path as a cross-check."""
    import pytorch_loss as P
    from oracle import losses as O
    g = torch.Generator().manual_seed(2024)
    n, c, h, w = 3, 7, 48, 44                                       # 2112 pixels per image: pipelined tiles
    base = torch.randn(n, c, h, w, generator=g)
    lab_few = torch.randint(0, 2, (n, h, w), generator=g)           # classes 2..6 absent everywhere
    lab_mixed = labels_with_ignores(g, (n, h, w), c, 255, 0.2)
    lab_mixed[1] = 255                                              # one image ignored entirely
    lab_mixed[2][lab_mixed[2] == 3] = 4                             # class 3 absent from image 2 only
    saturated = base.clone()
    saturated[0, :, 0, 0] = -40.0
    saturated[0, int(lab_mixed[0, 0, 0]) if lab_mixed[0, 0, 0] != 255 else 0, 0, 0] = 40.0
    lab_sat = lab_mixed.clone()
    if lab_sat[0, 0, 0] == 255:
        lab_sat[0, 0, 0] = 0
    cases = [(base, lab_few), (base * 6.0, lab_mixed), (saturated, lab_sat)]
    for logits, labels in cases:
        for per_image in (False, True):
            want_loss, want_grad = O.lovasz_softmax(logits, labels, 255, 'none', per_image, dtype=torch.float64)
            crit = P.LovaszSoftmaxV3('none', 255, per_image=per_image)
            loss, grad = run_module(crit, logits.cuda(), labels.cuda())
            assert_loss_close(loss, want_loss.float(), atol=1e-6)
            assert_grad_close(grad, want_grad.float())
            monkeypatch.setenv("B200_LOVASZ_NO_PRUNE", "1")
            monkeypatch.setenv("B200_LOVASZ_EXACT", "1")
            loss_full, grad_full = run_module(crit, logits.cuda(), labels.cuda())
            monkeypatch.delenv("B200_LOVASZ_NO_PRUNE")
            loss_pruned, grad_pruned = run_module(crit, logits.cuda(), labels.cuda())
            monkeypatch.delenv("B200_LOVASZ_EXACT")
            assert_loss_close(loss_full, loss, atol=1e-6)
            assert_grad_close(grad_full, grad, atol=1e-7)
            assert torch.equal(grad_full, grad_pruned)              # same ranks, same dJ, same gradient


def test_sorted_order_properties():
    """Size-independent checks on the raw C-ABI outputs: per segment the Jaccard gradients
    are non-negative and sum to 1 (J runs from 0 to 1) and the loss lies in [0, 1]."""
    from pytorch_loss import lovasz_softmax as L
    g = torch.Generator().manual_seed(78)
    logits = torch.randn(2, 6, 120, 150, generator=g).cuda()
    labels = labels_with_ignores(g, (2, 120, 150), 6, 255, 0.05).cuda()
    for per_image in (False, True):
        loss, jacc, _, _ = L.lovasz_forward(logits, labels, 255, per_image)
        seg = jacc.reshape(-1, jacc.shape[-1]).double()
        assert bool((seg >= 0).all())
        torch.testing.assert_close(seg.sum(1), torch.ones_like(seg[:, 0]), rtol=0, atol=1e-4)
        assert bool(((loss >= 0) & (loss <= 1)).all())


def test_all_ignored_and_reference_function_signature():
    import pytorch_loss as P
    logits = torch.randn(1, 4, 8, 8).cuda().requires_grad_(True)
    labels = torch.full((1, 8, 8), 255, dtype=torch.int64).cuda()
    loss = P.LovaszSoftmaxFunctionV3.apply(logits, labels, 255)
    assert loss.shape == (4,) and bool((loss == 0).all())
    loss.sum().backward()
    assert bool((logits.grad == 0).all())


def test_backward_twice_and_fp16_input():
    import pytorch_loss as P
    from oracle import losses as O
    g = torch.Generator().manual_seed(79)
    logits = torch.randn(2, 5, 20, 24, generator=g)
    labels = labels_with_ignores(g, (2, 20, 24), 5, 255, 0.1)
    x = logits.cuda().requires_grad_(True)
    loss = P.LovaszSoftmaxV3(ignore_index=255)(x, labels.cuda())
    g1, = torch.autograd.grad(loss, x, retain_graph=True)
    g2, = torch.autograd.grad(loss, x)
    assert torch.equal(g1, g2)                 # saved tensors are not clobbered
    want_loss, want_grad = O.lovasz_softmax(logits.half().float(), labels, 255, 'mean')
    loss16, grad16 = run_module(P.LovaszSoftmaxV3(ignore_index=255), logits.half().cuda(), labels.cuda())
    assert grad16.dtype == torch.float16
    assert_loss_close(loss16, want_loss, rtol=2e-3)
    assert_grad_close(grad16, want_grad, atol=2e-3 * float(want_grad.abs().max()), rtol=2e-3)


def test_unsupported_shapes_raise():
    import pytorch_loss as P
    with pytest.raises(RuntimeError):
        P.LovaszSoftmaxV3()(torch.randn(1, 1100, 4, 4).cuda(), torch.zeros(1, 4, 4, dtype=torch.int64).cuda())
    with pytest.raises(ValueError):
        P.LovaszSoftmaxV3(process_group=True)
