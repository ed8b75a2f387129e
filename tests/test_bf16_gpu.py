"""bfloat16 logits (storage type; arithmetic stays fp32): every loss against the CPU oracle evaluated
on the same bf16-rounded inputs.  The reduced loss is formed in fp32/fp64, so it keeps the fp32
tolerance; gradients leave rounded to bf16 (8 mantissa bits): 2^-8 relative."""
import pytest
import torch

from helpers import assert_grad_close, assert_loss_close, labels_with_ignores, run_module

pytestmark = pytest.mark.gpu

BF16_RTOL = 2.0 ** -8


def _grad_close(grad, want, what, roundings=1):
    assert grad.dtype == torch.bfloat16
    tol = roundings * BF16_RTOL
    assert_grad_close(grad.float(), want, atol=tol * float(want.abs().max()), rtol=tol, what=what)


@pytest.mark.parametrize("shape", [(2, 19, 40, 52), (1, 150, 24, 44), (2, 7, 9, 5), (6, 4096), (64, 10)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("kind", ["lsr", "lmargin", "pc"])
@pytest.mark.parametrize("reduction", ["mean", "none"])
def test_softmax_losses_bf16(shape, kind, reduction):
    import pytorch_loss as P
    from oracle import losses as O
    from oracle import pc_softmax as PC
    g = torch.Generator().manual_seed(800 + shape[1])
    logits = (torch.randn(shape, generator=g) * 1.5).bfloat16()
    labels = labels_with_ignores(g, shape[:1] + shape[2:], shape[1], 255, 0.1)
    x32 = logits.float()
    if kind == "lsr":
        crit, (want_loss, want_grad) = P.LabelSmoothSoftmaxCEV3(0.1, reduction, 255), O.label_smooth_ce(x32, labels, 0.1, 255, reduction)
    elif kind == "lmargin":
        crit, (want_loss, want_grad) = P.LargeMarginSoftmaxV3(0.3, reduction, 255), O.large_margin_softmax(x32, labels, 0.3, 255, reduction)
    else:
        prop = (torch.rand(shape[1], generator=g) + 0.05)
        prop = (prop / prop.sum()).tolist()
        crit, (want_loss, want_grad) = P.PCSoftmaxCrossEntropyV2(prop, reduction, 255), PC.pc_softmax_ce(x32, labels, prop, 255, reduction)
    loss, grad = run_module(crit, logits.cuda(), labels.cuda())
    if reduction == "mean":
        # (PC softmax rounds its per-pixel losses to bf16 before they are summed: unbiased, ~1e-4 left)
        assert_loss_close(loss.float(), want_loss, rtol=2e-5 if kind != "pc" else 1e-3, what=kind + " loss")
    else:
        assert_loss_close(loss.float(), want_loss, rtol=BF16_RTOL, atol=BF16_RTOL, what=kind + " per-pixel loss")
    # (PC softmax scales its bf16 gradient by the upstream gradient in a second pass: two roundings)
    _grad_close(grad, want_grad, kind + " grad", roundings=2 if kind == "pc" else 1)
    assert bool((grad.float().cpu().transpose(0, 1)[:, labels == 255] == 0).all())


@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_focal_bf16(reduction):
    import pytorch_loss as P
    from oracle import losses as O
    g = torch.Generator().manual_seed(810)
    logits = (torch.randn(3, 2, 41, 67, generator=g) * 2).bfloat16()
    labels = (torch.rand(3, 2, 41, 67, generator=g) < 0.2).bfloat16()
    want_loss, want_grad = O.focal_loss(logits.float(), labels.float(), 0.25, 2.0, reduction)
    loss, grad = run_module(P.FocalLossV3(reduction=reduction), logits.cuda(), labels.cuda())
    if reduction == "none":
        assert_loss_close(loss.float(), want_loss, rtol=BF16_RTOL, atol=1e-4)
    else:
        assert_loss_close(loss.float(), want_loss, rtol=2e-5)
    _grad_close(grad, want_grad, "focal grad")


def test_lovasz_bf16():
    import pytorch_loss as P
    from oracle import losses as O
    g = torch.Generator().manual_seed(811)
    logits = torch.randn(2, 5, 20, 24, generator=g).bfloat16()
    labels = labels_with_ignores(g, (2, 20, 24), 5, 255, 0.1)
    want_loss, want_grad = O.lovasz_softmax(logits.float(), labels, 255, 'mean')
    loss, grad = run_module(P.LovaszSoftmaxV3(ignore_index=255), logits.cuda(), labels.cuda())
    assert_loss_close(loss.float(), want_loss, rtol=1e-4)      # bf16 inputs tie often: order among equal errors is free
    _grad_close(grad, want_grad, "lovasz grad")
