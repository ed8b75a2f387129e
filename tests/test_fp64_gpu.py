"""float64 logits: label smooth, large margin and focal run double-precision kernels (the reference
dispatches its kernels over double too).  Compared with the oracle evaluated in float64; the
hyper-parameters cross the C boundary as float, as in the reference, so the oracle gets the same
float values.  Tolerance 1e-10: both sides are double arithmetic."""
import numpy as np
import pytest
import torch

from helpers import assert_grad_close, assert_loss_close, labels_with_ignores, run_module

pytestmark = pytest.mark.gpu

F = lambda v: float(np.float32(v))


@pytest.mark.parametrize("shape", [(2, 19, 9, 11), (1, 150, 6, 7), (7, 10), (2, 3, 40, 33)], ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("kind", ["lsr", "lmargin"])
@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_softmax_losses_fp64(shape, kind, reduction):
    import pytorch_loss as P
    from oracle import losses as O
    g = torch.Generator().manual_seed(950 + shape[1])
    logits = torch.randn(shape, generator=g, dtype=torch.float64) * 2.0
    labels = labels_with_ignores(g, shape[:1] + shape[2:], shape[1], 255, 0.15)
    if kind == "lsr":
        crit = P.LabelSmoothSoftmaxCEV3(0.1, reduction, 255)
        want_loss, want_grad = O.label_smooth_ce(logits, labels, F(0.1), 255, reduction, dtype=torch.float64)
    else:
        crit = P.LargeMarginSoftmaxV3(0.3, reduction, 255)
        want_loss, want_grad = O.large_margin_softmax(logits, labels, F(0.3), 255, reduction, dtype=torch.float64)
    loss, grad = run_module(crit, logits.cuda(), labels.cuda())
    assert loss.dtype == torch.float64 and grad.dtype == torch.float64
    assert_loss_close(loss, want_loss, rtol=1e-10, atol=1e-12)
    assert_grad_close(grad, want_grad, atol=1e-12, rtol=1e-10)
    assert bool((grad.cpu().transpose(0, 1)[:, labels == 255] == 0).all())


@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
@pytest.mark.parametrize("gamma", [2.0, 1.5])
def test_focal_fp64(reduction, gamma):
    import pytorch_loss as P
    from oracle import losses as O
    g = torch.Generator().manual_seed(960)
    logits = torch.randn(3, 2, 17, 9, generator=g, dtype=torch.float64) * 3
    labels = (torch.rand(3, 2, 17, 9, generator=g) < 0.2).double()
    want_loss, want_grad = O.focal_loss(logits, labels, F(0.25), gamma, reduction, dtype=torch.float64)
    loss, grad = run_module(P.FocalLossV3(0.25, gamma, reduction), logits.cuda(), labels.cuda())
    assert loss.dtype == torch.float64 and grad.dtype == torch.float64
    assert_loss_close(loss, want_loss, rtol=1e-10, atol=1e-12)
    assert_grad_close(grad, want_grad, atol=1e-12, rtol=1e-9)
    for fn in (P.FocalSigmoidLossFuncV3, P.FocalSigmoidLossFuncV3FB):
        x = logits.cuda().requires_grad_(True)
        up = torch.randn(3, 2, 17, 9, generator=g, dtype=torch.float64)
        fn.apply(x, labels.cuda(), 0.25, gamma).backward(up.cuda())
        _, g_none = O.focal_loss(logits, labels, F(0.25), gamma, "none", dtype=torch.float64)
        assert_grad_close(x.grad, g_none * up, atol=1e-12, rtol=1e-9)


def test_gradcheck_fp64():
    """torch.autograd.gradcheck on the double kernels: analytic gradients against finite differences."""
    import pytorch_loss as P
    g = torch.Generator().manual_seed(970)
    x = (torch.randn(2, 5, 3, 4, generator=g, dtype=torch.float64)).cuda().requires_grad_(True)
    y = labels_with_ignores(g, (2, 3, 4), 5, 255, 0.2).cuda()
    assert torch.autograd.gradcheck(lambda t: P.LSRCrossEntropyFunctionV3.apply(t, y, 0.1, 255), (x,), eps=1e-6, atol=1e-6)
    assert torch.autograd.gradcheck(lambda t: P.LargeMarginSoftmaxFuncV3.apply(t, y, 0.3, 255), (x,), eps=1e-6, atol=1e-6)
    yf = (torch.rand(2, 5, 3, 4, generator=g) < 0.3).double().cuda()
    assert torch.autograd.gradcheck(lambda t: P.FocalSigmoidLossFuncV3.apply(t, yf, 0.25, 2.0), (x,), eps=1e-6, atol=1e-6)
