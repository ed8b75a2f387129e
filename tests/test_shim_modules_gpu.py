"""The reference-named extension modules (`lsr_cpp`, `focal_cpp`, `large_margin_cpp`,
`lovasz_softmax_cpp`) executed on the GPU with the reference's argument orders
(csrc/lsr_kernel.cu:319-322, csrc/focal_kernel.cu:337-341, csrc/large_margin_kernel.cu:834-838,
csrc/lovasz_softmax.cu:799-802) and compared with the CPU oracle.  These modules are what the
reference's own Python classes import, so this is the zero-change route of a drop-in."""
import pytest
import torch

from helpers import assert_grad_close, assert_loss_close, labels_with_ignores

pytestmark = pytest.mark.gpu


def _inputs(c=19, shape=(3, 40, 52), seed=31):
    g = torch.Generator().manual_seed(seed)
    n = shape[0]
    logits = torch.randn((n, c) + shape[1:], generator=g) * 1.5
    labels = labels_with_ignores(g, shape, c, 255, 0.1)
    return logits, labels


@pytest.mark.parametrize("c", [19, 150])
def test_lsr_cpp(c):
    import lsr_cpp
    from oracle import losses as O
    logits, labels = _inputs(c)
    want_loss, want_grad = O.label_smooth_ce(logits, labels, 0.1, 255, 'none')
    # lsr_forward(logits, labels, ignore_index, smooth)
    loss = lsr_cpp.lsr_forward(logits.cuda(), labels.cuda(), 255, 0.1)
    grad = lsr_cpp.lsr_backward(logits.cuda(), labels.cuda(), 255, 0.1)
    assert loss.shape == labels.shape and grad.shape == logits.shape
    assert_loss_close(loss, want_loss, atol=2e-6)
    assert_grad_close(grad, want_grad)


def test_focal_cpp():
    import focal_cpp
    from oracle import losses as O
    g = torch.Generator().manual_seed(32)
    logits = torch.randn(2, 3, 33, 41, generator=g) * 2
    labels = (torch.rand(2, 3, 33, 41, generator=g) < 0.2).float()
    want_loss, want_grad = O.focal_loss(logits, labels, 0.3, 1.5, 'none')
    x, y = logits.cuda(), labels.cuda()
    # note the order at this boundary: (logits, labels, gamma, alpha)
    loss = focal_cpp.focalloss_forward(x, y, 1.5, 0.3)
    grad = focal_cpp.focalloss_backward(x, y, 1.5, 0.3)
    loss2, grad2 = focal_cpp.focalloss_forward_backward(x, y, 1.5, 0.3)
    assert_loss_close(loss, want_loss, atol=1e-6)
    assert_grad_close(grad, want_grad)
    assert torch.equal(loss, loss2)
    assert_grad_close(grad2, want_grad)
    with pytest.raises(RuntimeError):
        focal_cpp.focalloss_forward(x, y.long(), 1.5, 0.3)         # labels must have the logits' dtype


@pytest.mark.parametrize("c", [19, 150])
def test_large_margin_cpp(c):
    import large_margin_cpp
    from oracle import losses as O
    logits, labels = _inputs(c, seed=33)
    want_loss, want_grad = O.large_margin_softmax(logits, labels, 0.3, 255, 'none')
    x, y = logits.cuda(), labels.cuda()
    # l_margin_*(logits, labels, lam, ignore_index)
    loss = large_margin_cpp.l_margin_forward(x, y, 0.3, 255)
    grad = large_margin_cpp.l_margin_backward(x, y, 0.3, 255)
    loss2, grad2, cnt = large_margin_cpp.l_margin_forward_backward(x, y, 0.3, 255)
    assert_loss_close(loss, want_loss, atol=2e-6)
    assert_grad_close(grad, want_grad)
    assert_loss_close(loss2, want_loss, atol=2e-6)
    assert_grad_close(grad2, want_grad)
    assert cnt.dtype == torch.int64 and cnt.shape == (1,) and int(cnt) == int((labels != 255).sum())


def test_lovasz_softmax_cpp():
    import lovasz_softmax_cpp
    from oracle import losses as O
    from oracle.losses import _lovasz_group
    logits, labels = _inputs(7, shape=(2, 60, 70), seed=34)
    want_loss, _ = O.lovasz_softmax(logits, labels, 255, 'none', dtype=torch.float64)
    x, y = logits.cuda(), labels.cuda()
    loss, jacc = lovasz_softmax_cpp.lovasz_softmax_forward(x, y, 255)
    assert loss.shape == (7,) and jacc.shape == (7, labels.numel())
    up = torch.linspace(0.5, 2.0, 7)
    keep = jacc.clone()
    grad = lovasz_softmax_cpp.lovasz_softmax_backward(up.cuda(), x, y, jacc, 255)
    grad_again = lovasz_softmax_cpp.lovasz_softmax_backward(up.cuda(), x, y, jacc, 255)
    assert torch.equal(jacc, keep) and torch.equal(grad, grad_again)      # the saved tensor is only read
    assert_loss_close(loss, want_loss.float(), atol=1e-6)
    # the oracle's gradient for a per-class upstream gradient: d(sum_c up_c * loss_c)/d(logits)
    _, want_weighted = _lovasz_group(logits.double(), labels, 255, upstream=up.double())
    assert_grad_close(grad, want_weighted.float())
