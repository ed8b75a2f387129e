"""Memory layouts and size limits: channels-last logits are consumed in place (every pixel is a
row of C contiguous logits -- no `.contiguous()` copy as in the reference, csrc/lsr_kernel.cu:222-224)
and give channels-last gradients; arbitrary strided views still work through a copy; Lovasz refuses
inputs whose pixel count does not fit its 32-bit pixel indices."""
import pytest
import torch

from helpers import assert_grad_close, assert_loss_close, labels_with_ignores, run_module

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("c", [19, 150, 1024])
@pytest.mark.parametrize("kind", ["lsr", "lmargin"])
@pytest.mark.parametrize("reduction", ["mean", "none"])
def test_channels_last_softmax_losses(c, kind, reduction):
    import pytorch_loss as P
    from pytorch_loss import _softmax_family as SF
    from oracle import losses as O
    g = torch.Generator().manual_seed(900 + c)
    logits = torch.randn(2, c, 12, 20, generator=g) * 1.5
    labels = labels_with_ignores(g, (2, 12, 20), c, 255, 0.15)
    if kind == "lsr":
        crit, (want_loss, want_grad) = P.LabelSmoothSoftmaxCEV3(0.1, reduction, 255), O.label_smooth_ce(logits, labels, 0.1, 255, reduction)
    else:
        crit, (want_loss, want_grad) = P.LargeMarginSoftmaxV3(0.3, reduction, 255), O.large_margin_softmax(logits, labels, 0.3, 255, reduction)
    x = logits.cuda().contiguous(memory_format=torch.channels_last)
    assert not x.is_contiguous()
    same, n, cc, m = SF.kernel_layout(x)
    assert same.data_ptr() == x.data_ptr() and (n, cc, m) == (2 * 12 * 20, c, 1)      # consumed in place as rows
    loss, grad = run_module(crit, x, labels.cuda())
    assert_loss_close(loss, want_loss, atol=2e-6 if reduction == "none" else 1e-7)
    assert_grad_close(grad, want_grad)
    assert grad.is_contiguous(memory_format=torch.channels_last)


def test_channels_last_focal_and_strided_views():
    import pytorch_loss as P
    from oracle import losses as O
    g = torch.Generator().manual_seed(901)
    logits = torch.randn(2, 6, 17, 9, generator=g) * 2
    labels = (torch.rand(2, 6, 17, 9, generator=g) < 0.2).float()
    for reduction in ("mean", "none"):
        want_loss, want_grad = O.focal_loss(logits, labels, 0.25, 2.0, reduction)
        x = logits.cuda().contiguous(memory_format=torch.channels_last)
        y = labels.cuda().contiguous(memory_format=torch.channels_last)
        loss, grad = run_module(P.FocalLossV3(reduction=reduction), x, y)
        assert_loss_close(loss, want_loss, atol=1e-6)
        assert_grad_close(grad, want_grad)
        assert grad.is_contiguous(memory_format=torch.channels_last)
        # mixed layouts and a per-element upstream gradient
        xg = x.detach().clone(memory_format=torch.preserve_format).requires_grad_(True)
        out = P.FocalSigmoidLossFuncV3.apply(xg, labels.cuda(), 0.25, 2.0)
        up = torch.randn(2, 6, 17, 9, generator=g)
        out.backward(up.cuda())
        _, g_none = O.focal_loss(logits, labels, 0.25, 2.0, "none")
        assert_grad_close(xg.grad, g_none * up)
    # a strided view (every other column): copied, still right
    wide = torch.randn(2, 5, 8, 20, generator=g)
    lab = labels_with_ignores(g, (2, 8, 10), 5, 255, 0.1)
    view = wide.cuda()[..., ::2]
    want_loss, want_grad = O.label_smooth_ce(wide[..., ::2], lab, 0.1, 255, "mean")
    loss, grad = run_module(P.LabelSmoothSoftmaxCEV3(0.1, "mean", 255), view, lab.cuda())
    assert_loss_close(loss, want_loss)
    assert_grad_close(grad, want_grad)


def test_lovasz_refuses_pixel_counts_beyond_32_bits():
    """The reference asserts numel < 2^31 (csrc/lovasz_softmax.cu:664); here the pixel index of the
    sort is 32 bits wide, so N*M >= 2^31 is refused with a message before anything is launched
    (checked through the C ABI with null data pointers: nothing is dereferenced)."""
    from pytorch_loss import _cabi
    lib = _cabi.load_library()
    big_n, m = 1 << 12, 1 << 19                       # 2^31 pixels
    assert int(lib.b200_lovasz_workspace_bytes(big_n, 2, m, 0)) == 0
    rc = lib.b200_lovasz_forward(None, None, None, None, None, 0, big_n, 2, m, _cabi.F32, 255, 0, None)
    assert rc != 0 and b"2^31" in lib.b200_last_error()
    assert lib.b200_lovasz_backward(None, None, None, None, None, big_n, 2, m, _cabi.F32, 255, 0, None) != 0
