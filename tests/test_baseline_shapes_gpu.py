"""Parity at the shapes the benchmark measures: the five baseline configurations at their full
per-item size (reduced batch where the CPU oracle would otherwise take minutes), inputs from the
benchmark's own generator (bench_workloads.Workload.make), so every launch geometry the bench
times -- persistent loops that wrap, 262 144-pixel images, 64 KB rows, 1 048 576-pixel Lovasz
segments of 128 sort tiles -- is compared with the CPU oracle.

'mean' divides O(1) gradients by millions of pixels, where the absolute tolerance would pass
anything; so every case also runs reduction 'sum' (or 'none'), whose gradients are O(1), and the
'mean' gradients are checked relative to their own largest magnitude.
Tolerances: fp32 loss 1e-5 relative, gradients 1e-5 abs + 1e-5 rel; fp16 2e-3."""
import pytest
import torch

import bench_workloads as BW
from helpers import assert_grad_close, assert_loss_close, run_module, TOL_F16

pytestmark = pytest.mark.gpu


def _oracle():
    from oracle import losses as O
    return O


def _check_scaled(grad, want, what, units=1e-5):
    """|got - want| <= units * max|want| + 1e-5 * |want|: the stated tolerance in units of the
    largest gradient, for reductions that shrink every gradient far below the absolute 1e-5."""
    scale = float(want.abs().max())
    assert_grad_close(grad, want, atol=units * scale, rtol=1e-5, what=what)


# Segments with at least 4096 foreground pixels are sorted on the top 20 bits of an error (2^-13
# relative): pixels whose errors agree that closely may come out in either order, which moves a
# pixel's dJ by up to ~8e-5 of the largest dJ of its class on 1 Mpixel segments (csrc/lovasz.cu,
# "Key bits").  The stated tolerance (1e-5 absolute) is four orders wider; the checks below hold
# the gradients to 2e-4 of their largest, and to 1e-5 of it with B200_LOVASZ_EXACT=1 (all 30 bits).
LOVASZ_RANK_UNITS = 2e-4


@pytest.mark.parametrize("items", [2, 5, 9])
def test_config1_label_smooth(items):
    """[items,19,512,512], 5 % ignored.  Up to 40 M elements (2 and 5 images) the fused step is the
    register-resident kernel; 9 images (44.8 M) take the tile pipeline of the full configuration:
    two-box TMA tiles, 512 tiles per image."""
    import pytorch_loss as P
    O = _oracle()
    x, y = BW.WORKLOADS["lsr"].make(items=items)
    for red in ("sum", "mean"):
        want_loss, want_grad = O.label_smooth_ce(x, y, 0.1, 255, red, dtype=torch.float64)
        loss, grad = run_module(P.LabelSmoothSoftmaxCEV3(0.1, red, 255), x.cuda(), y.cuda())
        assert_loss_close(loss, want_loss, what="config 1 %s loss" % red)
        (assert_grad_close if red == "sum" else _check_scaled)(grad, want_grad, what="config 1 %s grad" % red)
        assert bool((grad.cpu().transpose(0, 1)[:, y == 255] == 0).all())
    want_px, _ = O.label_smooth_ce(x, y, 0.1, 255, "none")
    px, _ = run_module(P.LabelSmoothSoftmaxCEV3(0.1, "none", 255), x.cuda(), y.cuda())
    assert_loss_close(px, want_px, atol=2e-6, what="config 1 per-pixel loss")


def test_config2_focal_full_size_and_wrapping_grid():
    """The whole of config 2 (16.7 M elements) and four times that, where the persistent grid of the
    fused step makes several trips; upstream gradients 1 and 2 (the rescale pass)."""
    import pytorch_loss as P
    O = _oracle()
    for items in (16, 64):
        x, y = BW.WORKLOADS["focal"].make(items=items)
        for red in ("sum", "mean"):
            want_loss, want_grad = O.focal_loss(x, y, 0.25, 2.0, red, dtype=torch.float64)
            crit = P.FocalLossV3(0.25, 2, red)
            loss, grad = run_module(crit, x.cuda(), y.cuda())
            assert_loss_close(loss, want_loss, what="config 2 x%d %s loss" % (items, red))
            (assert_grad_close if red == "sum" else _check_scaled)(grad, want_grad, what="config 2 %s grad" % red)
        xg = x.cuda().requires_grad_(True)
        (P.FocalLossV3(0.25, 2, "sum")(xg, y.cuda()) * 2.0).backward()
        want_loss, want_grad = O.focal_loss(x, y, 0.25, 2.0, "sum", dtype=torch.float64)
        assert_grad_close(xg.grad, 2.0 * want_grad, atol=2e-5, what="config 2 upstream 2.0")
    want_el, _ = O.focal_loss(x[:2], y[:2], 0.25, 2.0, "none")
    el, _ = run_module(P.FocalLossV3(0.25, 2, "none"), x[:2].cuda(), y[:2].cuda())
    assert_loss_close(el, want_el, atol=1e-6, what="config 2 per-element loss")


@pytest.mark.parametrize("items", [1, 2])
def test_config3_large_margin(items):
    """[items,150,512,512], 10 % ignored: the 150-class fused step and the chunked forward/backward."""
    import pytorch_loss as P
    O = _oracle()
    x, y = BW.WORKLOADS["lmargin"].make(items=items)
    for red in ("sum", "mean"):
        want_loss, want_grad = O.large_margin_softmax(x, y, 0.3, 255, red, dtype=torch.float64)
        loss, grad = run_module(P.LargeMarginSoftmaxV3(0.3, red, 255), x.cuda(), y.cuda())
        assert_loss_close(loss, want_loss, what="config 3 %s loss" % red)
        (assert_grad_close if red == "sum" else _check_scaled)(grad, want_grad, what="config 3 %s grad" % red)
        assert bool((grad.cpu().transpose(0, 1)[:, y == 255] == 0).all())
    # the separate kernels (per-pixel losses out, per-pixel upstream gradient in)
    want_px, want_grad = O.large_margin_softmax(x, y, 0.3, 255, "none")
    px, grad = run_module(P.LargeMarginSoftmaxV3(0.3, "none", 255), x.cuda(), y.cuda())
    assert_loss_close(px, want_px, atol=2e-6, what="config 3 per-pixel loss")
    assert_grad_close(grad, want_grad, what="config 3 per-pixel grad")


@pytest.mark.parametrize("name", ["lovasz", "lovasz_full"])
def test_config4_lovasz_per_image(name, monkeypatch):
    """[1,19,1024,1024] per image with the bench's blocky labels: segments of 1 048 576 pixels =
    128 sort tiles.  `lovasz` lets the pruning drop ~93 % of the elements; `lovasz_full` has one
    saturated foreground pixel per class, so every valid element is ranked.  Both the 20-bit
    two-pass sort these segments take by default and the 30-bit three-pass sort."""
    import pytorch_loss as P
    O = _oracle()
    x, y = BW.WORKLOADS[name].make(items=1)
    want_loss, want_grad = O.lovasz_softmax(x, y, 255, "none", per_image=True, dtype=torch.float64)
    crit = P.LovaszSoftmaxV3("none", 255, per_image=True)
    loss, grad = run_module(crit, x.cuda(), y.cuda())
    assert_loss_close(loss, want_loss.float(), what="config 4 (%s) loss" % name)
    # dJ of a foreground element is 1/union ~ 2e-5 here: compare in units of the largest gradient
    assert_grad_close(grad, want_grad.float(), what="config 4 (%s) grad, stated tolerance" % name)
    _check_scaled(grad, want_grad.float(), "config 4 (%s) grad" % name, LOVASZ_RANK_UNITS)
    assert bool((grad.cpu().transpose(0, 1)[:, y == 255] == 0).all())
    again = run_module(crit, x.cuda(), y.cuda())
    assert torch.equal(again[0], loss) and torch.equal(again[1], grad)        # reproducible bit for bit
    monkeypatch.setenv("B200_LOVASZ_EXACT", "1")
    loss30, grad30 = run_module(crit, x.cuda(), y.cuda())
    monkeypatch.delenv("B200_LOVASZ_EXACT")
    assert_loss_close(loss30, want_loss.float(), what="config 4 (%s) loss, 30-bit sort" % name)
    _check_scaled(grad30, want_grad.float(), "config 4 (%s) grad, 30-bit sort" % name)
    want_mean, _ = O.lovasz_softmax(x, y, 255, "mean", per_image=True, dtype=torch.float64)
    mean, _ = run_module(P.LovaszSoftmaxV3("mean", 255, per_image=True), x.cuda(), y.cuda())
    assert_loss_close(mean, want_mean.float(), what="config 4 (%s) mean" % name)


def test_config4_lovasz_batch_global_two_images():
    """The reference's batch-global sort over 2 images of config 4: segments of 2 097 152 pixels."""
    import pytorch_loss as P
    O = _oracle()
    x, y = BW.WORKLOADS["lovasz"].make(items=2)
    want_loss, want_grad = O.lovasz_softmax(x, y, 255, "none", dtype=torch.float64)
    loss, grad = run_module(P.LovaszSoftmaxV3("none", 255), x.cuda(), y.cuda())
    assert_loss_close(loss, want_loss.float(), what="batch-global loss")
    _check_scaled(grad, want_grad.float(), "batch-global grad", LOVASZ_RANK_UNITS)


def test_config5_label_smooth_rows_fp16():
    """[256,32768] fp16 rows of 64 KB: the whole-row fused step and the warp-per-row forward."""
    import pytorch_loss as P
    O = _oracle()
    x, y = BW.WORKLOADS["lsr_rows"].make(items=256)
    for red in ("sum", "mean"):
        want_loss, want_grad = O.label_smooth_ce(x.float(), y, 0.1, -100, red, dtype=torch.float64)
        loss, grad = run_module(P.LabelSmoothSoftmaxCEV3(0.1, red, -100), x.cuda(), y.cuda())
        assert grad.dtype == torch.float16
        assert_loss_close(loss, want_loss, rtol=TOL_F16, what="config 5 %s loss" % red)
        scale = float(want_grad.abs().max())
        assert_grad_close(grad.float(), want_grad, atol=TOL_F16 * scale, rtol=TOL_F16, what="config 5 %s grad" % red)
    want_px, _ = O.label_smooth_ce(x.float(), y, 0.1, -100, "none")
    px, _ = run_module(P.LabelSmoothSoftmaxCEV3(0.1, "none", -100), x.cuda(), y.cuda())
    assert_loss_close(px.float(), want_px, rtol=TOL_F16, what="config 5 per-row loss")


def test_pc_softmax_at_config1_shape():
    """PCSoftmaxCrossEntropyV2 at [2,19,512,512] with the benchmark's inputs and class proportions:
    the fused step on the tile pipeline ('mean', 'sum') and the per-pixel kernel ('none')."""
    import pytorch_loss as P
    from oracle import pc_softmax as PC
    wl = BW.WORKLOADS["pc_softmax"]
    x, y = wl.make(items=2)
    prop = wl.proportions()
    for red in ("sum", "mean", "none"):
        want_loss, want_grad = PC.pc_softmax_ce(x, y, prop, 255, red, dtype=torch.float64)
        loss, grad = run_module(P.PCSoftmaxCrossEntropyV2(prop, red, 255), x.cuda(), y.cuda())
        assert_loss_close(loss, want_loss, atol=2e-6 if red == "none" else 1e-7, what="pc softmax %s loss" % red)
        (_check_scaled if red == "mean" else assert_grad_close)(grad, want_grad, what="pc softmax %s grad" % red)
        assert bool((grad.cpu().transpose(0, 1)[:, y == 255] == 0).all())


@pytest.mark.parametrize("shape", [(2, 19, 512, 512), (1, 150, 512, 512)], ids=["19ch", "150ch"])
@pytest.mark.parametrize("use_log", [False, True])
def test_taylor_softmax_at_bench_shapes(shape, use_log):
    """The two Taylor workloads of the benchmark at full per-item size: all channels of a pixel pair
    in one thread's registers (19), channel slices over the threads of a block (150)."""
    import pytorch_loss as P
    from oracle import taylor as OT
    g = torch.Generator().manual_seed(77 + shape[1])
    x = torch.randn(shape, generator=g) * 1.4
    up = torch.randn(shape, generator=g)
    want, want_grad = OT.taylor_softmax(x, 1, 2, use_log, upstream=up, dtype=torch.float64)
    xg = x.cuda().requires_grad_(True)
    out = (P.LogTaylorSoftmaxV3 if use_log else P.TaylorSoftmaxV3)(dim=1, n=2)(xg)
    out.backward(up.cuda())
    assert_loss_close(out.detach(), want, atol=2e-6, what="taylor output")
    assert_grad_close(xg.grad, want_grad, what="taylor gradient")
