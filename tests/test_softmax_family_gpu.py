"""LabelSmoothSoftmaxCEV3 and LargeMarginSoftmaxV3 (CUDA, through the C ABI) against the
CPU oracle and the golden files, over every access regime of the kernels:
pixel tiles with and without TMA (M multiple of 4 or not), rows (M == 1, large C) and the
strided sweep (M == 1 with few classes, very large C with M > 1)."""
import os

import numpy as np
import pytest
import torch

from helpers import (assert_grad_close, assert_loss_close, labels_with_ignores, run_module, TOL_F16)

pytestmark = pytest.mark.gpu

# (N, C, spatial) — C in {2,3,19,32,33,64,150,256,500}, M in {1, odd, not multiple of 4, large}
SHAPES = [
    (2, 2, (8, 8)), (3, 3, (5, 7)), (2, 19, (32, 36)), (2, 19, (33, 35)), (1, 32, (64, 66)),
    (2, 33, (17,)), (2, 64, (8, 12)), (2, 150, (24, 24)), (1, 150, (13, 11)), (1, 256, (16, 8)),
    (1, 257, (8, 8)), (1, 500, (6, 10)), (4, 19, (300, 300)),
    (6, 5, ()), (16, 19, ()), (5, 300, ()), (3, 1000, ()), (2, 4099, ()), (2, 2000, (3, 5)),
    # forward in channel chunks (more than 20 classes, >= 512 pixels): last chunk of 9 / 1 / 5 channels,
    # ragged second box, several tiles per image
    (2, 41, (20, 30)), (1, 33, (16, 36)), (3, 21, (26, 30)), (1, 150, (40, 52)),
    # long rows (M == 1, >= 8 KB): one warp per row, 4 KB chunks; whole chunks, ragged last chunk,
    # more rows than warps in flight
    (5, 4096, ()), (3, 5000, ()), (700, 2048, ()),
]


def _crit(kind, reduction, ignore):
    import pytorch_loss as P
    from oracle import losses as O
    if kind == "lsr":
        return P.LabelSmoothSoftmaxCEV3(0.1, reduction, ignore), \
            lambda x, y: O.label_smooth_ce(x, y, 0.1, ignore, reduction)
    return P.LargeMarginSoftmaxV3(0.3, reduction, ignore), \
        lambda x, y: O.large_margin_softmax(x, y, 0.3, ignore, reduction)


@pytest.mark.parametrize("kind", ["lsr", "lmargin"])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, (s[0], s[1]) + s[2])))
@pytest.mark.parametrize("reduction", ["mean", "none"])
def test_matches_oracle(kind, shape, reduction):
    n, c, sp = shape
    g = torch.Generator().manual_seed(1000 + c)
    logits = torch.randn((n, c) + sp, generator=g) * 1.5
    labels = labels_with_ignores(g, (n,) + sp, c, 255, 0.15)
    crit, oracle = _crit(kind, reduction, 255)
    want_loss, want_grad = oracle(logits, labels)
    loss, grad = run_module(crit, logits.cuda(), labels.cuda())
    assert_loss_close(loss, want_loss, atol=2e-6 if reduction == "none" else 1e-7)
    assert_grad_close(grad, want_grad)
    ign = (labels == 255)
    if reduction == "none":
        assert bool((loss.cpu()[ign] == 0).all())
    assert bool((grad.cpu().transpose(0, 1)[:, ign] == 0).all()), "ignored pixels must have exactly zero gradient"


@pytest.mark.parametrize("kind", ["lsr", "lmargin"])
def test_sum_and_ignore_patterns(kind):
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(3, 7, 16, 20, generator=g)
    for pattern in ("none", "rows", "image", "all"):
        labels = torch.randint(0, 7, (3, 16, 20), generator=g)
        if pattern == "rows":
            labels[:, 3:9] = 255
        elif pattern == "image":
            labels[1] = 255
        elif pattern == "all":
            labels[:] = 255
        for reduction in ("sum", "mean"):
            crit, oracle = _crit(kind, reduction, 255)
            want_loss, want_grad = oracle(logits, labels)
            loss, grad = run_module(crit, logits.cuda(), labels.cuda())
            assert_loss_close(loss, want_loss, what=f"{pattern}/{reduction}")
            if pattern == "all" and reduction == "mean":
                assert torch.isnan(loss)            # 0 / 0, as the reference
                assert bool((grad == 0).all())
            else:
                assert_grad_close(grad, want_grad, what=f"{pattern}/{reduction}")


@pytest.mark.parametrize("kind", ["lsr", "lmargin"])
def test_ignore_index_inside_class_range(kind):
    g = torch.Generator().manual_seed(6)
    logits = torch.randn(2, 6, 9, 8, generator=g)
    labels = torch.randint(0, 6, (2, 9, 8), generator=g)
    crit, oracle = _crit(kind, "mean", 3)
    want_loss, want_grad = oracle(logits, labels)
    loss, grad = run_module(crit, logits.cuda(), labels.cuda())
    assert_loss_close(loss, want_loss)
    assert_grad_close(grad, want_grad)


@pytest.mark.parametrize("name,kind", [("label_smooth", "lsr"), ("large_margin", "lmargin")])
def test_golden(golden_dir, name, kind):
    import pytorch_loss as P
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    for i in range(int(z["n_cases"])):
        hp, ign = z[f"c{i}_hyper"]
        red = str(z[f"c{i}_reduction"])
        logits, labels = torch.from_numpy(z[f"c{i}_logits"]), torch.from_numpy(z[f"c{i}_labels"])
        crit = (P.LabelSmoothSoftmaxCEV3(float(hp), red, int(ign)) if kind == "lsr"
                else P.LargeMarginSoftmaxV3(float(hp), red, int(ign)))
        loss, grad = run_module(crit, logits.cuda(), labels.cuda())
        assert_loss_close(loss, torch.from_numpy(z[f"c{i}_loss_v2"]), atol=2e-6, what=f"{name} c{i} loss")
        assert_grad_close(grad, torch.from_numpy(z[f"c{i}_grad_v2"]), what=f"{name} c{i} grad")


@pytest.mark.parametrize("kind", ["lsr", "lmargin"])
def test_public_functions_per_pixel_upstream_gradient(kind):
    """The reference-facing autograd Functions: per-pixel loss out, per-pixel grad_output in."""
    import pytorch_loss as P
    from oracle import losses as O
    g = torch.Generator().manual_seed(8)
    logits = torch.randn(2, 11, 10, 12, generator=g)
    labels = labels_with_ignores(g, (2, 10, 12), 11, 255, 0.2)
    up = torch.randn(2, 10, 12, generator=g)
    x = logits.cuda().requires_grad_(True)
    if kind == "lsr":
        want_loss, want_grad = O.label_smooth_ce(logits, labels, 0.1, 255, "none")
        loss = P.LSRCrossEntropyFunctionV3.apply(x, labels.cuda(), 0.1, 255)
    else:
        want_loss, want_grad = O.large_margin_softmax(logits, labels, 0.3, 255, "none")
        loss = P.LargeMarginSoftmaxFuncV3.apply(x, labels.cuda(), 0.3, 255)
    loss.backward(up.cuda())
    assert_loss_close(loss, want_loss, atol=2e-6)
    assert_grad_close(x.grad, want_grad * up.unsqueeze(1))


def test_large_margin_fb_function_returns_count():
    import pytorch_loss as P
    from oracle import losses as O
    g = torch.Generator().manual_seed(9)
    logits = torch.randn(2, 9, 6, 8, generator=g)
    labels = labels_with_ignores(g, (2, 6, 8), 9, 255, 0.25)
    x = logits.cuda().requires_grad_(True)
    losses, cnt = P.LargeMarginSoftmaxFuncV3FB.apply(x, labels.cuda(), 0.3, 255)
    assert int(cnt.item()) == int((labels != 255).sum())
    (losses.sum() / cnt).backward()
    want_loss, want_grad = O.large_margin_softmax(logits, labels, 0.3, 255, "mean")
    assert_loss_close((losses.sum() / cnt).reshape(()), want_loss)
    assert_grad_close(x.grad, want_grad)


@pytest.mark.parametrize("kind", ["lsr", "lmargin"])
@pytest.mark.parametrize("shape", [(2, 19, (16, 24)), (3, 150, (8, 8)), (4, 4096, ()), (2, 21, (5, 7)),
                                   (2, 150, (24, 28)), (1, 45, (32, 40))],
                         ids=["tile19", "tile150", "rows4096", "unaligned", "chunks150", "chunks45"])
def test_fp16_io(kind, shape):
    n, c, sp = shape
    g = torch.Generator().manual_seed(10)
    logits = torch.randn((n, c) + sp, generator=g).half()
    labels = labels_with_ignores(g, (n,) + sp, c, 255, 0.1)
    crit, oracle = _crit(kind, "mean", 255)
    want_loss, want_grad = oracle(logits.float(), labels)
    loss, grad = run_module(crit, logits.cuda(), labels.cuda())
    assert grad.dtype == torch.float16
    assert_loss_close(loss, want_loss, rtol=TOL_F16)
    assert_grad_close(grad, want_grad, atol=TOL_F16 * float(want_grad.abs().max()), rtol=TOL_F16)


def test_autocast_casts_to_fp32():
    import pytorch_loss as P
    from oracle import losses as O
    g = torch.Generator().manual_seed(11)
    logits = torch.randn(2, 19, 8, 8, generator=g)
    labels = torch.randint(0, 19, (2, 8, 8), generator=g)
    x = logits.cuda().half().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.float16):
        loss = P.LabelSmoothSoftmaxCEV3()(x, labels.cuda())
    loss.backward()
    want_loss, want_grad = O.label_smooth_ce(logits.half().float(), labels, 0.1, -100, "mean")
    assert loss.dtype == torch.float32
    assert_loss_close(loss, want_loss)
    assert_grad_close(x.grad.float(), want_grad, atol=1e-5, rtol=2e-3)


def test_non_contiguous_and_empty_inputs():
    import pytorch_loss as P
    from oracle import losses as O
    g = torch.Generator().manual_seed(12)
    nhwc = torch.randn(2, 8, 10, 19, generator=g)
    logits = nhwc.permute(0, 3, 1, 2)                      # channels-last view
    labels = torch.randint(0, 19, (2, 8, 10), generator=g)
    want_loss, want_grad = O.label_smooth_ce(logits, labels, 0.1, -100, "mean")
    loss, grad = run_module(P.LabelSmoothSoftmaxCEV3(), nhwc.cuda().permute(0, 3, 1, 2), labels.cuda())
    assert_loss_close(loss, want_loss)
    assert_grad_close(grad, want_grad)
    empty = P.LabelSmoothSoftmaxCEV3(reduction="none")(torch.zeros(0, 5, 4, 4).cuda(),
                                                       torch.zeros(0, 4, 4, dtype=torch.int64).cuda())
    assert empty.shape == (0, 4, 4)


def test_bad_arguments_raise():
    import pytorch_loss as P
    crit = P.LabelSmoothSoftmaxCEV3()
    with pytest.raises(RuntimeError):
        crit(torch.randn(2, 5, 4, 4), torch.zeros(2, 4, 4, dtype=torch.int64))          # CPU tensors
    with pytest.raises(RuntimeError):
        crit(torch.randn(2, 5, 4, 4).cuda(), torch.zeros(2, 4, 5, dtype=torch.int64).cuda())  # shape
    with pytest.raises(RuntimeError):
        crit(torch.randn(2, 5, 4, 4).cuda(), torch.zeros(2, 4, 4, dtype=torch.int32).cuda())  # dtype
    with pytest.raises(RuntimeError):
        crit(torch.randint(0, 5, (2, 5, 4, 4)).cuda(), torch.zeros(2, 4, 4, dtype=torch.int64).cuda())   # integer logits


def test_deterministic_and_status_clean():
    import pytorch_loss as P
    from pytorch_loss import _cabi
    g = torch.Generator().manual_seed(13)
    logits = torch.randn(4, 19, 128, 128, generator=g).cuda()
    labels = labels_with_ignores(g, (4, 128, 128), 19, 255, 0.05).cuda()
    for crit in (P.LabelSmoothSoftmaxCEV3(ignore_index=255), P.LargeMarginSoftmaxV3()):
        first, g1 = run_module(crit, logits, labels)
        for _ in range(3):
            again, g2 = run_module(crit, logits, labels)
            assert again.item() == first.item()
            assert torch.equal(g1, g2)
    _cabi.read_status(logits.device)


@pytest.mark.parametrize("kind", ["lsr", "lmargin"])
def test_statistics_backward_equals_recomputing_backward(kind):
    """Many classes: the backward that uses the forward's saved statistics against the one that
    recomputes the softmax, for every upstream-gradient mode (none, device scalar, per pixel)."""
    from pytorch_loss import _cabi
    lib = _cabi.load_library()
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(21)
    n, c, h, w = 2, 70, 24, 28                      # 672 pixels per image, 5 chunks (last of 6 channels)
    x = (torch.randn(n, c, h, w, generator=g) * 2).to(dev)
    y = labels_with_ignores(g, (n, h, w), c, 255, 0.1).to(dev)
    m = h * w
    hp = 0.1 if kind == "lsr" else 0.3
    P, st = _cabi.ptr, _cabi.stream_ptr(dev)
    assert lib.b200_softmax_stats_path(P(x), P(y), None, n, c, m, _cabi.F32) == 1
    stats = torch.empty(n * m, 4, device=dev)
    losses = torch.empty(n, h, w, device=dev)
    fwd = getattr(lib, "b200_%s_forward_ex" % kind)
    _cabi.check(fwd(P(x), P(y), P(losses), None, None, 0, P(stats), n, c, m, _cabi.F32, 255, hp, st))
    ref_losses = torch.empty_like(losses)
    _cabi.check(getattr(lib, "b200_%s_forward" % kind)(P(x), P(y), P(ref_losses), None, None, 0, n, c, m,
                                                       _cabi.F32, 255, hp, st))
    assert torch.allclose(losses, ref_losses, atol=1e-6, rtol=1e-6)
    scalar = torch.tensor([0.37], device=dev)
    per_px = torch.randn(n, h, w, generator=g).to(dev)
    denom = torch.tensor([3.0], dtype=torch.float64, device=dev)
    for mode, gout, dn in ((0, None, None), (1, scalar, denom), (2, per_px, None)):
        got, want = torch.empty_like(x), torch.empty_like(x)
        _cabi.check(getattr(lib, "b200_%s_backward_ex" % kind)(
            P(x), P(y), P(stats), P(gout), mode, P(dn), P(got), n, c, m, _cabi.F32, 255, hp, st))
        _cabi.check(getattr(lib, "b200_%s_backward" % kind)(
            P(x), P(y), P(gout), mode, P(dn), P(want), n, c, m, _cabi.F32, 255, hp, st))
        assert torch.allclose(got, want, atol=2e-6, rtol=1e-5), (kind, mode, float((got - want).abs().max()))
    _cabi.read_status(dev)


@pytest.mark.parametrize("kind", ["lsr", "lmargin"])
@pytest.mark.parametrize("shape", [(2, 19, (32, 36)), (3, 7, (16, 20)), (1, 150, (40, 52)), (2, 64, (8, 12)),
                                   (5, 4096, ()), (700, 2048, ()), (3, 1000, ())],
                         ids=lambda s: "x".join(map(str, (s[0], s[1]) + s[2])))
@pytest.mark.parametrize("reduction", ["mean", "sum"])
def test_fused_step(kind, shape, reduction, monkeypatch):
    """The training step that reads the logits once (loss sum + final gradient in the backward tile
    kernel): upstream gradient other than 1, a second backward through the same graph, a forward
    without gradient, and the same numbers as the separate forward and backward kernels."""
    import pytorch_loss  # noqa: F401
    from pytorch_loss import _cabi
    n, c, sp = shape
    g = torch.Generator().manual_seed(77 + c)
    logits = torch.randn((n, c) + sp, generator=g) * 1.5
    labels = labels_with_ignores(g, (n,) + sp, c, 255, 0.2)
    crit, oracle = _crit(kind, reduction, 255)
    want_loss, want_grad = oracle(logits, labels)
    lib = _cabi.load_library()
    xg, yg = logits.cuda(), labels.cuda()
    assert lib.b200_softmax_fused_step_path(_cabi.ptr(xg), _cabi.ptr(yg), _cabi.ptr(torch.empty_like(xg)),
                                            n, c, labels[0].numel(), 0) == 1

    x = xg.clone().requires_grad_(True)
    loss = crit(x, yg)
    (loss * 0.5).backward(retain_graph=True)
    assert_loss_close(loss, want_loss)
    assert_grad_close(x.grad, want_grad * 0.5)
    x.grad = None
    loss.backward()
    assert_grad_close(x.grad, want_grad)
    with torch.no_grad():
        assert_loss_close(crit(xg, yg), want_loss)

    fused_loss, fused_grad = run_module(crit, xg, yg)
    monkeypatch.setenv("B200_SOFTMAX_FUSED", "0")
    plain_loss, plain_grad = run_module(crit, xg, yg)
    assert_loss_close(fused_loss, plain_loss.cpu(), rtol=2e-6)
    assert_grad_close(fused_grad, plain_grad.cpu())


@pytest.mark.parametrize("kind", ["lsr", "lmargin"])
def test_empty_batch_reduced(kind):
    """No pixels at all: 'sum' is 0, 'mean' is 0/0 = NaN as in the reference, the gradient is empty."""
    for reduction in ("sum", "mean"):
        crit, _ = _crit(kind, reduction, 255)
        x = torch.randn(0, 5, 4, 4).cuda().requires_grad_(True)
        loss = crit(x, torch.zeros(0, 4, 4, dtype=torch.int64).cuda())
        loss.backward()
        assert x.grad.shape == x.shape
        assert torch.isnan(loss.detach()) if reduction == "mean" else float(loss.detach()) == 0.0
