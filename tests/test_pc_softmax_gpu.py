"""PCSoftmaxCrossEntropyV2 (CUDA, through the C ABI) against the CPU oracle and the golden file
recorded from the reference's V1 class."""
import os

import numpy as np
import pytest
import torch

from helpers import assert_grad_close, assert_loss_close, labels_with_ignores, run_module, TOL_F16

pytestmark = pytest.mark.gpu

SHAPES = [(2, 5, (6, 7)), (3, 19, (16, 20)), (2, 19, (33, 35)), (1, 150, (12, 16)), (7, 10, ()), (3, 1000, ()),
          (2, 4, (5,)), (4, 19, (128, 128))]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, (s[0], s[1]) + s[2])))
@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
def test_matches_oracle(shape, reduction):
    import pytorch_loss as P
    from oracle import pc_softmax as PC
    n, c, sp = shape
    g = torch.Generator().manual_seed(700 + c + len(sp))
    logits = torch.randn((n, c) + sp, generator=g) * 2.0
    labels = labels_with_ignores(g, (n,) + sp, c, 255, 0.15)
    prop = torch.rand(c, generator=g) + 0.05
    prop = (prop / prop.sum()).tolist()
    want_loss, want_grad = PC.pc_softmax_ce(logits, labels, prop, 255, reduction)
    loss, grad = run_module(P.PCSoftmaxCrossEntropyV2(prop, reduction, 255), logits.cuda(), labels.cuda())
    assert_loss_close(loss, want_loss, atol=2e-6 if reduction == "none" else 1e-7)
    assert_grad_close(grad, want_grad)
    ign = labels == 255
    assert bool((grad.cpu().transpose(0, 1)[:, ign] == 0).all())
    if reduction == "none":
        assert bool((loss.cpu()[ign] == 0).all())


def test_golden(golden_dir):
    import pytorch_loss as P
    z = np.load(os.path.join(golden_dir, "pc_softmax.npz"))
    for i in range(int(z["n_cases"])):
        x, y = torch.from_numpy(z[f"c{i}_logits"]), torch.from_numpy(z[f"c{i}_labels"])
        red, ign = str(z[f"c{i}_reduction"]), int(z[f"c{i}_hyper"][0])
        crit = P.PCSoftmaxCrossEntropyV2(z[f"c{i}_proportion"].tolist(), red, ign)
        loss, grad = run_module(crit, x.cuda(), y.cuda())
        assert_loss_close(loss, torch.from_numpy(z[f"c{i}_loss_v1"]), atol=2e-6, what=f"c{i} loss")
        assert_grad_close(grad, torch.from_numpy(z[f"c{i}_grad_v1"]), what=f"c{i} grad")


def test_fp16_per_pixel_upstream_gradient_and_errors():
    import pytorch_loss as P
    from oracle import pc_softmax as PC
    g = torch.Generator().manual_seed(710)
    logits = (torch.randn(2, 6, 9, 8, generator=g) * 2).half()
    labels = labels_with_ignores(g, (2, 9, 8), 6, 255, 0.1)
    prop = [0.3, 0.1, 0.2, 0.15, 0.05, 0.2]
    want_loss, want_grad = PC.pc_softmax_ce(logits.float(), labels, prop, 255, 'none')
    up = torch.randn(2, 9, 8, generator=g)
    x = logits.cuda().requires_grad_(True)
    loss = P.PCSoftmaxCrossEntropyFunction.apply(x, labels.cuda(), prop, 'none', 255)
    loss.backward(up.cuda().half())
    assert_loss_close(loss.float(), want_loss, rtol=TOL_F16, atol=TOL_F16)
    assert_grad_close(x.grad.float(), want_grad * up.unsqueeze(1), atol=4 * TOL_F16, rtol=4 * TOL_F16)
    with pytest.raises(RuntimeError):
        P.PCSoftmaxCrossEntropyV2([0.5, 0.5])(torch.randn(2, 3, 4, 4).cuda(), torch.zeros(2, 4, 4, dtype=torch.int64).cuda())
    with pytest.raises(RuntimeError):
        P.PCSoftmaxCrossEntropyV2([0.5, 0.5])(torch.randn(2, 2, 4, 4), torch.zeros(2, 4, 4, dtype=torch.int64))


@pytest.mark.parametrize("c", [8, 20, 32, 33])
def test_scalar_upstream_gradient_and_second_backward(c):
    """'mean' leaves the kernel divided by the valid count; backward rescales in place once, and a
    second trip through the graph recomputes instead of scaling twice."""
    import pytorch_loss as P
    from oracle import pc_softmax as PC
    g = torch.Generator().manual_seed(720 + c)
    logits = torch.randn(2, c, 10, 12, generator=g) * 2.0
    labels = labels_with_ignores(g, (2, 10, 12), c, 255, 0.2)
    prop = torch.rand(c, generator=g) + 0.05
    prop = (prop / prop.sum()).tolist()
    for reduction in ("mean", "sum"):
        want_loss, want_grad = PC.pc_softmax_ce(logits, labels, prop, 255, reduction)
        x = logits.cuda().requires_grad_(True)
        loss = P.PCSoftmaxCrossEntropyV2(prop, reduction, 255)(x, labels.cuda())
        (loss * 3.0).backward(retain_graph=True)
        assert_loss_close(loss.detach(), want_loss, atol=1e-7)
        assert_grad_close(x.grad, want_grad * 3.0)
        x.grad = None
        (loss * -0.5).backward()
        assert_grad_close(x.grad, want_grad * -0.5)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(2, 19, (32, 40)), (1, 150, (16, 32)), (2, 256, (8, 16)), (2, 257, (8, 16))],
                         ids=lambda s: "x".join(map(str, (s[0], s[1]) + s[2])))
def test_half_logits_reduced_step(shape, dtype):
    """'mean' / 'sum' with a gradient: the fused step on the tile pipeline (up to 256 classes; 257
    takes the per-pixel kernel), half storage, fp32 arithmetic."""
    import pytorch_loss as P
    from oracle import pc_softmax as PC
    n, c, sp = shape
    g = torch.Generator().manual_seed(730 + c)
    logits = (torch.randn((n, c) + sp, generator=g) * 2.0).to(dtype)
    labels = labels_with_ignores(g, (n,) + sp, c, 255, 0.15)
    prop = torch.rand(c, generator=g) + 0.05
    prop = (prop / prop.sum()).tolist()
    tol = TOL_F16 if dtype == torch.float16 else 2.0 ** -7
    for reduction in ("mean", "sum"):
        want_loss, want_grad = PC.pc_softmax_ce(logits.float(), labels, prop, 255, reduction)
        loss, grad = run_module(P.PCSoftmaxCrossEntropyV2(prop, reduction, 255), logits.cuda(), labels.cuda())
        assert grad.dtype == dtype
        assert_loss_close(loss.float(), want_loss, rtol=tol, atol=tol)
        assert_grad_close(grad.float(), want_grad, atol=tol, rtol=tol)
        ign = labels == 255
        assert bool((grad.cpu().transpose(0, 1)[:, ign] == 0).all())


def test_zero_proportion_class():
    """A class with proportion 0 drops out of the sum (its exponential is weighted by 0)."""
    import pytorch_loss as P
    from oracle import pc_softmax as PC
    g = torch.Generator().manual_seed(740)
    logits = torch.randn(2, 6, 8, 12, generator=g) * 2.0
    labels = torch.randint(1, 6, (2, 8, 12), generator=g)          # class 0 never is the label
    prop = [0.0, 0.3, 0.2, 0.2, 0.1, 0.2]
    for reduction in ("mean", "none"):
        want_loss, want_grad = PC.pc_softmax_ce(logits, labels, prop, 255, reduction)
        loss, grad = run_module(P.PCSoftmaxCrossEntropyV2(prop, reduction, 255), logits.cuda(), labels.cuda())
        assert_loss_close(loss, want_loss, atol=2e-6)
        assert_grad_close(grad, want_grad)
        assert bool((grad[:, 0] == 0).all())
