"""Taylor softmax / log-Taylor softmax / Taylor cross entropy (CUDA, through the C ABI) against
the CPU oracle and the golden file made from the reference's V1 functions."""
import os

import numpy as np
import pytest
import torch

from helpers import labels_with_ignores

pytestmark = pytest.mark.gpu

# (shape, dim): 16-byte path, scalar path (odd inner size), one warp per row (dim last), dim 0
CASES = [((2, 19, 16, 24), 1), ((3, 7, 5, 7), 1), ((6, 33), 1), ((64, 1000), -1), ((5, 4, 6), 0),
         ((2, 3, 4, 40), 2), ((2, 150, 12, 12), 1), ((1, 2, 1, 1), 1),
         # 33..320 channels: channel slices over the threads of a block (4 slices to 160, 8 beyond), ragged ends
         ((1, 33, 5, 9), 1), ((2, 33, 6, 12), 1), ((3, 40, 70), 1), ((2, 161, 4, 10), 1), ((1, 161, 10, 10), 1),
         ((1, 320, 8, 8), 1), ((1, 321, 8, 8), 1),
         # rows of 64..1024 floats stay in a warp's registers (2 or 8 vectors per lane); 1028 does not
         ((40, 64), 1), ((33, 256), -1), ((9, 260), 1), ((17, 1024), 1), ((5, 1028), 1)]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "x".join(map(str, c[0])) + "_d%d" % c[1])
@pytest.mark.parametrize("order", [2, 4, 8])
@pytest.mark.parametrize("use_log", [False, True])
def test_matches_oracle(case, order, use_log):
    import pytorch_loss as P
    from oracle import taylor as OT
    shape, dim = case
    g = torch.Generator().manual_seed(sum(shape) + order)
    x = torch.randn(shape, generator=g) * 1.5
    up = torch.randn(shape, generator=g)
    want_out, want_grad = OT.taylor_softmax(x, dim, order, use_log, upstream=up, dtype=torch.float64)
    xc = x.cuda().requires_grad_(True)
    out = P.taylor_softmax_v3(xc, dim, order, use_log)
    out.backward(up.cuda())
    assert out.shape == x.shape
    assert torch.allclose(out.detach().cpu().double(), want_out, atol=1e-6, rtol=1e-5)
    assert torch.allclose(xc.grad.cpu().double(), want_grad, atol=1e-5, rtol=1e-4)


def test_golden_and_modules(golden_dir):
    import pytorch_loss as P
    import taylor_softmax_cpp
    z = np.load(os.path.join(golden_dir, "taylor.npz"))
    for i in range(int(z["n_cases"])):
        dim, order, use_log = (int(v) for v in z[f"c{i}_hyper"])
        x, up = torch.from_numpy(z[f"c{i}_x"]).cuda(), torch.from_numpy(z[f"c{i}_up"]).cuda()
        out = taylor_softmax_cpp.taylor_softmax_forward(x, dim, order, bool(use_log))
        grad = taylor_softmax_cpp.taylor_softmax_backward(up, x, dim, order, bool(use_log))
        assert torch.allclose(out.cpu(), torch.from_numpy(z[f"c{i}_out"]), atol=1e-6, rtol=1e-5), i
        assert torch.allclose(grad.cpu(), torch.from_numpy(z[f"c{i}_grad"]), atol=1e-5, rtol=1e-4), i
    for i in range(int(z["n_ce_cases"])):
        order, ign = (int(v) for v in z[f"ce{i}_hyper"])
        logits = torch.from_numpy(z[f"ce{i}_logits"]).cuda().requires_grad_(True)
        labels = torch.from_numpy(z[f"ce{i}_labels"]).cuda()
        crit = P.TaylorCrossEntropyLossV3(n=order, ignore_index=ign, reduction=str(z[f"ce{i}_reduction"]))
        loss = crit(logits, labels)
        loss.backward()
        assert torch.allclose(loss.detach().cpu(), torch.from_numpy(z[f"ce{i}_loss"]), atol=1e-6, rtol=1e-5), i
        assert torch.allclose(logits.grad.cpu(), torch.from_numpy(z[f"ce{i}_grad"]), atol=1e-6, rtol=1e-5), i
    mod = P.TaylorSoftmaxV3(dim=1, n=4)
    y = mod(torch.randn(2, 5, 3, 3).cuda())
    assert torch.allclose(y.sum(dim=1), torch.ones(2, 3, 3).cuda(), atol=1e-6)
    y = P.LogTaylorSoftmaxV3(dim=1, n=2)(torch.randn(2, 5, 3, 3).cuda())
    assert torch.allclose(y.exp().sum(dim=1), torch.ones(2, 3, 3).cuda(), atol=1e-5)


def test_fp16_autocast_noncontiguous_empty_and_errors():
    import pytorch_loss as P
    from oracle import taylor as OT
    g = torch.Generator().manual_seed(4)
    x = torch.randn(2, 9, 6, 8, generator=g)
    want, _ = OT.taylor_softmax(x.half().float(), 1, 4, False)
    got = P.taylor_softmax_v3(x.half().cuda(), 1, 4, False)
    assert got.dtype == torch.float16
    assert torch.allclose(got.float().cpu(), want, atol=2e-3, rtol=2e-3)
    with torch.autocast("cuda", dtype=torch.float16):
        got = P.taylor_softmax_v3(x.half().cuda(), 1, 4, True)
    assert got.dtype == torch.float32                      # inputs are cast to fp32 under autocast
    xt = x.cuda().transpose(1, 3)                          # non-contiguous input
    want, _ = OT.taylor_softmax(x.transpose(1, 3), 1, 2, True)
    assert torch.allclose(P.taylor_softmax_v3(xt, 1, 2, True).cpu(), want, atol=1e-6, rtol=1e-5)
    assert P.taylor_softmax_v3(torch.empty(0, 5, 3).cuda(), 1, 2).shape == (0, 5, 3)
    with pytest.raises(RuntimeError):
        P.taylor_softmax_v3(x, 1, 4)                       # CPU tensor: gpu only
    with pytest.raises(RuntimeError):
        P.TaylorSoftmaxFunc.apply(x.cuda(), 1, 18, False)  # order above the supported 16
