"""More than 2^31 logit elements in one call (64-bit indexing).

The reference's label-smooth, large-margin and focal kernels index with int64 and take any size
(csrc/lsr_kernel.cu:66-185, csrc/large_margin_kernel.cu:354-599, csrc/focal_kernel.cu:26-163; only
Lovasz asserts numel < 2^31, csrc/lovasz_softmax.cu:664).  A CPU oracle of 2^31 elements is out of
reach of a test, so these cases use what does not depend on the size:

* additivity: the 'sum' loss of the whole tensor equals the sum of the losses of its images (each
  below 2^31 elements), computed by separate calls;
* spot checks against the oracle on windows of pixels at the very start, across the 2^31-element
  offset and at the very end of the tensor, loss values and gradients;
* gradients at ignored pixels are exactly 0 in those windows.

Half-precision logits keep the tensors at 4.3 GB each.
"""
import pytest
import torch

from helpers import TOL_F16

pytestmark = pytest.mark.gpu

N, C, M = 4, 16, (1 << 25) + (1 << 10)            # 4 x 16 x 33 555 456 = 2 147 549 184 elements
WINDOW = 1024


def _need_memory(gib):
    free, _ = torch.cuda.mem_get_info()
    if free < gib * (1 << 30):
        pytest.skip("needs %d GiB of free device memory" % gib)


def _windows():
    """(image, first pixel) of the windows checked against the oracle: the tensor's first and last
    pixels and the pixels whose channel-0 element offset straddles 2^31."""
    per_image = C * M
    n_cross = (1 << 31) // per_image                       # image that holds element 2^31 ...
    px = ((1 << 31) - n_cross * per_image) % M             # ... at this pixel of one of its channels
    p_cross = max(0, min(px - WINDOW // 2, M - WINDOW))
    return [(0, 0), (n_cross, 0), (n_cross, p_cross), (N - 1, M - WINDOW)]


def _softmax_inputs():
    g = torch.Generator(device="cuda").manual_seed(31)
    logits = torch.empty((N, C, M), dtype=torch.float16, device="cuda")
    for n in range(N):                                      # (fp32 randn of one image at a time: 2 GB)
        logits[n] = (torch.randn((C, M), generator=g, device="cuda") * 2.0).half()
    labels = torch.randint(0, C, (N, M), generator=g, device="cuda")
    labels[torch.rand((N, M), generator=g, device="cuda") < 0.1] = 255
    return logits, labels


@pytest.mark.parametrize("kind", ["lsr", "lmargin"])
def test_softmax_losses_beyond_2g_elements(kind):
    import pytorch_loss as P
    from oracle import losses as O
    _need_memory(24)
    assert N * C * M > (1 << 31)
    logits, labels = _softmax_inputs()
    if kind == "lsr":
        crit = P.LabelSmoothSoftmaxCEV3(0.1, 'sum', 255)
        oracle = lambda x, y: O.label_smooth_ce(x, y, 0.1, 255, 'sum')
    else:
        crit = P.LargeMarginSoftmaxV3(0.3, 'sum', 255)
        oracle = lambda x, y: O.large_margin_softmax(x, y, 0.3, 255, 'sum')
    x = logits.requires_grad_(True)
    loss = crit(x, labels)
    loss.backward()
    grad = x.grad
    assert grad.shape == x.shape and grad.dtype == torch.float16
    # additivity over the images
    parts = 0.0
    with torch.no_grad():
        for n in range(N):
            parts += float(crit(logits[n:n + 1].detach(), labels[n:n + 1]))
    assert abs(float(loss.detach()) - parts) <= 1e-5 * abs(parts)
    # windows against the oracle (float32 arithmetic on the half inputs)
    total = 0.0
    for n, p0 in _windows():
        xw = logits[n:n + 1, :, p0:p0 + WINDOW].detach().float().cpu()
        yw = labels[n:n + 1, p0:p0 + WINDOW].cpu()
        _, want = oracle(xw, yw)
        got = grad[n:n + 1, :, p0:p0 + WINDOW].float().cpu()
        err = (got - want).abs() - (TOL_F16 + TOL_F16 * want.abs())
        assert bool((err <= 0).all()), "gradient window (%d, %d): max violation %g" % (n, p0, float(err.max()))
        ign = yw[0] == 255
        assert bool((got[0][:, ign] == 0).all())
        total += float(ign.sum())
    assert total > 0                                        # the windows did hold ignored pixels


def test_focal_beyond_2g_elements():
    import pytorch_loss as P
    from oracle import losses as O
    _need_memory(24)
    e_half = (1 << 30) + (1 << 12)
    g = torch.Generator(device="cuda").manual_seed(32)
    logits = torch.empty((2, e_half), dtype=torch.float16, device="cuda")
    labels = torch.empty((2, e_half), dtype=torch.float16, device="cuda")
    for n in range(2):
        logits[n] = (torch.randn(e_half, generator=g, device="cuda") * 1.7).half()
        labels[n] = (torch.rand(e_half, generator=g, device="cuda") < 0.1).half()
    assert logits.numel() > (1 << 31)
    crit = P.FocalLossV3(0.25, 2, 'sum')
    x = logits.requires_grad_(True)
    loss = crit(x, labels)
    loss.backward()
    parts = 0.0
    with torch.no_grad():
        for n in range(2):
            parts += float(crit(logits[n:n + 1].detach(), labels[n:n + 1]))
    assert abs(float(loss.detach()) - parts) <= 1e-5 * abs(parts)
    for n, p0 in ((0, 0), (0, e_half - WINDOW), (1, 0), (1, e_half - WINDOW)):   # (1, 0) starts past element 2^30; the last window ends the tensor
        xw = logits[n:n + 1, p0:p0 + WINDOW].detach().float().cpu()
        yw = labels[n:n + 1, p0:p0 + WINDOW].float().cpu()
        _, want = O.focal_loss(xw, yw, 0.25, 2.0, 'sum')
        got = x.grad[n:n + 1, p0:p0 + WINDOW].float().cpu()
        err = (got - want).abs() - (TOL_F16 + TOL_F16 * want.abs())
        assert bool((err <= 0).all()), "focal gradient window (%d, %d): max violation %g" % (n, p0, float(err.max()))
    # 'mean' divides by the element count, which does not fit 32 bits
    x.grad = None
    crit_mean = P.FocalLossV3(0.25, 2, 'mean')
    lm = crit_mean(x, labels)
    lm.backward()
    assert abs(float(lm.detach()) - parts / logits.numel()) <= 1e-5 * abs(parts / logits.numel())


def test_taylor_beyond_2g_elements():
    import pytorch_loss as P
    from oracle import taylor as OT
    _need_memory(24)
    g = torch.Generator(device="cuda").manual_seed(33)
    x = torch.empty((N, C, M), dtype=torch.float16, device="cuda")
    for n in range(N):
        x[n] = torch.randn((C, M), generator=g, device="cuda").half()
    out = P.TaylorSoftmaxV3(dim=1, n=2)(x)
    assert out.shape == x.shape
    for n, p0 in _windows():
        want, _ = OT.taylor_softmax(x[n:n + 1, :, p0:p0 + WINDOW].float().cpu(), 1, 2, False)
        got = out[n:n + 1, :, p0:p0 + WINDOW].float().cpu()
        assert bool(((got - want).abs() <= TOL_F16).all()), "taylor window (%d, %d)" % (n, p0)


def test_label_smooth_rows_beyond_2g_elements():
    """[rows, 32768] half logits, one row per pixel (the rows kernels): 65 552 rows pass 2^31 elements."""
    import pytorch_loss as P
    from oracle import losses as O
    _need_memory(24)
    rows, cols = (1 << 16) + 16, 1 << 15
    g = torch.Generator(device="cuda").manual_seed(34)
    logits = torch.empty((rows, cols), dtype=torch.float16, device="cuda")
    step = 1 << 13
    for r in range(0, rows, step):
        logits[r:r + step] = (torch.randn((min(step, rows - r), cols), generator=g, device="cuda") * 2.0).half()
    labels = torch.randint(0, cols, (rows,), generator=g, device="cuda")
    labels[torch.rand((rows,), generator=g, device="cuda") < 0.1] = -100
    assert logits.numel() > (1 << 31)
    crit = P.LabelSmoothSoftmaxCEV3(0.1, 'sum', -100)
    x = logits.requires_grad_(True)
    loss = crit(x, labels)
    loss.backward()
    half = rows // 2
    with torch.no_grad():
        parts = float(crit(logits[:half].detach(), labels[:half])) + float(crit(logits[half:].detach(), labels[half:]))
    assert abs(float(loss.detach()) - parts) <= 1e-5 * abs(parts)
    for r0 in (0, (1 << 16) - 8, rows - 16):                 # first rows, the rows around element 2^31, last rows
        xw = logits[r0:r0 + 16].detach().float().cpu()
        yw = labels[r0:r0 + 16].cpu()
        _, want = O.label_smooth_ce(xw, yw, 0.1, -100, 'sum')
        got = x.grad[r0:r0 + 16].float().cpu()
        err = (got - want).abs() - (TOL_F16 + TOL_F16 * want.abs())
        assert bool((err <= 0).all()), "rows window %d: max violation %g" % (r0, float(err.max()))
        assert bool((got[yw == -100] == 0).all())
