"""FocalLossV3 (CUDA, through the C ABI) against the CPU oracle and the golden files."""
import os

import numpy as np
import pytest
import torch

from helpers import assert_grad_close, assert_loss_close, run_module, TOL_F16

pytestmark = pytest.mark.gpu


def _mods():
    import pytorch_loss
    from oracle import losses as O
    return pytorch_loss, O


@pytest.mark.parametrize("shape", [(2, 3, 7, 5), (16, 1, 64, 64), (1, 1, 1), (3, 5, 1023), (2, 2, 4096, 33)])
@pytest.mark.parametrize("reduction", ["mean", "sum", "none"])
@pytest.mark.parametrize("gamma", [2, 1.5])
def test_focal_matches_oracle(shape, reduction, gamma):
    P, O = _mods()
    g = torch.Generator().manual_seed(11)
    logits = torch.randn(shape, generator=g) * 3 ** 0.5
    labels = (torch.rand(shape, generator=g) < 0.1).float()
    want_loss, want_grad = O.focal_loss(logits, labels, 0.25, gamma, reduction)
    loss, grad = run_module(P.FocalLossV3(0.25, gamma, reduction), logits.cuda(), labels.cuda())
    assert_loss_close(loss, want_loss, atol=1e-6 if reduction == "none" else 1e-7)
    assert_grad_close(grad, want_grad)


def test_focal_soft_labels_and_extremes():
    P, O = _mods()
    g = torch.Generator().manual_seed(12)
    logits = torch.randn(4, 3, 50, generator=g) * 10
    logits[0, 0, :6] = torch.tensor([-100., 100., -30., 30., 0., -0.])
    labels = torch.sigmoid(torch.randn(4, 3, 50, generator=g))
    want_loss, want_grad = O.focal_loss(logits, labels, 0.4, 2.0, "sum")
    loss, grad = run_module(P.FocalLossV3(0.4, 2.0, "sum"), logits.cuda(), labels.cuda())
    assert_loss_close(loss, want_loss)
    assert_grad_close(grad, want_grad)


def test_focal_golden(golden_dir):
    P, _ = _mods()
    z = np.load(os.path.join(golden_dir, "focal.npz"))
    for i in range(int(z["n_cases"])):
        al, ga = z[f"c{i}_hyper"]
        red = str(z[f"c{i}_reduction"])
        logits, labels = torch.from_numpy(z[f"c{i}_logits"]), torch.from_numpy(z[f"c{i}_labels"])
        loss, grad = run_module(P.FocalLossV3(float(al), float(ga), red), logits.cuda(), labels.cuda())
        assert_loss_close(loss, torch.from_numpy(z[f"c{i}_loss_v2"]), atol=1e-6, what=f"golden c{i} loss")
        assert_grad_close(grad, torch.from_numpy(z[f"c{i}_grad_v2"]), what=f"golden c{i} grad")


def test_focal_functions_match_reference_contract():
    """The two public autograd Functions: per-element loss, gradient scaled by grad_output."""
    P, O = _mods()
    g = torch.Generator().manual_seed(13)
    logits = torch.randn(3, 2, 17, generator=g)
    labels = (torch.rand(3, 2, 17, generator=g) < 0.3).float()
    up = torch.randn(3, 2, 17, generator=g)
    want_loss, want_grad = O.focal_loss(logits, labels, 0.25, 2.0, "none")
    for fn in (P.FocalSigmoidLossFuncV3, P.FocalSigmoidLossFuncV3FB):
        x = logits.cuda().requires_grad_(True)
        loss = fn.apply(x, labels.cuda(), 0.25, 2.0)
        loss.backward(up.cuda())
        assert_loss_close(loss, want_loss, atol=1e-6)
        assert_grad_close(x.grad, want_grad * up)


def test_focal_fp16_io():
    P, O = _mods()
    g = torch.Generator().manual_seed(14)
    logits = (torch.randn(2, 4, 31, 8, generator=g) * 2).half()
    labels = (torch.rand(2, 4, 31, 8, generator=g) < 0.2).half()
    want_loss, want_grad = O.focal_loss(logits.float(), labels.float(), 0.25, 2.0, "mean")
    loss, grad = run_module(P.FocalLossV3(), logits.cuda(), labels.cuda())
    assert grad.dtype == torch.float16
    assert_loss_close(loss, want_loss, rtol=TOL_F16)
    assert_grad_close(grad, want_grad, atol=TOL_F16 * float(want_grad.abs().max()), rtol=TOL_F16)


@pytest.mark.parametrize("reduction", ["mean", "sum"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_focal_fused_step(reduction, dtype, monkeypatch):
    """The training step whose forward kernel already writes the gradient: an upstream gradient
    other than 1 (rescale kernel, vector body and ragged tail), a second backward through the
    same graph (recomputing kernel), a forward that needs no gradient, and equality with the
    two-kernel path."""
    P, O = _mods()
    g = torch.Generator().manual_seed(16)
    shape = (3, 2, 41, 67)                                   # 16482 elements: not a multiple of 4 or 8
    logits = (torch.randn(shape, generator=g) * 2).to(dtype)
    labels = (torch.rand(shape, generator=g) < 0.2).to(dtype)
    want_loss, want_grad = O.focal_loss(logits.float(), labels.float(), 0.25, 2.0, reduction)
    tol = dict(atol=TOL_F16 * float(want_grad.abs().max()) * 3, rtol=TOL_F16) if dtype == torch.float16 else {}
    crit = P.FocalLossV3(reduction=reduction)

    x = logits.cuda().requires_grad_(True)
    loss = crit(x, labels.cuda())
    (loss * 3.0).backward(retain_graph=True)
    assert_loss_close(loss, want_loss, rtol=TOL_F16 if dtype == torch.float16 else 1e-5)
    assert_grad_close(x.grad.float(), want_grad * 3.0, **({k: v * 3 if k == "atol" else v for k, v in tol.items()}))
    x.grad = None
    loss.backward()                                          # second trip: recomputed, not the saved tensor
    assert_grad_close(x.grad.float(), want_grad, **tol)

    with torch.no_grad():
        assert_loss_close(crit(logits.cuda(), labels.cuda()), want_loss, rtol=TOL_F16 if dtype == torch.float16 else 1e-5)

    fused_loss, fused_grad = run_module(crit, logits.cuda(), labels.cuda())
    monkeypatch.setenv("B200_FOCAL_FUSED", "0")
    plain_loss, plain_grad = run_module(crit, logits.cuda(), labels.cuda())
    assert float(fused_loss) == float(plain_loss)
    assert_grad_close(fused_grad.float(), plain_grad.float(), atol=1e-9 if dtype == torch.float32 else 1e-6, rtol=2e-3 if dtype == torch.float16 else 1e-6)


def test_focal_rejects_cpu_and_bad_dtype():
    P, _ = _mods()
    crit = P.FocalLossV3()
    with pytest.raises(RuntimeError):
        crit(torch.randn(2, 3), torch.zeros(2, 3))
    with pytest.raises(RuntimeError):
        crit(torch.randn(2, 3).cuda(), torch.zeros(2, 3, dtype=torch.int64).cuda())


def test_focal_deterministic_and_workspace_rearmed():
    P, _ = _mods()
    g = torch.Generator().manual_seed(15)
    logits = torch.randn(8, 1, 256, 256, generator=g).cuda()
    labels = (torch.rand(8, 1, 256, 256, generator=g) < 0.1).float().cuda()
    crit = P.FocalLossV3()
    first = crit(logits, labels).item()
    for _ in range(5):
        assert crit(logits, labels).item() == first
    from pytorch_loss import _cabi
    _cabi.read_status(logits.device)


def test_exchange_single_rank_and_bounded_wait():
    """The in-kernel cross-GPU sum on one GPU: a world of one rank gives the local sums, and a
    context whose peer never writes makes the bounded wait give up: status word set, record NaN
    (never a silently local number), no hang."""
    import pytorch_loss  # noqa: F401  (loads the library)
    from pytorch_loss import _cabi, _p2p
    from oracle import losses as O
    dev = torch.device("cuda", 0)
    lib = _cabi.load_library()
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(3, 1, 40, 50, generator=g)
    labels = (torch.rand(3, 1, 40, 50, generator=g) < 0.2).float()
    want, _ = O.focal_loss(logits, labels, 0.25, 2.0, 'sum')
    x, y = logits.to(dev), labels.to(dev)

    def run(exchange, calls=6):
        rec = _cabi.new_record(dev)
        ws = exchange.workspace()
        for _ in range(calls):          # every slot set, and the first one again
            _cabi.check(lib.b200_focal_forward(_cabi.ptr(x), _cabi.ptr(y), None, _cabi.ptr(rec), _cabi.ptr(ws),
                                               ws.numel(), x.numel(), _cabi.F32, 2.0, 0.25, _cabi.stream_ptr(dev)))
        return rec, ws

    rec, ws = run(_p2p.local_exchange_for_tests(dev, 1, 0, 1000))
    _cabi.check(lib.b200_read_status(_cabi.ptr(ws), _cabi.stream_ptr(dev)))
    sums = rec[:4].view(torch.float64).cpu()
    assert abs(float(sums[0]) - float(want)) <= 1e-5 * abs(float(want))
    assert float(sums[1]) == x.numel()

    rec, ws = run(_p2p.local_exchange_for_tests(dev, 2, 0, 200), calls=2)     # rank 1 never shows up
    rc = lib.b200_read_status(_cabi.ptr(ws), _cabi.stream_ptr(dev))
    assert rc == 4, "expected B200_ERR_STATUS, got %d" % rc          # the wait ran out and said so
    assert b"0x100" in lib.b200_last_error()
    assert bool(torch.isnan(rec[:4].view(torch.float64)).all()) and bool(torch.isnan(rec[4]))
    assert lib.b200_read_status(_cabi.ptr(ws), _cabi.stream_ptr(dev)) == 0    # cleared by the read


def test_exchange_foreign_tag_is_reported():
    """Ranks whose call sequences differ: this rank waits for a loss sum where its peer's slot
    holds a label count with the same sequence number.  The message is refused (status 0x200,
    NaN record) instead of being added as if it were a sum."""
    import pytorch_loss  # noqa: F401
    from pytorch_loss import _cabi, _p2p
    dev = torch.device("cuda", 0)
    lib = _cabi.load_library()
    ex = _p2p.local_exchange_for_tests(dev, 2, 0, 200)
    ws = ex.workspace()
    st = _cabi.stream_ptr(dev)
    # play rank 1: a context of its own whose "peer 0" array is rank 0's local array, so its
    # count message lands where rank 0 will look for rank 1's first message
    other = _p2p.Exchange(dev, 2, 1, ex.stand_ins[0], {0: ex.local_slots.data_ptr()}, 200)
    cnt = _cabi.new_record(dev)
    labels = torch.zeros(64, dtype=torch.int64, device=dev)
    wo = other.workspace()
    _cabi.check(lib.b200_count_valid(_cabi.ptr(labels), 64, 255, _cabi.ptr(cnt), _cabi.ptr(wo), wo.numel(), st))
    x = torch.randn(256, device=dev)
    y = torch.zeros(256, device=dev)
    rec = _cabi.new_record(dev)
    _cabi.check(lib.b200_focal_forward(_cabi.ptr(x), _cabi.ptr(y), None, _cabi.ptr(rec), _cabi.ptr(ws), ws.numel(),
                                       256, _cabi.F32, 2.0, 0.25, st))
    assert lib.b200_read_status(_cabi.ptr(ws), st) == 4
    assert b"0x200" in lib.b200_last_error()
    assert bool(torch.isnan(rec[4]))


def test_two_emulated_ranks_exchange_the_label_count():
    """Two emulated ranks on one GPU: two exchange contexts over each other's slot arrays, their
    kernels launched one after the other, so no kernel ever waits on one that has not run.  Rank 1's
    count kernel runs first: it posts its count and gives up waiting for rank 0 (bounded, NaN, status
    bit).  Rank 0's count kernel then finds both messages and gets the GLOBAL count, which its fused
    label-smooth step divides by; that step's own sum exchange times out (rank 1 posts no sum)."""
    import pytorch_loss  # noqa: F401
    from pytorch_loss import _cabi, _p2p
    from oracle import losses as O
    dev = torch.device("cuda", 0)
    lib = _cabi.load_library()
    st = _cabi.stream_ptr(dev)
    nbytes = int(lib.b200_exchange_slot_bytes(2))
    arrays = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(2)]
    ranks = [_p2p.Exchange(dev, 2, r, arrays[r], {1 - r: arrays[1 - r].data_ptr()}, 500) for r in range(2)]
    g = torch.Generator().manual_seed(91)
    logits = torch.randn(4, 19, 32, 32, generator=g)
    labels = torch.randint(0, 19, (4, 32, 32), generator=g)
    labels[0, :11] = 255                                       # uneven valid counts per rank
    want_loss, want_grad = O.label_smooth_ce(logits, labels, 0.1, 255, 'mean')
    xs = [logits[2 * r:2 * r + 2].to(dev) for r in range(2)]
    ys = [labels[2 * r:2 * r + 2].to(dev) for r in range(2)]
    cnts = [_cabi.new_record(dev) for _ in range(2)]
    for r in (1, 0):
        ws = ranks[r].workspace()
        _cabi.check(lib.b200_count_valid(_cabi.ptr(ys[r]), ys[r].numel(), 255, _cabi.ptr(cnts[r]), _cabi.ptr(ws),
                                         ws.numel(), st))
    torch.cuda.synchronize()
    w1 = ranks[1].workspace()
    assert lib.b200_read_status(_cabi.ptr(w1), st) == 4 and b"0x100" in lib.b200_last_error()
    assert bool(torch.isnan(cnts[1][:4].view(torch.float64)[1]))
    assert float(cnts[0][:4].view(torch.float64)[1]) == float((labels != 255).sum())   # the GLOBAL count
    grad = torch.empty_like(xs[0])
    rec = _cabi.new_record(dev)
    ws = ranks[0].workspace()
    _cabi.check(lib.b200_lsr_forward_backward_reduced(
        _cabi.ptr(xs[0]), _cabi.ptr(ys[0]), _cabi.ptr(grad), _cabi.ptr(rec), _cabi.ptr(ws), ws.numel(),
        _cabi._vp(cnts[0].data_ptr() + 8), 2, 19, 32 * 32, _cabi.F32, 255, 0.1, 0, st))
    torch.cuda.synchronize()
    assert_grad_close(grad, want_grad[:2])
    assert lib.b200_read_status(_cabi.ptr(ws), st) == 4 and b"0x100" in lib.b200_last_error()
    assert bool(torch.isnan(rec[4]))


def test_focal_predicted_count_correction():
    """The sharded fused step divides by the global element count of the PREVIOUS call and leaves
    predicted / actual for the rescale kernel.  One rank (a world of one) whose batch changes size
    between calls: the loss is right at once, `correction` != 1, the rescaled gradient matches the
    oracle, and the state holds the new count."""
    import pytorch_loss as P
    from pytorch_loss import _cabi, _p2p
    from oracle import losses as O
    dev = torch.device("cuda", 0)
    lib = _cabi.load_library()
    st = _cabi.stream_ptr(dev)
    ex = _p2p.local_exchange_for_tests(dev, 1, 0, 1000)
    ws = ex.workspace()
    g = torch.Generator().manual_seed(92)
    state = torch.tensor([3.0 * 5 * 77], dtype=torch.float64, device=dev)     # count of an earlier, larger batch
    for shape in ((2, 5, 77), (3, 5, 77), (3, 5, 77)):
        logits = torch.randn(shape, generator=g) * 2
        labels = (torch.rand(shape, generator=g) < 0.3).float()
        want_loss, want_grad = O.focal_loss(logits, labels, 0.25, 2.0, 'mean')
        x, y = logits.to(dev), labels.to(dev)
        predicted = float(state)
        grad = torch.empty_like(x)
        rec = _cabi.new_record(dev)
        corr = torch.zeros(1, dtype=torch.float32, device=dev)
        _cabi.check(lib.b200_focal_forward_backward_predicted(
            _cabi.ptr(x), _cabi.ptr(y), _cabi.ptr(grad), _cabi.ptr(rec), _cabi.ptr(ws), ws.numel(),
            _cabi.ptr(state), _cabi.ptr(corr), x.numel(), _cabi.F32, 2.0, 0.25, 0, st))
        one = torch.ones(1, dtype=torch.float32, device=dev)
        _cabi.check(lib.b200_rescale_gradient(_cabi.ptr(grad), _cabi.ptr(one), _cabi.ptr(corr), x.numel(),
                                              _cabi.F32, st))
        assert_loss_close(rec[4], want_loss)
        assert abs(float(corr) - predicted / x.numel()) <= 1e-6 * predicted / x.numel()
        assert float(state) == x.numel()
        assert_grad_close(grad, want_grad, atol=1e-7)
    _cabi.check(lib.b200_read_status(_cabi.ptr(ws), st))


def test_deferred_sum_is_completed_by_the_rescale_kernel():
    """`defer`: the fused step posts its sums and leaves the record incomplete (NaN mean, no
    correction); the rescale kernel that follows collects them, completes the record, writes the
    correction and rescales with it.  A world of one rank, batch size changing between calls.
    Also the stand-alone completion (loss read without backward), which may be called twice."""
    from pytorch_loss import _cabi, _p2p
    from oracle import losses as O
    dev = torch.device("cuda", 0)
    lib = _cabi.load_library()
    st = _cabi.stream_ptr(dev)
    ex = _p2p.local_exchange_for_tests(dev, 1, 0, 1000)
    ws = ex.workspace()
    g = torch.Generator().manual_seed(93)
    state = torch.tensor([2.0 * 5 * 77], dtype=torch.float64, device=dev)
    for i, shape in enumerate(((3, 5, 77), (3, 5, 77), (2, 5, 77))):
        logits = torch.randn(shape, generator=g) * 2
        labels = (torch.rand(shape, generator=g) < 0.3).float()
        want_loss, want_grad = O.focal_loss(logits, labels, 0.25, 2.0, 'mean')
        x, y = logits.to(dev), labels.to(dev)
        grad = torch.empty_like(x)
        rec = _cabi.new_record(dev)
        corr = torch.full((1,), float("nan"), dtype=torch.float32, device=dev)
        _cabi.check(lib.b200_focal_forward_backward_predicted(
            _cabi.ptr(x), _cabi.ptr(y), _cabi.ptr(grad), _cabi.ptr(rec), _cabi.ptr(ws), ws.numel(),
            _cabi.ptr(state), _cabi.ptr(corr), x.numel(), _cabi.F32, 2.0, 0.25, 1, st))
        torch.cuda.synchronize()
        assert bool(torch.isnan(rec[4])) and bool(torch.isnan(corr[0]))           # posted, not collected
        up = torch.full((1,), 2.0, dtype=torch.float32, device=dev)
        if i == 2:                       # the loss is read first: stand-alone completion, twice
            for _ in range(2):
                _cabi.check(lib.b200_exchange_finish(_cabi.ptr(ws), _cabi.ptr(rec), _cabi.ptr(state), _cabi.ptr(corr), st))
            assert_loss_close(rec[4], want_loss)
        _cabi.check(lib.b200_rescale_gradient_finish(_cabi.ptr(grad), _cabi.ptr(up), _cabi.ptr(corr), x.numel(),
                                                     _cabi.F32, _cabi.ptr(ws), _cabi.ptr(rec), _cabi.ptr(state), st))
        assert_loss_close(rec[4], want_loss)
        assert float(rec[:4].view(torch.float64)[1]) == x.numel() == float(state)
        assert_grad_close(grad, 2.0 * want_grad, atol=1e-7)
    _cabi.check(lib.b200_read_status(_cabi.ptr(ws), st))
