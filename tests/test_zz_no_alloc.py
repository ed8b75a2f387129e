"""The allocation-free focal forward (b200_focal_forward_noalloc), called through the C ABI.

Who needs it: a program that cannot give the library a workspace -- for instance one that
reserved the whole GPU for its own memory pool when it started, so any later cudaMalloc
would fail, or a thin FFI caller with no device allocator of its own.  The entry point keeps
the reduction's scratch in a fixed array inside the library, so the caller passes only its
inputs and outputs.

What is checked: on two calls in a row (the second on different data, so stale scratch from
the first would show), its reduction record equals the one the ordinary entry point
(b200_focal_forward with a caller-provided workspace) produces, within the tolerance the
other focal tests use (1e-5 relative on the loss), and both equal the CPU oracle's sum within
that same tolerance; the count is exact; oversize inputs are refused with a message.  This file sorts last on purpose: a run that stops at the first
failure has then already executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_ELEMS = 1 << 28


def _records(lib, logits, labels, gamma, alpha):
    """(record of the no-alloc entry, record of the workspace entry) as float64 [sum, count] + float32 mean."""
    from pytorch_loss import _cabi
    dev = logits.device
    stream = _cabi.stream_ptr(dev)
    out_new = torch.full((8,), float("nan"), dtype=torch.float32, device=dev)
    out_ref = torch.full((8,), float("nan"), dtype=torch.float32, device=dev)
    ws = torch.zeros(int(lib.b200_reduce_workspace_bytes()), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = lib.b200_focal_forward_noalloc(_cabi.ptr(logits), _cabi.ptr(labels), None, _cabi.ptr(out_new),
                                            logits.numel(), _cabi.dtype_code(logits), gamma, alpha, stream)
        assert rc == 0, lib.b200_last_error()
        _cabi.check(lib.b200_focal_forward(_cabi.ptr(logits), _cabi.ptr(labels), None, _cabi.ptr(out_ref),
                                           _cabi.ptr(ws), ws.numel(), logits.numel(),
                                           _cabi.dtype_code(logits), gamma, alpha, stream))
    torch.cuda.synchronize(dev)
    return out_new.cpu(), out_ref.cpu()


def test_no_alloc_entry_matches_workspace_entry_on_two_calls():
    from pytorch_loss import _cabi
    from oracle import losses as O
    lib = _cabi.load_library()
    g = torch.Generator().manual_seed(2024)
    for call, shape in enumerate([(4, 3, 257, 129), (2, 1, 1024, 1024)]):
        logits = torch.randn(shape, generator=g) * 3 ** 0.5
        labels = (torch.rand(shape, generator=g) < 0.1).float()
        want_sum = float(O.focal_loss(logits, labels, 0.25, 2.0, 'sum', dtype=torch.float64)[0])
        logits, labels = logits.cuda(), labels.cuda()
        new, ref = _records(lib, logits, labels, 2.0, 0.25)
        assert abs(float(new[:4].view(torch.float64)[0]) - want_sum) <= 1e-5 * abs(want_sum), "call %d: oracle" % call
        new_sc, ref_sc = new[:4].view(torch.float64), ref[:4].view(torch.float64)
        assert float(new_sc[1]) == float(ref_sc[1]) == logits.numel(), "call %d: count" % call
        assert abs(float(new_sc[0]) - float(ref_sc[0])) <= 1e-5 * abs(float(ref_sc[0])), "call %d: sum" % call
        assert abs(float(new[4]) - float(ref[4])) <= 1e-5 * abs(float(ref[4])), "call %d: mean" % call


def test_no_alloc_entry_writes_losses_and_handles_fp16_and_general_gamma():
    from pytorch_loss import _cabi
    lib = _cabi.load_library()
    g = torch.Generator().manual_seed(2025)
    logits = torch.randn(3, 5, 77, generator=g).half().cuda()
    labels = (torch.rand(3, 5, 77, generator=g) < 0.3).half().cuda()
    losses_new = torch.empty_like(logits)
    losses_ref = torch.empty_like(logits)
    out = torch.empty(8, dtype=torch.float32, device=logits.device)
    stream = _cabi.stream_ptr(logits.device)
    assert lib.b200_focal_forward_noalloc(_cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(losses_new),
                                          _cabi.ptr(out), logits.numel(), _cabi.F16, 1.5, 0.4, stream) == 0
    _cabi.check(lib.b200_focal_forward(_cabi.ptr(logits), _cabi.ptr(labels), _cabi.ptr(losses_ref), None, None, 0,
                                       logits.numel(), _cabi.F16, 1.5, 0.4, stream))
    torch.cuda.synchronize()
    assert torch.equal(losses_new, losses_ref)
    assert abs(float(out[5]) - float(losses_ref.float().sum())) <= 2e-3 * abs(float(losses_ref.float().sum()))


def test_no_alloc_entry_refuses_oversize_and_bad_arguments():
    from pytorch_loss import _cabi
    lib = _cabi.load_library()
    out = torch.empty(8, dtype=torch.float32, device="cuda")
    x = torch.zeros(16, device="cuda")
    rc = lib.b200_focal_forward_noalloc(_cabi.ptr(x), _cabi.ptr(x), None, _cabi.ptr(out), MAX_ELEMS + 1, _cabi.F32,
                                        2.0, 0.25, None)
    assert rc == 2 and b"maximum" in lib.b200_last_error()
    assert lib.b200_focal_forward_noalloc(_cabi.ptr(x), _cabi.ptr(x), None, None, 16, _cabi.F32, 2.0, 0.25, None) == 1
    assert lib.b200_focal_forward_noalloc(None, None, None, _cabi.ptr(out), 16, _cabi.F32, 2.0, 0.25, None) == 1
