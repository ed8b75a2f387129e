"""CPU-only checks of the C-ABI boundary: the library builds/loads without a GPU, exports
every function include/b200loss.h declares (and nothing is declared only on one side), and
rejects bad arguments before touching the device."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


def _header_functions():
    text = open(os.path.join(ROOT, "include", "b200loss.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_\w+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    import sys
    sys.path.insert(0, os.path.join(ROOT, "pytorch-loss_b200"))
    import build as b200_build
    b200_build.build()
    from pytorch_loss import _cabi
    return _cabi.load_library()


def test_header_and_binding_agree(lib):
    from pytorch_loss import _cabi
    declared = _header_functions()
    assert declared, "no declarations found in include/b200loss.h"
    assert sorted(_cabi.SIGNATURES) == declared


def test_every_declared_symbol_is_exported(lib):
    for name in _header_functions():
        assert hasattr(lib, name), "libb200loss.so does not export %s" % name


def test_version_and_workspace_queries(lib):
    from pytorch_loss import _cabi
    assert lib.b200_abi_version() == _cabi.ABI_VERSION
    assert lib.b200_reduce_workspace_bytes() >= 64 + 16 * 1024
    assert lib.b200_lovasz_workspace_bytes(2, 19, 1024, 1) > 0
    assert lib.b200_lovasz_workspace_bytes(2, 19, 1024, 0) > 0


def test_argument_errors_do_not_need_a_device(lib):
    # negative sizes / missing outputs are refused with a message, no CUDA call is made
    assert lib.b200_focal_forward(None, None, None, None, None, 0, -1, 0, 2.0, 0.25, None) == 1
    assert b"E >= 0" in lib.b200_last_error()
    assert lib.b200_lsr_forward(None, None, None, None, None, 0, 2, 0, 4, 0, -100, 0.1, None) == 1
    assert lib.b200_lsr_forward(None, None, None, ctypes.c_void_p(8), None, 0, 2, 3, 4, 0, -100, 0.1, None) == 5
    assert lib.b200_lmargin_backward(None, None, None, 7, None, None, 2, 3, 4, 0, 255, 0.3, None) == 1
    assert lib.b200_lovasz_forward(None, None, None, None, None, 0, 2, 600, 4, 0, 255, 0, None) != 0


def test_missing_library_fails_loudly(tmp_path):
    from pytorch_loss import _cabi
    with pytest.raises(RuntimeError, match="no fallback"):
        _cabi.load_library(str(tmp_path / "libb200loss.so"))


def test_fused_step_path_queries(lib):
    """Which layouts have a one-pass training step: pure pointer/shape arithmetic, no device needed.
    Addresses are made up (never dereferenced by the queries)."""
    A, U = 0x7f0000001000, 0x7f0000001004            # 16-byte aligned / only 4-byte aligned
    F32, F16 = 0, 1
    q = lambda x, y, g, n, c, m, dt: lib.b200_softmax_fused_step_path(
        ctypes.c_void_p(x), ctypes.c_void_p(y), ctypes.c_void_p(g), n, c, m, dt)
    # images: the tile pipeline (aligned rows), the any-alignment kernel (float32, <= 320 classes)
    assert q(A, A, A, 2, 19, 1024, F32) == 1
    assert q(A, A, A, 2, 19, 769 * 769, F32) == 1          # odd pixel count
    assert q(U, A, U, 2, 150, 1024, F32) == 1              # unaligned pointers
    assert q(A, A, A, 2, 19, 769 * 769, F16) == 0          # half logits need 16-byte aligned rows
    assert q(A, A, A, 2, 19, 1024, F16) == 1
    assert q(A, A, A, 2, 400, 1023, F32) == 0              # too many classes for the unaligned kernel
    # rows (M == 1): short rows up to 2048 classes, whole rows in shared memory beyond (16-byte rows)
    assert q(A, A, A, 4096, 1000, 1, F32) == 1
    assert q(A, A, A, 4096, 19, 1, F32) == 1
    assert q(A, A, A, 256, 32768, 1, F16) == 1
    assert q(A, A, A, 256, 4099, 1, F32) == 0              # 16 396-byte rows: no bulk copy
    assert q(A, A, A, 0, 19, 1024, F32) == 0               # empty batch
    p = lambda x, y, g, n, c, m, dt: lib.b200_pc_softmax_step_path(
        ctypes.c_void_p(x), ctypes.c_void_p(y), ctypes.c_void_p(g), n, c, m, dt)
    assert p(A, A, A, 2, 19, 1024, F32) == 1
    assert p(A, A, A, 2, 256, 1024, F16) == 1
    assert p(A, A, A, 2, 257, 1024, F32) == 0              # class weights for at most 256 classes
    assert p(A, A, A, 2, 19, 1023, F32) == 0               # the tile pipeline only
    assert p(A, A, A, 64, 19, 1, F32) == 0
