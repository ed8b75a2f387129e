"""ctypes binding of libb200loss.so (declared in include/b200loss.h) and the small
amount of host logic every op shares: dtype codes, contiguity, per-stream
workspaces, error translation.

There is no CPU or eager fallback: if the library is missing or a tensor is not
on a CUDA device, the call raises.
"""
import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200loss.so")

ABI_VERSION = 3
STEP_DEFER, STEP_AFTER_COUNT = 1, 2      # bits of the fused steps' `defer` argument (b200loss.h)
F32, F16, BF16, F64 = 0, 1, 2, 3

_c = ctypes
_vp, _i64, _int, _f32, _f64, _sz = _c.c_void_p, _c.c_int64, _c.c_int, _c.c_float, _c.c_double, _c.c_size_t

# name -> (restype, argtypes); mirrors include/b200loss.h one to one.
SIGNATURES = {
    "b200_abi_version": (_int, []),
    "b200_last_error": (_c.c_char_p, []),
    "b200_kernel_launch_count": (_c.c_uint64, []),
    "b200_reduce_workspace_bytes": (_sz, []),
    "b200_read_status": (_int, [_vp, _vp]),
    "b200_enable_peer_access": (_int, [_int]),
    "b200_ipc_export": (_int, [_vp, _vp, _vp]),
    "b200_ipc_open": (_int, [_vp, _c.c_uint64, _vp]),
    "b200_ipc_close": (_int, [_vp, _c.c_uint64]),
    "b200_exchange_ctx_bytes": (_sz, []),
    "b200_exchange_slot_bytes": (_sz, [_int]),
    "b200_reduce_attach_exchange": (_int, [_vp, _vp, _vp]),
    "b200_focal_forward": (_int, [_vp, _vp, _vp, _vp, _vp, _sz, _i64, _int, _f32, _f32, _vp]),
    "b200_focal_backward": (_int, [_vp, _vp, _vp, _int, _vp, _vp, _i64, _int, _f32, _f32, _vp]),
    "b200_focal_forward_backward": (_int, [_vp, _vp, _vp, _vp, _i64, _int, _f32, _f32, _vp]),
    "b200_focal_forward_backward_reduced": (_int, [_vp, _vp, _vp, _vp, _vp, _sz, _vp, _f32, _i64, _int, _f32, _f32, _int, _vp]),
    "b200_focal_forward_backward_predicted": (_int, [_vp, _vp, _vp, _vp, _vp, _sz, _vp, _vp, _i64, _int, _f32, _f32, _int, _vp]),
    "b200_rescale_gradient": (_int, [_vp, _vp, _vp, _i64, _int, _vp]),
    "b200_rescale_gradient_finish": (_int, [_vp, _vp, _vp, _i64, _int, _vp, _vp, _vp, _vp]),
    "b200_exchange_finish": (_int, [_vp, _vp, _vp, _vp, _vp]),
    "b200_exchange_count": (_int, [_f64, _vp, _vp, _sz, _vp]),
    "b200_softmax_fused_step_path": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _int]),
    "b200_count_valid": (_int, [_vp, _i64, _i64, _vp, _vp, _sz, _vp]),
    "b200_lsr_forward_backward_reduced": (_int, [_vp, _vp, _vp, _vp, _vp, _sz, _vp, _i64, _i64, _i64, _int, _i64, _f32, _int, _vp]),
    "b200_lmargin_forward_backward_reduced": (_int, [_vp, _vp, _vp, _vp, _vp, _sz, _vp, _i64, _i64, _i64, _int, _i64, _f32, _int, _vp]),
    "b200_focal_forward_noalloc": (_int, [_vp, _vp, _vp, _vp, _i64, _int, _f32, _f32, _vp]),
    "b200_lsr_forward": (_int, [_vp, _vp, _vp, _vp, _vp, _sz, _i64, _i64, _i64, _int, _i64, _f32, _vp]),
    "b200_lsr_backward": (_int, [_vp, _vp, _vp, _int, _vp, _vp, _i64, _i64, _i64, _int, _i64, _f32, _vp]),
    "b200_lmargin_forward": (_int, [_vp, _vp, _vp, _vp, _vp, _sz, _i64, _i64, _i64, _int, _i64, _f32, _vp]),
    "b200_lmargin_backward": (_int, [_vp, _vp, _vp, _int, _vp, _vp, _i64, _i64, _i64, _int, _i64, _f32, _vp]),
    "b200_softmax_stats_path": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _int]),
    "b200_lsr_forward_ex": (_int, [_vp, _vp, _vp, _vp, _vp, _sz, _vp, _i64, _i64, _i64, _int, _i64, _f32, _vp]),
    "b200_lsr_backward_ex": (_int, [_vp, _vp, _vp, _vp, _int, _vp, _vp, _i64, _i64, _i64, _int, _i64, _f32, _vp]),
    "b200_lmargin_forward_ex": (_int, [_vp, _vp, _vp, _vp, _vp, _sz, _vp, _i64, _i64, _i64, _int, _i64, _f32, _vp]),
    "b200_lmargin_backward_ex": (_int, [_vp, _vp, _vp, _vp, _int, _vp, _vp, _i64, _i64, _i64, _int, _i64, _f32, _vp]),
    "b200_lovasz_workspace_bytes": (_sz, [_i64, _i64, _i64, _int]),
    "b200_lovasz_forward": (_int, [_vp, _vp, _vp, _vp, _vp, _sz, _i64, _i64, _i64, _int, _i64, _int, _vp]),
    "b200_lovasz_backward": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _i64, _int, _vp]),
    "b200_taylor_softmax_forward": (_int, [_vp, _vp, _i64, _i64, _i64, _int, _int, _int, _vp]),
    "b200_taylor_softmax_backward": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _int, _vp]),
    "b200_pc_softmax_ce": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _i64, _vp]),
    "b200_pc_softmax_step_path": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _int]),
    "b200_pc_softmax_step": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _sz, _vp, _i64, _i64, _i64, _int, _i64, _int, _vp]),
    "b200_pc_softmax_ce_scaled": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _i64, _vp]),
    "b200_ohem_workspace_bytes": (_sz, [_i64, _i64]),
    "b200_ohem_label": (_int, [_vp, _vp, _vp, _vp, _sz, _i64, _i64, _i64, _int, _i64, _f32, _i64, _vp]),
}

_lib = None
_lib_lock = threading.Lock()


def load_library(path=None):
    """Loads libb200loss.so once and declares every prototype.  Raises RuntimeError with
    build instructions if the file is missing: nothing here can run without it."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    with _lib_lock:
        if _lib is not None and path is None:
            return _lib
        p = path or LIB_PATH
        if not os.path.exists(p):
            raise RuntimeError(
                "libb200loss.so not found at %s; build it with "
                "`python pytorch-loss_b200/build.py` (needs nvcc). There is no fallback path." % p)
        lib = ctypes.CDLL(p)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)          # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        ver = lib.b200_abi_version()
        if ver != ABI_VERSION:
            raise RuntimeError("libb200loss.so ABI version %d, Python side expects %d" % (ver, ABI_VERSION))
        if path is None:
            _lib = lib
        return lib


class B200LossError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, code, message):
        super().__init__("libb200loss error %d: %s" % (code, message))
        self.code = code


def check(code):
    if code != 0:
        msg = load_library().b200_last_error()
        raise B200LossError(code, msg.decode("utf-8", "replace") if msg else "")


def dtype_code(t, allow_f64=False):
    """The library's code of a tensor's dtype.  float64 only where the caller has a double path
    (per-pixel label-smooth / large-margin / focal kernels)."""
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.float64 and allow_f64:
        return F64
    if t.dtype == torch.float16:
        return F16
    if t.dtype == torch.bfloat16:
        return BF16
    raise RuntimeError("libb200loss supports float32, float16 and bfloat16 logits, got %s" % t.dtype)


def require_cuda(*tensors):
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("this loss only supports gpu mode: got a tensor on %s" % t.device)
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError("tensors are on different devices: %s vs %s" % (dev, t.device))
    return dev


def ptr(t):
    return None if t is None else _vp(t.data_ptr())


def stream_ptr(device):
    return _vp(torch.cuda.current_stream(device).cuda_stream)


# --- per-(device, stream) reduction workspace -----------------------------------------
# The reducing kernels need a zero-initialised scratch whose header they leave zero
# again, so one buffer per stream is allocated (and zeroed) once and then reused.

_workspaces = {}
_ws_lock = threading.Lock()


def reduce_workspace(device):
    stream = torch.cuda.current_stream(device)
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream.cuda_stream)
    ws = _workspaces.get(key)
    if ws is None:
        nbytes = int(load_library().b200_reduce_workspace_bytes())
        with _ws_lock:
            ws = _workspaces.get(key)
            if ws is None:
                ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)
                _workspaces[key] = ws
    return ws


def read_status(device):
    """Synchronises the current stream and raises if a kernel recorded a failed wait."""
    ws = reduce_workspace(device)
    check(load_library().b200_read_status(ptr(ws), stream_ptr(device)))


def new_record(device):
    """32-byte reduction record as 8 float32 (views: [:4]->2 doubles sum,count; [4] mean; [5] sum)."""
    return torch.empty(8, dtype=torch.float32, device=device)


def split_shape(logits, labels=None):
    """(N, C, M) of a [N, C, *spatial] tensor; checks the labels' shape when given."""
    if logits.dim() < 2:
        raise RuntimeError("logits must be [N, C, ...], got shape %s" % (tuple(logits.shape),))
    n, c = logits.shape[0], logits.shape[1]
    m = 1
    for d in logits.shape[2:]:
        m *= d
    if labels is not None:
        want = (n,) + tuple(logits.shape[2:])
        if tuple(labels.shape) != want:
            raise RuntimeError("labels shape %s does not match logits %s (expected %s)"
                               % (tuple(labels.shape), tuple(logits.shape), want))
        if labels.dtype != torch.int64:
            raise RuntimeError("labels must be int64, got %s" % labels.dtype)
    return n, c, m


def grad_mode_of(grad_output, pixel_shape):
    """Classifies an upstream gradient: (mode, tensor) with mode 1 = one scalar broadcast
    over all pixels (what autograd delivers below .sum()/.mean()), mode 2 = per pixel."""
    if grad_output.numel() == 1 or all(s == 0 for s in grad_output.stride()):
        scalar = grad_output.reshape(-1)[:1] if grad_output.numel() == 1 else grad_output.as_strided((1,), (1,))
        return 1, scalar.to(torch.float32).contiguous()
    if tuple(grad_output.shape) != tuple(pixel_shape):
        grad_output = grad_output.expand(pixel_shape)
    return 2, grad_output.contiguous()


# --- per-call device timing (used by the benchmark, off by default) ---------------------

class CallTimer:
    """Context manager: while active, every kernel-launching C-ABI call made through
    `load_library()` is bracketed by CUDA events on the current stream.  `summary()`
    returns {entry point: (calls, total milliseconds)} after a synchronise."""

    def __init__(self):
        self.records = []

    def __enter__(self):
        global _lib
        self._real = load_library()
        timer = self

        class _Proxy:
            def __getattr__(self, name):
                fn = getattr(timer._real, name)
                if not name.endswith(("_forward", "_backward", "_forward_backward")):
                    return fn

                def timed(*args):
                    a = torch.cuda.Event(enable_timing=True)
                    b = torch.cuda.Event(enable_timing=True)
                    a.record()
                    rc = fn(*args)
                    b.record()
                    timer.records.append((name, a, b))
                    return rc
                return timed

        _lib = _Proxy()
        return self

    def __exit__(self, *exc):
        global _lib
        _lib = self._real
        return False

    def summary(self):
        torch.cuda.synchronize()
        out = {}
        for name, a, b in self.records:
            n, ms = out.get(name, (0, 0.0))
            out[name] = (n + 1, ms + a.elapsed_time(b))
        return out
