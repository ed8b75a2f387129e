"""Stand-in for the reference's `taylor_softmax_cpp` extension module
(csrc/taylor_softmax.cu:419-422)."""
from pytorch_loss import taylor_softmax as _ts


def taylor_softmax_forward(feat, dim, n, use_log):
    return _ts.taylor_softmax_forward(feat, dim, n, use_log)


def taylor_softmax_backward(grad, feat, dim, n, use_log):
    return _ts.taylor_softmax_backward(grad, feat, dim, n, use_log)
