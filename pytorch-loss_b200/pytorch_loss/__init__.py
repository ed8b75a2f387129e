"""pytorch_loss — the fused V3 per-pixel losses of CoinCheung/pytorch-loss, rebuilt for
NVIDIA B200 (sm_100a) on a C-ABI CUDA library (libb200loss.so, include/b200loss.h).

Same import surface as the reference package for this path (reference
pytorch_loss/__init__.py:12,13,16,23):

    from pytorch_loss import LabelSmoothSoftmaxCEV3, FocalLossV3, LargeMarginSoftmaxV3, LovaszSoftmaxV3
"""
from .focal_loss import FocalLossV3, FocalSigmoidLossFuncV3, FocalSigmoidLossFuncV3FB
from .label_smooth import LabelSmoothSoftmaxCEV3, LSRCrossEntropyFunctionV3
from .large_margin_softmax import (LargeMarginSoftmaxV3, LargeMarginSoftmaxFuncV3,
                                   LargeMarginSoftmaxFuncV3FB)

__all__ = [
    "FocalLossV3", "FocalSigmoidLossFuncV3", "FocalSigmoidLossFuncV3FB",
    "LabelSmoothSoftmaxCEV3", "LSRCrossEntropyFunctionV3",
    "LargeMarginSoftmaxV3", "LargeMarginSoftmaxFuncV3", "LargeMarginSoftmaxFuncV3FB",
]
from .lovasz_softmax import LovaszSoftmaxV3, LovaszSoftmaxFunctionV3

__all__ += ["LovaszSoftmaxV3", "LovaszSoftmaxFunctionV3"]
from .ohem_loss import OhemCELoss, OhemLargeMarginLoss

__all__ += ["OhemCELoss", "OhemLargeMarginLoss"]
from .taylor_softmax import (TaylorSoftmaxV3, LogTaylorSoftmaxV3, TaylorCrossEntropyLossV3, TaylorSoftmaxFunc,
                             taylor_softmax_v3)

__all__ += ["TaylorSoftmaxV3", "LogTaylorSoftmaxV3", "TaylorCrossEntropyLossV3", "TaylorSoftmaxFunc",
            "taylor_softmax_v3"]
from .pc_softmax import PCSoftmaxCrossEntropyV2, PCSoftmaxCrossEntropyFunction

__all__ += ["PCSoftmaxCrossEntropyV2", "PCSoftmaxCrossEntropyFunction"]
