"""CPU-only tests of the host-side logic: shape/dtype checks, upstream-gradient
classification, shard arithmetic, module surface (names, defaults, attributes) and the
refusal to run without a CUDA device."""
import inspect

import pytest
import torch


def test_module_surface_matches_reference_names():
    import pytorch_loss as P
    for name in ("LabelSmoothSoftmaxCEV3", "LSRCrossEntropyFunctionV3", "FocalLossV3",
                 "FocalSigmoidLossFuncV3", "FocalSigmoidLossFuncV3FB", "LargeMarginSoftmaxV3",
                 "LargeMarginSoftmaxFuncV3", "LargeMarginSoftmaxFuncV3FB", "LovaszSoftmaxV3",
                 "LovaszSoftmaxFunctionV3"):
        assert hasattr(P, name), name
    lsr = P.LabelSmoothSoftmaxCEV3()
    assert (lsr.lb_smooth, lsr.reduction, lsr.lb_ignore) == (0.1, 'mean', -100)
    fo = P.FocalLossV3()
    assert (fo.alpha, fo.gamma, fo.reduction) == (0.25, 2, 'mean')
    lm = P.LargeMarginSoftmaxV3()
    assert (lm.lam, lm.reduction, lm.ignore_index, lm.fb) == (0.3, 'mean', 255, True)
    lv = P.LovaszSoftmaxV3()
    assert (lv.reduction, lv.lb_ignore) == ('mean', -100)
    for m in (lsr, fo, lm, lv):
        assert len(m.state_dict()) == 0          # stateless, like the reference
    # positional constructor orders of the reference
    assert list(inspect.signature(P.LabelSmoothSoftmaxCEV3).parameters)[:3] == ['lb_smooth', 'reduction', 'ignore_index']
    assert list(inspect.signature(P.FocalLossV3).parameters)[:3] == ['alpha', 'gamma', 'reduction']
    assert list(inspect.signature(P.LargeMarginSoftmaxV3).parameters)[:4] == ['lam', 'reduction', 'ignore_index', 'fb']
    assert list(inspect.signature(P.LovaszSoftmaxV3).parameters)[:2] == ['reduction', 'ignore_index']


def test_extension_shims_expose_reference_entry_points():
    import lsr_cpp, focal_cpp, large_margin_cpp, lovasz_softmax_cpp
    assert callable(lsr_cpp.lsr_forward) and callable(lsr_cpp.lsr_backward)
    for f in ("focalloss_forward", "focalloss_backward", "focalloss_forward_backward"):
        assert callable(getattr(focal_cpp, f))
    for f in ("l_margin_forward", "l_margin_backward", "l_margin_forward_backward"):
        assert callable(getattr(large_margin_cpp, f))
    for f in ("lovasz_softmax_forward", "lovasz_softmax_backward"):
        assert callable(getattr(lovasz_softmax_cpp, f))


def test_cpu_tensors_are_refused_not_computed():
    import pytorch_loss as P
    x = torch.randn(2, 5, 4, 4)
    y = torch.randint(0, 5, (2, 4, 4))
    for crit in (P.LabelSmoothSoftmaxCEV3(), P.LargeMarginSoftmaxV3(), P.LovaszSoftmaxV3()):
        with pytest.raises(RuntimeError, match="gpu"):
            crit(x, y)
    with pytest.raises(RuntimeError, match="gpu"):
        P.FocalLossV3()(x, torch.zeros_like(x))


def test_split_shape_and_label_checks():
    from pytorch_loss import _cabi
    assert _cabi.split_shape(torch.zeros(2, 3, 4, 5)) == (2, 3, 20)
    assert _cabi.split_shape(torch.zeros(7, 9)) == (7, 9, 1)
    assert _cabi.split_shape(torch.zeros(2, 3, 4), torch.zeros(2, 4, dtype=torch.int64)) == (2, 3, 4)
    with pytest.raises(RuntimeError):
        _cabi.split_shape(torch.zeros(5))
    with pytest.raises(RuntimeError):
        _cabi.split_shape(torch.zeros(2, 3, 4), torch.zeros(2, 5, dtype=torch.int64))
    with pytest.raises(RuntimeError):
        _cabi.split_shape(torch.zeros(2, 3, 4), torch.zeros(2, 4, dtype=torch.int32))
    with pytest.raises(RuntimeError):
        _cabi.dtype_code(torch.zeros(1, dtype=torch.float64))


def test_grad_mode_classification():
    from pytorch_loss import _cabi
    scalar = torch.tensor(2.0)
    mode, g = _cabi.grad_mode_of(scalar.expand(2, 3, 4), (2, 3, 4))
    assert mode == 1 and g.shape == (1,) and float(g) == 2.0
    mode, g = _cabi.grad_mode_of(scalar, (2, 3, 4))
    assert mode == 1 and float(g) == 2.0
    per = torch.arange(24.).reshape(2, 3, 4)
    mode, g = _cabi.grad_mode_of(per.transpose(1, 2).transpose(1, 2), (2, 3, 4))
    assert mode == 2 and g.is_contiguous() and torch.equal(g, per)


def test_shard_bounds_cover_the_batch():
    from pytorch_loss import _sharding
    for n in (0, 1, 7, 8, 16, 17):
        for world in (1, 2, 3, 4, 8):
            spans = [_sharding.shard_bounds(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c and b - a >= d - c >= 0
    with pytest.raises(ValueError):
        _sharding.shard_bounds(4, 2, 2)


def test_combine_mean_and_group_flags():
    from pytorch_loss import _sharding
    sc = torch.tensor([6.0, 4.0], dtype=torch.float64)
    assert float(_sharding.combine_mean(sc)) == 1.5
    assert torch.isnan(_sharding.combine_mean(torch.zeros(2, dtype=torch.float64)))
    assert not _sharding.group_is_active(None)
    with pytest.raises(RuntimeError):
        _sharding.group_is_active(True)          # no process group initialised here
    with pytest.raises(RuntimeError):
        _sharding.allreduce_sum_count(torch.zeros(3, dtype=torch.float64), None)


def test_ohem_oracle_rule():
    """The oracle's relabelling on a hand-made case: the n_min hardest always stay, pixels at or
    below the threshold stay, ignored pixels score 1 and stay ignored."""
    import torch
    from oracle import ohem as OH
    logits = torch.zeros(1, 2, 1, 6)
    # softmax score of class 0 per pixel: sigmoid(x0 - x1)
    logits[0, 0, 0] = torch.tensor([-3.0, -1.0, 0.0, 1.0, 3.0, 5.0])
    labels = torch.tensor([[[0, 0, 0, 0, 0, 255]]])
    new, scores = OH.score_ohem_label(logits, labels, 255, 0.6, 0)
    assert new.tolist() == [[[0, 0, 0, 255, 255, 255]]]          # scores .05 .27 .5 | .73 .95, ignored
    new, _ = OH.score_ohem_label(logits, labels, 255, 0.1, 3)
    assert new.tolist() == [[[0, 0, 0, 255, 255, 255]]]          # threshold keeps 1, n_min keeps 3
    new, _ = OH.score_ohem_label(logits, labels, 255, 0.1, 6)
    assert new.tolist() == labels.tolist()                       # n_min >= pixels: unchanged
    assert float(scores[0, 0, 5]) == 1.0
