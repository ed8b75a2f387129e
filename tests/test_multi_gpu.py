"""Batch sharded over 2 GPUs (one process each, NCCL): the modules built with
`process_group=True` return the loss of the concatenated batch and its gradient on the local
shard.  Skipped on boxes with fewer than two GPUs."""
import datetime
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG_PARENT, ROOT

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out, p2p):
    for p in (ROOT, PKG_PARENT):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      B200_LOSS_P2P="1" if p2p else "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=120))
    import pytorch_loss as P
    from pytorch_loss import _sharding
    from oracle import losses as O
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(4, 19, 32, 32, generator=g)
    labels = torch.randint(0, 19, (4, 32, 32), generator=g)
    labels[0, :20] = 255                                    # uneven ignore counts across ranks
    flabels = (torch.rand(4, 19, 32, 32, generator=g) < 0.2).float()
    lo, hi = _sharding.shard_bounds(4, world, rank)
    cases = [
        (P.LabelSmoothSoftmaxCEV3(0.1, 'mean', 255, process_group=True), labels,
         O.label_smooth_ce(logits, labels, 0.1, 255, 'mean')),
        (P.LargeMarginSoftmaxV3(0.3, 'mean', 255, process_group=True), labels,
         O.large_margin_softmax(logits, labels, 0.3, 255, 'mean')),
        (P.FocalLossV3(0.25, 2, 'mean', process_group=True), flabels,
         O.focal_loss(logits, flabels, 0.25, 2.0, 'mean')),
        (P.LovaszSoftmaxV3('mean', 255, per_image=True, process_group=True), labels,
         O.lovasz_softmax(logits, labels, 255, 'mean', per_image=True)),
    ]
    errs = []
    for crit, lab, (want_loss, want_grad) in cases:
        x = logits[lo:hi].to(dev).requires_grad_(True)
        loss = crit(x, lab[lo:hi].to(dev))
        loss.backward()
        errs.append((abs(float(loss) - float(want_loss)) / abs(float(want_loss)),
                     float((x.grad.cpu() - want_grad[lo:hi]).abs().max())))
    # run the sharded step a few more times: the exchange alternates between its two slot sets
    crit, lab, (want_loss, _) = cases[0]
    for _ in range(5):
        loss = crit(logits[lo:hi].to(dev), lab[lo:hi].to(dev))
    errs.append((abs(float(loss) - float(want_loss)) / abs(float(want_loss)), 0.0))
    # focal 'mean' divides by a predicted global element count: right on a repeated call, wrong
    # when a rank's shard changes size (the rescale kernel then corrects the gradient), right again
    fcrit = cases[2][0]
    uneven = [(0, 1), (1, 4)] if world == 2 else [_sharding.shard_bounds(4, world, r) for r in range(world)]
    for bounds in ([(lo, hi)] * 2 + [uneven[rank]] * 2 + [(lo, hi)]):
        a, b = bounds
        x = logits[a:b].to(dev).requires_grad_(True)
        loss = fcrit(x, flabels[a:b].to(dev))
        loss.backward()
        want_loss, want_grad = cases[2][2]
        errs.append((abs(float(loss) - float(want_loss)) / abs(float(want_loss)),
                     float((x.grad.cpu() - want_grad[a:b]).abs().max())))
    # A sharded fused step leaves its cross-GPU sum in flight for backward to collect; the loss it
    # returns completes itself when it is read first.  Both orders, for all three losses.
    from pytorch_loss import _p2p as P2P
    for crit, lab, (want_loss, want_grad) in cases[:3]:
        for read_first in (True, False):
            x = logits[lo:hi].to(dev).requires_grad_(True)
            loss = crit(x, lab[lo:hi].to(dev))
            if p2p:
                assert isinstance(loss, P2P.DeferredLoss), type(loss)
            early = float(loss) if read_first else float(want_loss)
            loss.backward()
            errs.append((abs(early - float(want_loss)) / abs(float(want_loss)), 0.0))
            errs.append((abs(float(loss) - float(want_loss)) / abs(float(want_loss)),
                         float((x.grad.cpu() - want_grad[lo:hi]).abs().max())))
            assert type(loss * 2.0) is torch.Tensor
    # Ranks that take different kernels still make the same sequence of exchanges: an EMPTY shard
    # on the last rank (the others hold the whole batch between them), and a rank that needs no
    # gradient (unfused forward) beside ranks that run the fused step.
    if world == 2:
        for crit, lab, (want_loss, want_grad) in cases[:2]:
            a, b = (0, 4) if rank == 0 else (4, 4)
            x = logits[a:b].to(dev).requires_grad_(True)
            loss = crit(x, lab[a:b].to(dev))
            loss.backward()
            gerr = float((x.grad.cpu() - want_grad[a:b]).abs().max()) if b > a else 0.0
            errs.append((abs(float(loss) - float(want_loss)) / abs(float(want_loss)), gerr))
            x = logits[lo:hi].to(dev).requires_grad_(rank == 0)
            if rank == 0:
                loss = crit(x, lab[lo:hi].to(dev))
                loss.backward()
                gerr = float((x.grad.cpu() - want_grad[lo:hi]).abs().max())
            else:
                with torch.no_grad():
                    loss = crit(x, lab[lo:hi].to(dev))
                gerr = 0.0
            errs.append((abs(float(loss) - float(want_loss)) / abs(float(want_loss)), gerr))
    from pytorch_loss import _cabi, _p2p
    _cabi.read_status(dev)
    for ex in _p2p._contexts.values():
        if ex is not None:
            _cabi.check(_cabi.load_library().b200_read_status(_cabi.ptr(ex.workspace()), _cabi.stream_ptr(dev)))
    mode = "p2p" if any(ex is not None for ex in _p2p._contexts.values()) else "nccl"
    torch.save((mode, errs), "%s.%d" % (out, rank))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("p2p", [True, False], ids=["peer_exchange", "nccl_allreduce"])
def test_sharded_losses_match_concatenated_batch(tmp_path, p2p):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    out = str(tmp_path / "errs")
    mp.spawn(_worker, args=(2, _free_port(), out, p2p), nprocs=2, join=True)
    for rank in range(2):
        mode, errs = torch.load("%s.%d" % (out, rank))
        assert mode == ("p2p" if p2p else "nccl"), "the sums went through %s" % mode
        for loss_err, grad_err in errs:
            assert loss_err <= 1e-5, loss_err
            assert grad_err <= 1e-5, grad_err
