"""Two CPU ranks over gloo: the host-side sharding logic of the losses.

The kernels need a GPU, so the per-rank `[sum, count]` pairs come from the CPU oracle here; what
is under test is everything between the kernels of different ranks: the 16-byte all-reduce, the
combined mean, its equality with the single-process loss of the concatenated batch (which is NOT
the mean of per-rank means when ranks hold different numbers of ignored pixels), the gradient
rule of the Lovasz all-reduce Function, and what happens when a rank never shows up.
"""
import datetime
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG_PARENT, ROOT


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _setup(rank, world, port, timeout_s=60):
    for p in (ROOT, PKG_PARENT):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=timeout_s))


def _inputs():
    g = torch.Generator().manual_seed(99)
    logits = torch.randn(6, 7, 5, 4, generator=g)
    labels = torch.randint(0, 7, (6, 5, 4), generator=g)
    labels[0] = 255                      # rank 0's shard is mostly ignored: counts differ per rank
    labels[1, :3] = 255
    return logits, labels


def _worker_mean(rank, world, port, out):
    _setup(rank, world, port)
    from pytorch_loss import _sharding
    from oracle import losses as O
    logits, labels = _inputs()
    lo, hi = _sharding.shard_bounds(logits.shape[0], world, rank)
    res = {}
    for name, fn in (("lsr", lambda x, y, r: O.label_smooth_ce(x, y, 0.1, 255, r)),
                     ("lmargin", lambda x, y, r: O.large_margin_softmax(x, y, 0.3, 255, r))):
        local_sum, _ = fn(logits[lo:hi], labels[lo:hi], "sum")
        n_valid = (labels[lo:hi] != 255).sum()
        pair = torch.stack([local_sum.double(), n_valid.double()])
        assert _sharding.group_is_active(True)
        _sharding.allreduce_sum_count(pair, True)
        got = _sharding.combine_mean(pair)
        want, want_grad = fn(logits, labels, "mean")
        # gradient of the global mean on this shard = local 'sum' gradient / global count
        _, gsum = fn(logits[lo:hi], labels[lo:hi], "sum")
        res[name] = (float(got), float(want), float((gsum / pair[1] - want_grad[lo:hi]).abs().max()),
                     float(fn(logits[lo:hi], labels[lo:hi], "mean")[0]))
    if rank == 0:
        torch.save(res, out)
    dist.destroy_process_group()


def test_global_mean_equals_concatenated_batch(tmp_path):
    out = str(tmp_path / "res.pt")
    mp.spawn(_worker_mean, args=(2, _free_port(), out), nprocs=2, join=True)
    res = torch.load(out)
    for name, (got, want, gerr, local_mean) in res.items():
        assert abs(got - want) <= 1e-6 * abs(want), (name, got, want)
        assert gerr <= 1e-7, (name, gerr)
        assert abs(local_mean - want) > 1e-3     # the local mean is a different number


def _worker_lovasz_fn(rank, world, port, out):
    _setup(rank, world, port)
    from pytorch_loss.lovasz_softmax import _AllReduceSumCount
    local = torch.tensor([1.5 + rank, 4.0], dtype=torch.float64, requires_grad=True)
    tot = _AllReduceSumCount.apply(local, True)
    (tot[0] / tot[1]).backward()
    if rank == 0:
        torch.save((tot.detach(), local.grad), out)
    dist.destroy_process_group()


def test_allreduce_function_forward_and_gradient(tmp_path):
    out = str(tmp_path / "fn.pt")
    mp.spawn(_worker_lovasz_fn, args=(2, _free_port(), out), nprocs=2, join=True)
    tot, grad = torch.load(out)
    assert tot.tolist() == [4.0, 8.0]                    # (1.5 + 2.5, 4 + 4)
    assert grad.tolist() == [1.0 / 8.0, -4.0 / 64.0]     # d(sum/count) wrt this rank's pair


def _worker_missing_peer(rank, world, port, out):
    # rank 1 never joins: rank 0 must get an error from the rendezvous, not hang
    if rank == 1:
        return
    try:
        _setup(rank, world, port, timeout_s=3)
        ok = "joined"
    except Exception as exc:   # noqa: BLE001  any rendezvous failure is the expected outcome
        ok = "error: " + type(exc).__name__
    with open(out, "w") as fh:
        fh.write(ok)


def test_missing_rank_surfaces_as_error(tmp_path):
    out = str(tmp_path / "missing.txt")
    mp.spawn(_worker_missing_peer, args=(2, _free_port(), out), nprocs=2, join=True)
    assert open(out).read().startswith("error")


def test_process_group_flag_without_init_raises():
    from pytorch_loss import _sharding
    with pytest.raises(RuntimeError):
        _sharding.group_is_active(True)
