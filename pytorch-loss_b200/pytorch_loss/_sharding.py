"""Batch sharding of the fused losses across ranks (one process per GPU).

Pixels are independent, so a loss over a batch split along N only couples the ranks
through the final scalar: reduction='mean' divides the global loss sum by the global
number of valid pixels.  Each rank's forward kernel leaves `[sum, count]` as two
float64 in device memory; `allreduce_sum_count` adds them over the process group
with ONE 16-byte all-reduce (NCCL on GPUs, gloo in the CPU tests).  The backward
kernels read the reduced count from that same device buffer, so no host
synchronisation sits between the collective and the backward launch.

The result equals the single-process loss on the concatenated batch; note that
this is not what DistributedDataParallel over per-rank means gives when ranks hold
different numbers of ignored pixels (mean of local means).
"""
import torch
import torch.distributed as dist


def group_is_active(group):
    """True when `group` asks for cross-rank reduction and a process group exists."""
    if group is None or group is False:
        return False
    if not dist.is_available() or not dist.is_initialized():
        raise RuntimeError("a process group was requested but torch.distributed is not initialised")
    return True


def resolve_group(group):
    """`True` means the default (world) group; otherwise a ProcessGroup object."""
    return None if group is True else group


def allreduce_sum_count(sum_count, group):
    """In-place SUM all-reduce of a 2-element float64 tensor `[loss_sum, n_valid]`."""
    if sum_count.dtype != torch.float64 or sum_count.numel() != 2:
        raise RuntimeError("expected a 2-element float64 tensor [sum, count]")
    dist.all_reduce(sum_count, op=dist.ReduceOp.SUM, group=resolve_group(group))
    return sum_count


def shard_bounds(n_items, world_size, rank):
    """Even split of `n_items` batch items: rank r owns [lo, hi).  The first
    `n_items % world_size` ranks take one extra item."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError("bad rank %d / world size %d" % (rank, world_size))
    base, extra = divmod(n_items, world_size)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    return lo, hi


def combine_mean(sum_count):
    """loss = sum / count as a 0-dim float32 tensor (NaN when count == 0, as the
    reference's `losses.sum() / n_valid`)."""
    return (sum_count[0] / sum_count[1]).to(torch.float32)
