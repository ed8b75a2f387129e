"""In-kernel cross-GPU reduction of `[sum, count]` for losses sharded over the batch.

With one process per GPU on one node, the reducing forward kernels can add their partial
sums across the ranks themselves (plain stores into peer-mapped slots + a bounded wait, see
`include/b200loss.h`, "cross-GPU sum"), which replaces the 16-byte NCCL all-reduce between
the forward and the backward kernel and the small kernels that followed it.

`get_exchange(group, device)` sets this up once per (group, device):
  * every rank allocates its slot array and a call counter, and exports the slot array
    through CUDA IPC (`b200_ipc_export`);
  * the 64-byte handles travel through `all_gather_object`; each rank opens its peers' arrays
    with its own device current (`b200_ipc_open`), which maps them for its kernels;
  * all ranks agree (one MIN all-reduce) that the set-up worked everywhere; otherwise
    every rank falls back to the NCCL path.
Set `B200_LOSS_P2P=0` to keep the NCCL path.
"""
import os
import struct
import threading

import torch
import torch.distributed as dist

from . import _cabi
from . import _sharding

MAX_RANKS = 16
DEFAULT_POLL_LIMIT = 1 << 20          # polls of ~1 us each: gives up after roughly a second

_contexts = {}
_lock = threading.Lock()


class Exchange:
    """Device-side context of one (process group, device) plus the workspaces attached to it."""

    def __init__(self, device, world, rank, local_slots, peer_slots, poll_limit=DEFAULT_POLL_LIMIT):
        lib = _cabi.load_library()
        self.device, self.world, self.rank = device, world, rank
        self.local_slots = local_slots              # keeps the shared allocation alive
        self.peer_slots = peer_slots                # rank -> device address of that rank's array here
        self.seq = torch.zeros(8, dtype=torch.int64, device=device)   # the call counter (eight words reserved)
        ptrs = [0] * MAX_RANKS
        for p in range(world):
            ptrs[p] = local_slots.data_ptr() if p == rank else int(peer_slots[p])
        blob = struct.pack("<iiIIQ%dQ" % MAX_RANKS, world, rank, poll_limit, 0, self.seq.data_ptr(), *ptrs)
        assert len(blob) == int(lib.b200_exchange_ctx_bytes())
        self.ctx = torch.frombuffer(bytearray(blob), dtype=torch.uint8).to(device)
        self._workspaces = {}
        # a loss sum that a fused step has posted to the peers but nobody has collected yet:
        # (record, workspace, denom_state or None, correction or None)
        self.pending = None

    def defer(self, record, workspace, denom_state=None, correction=None):
        self.pending = (record, workspace, denom_state, correction)

    def take_pending(self, record):
        """The pending entry if it belongs to `record` (then it is cleared), else None."""
        p = self.pending
        if p is not None and p[0] is record:
            self.pending = None
            return p
        return None

    def finish_pending(self):
        """Completes a deferred record now (one small kernel): before the next exchange of this
        context, or when the loss is read ahead of backward."""
        p, self.pending = self.pending, None
        if p is None:
            return
        rec, ws, state, corr = p
        with torch.cuda.device(self.device):
            _cabi.check(_cabi.load_library().b200_exchange_finish(
                _cabi.ptr(ws), _cabi.ptr(rec), _cabi.ptr(state), _cabi.ptr(corr), _cabi.stream_ptr(self.device)))

    def workspace(self):
        """The reduction workspace of the current stream with this context attached.  Asking for
        it announces a new exchange: a deferred one is completed first."""
        self.finish_pending()
        stream = torch.cuda.current_stream(self.device)
        ws = self._workspaces.get(stream.cuda_stream)
        if ws is None:
            lib = _cabi.load_library()
            ws = torch.zeros(int(lib.b200_reduce_workspace_bytes()), dtype=torch.uint8, device=self.device)
            with torch.cuda.device(self.device):
                _cabi.check(lib.b200_reduce_attach_exchange(_cabi.ptr(ws), _cabi.ptr(self.ctx),
                                                            _cabi.stream_ptr(self.device)))
            self._workspaces[stream.cuda_stream] = ws
        return ws


class DeferredLoss(torch.Tensor):
    """The loss a sharded fused step returns while its cross-GPU sum is still in flight: the step's
    kernel has posted this rank's sums and left; backward's first kernel collects the peers' (so
    the wait overlaps the launch in between).  Anything that reads the VALUE before backward --
    `.item()`, `float()`, printing, arithmetic -- first completes the record with one small
    kernel; `backward()` and attribute reads (shape, dtype, grad_fn) do not.  Results of
    operations on it are plain tensors."""

    @staticmethod
    def wrap(tensor, exchange):
        out = tensor.as_subclass(DeferredLoss)
        out._b200_exchange = exchange
        return out

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        reads_value = func is not torch.Tensor.backward and getattr(func, "__name__", "") != "__get__"
        if reads_value:
            from torch.utils._pytree import tree_leaves
            for a in tree_leaves((args, kwargs)):
                ex = getattr(a, "_b200_exchange", None) if isinstance(a, DeferredLoss) else None
                if ex is not None:
                    ex.finish_pending()
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **kwargs)


def defer_enabled():
    """B200_LOSS_DEFER=0 keeps the wait for the peers' sums inside the step's own kernel."""
    return os.environ.get("B200_LOSS_DEFER", "1") != "0"


def local_exchange_for_tests(device, world, rank, poll_limit):
    """A context whose 'peers' are local buffers nobody writes: used to check that the bounded
    wait gives up and reports through the status word."""
    lib = _cabi.load_library()
    nbytes = int(lib.b200_exchange_slot_bytes(world))
    local = torch.zeros(nbytes, dtype=torch.uint8, device=device)
    stand_ins = [torch.zeros(nbytes, dtype=torch.uint8, device=device) for p in range(world) if p != rank]
    peers = {p: t.data_ptr() for p, t in zip([q for q in range(world) if q != rank], stand_ins)}
    ex = Exchange(device, world, rank, local, peers, poll_limit)
    ex.stand_ins = stand_ins                        # keep them alive
    return ex


def _build(group, device):
    import ctypes
    pg = _sharding.resolve_group(group)
    world, rank = dist.get_world_size(pg), dist.get_rank(pg)
    ok, handle, local = 1, None, None
    lib = _cabi.load_library()
    try:
        if world > MAX_RANKS or os.environ.get("B200_LOSS_P2P", "1") == "0" or dist.get_backend(pg) != "nccl":
            raise RuntimeError("peer exchange not applicable")
        nbytes = int(lib.b200_exchange_slot_bytes(world))
        local = torch.zeros(max(nbytes, 4096), dtype=torch.uint8, device=device)
        torch.cuda.synchronize(device)
        raw = ctypes.create_string_buffer(64)
        offset = ctypes.c_uint64(0)
        with torch.cuda.device(device):
            _cabi.check(lib.b200_ipc_export(_cabi.ptr(local), raw, ctypes.byref(offset)))
        handle = (bytes(raw.raw), int(offset.value))
    except Exception:                      # noqa: BLE001  any failure -> collective fallback, decided below
        ok, handle = 0, None
    handles = [None] * world
    dist.all_gather_object(handles, (ok, handle), group=pg)
    peers, exchange = {}, None
    if ok and all(h[0] for h in handles):
        try:
            with torch.cuda.device(device):            # the handle must be opened with MY device current
                for p, (_, (raw_bytes, off)) in enumerate(handles):
                    if p != rank:
                        mapped = ctypes.c_void_p(0)
                        _cabi.check(lib.b200_ipc_open(ctypes.create_string_buffer(raw_bytes, 64), off,
                                                      ctypes.byref(mapped)))
                        peers[p] = int(mapped.value)
            exchange = Exchange(device, world, rank, local, peers)
            torch.cuda.synchronize(device)
        except Exception:                  # noqa: BLE001
            ok, exchange = 0, None
    else:
        ok = 0
    flag = torch.tensor([ok], dtype=torch.int32, device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=pg)
    if int(flag.item()) == 0:
        return None
    # nobody may start exchanging before every rank has zeroed and published its slots
    dist.barrier(group=pg)
    return exchange


def get_exchange(group, device):
    """The Exchange of (group, device), or None when the NCCL path must be used.  Collective:
    the first call per group must be made by all ranks."""
    if not _sharding.group_is_active(group):
        return None
    pg = _sharding.resolve_group(group)
    if dist.get_world_size(pg) == 1:
        return None
    key = (id(pg) if pg is not None else 0, device.index)
    with _lock:
        if key not in _contexts:
            _contexts[key] = _build(group, device)
        return _contexts[key]


def wrap_if_deferred(loss, group, like):
    """`loss` as a DeferredLoss when the step that produced it left its cross-GPU sum pending."""
    if not like.is_cuda or not _sharding.group_is_active(group):
        return loss
    ex = get_exchange(group, like.device)
    if ex is not None and ex.pending is not None:
        return DeferredLoss.wrap(loss, ex)
    return loss
