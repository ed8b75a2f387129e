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

    def workspace(self):
        """The reduction workspace of the current stream with this context attached."""
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
