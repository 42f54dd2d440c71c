"""Peer-memory transport of the Ulysses exchange (GPUs of one node, NVLink / NVSwitch).

Each rank keeps a small control block and a pool of *slots* in symmetric memory (allocated and exchanged
through ``torch.distributed._symmetric_memory``); the library's push / pull / barrier / fetch kernels do
the rest (see ``csrc/peer_exchange.cu``).  Selected with ``TGT_EXCHANGE``:

* ``auto`` (default): peer memory when the tensors are CUDA, the group has 2..16 ranks and symmetric
  memory can be set up; otherwise one NCCL ``all_to_all_single`` with pack / unpack kernels;
* ``nccl``: always the collective;   * ``p2p``: peer memory or an error.

Slot discipline.  All ranks run the same program, so every rank takes and gives back slots in the same
order and the pools stay identical without any communication.  A slot that was given back can be handed
out again only after one more barrier has been enqueued: by then every rank has finished reading (or
writing) its old content, because a rank announces a barrier only after everything it enqueued before.
New slots are created on demand (a collective set-up step); that cannot happen while a CUDA graph is
being captured, so run one eager step first.

Slots keep the role they were created for: LANDING slots are written by the peers' pushes and read by
their owner; SOURCE slots are written by their owner's kernels and read by the peers' pulls.  With the
roles apart, the first write a training iteration makes to any slot is ordered behind a barrier that
every reader of the old content has already announced (a push at the start of an iteration follows the
previous iteration's last barrier, which the owner announced after its last read; the owner's kernels
write a SOURCE slot only after the first barrier of their own iteration, which every peer announces
after its last pull).  So CUDA graphs that each hold whole iterations of the fused layer can be replayed
in any order.  Graphs that hold bare ``_SeqAllToAll`` exchanges must be replayed in the order they were
captured.
"""
from __future__ import annotations

import ctypes
import os
import weakref
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist
from torch import Tensor

from .. import _cabi

_GRANULE = 2 << 20
DEFAULT_SPIN_LIMIT = 60_000_000  # polls of the barrier before it gives up (about a minute)


LANDING, SOURCE = "landing", "source"   # who writes a slot: the peers' pushes / its owner's kernels


class PeerExchangeTimeout(RuntimeError):
    pass


class Slot:
    """One peer-visible buffer of ``nbytes`` on every rank of the group."""

    def __init__(self, buffer: Tensor, handle, world: int, role: str = LANDING):
        self.buffer = buffer
        self.handle = handle
        self.role = role
        self.nbytes = buffer.numel()
        self.peers = (ctypes.c_void_p * world)(*[int(p) for p in handle.buffer_ptrs])
        self.free_epoch = -1          # barrier count at the moment it was last given back
        self.in_use = False
        self._shifted = {}

    def peers_at(self, offset_bytes: int):
        """Peer table of the slot's addresses ``offset_bytes`` further in (for filling it piece by piece)."""
        if offset_bytes == 0:
            return self.peers
        table = self._shifted.get(offset_bytes)
        if table is None:
            table = (ctypes.c_void_p * len(self.peers))(*[int(p) + offset_bytes for p in self.peers])
            self._shifted[offset_bytes] = table
        return table

    def view(self, offset_bytes: int, shape, dtype: torch.dtype) -> Tensor:
        """This rank's copy of the slot, ``shape`` elements of ``dtype`` starting at ``offset_bytes``."""
        n = 1
        for s in shape:
            n *= int(s)
        size = n * torch.empty((), dtype=dtype).element_size()
        return self.buffer[offset_bytes:offset_bytes + size].view(dtype).view(*shape)


class PeerExchange:
    """Control block + slot pool of one (process group, device)."""

    def __init__(self, group, device: torch.device):
        import torch.distributed._symmetric_memory as symm_mem
        self._symm = symm_mem
        self.group = group
        self.device = device
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.status = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.spin_limit = int(os.environ.get("TGT_P2P_SPIN_LIMIT", DEFAULT_SPIN_LIMIT))
        self.epoch = 0                 # barriers enqueued so far (host count, same on every rank)
        self.slots: List[Slot] = []
        self.side_stream = torch.cuda.Stream(device=device)   # pushes that overlap the caller's own work
        self.trace = None              # list of (label, CUDA event) while a caller measures the phases of a step
        lib = _cabi.load()
        control_bytes = max(int(lib.tgt_p2p_control_bytes()), 256)
        self.control = self._new_symmetric(control_bytes)

    # -- memory ------------------------------------------------------------------------------------
    def _new_symmetric(self, nbytes: int, role: str = LANDING) -> Slot:
        """Collective: every rank of the group allocates ``nbytes`` and learns the peers' addresses."""
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("the peer exchange needs a new slot while a CUDA graph is being captured; "
                               "run one eager step of the same shapes before capturing")
        torch.cuda.synchronize(self.device)
        buf = self._symm.empty(nbytes, dtype=torch.uint8, device=self.device)
        handle = self._symm.rendezvous(buf, self.group)
        buf.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)               # every rank's memory is zeroed before anyone uses it
        return Slot(buf, handle, self.world, role)

    def acquire(self, nbytes: int, role: str = LANDING) -> Slot:
        """A slot of at least ``nbytes`` and of this role that no rank is still using (same choice on
        every rank)."""
        want = (max(int(nbytes), 16) + _GRANULE - 1) // _GRANULE * _GRANULE
        best = None
        for slot in self.slots:
            if slot.role == role and not slot.in_use and slot.free_epoch < self.epoch and slot.nbytes >= want:
                if best is None or slot.nbytes < best.nbytes:
                    best = slot
        if best is None:
            best = self._new_symmetric(want, role)
            self.slots.append(best)
        best.in_use = True
        return best

    def mark(self, label: str) -> None:
        """Record a timing event on the current stream when tracing is on (see ``start_trace``)."""
        if self.trace is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(torch.cuda.current_stream(self.device))
            self.trace.append((label, ev))

    def start_trace(self) -> None:
        self.trace = []
        self.mark("start")

    def stop_trace(self):
        """Milliseconds between consecutive marks, as (label of the phase that ended, ms); waits for the device."""
        torch.cuda.synchronize(self.device)
        marks, self.trace = self.trace, None
        return [(marks[i][0], marks[i - 1][1].elapsed_time(marks[i][1])) for i in range(1, len(marks))]

    def release(self, slot: Slot) -> None:
        slot.in_use = False
        slot.free_epoch = self.epoch

    # -- kernels -----------------------------------------------------------------------------------
    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def push(self, xs: Sequence[Tensor], slot: Slot, outer_s: int, width_s_bytes: int, width_g_bytes: int,
             alias_rows: Optional[Tensor] = None, alias_row_bytes: int = 0, mode: int = _cabi.TGT_PUSH_FINAL,
             offset_bytes: int = 0) -> None:
        """Enqueue the push on the current stream; the tensors land ``offset_bytes`` into the peers' slots."""
        lib = _cabi.load()
        ptrs = [t.data_ptr() for t in xs] + [None] * (3 - len(xs))
        n_alias = 0 if alias_rows is None else int(alias_rows.numel())
        _cabi.check(lib.tgt_p2p_push(ptrs[0], ptrs[1], ptrs[2], len(xs), slot.peers_at(offset_bytes),
                                     slot.nbytes - offset_bytes, outer_s, width_s_bytes, width_g_bytes, self.world,
                                     self.rank, alias_rows.data_ptr() if n_alias else None, n_alias, alias_row_bytes,
                                     mode, self._stream()))

    def pull(self, slot: Slot, outs: Sequence[Tensor], outer: int, rows: int, width_bytes: int,
             alias_rows: Optional[Tensor] = None, offset_bytes: int = 0) -> None:
        """Enqueue the gather of this rank's rows of the tensors that start ``offset_bytes`` into the peers' slots."""
        lib = _cabi.load()
        ptrs = [t.data_ptr() for t in outs] + [None] * (3 - len(outs))
        n_alias = 0 if alias_rows is None else int(alias_rows.numel())
        _cabi.check(lib.tgt_p2p_pull(slot.peers_at(offset_bytes), slot.nbytes - offset_bytes, len(outs), ptrs[0],
                                     ptrs[1], ptrs[2], outer, rows, width_bytes, self.world, self.rank,
                                     alias_rows.data_ptr() if n_alias else None, n_alias, self._stream()))

    def barrier(self) -> None:
        lib = _cabi.load()
        _cabi.check(lib.tgt_p2p_barrier(self.control.peers, self.world, self.rank, self.spin_limit,
                                        self.status.data_ptr(), self._stream()))
        self.epoch += 1

    def fetch(self, slot: Slot, outs: Sequence[Tensor], nbytes: int, staged: int, width_g_bytes: int) -> None:
        lib = _cabi.load()
        ptrs = [t.data_ptr() for t in outs] + [None] * (3 - len(outs))
        _cabi.check(lib.tgt_p2p_fetch(slot.buffer.data_ptr(), slot.nbytes, len(outs), ptrs[0], ptrs[1], ptrs[2],
                                      nbytes, staged, self.world, width_g_bytes, self._stream()))

    # -- failure reporting -------------------------------------------------------------------------
    def check(self, wait: bool = False) -> None:
        """Raise if a barrier of this exchange gave up waiting for a peer.  The kernels of that step ran
        on incomplete data: discard the step.  ``wait=True`` first waits for the device, so that every
        barrier enqueued so far has reported; without it only barriers that already ran are seen."""
        if wait and not torch.cuda.is_current_stream_capturing():
            torch.cuda.synchronize(self.device)
        code = int(self.status[0])
        if code != 0:
            self.status[0] = 0
            raise PeerExchangeTimeout(f"rank {self.rank}: peer exchange gave up waiting for rank {code - 1}; "
                                      "the results of that step are invalid")

    # -- the general all-to-all --------------------------------------------------------------------
    def exchange(self, xs: Sequence[Tensor], out_shape, outer_s: int, width_s_bytes: int, width_g_bytes: int,
                 alias_rows: Optional[Tensor], alias_row_bytes: int) -> List[Tensor]:
        """push -> barrier -> fetch into ordinary tensors (any tensors, any axis pair)."""
        self.check()
        n_t = len(xs)
        nbytes = xs[0].numel() * xs[0].element_size()
        slot = self.acquire(n_t * nbytes)
        # small destination runs (narrow head slices) would become slow sub-128-byte NVLink stores: send
        # each rank's chunk as one block instead and concatenate while fetching
        staged = 1 if width_g_bytes < 128 else 0
        self.push(xs, slot, outer_s, width_s_bytes, width_g_bytes, alias_rows, alias_row_bytes,
                  _cabi.TGT_PUSH_STAGED if staged else _cabi.TGT_PUSH_FINAL)
        self.barrier()
        outs = [torch.empty(out_shape, dtype=xs[0].dtype, device=self.device) for _ in range(n_t)]
        self.fetch(slot, outs, nbytes, staged, width_g_bytes)
        self.release(slot)
        return outs


_exchanges: "weakref.WeakKeyDictionary" = weakref.WeakKeyDictionary()   # group -> {device index: PeerExchange}
_strong: Dict[int, object] = {}   # groups that cannot be weakly referenced are pinned here (id -> group)


def mode() -> str:
    m = os.environ.get("TGT_EXCHANGE", "auto").lower()
    if m not in ("auto", "nccl", "p2p"):
        raise ValueError("TGT_EXCHANGE must be auto, nccl or p2p")
    return m


def _table_for(group) -> dict:
    try:
        return _exchanges.setdefault(group, {})
    except TypeError:                       # not weak-referenceable: keep the group alive with its entry
        _strong[id(group)] = group
        return _exchanges_by_id.setdefault(id(group), {})


_exchanges_by_id: Dict[int, dict] = {}


def peer_exchange_for(group, device: torch.device) -> Optional[PeerExchange]:
    """The peer-memory transport of this group, or None when the collective should be used."""
    m = mode()
    if m == "nccl":
        return None
    table = _table_for(group)
    if device.index not in table:
        px = None
        try:
            world = dist.get_world_size(group)
            if not 2 <= world <= 16:
                raise RuntimeError(f"peer exchange supports 2..16 ranks, the group has {world}")
            if dist.get_backend(group) != "nccl":
                raise RuntimeError("peer exchange needs a CUDA (nccl) process group")
            px = PeerExchange(group, device)     # set-up (collective) happens here, once
        except Exception as exc:               # symmetric memory not available on this system
            if m == "p2p":
                raise
            px = None
            if os.environ.get("TGT_EXCHANGE_VERBOSE"):
                print(f"torchgt_b200: peer exchange unavailable ({exc!r}); using NCCL all-to-all")
        table[device.index] = px
    return table[device.index]


def all_peer_exchanges() -> List[PeerExchange]:
    found = []
    for table in list(_exchanges.values()) + list(_exchanges_by_id.values()):
        found += [px for px in table.values() if px is not None]
    return found


def check_peer_exchanges(wait: bool = True) -> None:
    """Raise ``PeerExchangeTimeout`` if any barrier enqueued so far gave up on a peer.  Call it where the
    program synchronises anyway (end of a step, before the optimizer step); ``wait=True`` waits for the
    device first."""
    for px in all_peer_exchanges():
        px.check(wait=wait)
        wait = False


def reset_peer_exchanges() -> None:
    """Forget every exchange (and with it the symmetric memory it holds).  Every rank must call it at the
    same point, with the device idle."""
    _exchanges.clear()
    _exchanges_by_id.clear()
    _strong.clear()
