"""Peer-memory transport of the Ulysses exchange (GPUs of one node, NVLink / NVSwitch).

Each rank keeps one landing area in symmetric memory (allocated and exchanged once per process group
through ``torch.distributed._symmetric_memory``, grown on demand); the library's push / barrier / fetch
kernels do the rest (see ``csrc/peer_exchange.cu``).  Selected with ``TGT_EXCHANGE``:

* ``auto`` (default): peer memory when the tensors are CUDA, the group has 2..16 ranks and symmetric
  memory can be set up; otherwise one NCCL ``all_to_all_single`` with pack / unpack kernels;
* ``nccl``: always the collective;   * ``p2p``: peer memory or an error.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist
from torch import Tensor

from .. import _cabi

_GROW_ALIGN = 2 << 20
DEFAULT_SPIN_LIMIT = 60_000_000  # polls of the barrier before it gives up (about a minute)


class PeerExchangeTimeout(RuntimeError):
    pass


class PeerExchange:
    """Landing area + peer table of one (process group, device)."""

    def __init__(self, group, device: torch.device):
        self.group = group
        self.device = device
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.half_bytes = 0
        self.buffer: Optional[Tensor] = None
        self.handle = None
        self.peers = None
        self.status = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.spin_limit = int(os.environ.get("TGT_P2P_SPIN_LIMIT", DEFAULT_SPIN_LIMIT))
        self.control_bytes = int(_cabi.load().tgt_p2p_control_bytes())

    def ensure(self, half_bytes: int) -> None:
        """Make each landing half at least ``half_bytes`` big.  Collective: every rank of the group must
        call it with the same size at the same point (true for the SPMD layers that use it)."""
        if half_bytes <= self.half_bytes:
            return
        import torch.distributed._symmetric_memory as symm_mem
        new_half = max(half_bytes, 2 * self.half_bytes)
        new_half = (new_half + _GROW_ALIGN - 1) // _GROW_ALIGN * _GROW_ALIGN
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)               # nobody is still using the old area
        buf = symm_mem.empty(self.control_bytes + 2 * new_half, dtype=torch.uint8, device=self.device)
        handle = symm_mem.rendezvous(buf, self.group)
        buf.zero_()                            # flags and epoch start at zero
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)               # every area is zeroed before anyone signals
        self.buffer, self.handle, self.half_bytes = buf, handle, new_half
        self.peers = (ctypes.c_void_p * self.world)(*[int(p) for p in handle.buffer_ptrs])

    def check(self) -> None:
        code = int(self.status[0])
        if code != 0:
            self.status[0] = 0
            raise PeerExchangeTimeout(f"rank {self.rank}: peer exchange gave up waiting for rank {code - 1}")

    def exchange(self, xs: Sequence[Tensor], out_shape, outer_s: int, width_s_bytes: int, width_g_bytes: int,
                 alias_rows: Optional[Tensor], alias_row_bytes: int) -> List[Tensor]:
        lib = _cabi.load()
        self.check()
        n_t = len(xs)
        nbytes = xs[0].numel() * xs[0].element_size()
        self.ensure(n_t * nbytes)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        ptrs = [t.data_ptr() for t in xs] + [None] * (3 - n_t)
        n_alias = 0 if alias_rows is None else int(alias_rows.numel())
        # small destination runs (narrow head slices) would become slow sub-128-byte NVLink stores: send
        # each rank's chunk as one block instead and concatenate while fetching
        staged = 1 if width_g_bytes < 128 else 0
        _cabi.check(lib.tgt_p2p_push(ptrs[0], ptrs[1], ptrs[2], n_t, self.peers, self.half_bytes, outer_s,
                                     width_s_bytes, width_g_bytes, self.world, self.rank,
                                     alias_rows.data_ptr() if n_alias else None, n_alias, alias_row_bytes, staged,
                                     stream))
        _cabi.check(lib.tgt_p2p_barrier(self.peers, self.world, self.rank, self.spin_limit,
                                        self.status.data_ptr(), stream))
        outs = [torch.empty(out_shape, dtype=xs[0].dtype, device=self.device) for _ in range(n_t)]
        optrs = [t.data_ptr() for t in outs] + [None] * (3 - n_t)
        _cabi.check(lib.tgt_p2p_fetch(self.buffer.data_ptr(), self.half_bytes, n_t, optrs[0], optrs[1], optrs[2],
                                      nbytes, staged, self.world, width_g_bytes, stream))
        return outs


_exchanges: Dict[tuple, Optional[PeerExchange]] = {}


def mode() -> str:
    m = os.environ.get("TGT_EXCHANGE", "auto").lower()
    if m not in ("auto", "nccl", "p2p"):
        raise ValueError("TGT_EXCHANGE must be auto, nccl or p2p")
    return m


def peer_exchange_for(group, device: torch.device) -> Optional[PeerExchange]:
    """The peer-memory transport of this group, or None when the collective should be used."""
    m = mode()
    if m == "nccl":
        return None
    key = (id(group), device.index)
    if key not in _exchanges:
        px = None
        try:
            world = dist.get_world_size(group)
            if not 2 <= world <= 16:
                raise RuntimeError(f"peer exchange supports 2..16 ranks, the group has {world}")
            if dist.get_backend(group) != "nccl":
                raise RuntimeError("peer exchange needs a CUDA (nccl) process group")
            px = PeerExchange(group, device)
            px.ensure(_GROW_ALIGN)             # set-up (collective) happens here, once
        except Exception as exc:               # symmetric memory not available on this system
            if m == "p2p":
                raise
            px = None
            if os.environ.get("TGT_EXCHANGE_VERBOSE"):
                print(f"torchgt_b200: peer exchange unavailable ({exc!r}); using NCCL all-to-all")
        _exchanges[key] = px
    return _exchanges[key]


def reset_peer_exchanges() -> None:
    _exchanges.clear()
