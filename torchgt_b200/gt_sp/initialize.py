"""Sequence-parallel process state read by the Ulysses layers.

Same getter/setter names as the reference's gt_sp/initialize.py:112-202 so code written against it
keeps working; state lives in one object instead of module globals.  ``initialize_distributed``
(gt_sp/initialize.py:24-66) is reproduced for both ``nccl`` (one process per GPU) and ``gloo``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from datetime import timedelta
from typing import List, Optional

import torch
import torch.distributed as dist


@dataclass
class _SequenceParallelState:
    group: Optional[object] = None
    world_size: Optional[int] = None
    rank: Optional[int] = None
    seq_length: Optional[int] = None
    seq_length_per_rank: Optional[int] = None
    global_token_indices: Optional[List[int]] = None
    global_token_indices_last_batch: Optional[List[int]] = None
    global_token_num: Optional[int] = None
    last_batch: bool = False
    device_rows: dict = field(default_factory=dict)  # cached device copies of the index lists


_state = _SequenceParallelState()


def initialize_distributed(args) -> None:
    """Join the default process group from RANK/WORLD_SIZE and create the sequence-parallel group that
    spans all ranks (the reference is "sp only", gt_sp/initialize.py:64)."""
    if dist.is_initialized():
        args.rank, args.world_size = dist.get_rank(), dist.get_world_size()
    else:
        args.rank, args.world_size = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        backend = getattr(args, "distributed_backend", "nccl")
        if backend == "nccl":
            n_dev = torch.cuda.device_count()
            if n_dev == 0:
                raise RuntimeError("the nccl backend needs at least one GPU")
            local = args.rank % n_dev
            if getattr(args, "local_rank", None) not in (None, local):
                raise RuntimeError("local_rank must equal rank % device_count")
            args.local_rank = local
            torch.cuda.set_device(local)
        minutes = getattr(args, "distributed_timeout_minutes", 10)
        dist.init_process_group(backend=backend, world_size=args.world_size, rank=args.rank,
                                timeout=timedelta(minutes=minutes))
    _state.global_token_num = getattr(args, "num_global_node", 1)
    args.sequence_parallel_size = args.world_size
    initialize_sequence_parallel(args.seq_len, 1, 1, args.sequence_parallel_size)


def initialize_sequence_parallel(seq_length: int, tensor_model_parallel_size: int = 1,
                                 pipeline_model_parallel_size: int = 1,
                                 sequence_parallel_size: Optional[int] = 1) -> None:
    """Create one process group per block of ``sequence_parallel_size`` consecutive ranks
    (gt_sp/initialize.py:69-106).  The tensor/pipeline sizes are accepted and ignored, as there."""
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed is not initialised")
    world = dist.get_world_size()
    sp = world if sequence_parallel_size is None else sequence_parallel_size
    if world % sp != 0:
        raise ValueError(f"world size {world} is not a multiple of sequence_parallel_size {sp}")
    if _state.group is not None:
        raise RuntimeError("sequence parallel group is already initialized")
    me = dist.get_rank()
    _state.seq_length = seq_length
    for first in range(0, world, sp):
        ranks = list(range(first, first + sp))
        group = dist.new_group(ranks)  # every rank must take part in every new_group call
        if me in ranks:
            _state.group, _state.rank, _state.world_size = group, ranks.index(me), sp
            _state.seq_length_per_rank = seq_length // sp


def destroy_sequence_parallel() -> None:
    """Forget all sequence-parallel state (tests create and tear down groups repeatedly)."""
    global _state
    from . import p2p
    p2p.reset_peer_exchanges()    # their symmetric memory and counters belong to the group being forgotten
    _state = _SequenceParallelState()


def sequence_parallel_is_initialized() -> bool:
    return _state.group is not None


def get_sequence_parallel_group():
    if _state.group is None:
        raise RuntimeError("sequence parallel group is not initialized")
    return _state.group


def get_sequence_parallel_world_size() -> int:
    if _state.world_size is not None:
        return _state.world_size
    return dist.get_world_size(group=get_sequence_parallel_group())


def get_sequence_parallel_rank() -> int:
    if _state.rank is not None:
        return _state.rank
    return dist.get_rank(group=get_sequence_parallel_group())


def get_sequence_parallel_src_rank() -> int:
    """Global rank of the first member of this rank's sequence-parallel group."""
    size = get_sequence_parallel_world_size()
    return (dist.get_rank() // size) * size


def get_sequence_length() -> int:
    if _state.seq_length is None:
        raise RuntimeError("sequence length is not initialized")
    return _state.seq_length


def get_sequence_length_per_rank() -> int:
    if _state.seq_length_per_rank is None:
        raise RuntimeError("subsequence length is not initialized")
    return _state.seq_length_per_rank


def set_global_token_num(n: int) -> None:
    _state.global_token_num = n


def get_global_token_num() -> int:
    if _state.global_token_num is None:
        raise RuntimeError("global token num is not initialized")
    return _state.global_token_num


def set_global_token_indices(global_token_indices) -> None:
    _state.global_token_indices = list(global_token_indices)


def set_last_batch_global_token_indices(global_token_indices_last_batch) -> None:
    _state.global_token_indices_last_batch = list(global_token_indices_last_batch)


def get_global_token_indices(last_batch: bool = False):
    if last_batch:
        return _state.global_token_indices_last_batch
    if _state.global_token_indices is None:
        raise RuntimeError("global token indices is not initialized")
    return _state.global_token_indices


def get_global_token_rows_on(device, last_batch: bool = False) -> torch.Tensor:
    """The active index list as an int32 tensor on ``device``, uploaded once and cached (the reference
    rebuilds a LongTensor and uploads it on every layer call, gt_sp/utils.py:836)."""
    indices = tuple(get_global_token_indices(last_batch))
    key = (str(device), indices)
    rows = _state.device_rows.get(key)
    if rows is None:
        if len(_state.device_rows) > 64:
            _state.device_rows.clear()
        rows = torch.tensor(indices, dtype=torch.int32, device=device)
        _state.device_rows[key] = rows
    return rows


def last_batch_flag(last_batch: bool = False) -> None:
    _state.last_batch = bool(last_batch)


def get_last_batch_flag() -> bool:
    return _state.last_batch
