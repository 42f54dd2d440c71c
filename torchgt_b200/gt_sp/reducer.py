"""Gradient averaging of the replicated weights across the sequence-parallel ranks.

The reference averages after every backward with one ``div_`` and one ``all_reduce`` per parameter
(main_sp_sparse_node_level.py:204-208: about eighty small collectives per step for the 4-layer
Graphormer) and carries an unfinished per-parameter ``Reducer`` (gt_sp/reducer.py:12-46, "TODO
communicate flatten tensor for high efficiency").  Here all gradients live in ONE flat buffer — every
``param.grad`` is a view into it, so nothing is copied in or out — and one ``all_reduce`` of that buffer,
started from the hook of the last gradient to arrive, runs while the rest of backward finishes.

Same results as the reference loop: each gradient is divided by the number of ranks and then summed
over the ranks; parameters that received no gradient in a step keep ``grad = None`` (so an optimizer
skips them, as it does in the reference).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .initialize import (get_sequence_parallel_group, get_sequence_parallel_src_rank,
                         get_sequence_parallel_world_size, sequence_parallel_is_initialized)


def sync_params_and_buffers(model: torch.nn.Module) -> None:
    """Broadcast every entry of the ``state_dict`` from the first rank of the sequence-parallel group
    (gt_sp/reducer.py:12-16)."""
    for _, param in model.state_dict().items():
        dist.broadcast(param.data, src=get_sequence_parallel_src_rank(), group=get_sequence_parallel_group())


class Reducer:
    """Flat-bucket gradient averager.

        reducer = Reducer(); reducer.init(model)
        for batch in ...:
            reducer.prepare()            # instead of optimizer.zero_grad()
            loss.backward()              # the all-reduce starts when the last gradient has arrived
            reducer.synchronize()        # averaged gradients are in param.grad
            optimizer.step()

    ``reduce(param, name, data)`` of the reference's class is kept: it marks ``param``'s gradient as
    complete, which is what the hooks installed by ``init`` do themselves."""

    def __init__(self, group=None, world_size: Optional[int] = None):
        self._group = group
        self._world = world_size
        self._params: List[torch.nn.Parameter] = []
        self._names: Dict[int, str] = {}
        self._views: List[torch.Tensor] = []
        self._flat: Optional[torch.Tensor] = None
        self._arrived: set = set()
        self._expected: Optional[frozenset] = None   # parameters a step gives gradients to (learnt from the first step)
        self._late = False
        self._work = None
        self._launched = False
        self._hooks = []

    # -- set-up ------------------------------------------------------------------------------------
    def init(self, model: torch.nn.Module) -> "Reducer":
        if self._group is None and sequence_parallel_is_initialized():
            self._group = get_sequence_parallel_group()
        if self._world is None:
            self._world = get_sequence_parallel_world_size() if sequence_parallel_is_initialized() else (
                dist.get_world_size(self._group) if dist.is_initialized() else 1)
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        if not named:
            raise ValueError("the model has no trainable parameters")
        first = named[0][1]
        for _, p in named:
            if p.dtype != first.dtype or p.device != first.device:
                raise ValueError("all trainable parameters must share dtype and device")
        self._params = [p for _, p in named]
        self._names = {id(p): n for n, p in named}
        # every view starts on a 16-byte boundary inside the flat buffer
        align = max(1, 16 // first.element_size())
        offsets, total = [], 0
        for p in self._params:
            offsets.append(total)
            total += (p.numel() + align - 1) // align * align
        self._flat = torch.zeros(total, dtype=first.dtype, device=first.device)
        self._views = [self._flat[o:o + p.numel()].view_as(p) for o, p in zip(offsets, self._params)]
        for p in self._params:
            self._hooks.append(p.register_post_accumulate_grad_hook(self._on_gradient))
        return self

    @property
    def flat_gradients(self) -> torch.Tensor:
        return self._flat

    # -- one step ------------------------------------------------------------------------------------
    def prepare(self) -> None:
        """Zero the flat buffer and point every ``param.grad`` into it (call before backward)."""
        self._flat.zero_()
        for p, view in zip(self._params, self._views):
            p.grad = view
        self._arrived.clear()
        self._work = None
        self._launched = False
        self._late = False

    def _on_gradient(self, param: torch.nn.Parameter) -> None:
        if self._launched and id(param) not in self._arrived:
            self._late = True           # a gradient nobody expected arrived after the all-reduce had started
        self._arrived.add(id(param))
        if self._expected is not None and not self._launched and self._arrived >= self._expected:
            self._launch()

    def reduce(self, param, name=None, data=None) -> None:
        """Reference-compatible entry (gt_sp/reducer.py:36-43): ``param``'s gradient is complete."""
        self._on_gradient(param)

    def _launch(self) -> None:
        self._launched = True
        if self._world > 1:
            self._flat.div_(self._world)
            self._work = dist.all_reduce(self._flat, op=dist.ReduceOp.SUM, group=self._group, async_op=True)

    def synchronize(self) -> None:
        """Wait for the averaged gradients; parameters without a gradient this step get ``grad = None``."""
        if not self._launched:          # first step (arrival count unknown yet) or a step with fewer gradients
            self._launch()
        if self._work is not None:
            self._work.wait()
            self._work = None
        if self._late:
            self._expected = None
            raise RuntimeError("a parameter that had no gradient in the first step received one after the "
                               "gradient all-reduce had started; this step's gradients are not averaged "
                               "correctly (the set of parameters is learnt again from the next step)")
        if self._expected is None:
            self._expected = frozenset(self._arrived)
        for p in self._params:
            if id(p) not in self._arrived:
                p.grad = None

    def average_gradients(self) -> None:
        """For loops that call the averaging explicitly after ``backward`` (as the reference's does)."""
        self.synchronize()

    def remove_hooks(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks = []
