"""Ulysses sequence-parallel attention layers with global-token handling (Graphormer family).

Class and function names, constructor arguments and forward signatures follow the reference's
gt_sp/layer.py so its models can import these in place of the originals.  Differences that do not
change results: q, k and v travel in one all-to-all instead of three, the index list of the global
token slots stays on the GPU, and with a single rank the exchange is skipped instead of copied.
"""
from __future__ import annotations

from typing import Any, Tuple

import torch
import torch.distributed as dist
from torch import Tensor
from torch.nn import Module

from . import fused, p2p
from .exchange import _exchange, seq_all_to_all_many
from .initialize import (get_global_token_rows_on, get_last_batch_flag, get_sequence_parallel_group,
                         get_sequence_parallel_rank, get_sequence_parallel_world_size)
from .utils import (copy_global_token0, extend_global_token, extend_global_token0, merge_global_token,
                    merge_global_token0)


class _SeqAllToAll(torch.autograd.Function):
    """``_SeqAllToAll.apply(group, input, scatter_idx, gather_idx)`` — gt_sp/layer.py:30-49."""

    @staticmethod
    def forward(ctx: Any, group, input: Tensor, scatter_idx: int, gather_idx: int) -> Tensor:
        ctx.group, ctx.scatter_idx, ctx.gather_idx = group, scatter_idx, gather_idx
        return _exchange(group, [input], scatter_idx, gather_idx)[0]

    @staticmethod
    def backward(ctx: Any, *grad_output: Tensor) -> Tuple[None, Tensor, None, None]:
        return (None, _SeqAllToAll.apply(ctx.group, *grad_output, ctx.gather_idx, ctx.scatter_idx), None, None)


class _SeqGather(torch.autograd.Function):
    """All-gather along ``gather_idx`` in forward, keep the own slice of dim 1 in backward
    (gt_sp/layer.py:52-96).  With one rank both directions are the identity; the reference's backward
    returns a single value there and autograd rejects it, this one returns the (grad, None) pair."""

    @staticmethod
    def forward(ctx, input_: Tensor, gather_idx: int) -> Tensor:
        world = get_sequence_parallel_world_size()
        ctx.world, ctx.rank, ctx.gather_idx = world, get_sequence_parallel_rank(), gather_idx
        if world == 1:
            return input_
        input_ = input_.contiguous()
        parts = [torch.empty_like(input_) for _ in range(world)]
        dist.all_gather(parts, input_, group=get_sequence_parallel_group())
        return torch.cat(parts, dim=gather_idx).contiguous()

    @staticmethod
    def backward(ctx, grad_output: Tensor):
        if ctx.world == 1:
            return grad_output, None
        size = grad_output.size(1) // ctx.world
        return grad_output.narrow(1, ctx.rank * size, size).contiguous(), None


class _SeqScatter(torch.autograd.Function):
    """Keep this rank's slice of dim 1 (heads) in forward, all-gather the gradient along dim 1 in
    backward (gt_sp/layer.py:99-139)."""

    @staticmethod
    def forward(ctx, input_: Tensor) -> Tensor:
        world, rank = get_sequence_parallel_world_size(), get_sequence_parallel_rank()
        if input_.size(1) % world != 0:
            raise ValueError(f"dim 1 of size {input_.size(1)} is not divisible by {world} ranks")
        size = input_.size(1) // world
        return input_.narrow(1, rank * size, size).contiguous()

    @staticmethod
    def backward(ctx, grad_output: Tensor) -> Tensor:
        world = get_sequence_parallel_world_size()
        if world == 1:
            return grad_output
        grad_output = grad_output.contiguous()
        parts = [torch.empty_like(grad_output) for _ in range(world)]
        dist.all_gather(parts, grad_output, group=get_sequence_parallel_group())
        return torch.cat(parts, dim=1).contiguous()


class _UlyssesBase(Module):
    def __init__(self, local_attention: Module, sequence_process_group, scatter_idx: int = 2,
                 gather_idx: int = 1) -> None:
        super().__init__()
        self.local_attn = local_attention
        self.spg = sequence_process_group
        self.scatter_idx = scatter_idx  # heads
        self.gather_idx = gather_idx    # sequence

    exchanges_in_eval = False   # layers that also exchange in evaluation mode set this

    def _peer_exchange(self, query: Tensor, attn_bias, edge_index, attn_type):
        """The peer-memory transport when this call can run as one autograd node (our CoreAttention, CUDA,
        sparse attention without a bias, transport available); else None."""
        from ..attn_module import CoreAttention
        if not isinstance(self.local_attn, CoreAttention):
            return None
        world = get_sequence_parallel_world_size()
        if not fused.eligible(query, attn_bias, edge_index, attn_type, world):
            return None
        return p2p.peer_exchange_for(self.spg, query.device)

    def start_exchange(self, query: Tensor, attn_bias, edge_index, attn_type):
        """Begin moving ``query`` to the peers while the caller computes key and value (models call this
        right after the first projection).  Returns a handle to ``add()`` the later tensors to and to pass
        to ``forward(..., pending=handle)``, or None when this call will not use the peer transport."""
        if not (self.training or self.exchanges_in_eval) or not query.is_cuda:
            return None
        if query.dim() != 4 or not query.is_contiguous():
            return None
        px = self._peer_exchange(query, attn_bias, edge_index, attn_type)
        return fused.PendingPush(px, query) if px is not None else None

    def _single_node(self, query: Tensor, key: Tensor, value: Tensor, attn_bias, edge_index, attn_type,
                     alias: bool, pending=None):
        """Exchange + sparse attention + exchange back as one autograd node over peer memory, or None."""
        px = pending.px if pending is not None else self._peer_exchange(query, attn_bias, edge_index, attn_type)
        if px is None:
            return None
        rows = get_global_token_rows_on(query.device, get_last_batch_flag()) if alias else None
        return fused.ulysses_sparse_attention(px, query, key, value, edge_index, rows, pending)

    def _gather_sequence(self, query: Tensor, key: Tensor, value: Tensor):
        """[b, s/p(+1), H, D] x3 -> [b, s(+p), H/p, D] x3 in one collective."""
        return seq_all_to_all_many(self.spg, [query, key, value], self.scatter_idx, self.gather_idx)

    def _scatter_sequence(self, context: Tensor, alias_rows=None) -> Tensor:
        """[b, s(+p), (H/p) D] -> [b, s/p(+1), H D]; rows listed in alias_rows travel as copies of row 0."""
        return seq_all_to_all_many(self.spg, [context], self.gather_idx, self.scatter_idx, alias_rows)[0]


class DistributedAttention(_UlyssesBase):
    """gt_sp/layer.py:142-218: the P copies of the global token are averaged into one row placed LAST;
    the bias is all-gathered along the sequence.  Exchange only in training mode."""

    def forward(self, query: Tensor, key: Tensor, value: Tensor, attn_bias: Tensor, *args: Any) -> Tensor:
        if not self.training:
            return self.local_attn(query, key, value, attn_bias, *args)
        q, k, v = (merge_global_token(t, merge_dim=1) for t in self._gather_sequence(query, key, value))
        bias = merge_global_token(_SeqGather.apply(attn_bias, self.gather_idx), merge_dim=1)
        context = self.local_attn(q, k, v, bias, *args)
        return self._scatter_sequence(extend_global_token(context, extend_dim=1))


class DistributedAttentionGlobal0(_UlyssesBase):
    """gt_sp/layer.py:221-301: as above with the merged global token at row 0 and an optional bias."""

    def forward(self, query: Tensor, key: Tensor, value: Tensor, attn_bias: Tensor, edge_index: Tensor,
                *args: Any) -> Tensor:
        if not self.training:
            return self.local_attn(query, key, value, attn_bias, edge_index, *args)
        q, k, v = (merge_global_token0(t, merge_dim=1) for t in self._gather_sequence(query, key, value))
        bias = attn_bias
        if bias is not None:
            bias = merge_global_token0(_SeqGather.apply(bias, self.gather_idx), merge_dim=1)
        context = self.local_attn(q, k, v, bias, edge_index, *args)
        return self._scatter_sequence(extend_global_token0(context, extend_dim=1))


class DistributedAttentionLocalBias(_UlyssesBase):
    """gt_sp/layer.py:304-375: every rank holds the full bias and keeps its head slice; the exchange
    runs in training and evaluation alike."""

    def forward(self, query: Tensor, key: Tensor, value: Tensor, attn_bias: Tensor, edge_index: Tensor,
                *args: Any) -> Tensor:
        q, k, v = (merge_global_token0(t, merge_dim=1) for t in self._gather_sequence(query, key, value))
        bias = _SeqScatter.apply(attn_bias) if attn_bias is not None else None
        context = self.local_attn(q, k, v, bias, edge_index, *args)
        return self._scatter_sequence(extend_global_token0(context, extend_dim=1))


class DistributedAttentionAll2all(_UlyssesBase):
    """gt_sp/layer.py:401-474: the bias [b, H, s/p+1, s+1] is exchanged too (heads scattered, rows
    gathered) and its global-token rows merged."""

    def forward(self, query: Tensor, key: Tensor, value: Tensor, attn_bias: Tensor, edge_index: Tensor,
                *args: Any) -> Tensor:
        q, k, v = (merge_global_token0(t, merge_dim=1) for t in self._gather_sequence(query, key, value))
        bias = attn_bias
        if bias is not None:
            bias = merge_global_token0(_SeqAllToAll.apply(self.spg, bias, 1, 2), merge_dim=2)
        context = self.local_attn(q, k, v, bias, edge_index, *args)
        return self._scatter_sequence(extend_global_token0(context, extend_dim=1))


class DistributedAttentionNoMerge(_UlyssesBase):
    """gt_sp/layer.py:477-550 — the variant the Graphormer models instantiate.  Every rank's copy of
    the global token keeps its own row (row r (L+1) of the gathered sequence); all global-token edges
    point at row 0, and after attention row 0's output is copied into the other slots."""

    def forward(self, query: Tensor, key: Tensor, value: Tensor, attn_bias: Tensor, edge_index: Tensor,
                attn_type, *args: Any, pending=None) -> Tensor:
        if not self.training:
            return self.local_attn(query, key, value, attn_bias, edge_index, attn_type, *args)
        out = self._single_node(query, key, value, attn_bias, edge_index, attn_type, alias=True, pending=pending)
        if out is not None:
            return out
        q, k, v = self._gather_sequence(query, key, value)
        bias = attn_bias
        if bias is not None:  # [b, s/p+1, s+1, H] -> [b, s+p, s+1, H/p] -> [b, s+p, s+p, H/p]
            bias = extend_global_token0(_SeqAllToAll.apply(self.spg, bias, 3, 1), extend_dim=2)
        context = self.local_attn(q, k, v, bias, edge_index, attn_type, *args)
        if context.is_cuda:
            # copy_global_token0 folded into the exchange: the slots are filled while the data moves
            rows = get_global_token_rows_on(context.device, get_last_batch_flag())
            return self._scatter_sequence(context, alias_rows=rows)
        context = copy_global_token0(context, extend_dim=1)
        return self._scatter_sequence(context)
