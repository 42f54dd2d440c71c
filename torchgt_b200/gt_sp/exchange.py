"""The Ulysses head<->sequence all-to-all: up to three tensors in ONE collective.

Rank r splits each input into P chunks along ``scatter_idx``, chunk r' goes to rank r', and what
arrives is concatenated along ``gather_idx`` (gt_sp/layer.py:30-49).  CUDA tensors are re-laid out by
the library's copy kernels into a peer-major staging buffer, exchanged with one
``all_to_all_single`` (NCCL over NVLink), and laid out again on arrival.  Host tensors (gloo ranks in
the multi-rank logic tests) take the same route with tensor views instead of kernels.
"""
from __future__ import annotations

import math
from typing import List, Sequence

import torch
import torch.distributed as dist
from torch import Tensor

from .. import _cabi
from . import p2p
from .initialize import get_sequence_parallel_world_size
from .utils import _elem


def _apply_alias(x: Tensor, alias_rows: Tensor) -> Tensor:
    """Rows of a [b, rows, width] tensor listed in alias_rows take the value of row 0 (new tensor)."""
    lib = _cabi.load()
    y = x.clone(memory_format=torch.contiguous_format)
    dtype, mult = _elem(y)
    b, rows, w = y.shape
    _cabi.check(lib.tgt_global_rows_broadcast(y.data_ptr(), alias_rows.data_ptr(), alias_rows.numel(), b, rows,
                                              w * mult, dtype, torch.cuda.current_stream(y.device).cuda_stream))
    return y


def _exchange_peer(px, xs: Sequence[Tensor], s: int, g: int, world: int, alias_rows) -> List[Tensor]:
    x0 = xs[0]
    shape = list(x0.shape)
    es = x0.element_size()
    chunk = shape.copy()
    chunk[s] //= world
    out_shape = chunk.copy()
    out_shape[g] *= world
    outer_s = math.prod(shape[:s])
    width_s_bytes = chunk[s] * math.prod(shape[s + 1:]) * es
    width_g_bytes = math.prod(chunk[g:]) * es
    alias_row_bytes = math.prod(shape[2:]) * es if alias_rows is not None else 0
    return px.exchange(xs, out_shape, outer_s, width_s_bytes, width_g_bytes, alias_rows, alias_row_bytes)


def _peer_eligible(xs: Sequence[Tensor], s: int, g: int, world: int) -> bool:
    x0 = xs[0]
    shape = list(x0.shape)
    es = x0.element_size()
    width_s_bytes = (shape[s] // world) * math.prod(shape[s + 1:]) * es
    chunk = shape.copy()
    chunk[s] //= world
    width_g_bytes = math.prod(chunk[g:]) * es
    return width_s_bytes % 16 == 0 and width_g_bytes % 16 == 0 and x0.numel() > 0


def _exchange_cuda(group, xs: Sequence[Tensor], s: int, g: int, world: int) -> List[Tensor]:
    lib = _cabi.load()
    x0 = xs[0]
    shape = list(x0.shape)
    n_t = len(xs)
    dtype, mult = _elem(x0)
    stream = torch.cuda.current_stream(x0.device).cuda_stream
    chunk = shape.copy()
    chunk[s] //= world
    per_peer = math.prod(chunk)
    outer_s = math.prod(shape[:s])                      # rows in front of the scatter axis
    width_s = chunk[s] * math.prod(shape[s + 1:])       # elements one peer gets from each such row
    out_shape = chunk.copy()
    out_shape[g] *= world
    outer_g = math.prod(chunk[:g])
    width_g = math.prod(chunk[g:])
    ptrs = [t.data_ptr() for t in xs] + [None] * (3 - n_t)

    if n_t == 1 and outer_s == 1:
        send = x0.reshape(world, per_peer)              # already peer-major
    else:
        send = torch.empty((world, n_t * per_peer), dtype=x0.dtype, device=x0.device)
        _cabi.check(lib.tgt_a2a_pack_heads(ptrs[0], ptrs[1], ptrs[2], n_t, send.data_ptr(), 1, outer_s,
                                           width_s * mult, world, dtype, stream))
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    if n_t == 1 and outer_g == 1:
        return [recv.view(out_shape)]                   # arrival order is the output order
    outs = [torch.empty(out_shape, dtype=x0.dtype, device=x0.device) for _ in range(n_t)]
    optrs = [t.data_ptr() for t in outs] + [None] * (3 - n_t)
    _cabi.check(lib.tgt_a2a_unpack_heads(recv.data_ptr(), n_t, optrs[0], optrs[1], optrs[2], 1, outer_g,
                                         width_g * mult, world, dtype, stream))
    return outs


def _exchange_host(group, xs: Sequence[Tensor], s: int, g: int, world: int) -> List[Tensor]:
    send = torch.stack([torch.stack(torch.tensor_split(x, world, dim=s)) for x in xs], dim=1).contiguous()
    recv = torch.empty_like(send)                       # [world, n_t, *chunk]
    dist.all_to_all_single(recv, send, group=group)
    outs = []
    for t in range(len(xs)):
        parts = recv[:, t]                              # [world, *chunk]
        outs.append(torch.cat(list(parts.unbind(0)), dim=g).contiguous())
    return outs


def _exchange(group, xs: Sequence[Tensor], s: int, g: int, alias_rows=None) -> List[Tensor]:
    """``alias_rows`` (device int32 indices into dim 1 of 3-D inputs, or None): those rows are sent with
    the value of row 0, i.e. copy_global_token0 (gt_sp/utils.py:817-838) applied on the way out."""
    world = get_sequence_parallel_world_size()
    xs = [x.contiguous() for x in xs]
    if alias_rows is not None and (len(xs) != 1 or xs[0].dim() != 3 or s % 3 != 1):
        raise ValueError("alias rows need a single [b, rows, width] tensor scattered along dim 1")
    if world == 1:
        return [_apply_alias(xs[0], alias_rows)] if alias_rows is not None else list(xs)
    first = xs[0]
    nd = first.dim()
    s, g = s % nd, g % nd
    if s == g:
        raise ValueError("scatter_idx and gather_idx must differ")
    for x in xs:
        if x.shape != first.shape or x.dtype != first.dtype or x.device != first.device:
            raise ValueError("tensors exchanged together must share shape, dtype and device")
    if first.shape[s] % world != 0:
        raise ValueError(f"dim {s} of size {first.shape[s]} is not divisible by the world size {world}")
    if first.is_cuda:
        px = p2p.peer_exchange_for(group, first.device) if _peer_eligible(xs, s, g, world) else None
        if px is not None:
            return _exchange_peer(px, xs, s, g, world, alias_rows)
        if alias_rows is not None:
            xs = [_apply_alias(xs[0], alias_rows)]
        return _exchange_cuda(group, xs, s, g, world)
    if alias_rows is not None:
        raise ValueError("alias rows are a CUDA-path feature")
    return _exchange_host(group, xs, s, g, world)


class _SeqAllToAllMany(torch.autograd.Function):
    @staticmethod
    def forward(ctx, group, scatter_idx: int, gather_idx: int, alias_rows, *tensors: Tensor):
        ctx.group, ctx.scatter_idx, ctx.gather_idx = group, scatter_idx, gather_idx
        ctx.alias_rows = alias_rows
        return tuple(_exchange(group, tensors, scatter_idx, gather_idx, alias_rows))

    @staticmethod
    def backward(ctx, *grads: Tensor):
        back = _SeqAllToAllMany.apply(ctx.group, ctx.gather_idx, ctx.scatter_idx, None, *grads)
        if ctx.alias_rows is not None:
            # gradient of "listed rows := row 0": row 0 collects the listed rows' gradients, they get 0
            lib = _cabi.load()
            dx = back[0]
            if any(dx.data_ptr() == g.data_ptr() for g in grads):
                # the exchange was the identity (one rank): the reduction below edits in place, and
                # autograd's gradient buffer may be shared with other branches
                dx = dx.clone()
                back = (dx,) + tuple(back[1:])
            if dx.dtype not in (torch.float32, torch.bfloat16):
                raise TypeError("alias rows support float32 and bfloat16 gradients")
            b, rows, w = dx.shape
            code = _cabi.TGT_F32 if dx.dtype == torch.float32 else _cabi.TGT_BF16
            _cabi.check(lib.tgt_global_rows_reduce(dx.data_ptr(), ctx.alias_rows.data_ptr(), ctx.alias_rows.numel(),
                                                   b, rows, w, code,
                                                   torch.cuda.current_stream(dx.device).cuda_stream))
        return (None, None, None, None, *back)


def seq_all_to_all_many(group, tensors: Sequence[Tensor], scatter_idx: int, gather_idx: int,
                        alias_rows=None) -> List[Tensor]:
    """Exchange up to three same-shaped tensors with one transfer; differentiable."""
    if not 1 <= len(tensors) <= 3:
        raise ValueError("between one and three tensors can share an exchange")
    return list(_SeqAllToAllMany.apply(group, scatter_idx, gather_idx, alias_rows, *tensors))
