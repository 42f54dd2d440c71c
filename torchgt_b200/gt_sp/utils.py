"""Edge-index construction and global-token bookkeeping around the Ulysses exchange.

Same function names and argument meaning as the reference's gt_sp/utils.py (and the copies in
data/collator_sp_sparse.py); the integer helpers are bit-exact with it for node ids below 2**24 (the
reference takes one floor in float32, see ``adjust_edge_index_nomerge``).
"""
from __future__ import annotations

from typing import List, Sequence

import torch
from torch import Tensor

from .. import _cabi
from .initialize import (get_global_token_indices, get_global_token_rows_on, get_last_batch_flag,
                         get_sequence_parallel_world_size)


# ---- edge-index helpers (host-side batch packing; integer, bit-exact) -----------------------------
def fix_edge_index(x: Tensor, num_node: int) -> Tensor:
    """gt_sp/utils.py:34-50: make room for the virtual node at id 0 (all ids + 1) and connect it to
    and from every node: appended columns are (i -> 0) for i = 1..num_node, then (0 -> i)."""
    nodes = torch.arange(1, num_node + 1, dtype=x.dtype, device=x.device)
    virtual = torch.zeros_like(nodes)
    return torch.cat([x + 1, torch.stack([nodes, virtual]), torch.stack([virtual, nodes])], dim=1)


def adjust_edge_index_nomerge(edge_index: Tensor, sub_seq_len: int) -> Tensor:
    """gt_sp/utils.py:53-58: every rank keeps its own copy of the virtual node in front of its
    ``sub_seq_len`` nodes, so node id i > 0 moves to row i + (i - 1) // sub_seq_len; id 0 stays.

    Integer arithmetic; the reference computes the quotient in float32, which agrees for ids < 2**24."""
    shift = torch.div(edge_index - 1, sub_seq_len, rounding_mode="floor")
    return torch.where(edge_index > 0, edge_index + shift, edge_index)


def flatten_edge_index_nopad(x: Sequence[Tensor], batch_node_num: int) -> Tensor:
    """data/collator_sp_sparse.py:126-133: concatenate the edge lists of a batch of graphs, graph g
    offset by g * batch_node_num, giving one block-diagonal edge list over the flattened batch."""
    return torch.cat([e + g * batch_node_num for g, e in enumerate(x)], dim=1)


# ---- global-token helpers -------------------------------------------------------------------------
def _active_global_rows() -> List[int]:
    return list(get_global_token_indices(last_batch=get_last_batch_flag()))


def split_tensor_along_second_dim(tensor: Tensor, num_partitions: int,
                                  contiguous_split_chunks: bool = False):
    """gt_sp/utils.py:688-716: equal chunks along dim 1."""
    chunks = torch.split(tensor, tensor.size(1) // num_partitions, dim=1)
    if contiguous_split_chunks:
        return tuple(c.contiguous() for c in chunks)
    return chunks


def _split_global(x_layer: Tensor, dim: int):
    rows = _active_global_rows()
    listed = torch.tensor(rows, dtype=torch.long, device=x_layer.device)
    keep = torch.ones(x_layer.size(dim), dtype=torch.bool, device=x_layer.device)
    keep[listed] = False
    rest = torch.index_select(x_layer, dim, keep.nonzero().flatten())
    mean = torch.index_select(x_layer, dim, listed).mean(dim=dim, keepdim=True)
    return mean, rest


def merge_global_token(x_layer: Tensor, merge_dim: int) -> Tensor:
    """gt_sp/utils.py:719-740: replace the per-rank copies of the global token by their mean,
    appended at the END of ``merge_dim``."""
    mean, rest = _split_global(x_layer, merge_dim)
    return torch.cat([rest, mean], dim=merge_dim).contiguous()


def merge_global_token0(x_layer: Tensor, merge_dim: int) -> Tensor:
    """gt_sp/utils.py:743-769: as above with the mean placed at index 0."""
    mean, rest = _split_global(x_layer, merge_dim)
    return torch.cat([mean, rest], dim=merge_dim).contiguous()


def extend_global_token(x_layer: Tensor, extend_dim: int) -> Tensor:
    """gt_sp/utils.py:772-790: [.., s + 1, ..] (token last) -> P chunks each followed by the token.

    The reference splits dim 1 into P equal chunks and appends the LAST chunk to each, which is only
    meaningful when extend_dim == 1; that behaviour is kept."""
    world = get_sequence_parallel_world_size()
    chunks = split_tensor_along_second_dim(x_layer, world)
    return torch.cat([torch.cat([chunks[i], chunks[-1]], dim=extend_dim) for i in range(world)],
                     dim=extend_dim).contiguous()


def extend_global_token0(x_layer: Tensor, extend_dim: int) -> Tensor:
    """gt_sp/utils.py:793-814: [.., 1 + s, ..] (token first) -> P chunks each preceded by the token."""
    world = get_sequence_parallel_world_size()
    body = x_layer.size(extend_dim) - 1
    if body % world != 0:
        raise ValueError(f"{body} rows cannot be split over {world} ranks")
    token, rest = torch.split(x_layer, [1, body], dim=extend_dim)
    pieces = []
    for chunk in torch.split(rest, body // world, dim=extend_dim):
        pieces += [token, chunk]
    return torch.cat(pieces, dim=extend_dim).contiguous()


class _CopyGlobalToken0(torch.autograd.Function):
    """``y = x; y[:, rows, :] = x[:, 0:1, :]`` on the device, index list resident on the GPU.

    Returns a new tensor: the input is the attention output, which the attention backward needs
    unchanged (it recomputes the softmax gradient from it), so it must not be edited in place."""

    @staticmethod
    def forward(ctx, x: Tensor, rows: Tensor):
        lib = _cabi.load()
        y = x.clone(memory_format=torch.contiguous_format)
        b, s, w = y.shape
        dtype, mult = _elem(y)
        _cabi.check(lib.tgt_global_rows_broadcast(y.data_ptr(), rows.data_ptr(), rows.numel(), b, s,
                                                  w * mult, dtype,
                                                  torch.cuda.current_stream(y.device).cuda_stream))
        ctx.save_for_backward(rows)
        return y

    @staticmethod
    def backward(ctx, grad: Tensor):
        lib = _cabi.load()
        (rows,) = ctx.saved_tensors
        grad = grad.contiguous().clone()
        if grad.dtype not in (torch.float32, torch.bfloat16):
            raise TypeError("copy_global_token0 backward supports float32 and bfloat16")
        b, s, w = grad.shape
        code = _cabi.TGT_F32 if grad.dtype == torch.float32 else _cabi.TGT_BF16
        _cabi.check(lib.tgt_global_rows_reduce(grad.data_ptr(), rows.data_ptr(), rows.numel(), b, s, w,
                                               code, torch.cuda.current_stream(grad.device).cuda_stream))
        return grad, None


def _elem(t: Tensor):
    """(dtype code, width multiplier) describing the element size to the byte-moving kernels."""
    size = t.element_size()
    if size == 4:
        return _cabi.TGT_F32, 1
    if size == 2:
        return _cabi.TGT_BF16, 1
    if size == 8:
        return _cabi.TGT_F32, 2
    raise TypeError(f"unsupported element size {size}")


def copy_global_token0(x_layer: Tensor, extend_dim: int) -> Tensor:
    """gt_sp/utils.py:817-838: x_layer [b, s + p, hp]; every rank's slot of the global token (rows
    ``get_global_token_indices``) takes the value computed at row 0.  Host tensors are edited in place
    like the reference does; CUDA tensors come back as a new tensor (see ``_CopyGlobalToken0``)."""
    world = get_sequence_parallel_world_size()
    if extend_dim != 1 or x_layer.dim() != 3:
        raise ValueError("copy_global_token0 expects [b, s+p, hp] and extend_dim == 1")
    if x_layer.size(1) % world != 0:
        raise ValueError(f"{x_layer.size(1)} rows cannot be split over {world} ranks")
    if x_layer.is_cuda:
        rows = get_global_token_rows_on(x_layer.device, get_last_batch_flag())
        return _CopyGlobalToken0.apply(x_layer, rows)
    # host tensors (multi-rank logic tests on gloo): plain indexing
    rows = torch.tensor(_active_global_rows(), dtype=torch.long)
    x_layer[:, rows, :] = x_layer[:, 0:1, :].expand(-1, rows.numel(), -1)
    return x_layer.contiguous()


# Batch construction (induced sub-graph, cluster-sparse blocks, per-rank slicing) lives in its own module,
# which builds on the helpers above; its names resolve here too, where the reference has them
# (gt_sp/utils.py:61-82,187-520).
_BATCHING_NAMES = ("create_pairs", "gen_sub_edge_index", "generate_new_edges_optimized", "get_batch_reorder_blockize",
                   "pad_2d", "pad_y", "random_split_idx", "reformat_graph")


def __getattr__(name: str):
    if name in _BATCHING_NAMES:
        from . import batching
        return getattr(batching, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
