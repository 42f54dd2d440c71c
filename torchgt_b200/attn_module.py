"""Drop-in ``CoreAttention`` for the reference's sparse branch.

Mirrors the constructor and call signatures of the reference class in all of its copies
(attn_module.py:87-229, models/graphormer_dist_node_level.py:42-221, models/gt_dist_node_level.py:30-166,
models/graphormer_dist_graph_level.py:185-316, models/gt_dist_graph_level.py:30-161) and routes the
``"sparse"`` attention type to the fused CUDA kernels.  The module owns no parameters or buffers, so
model ``state_dict``s are unchanged.  The dense ``"full"`` and ``"flash"`` branches of the reference
are baselines, not part of this library, and raise.
"""
from __future__ import annotations

import math
from typing import Optional, Union

import torch
from torch import nn

from .graph import SparseGraph
from .gt_sp.initialize import get_sequence_parallel_world_size, sequence_parallel_is_initialized
from .sparse_attn import sparse_graph_attention


def _is_edge_argument(x) -> bool:
    if isinstance(x, SparseGraph):
        return True
    return (isinstance(x, torch.Tensor) and not x.is_floating_point() and x.dim() == 2 and x.shape[0] == 2)


def edge_bias_from_dense(attn_bias: torch.Tensor, edge_index: torch.Tensor, batch: int, nodes: int,
                         heads: int, layout: Optional[str] = None) -> torch.Tensor:
    """Per-edge [E, heads] bias from the reference's dense forms.

    ``layout="graph"``: [b, heads, N, N] (models/graphormer_dist_graph_level.py:262-267): edge (s, d) in
    flattened row numbering reads ``attn_bias[s // N, :, s % N, d % N]``.  ``layout="node"``:
    [b, N, N, heads] (models/graphormer_dist_node_level.py:100-106) reads ``attn_bias[s // N, s % N,
    d % N, :]``.  ``layout=None`` tells the form from the shape and raises when the shape fits both
    (heads == N), instead of guessing.
    """
    src, dst = edge_index[0].long(), edge_index[1].long()
    if attn_bias.dim() != 4 or attn_bias.shape[0] != batch:
        raise ValueError(f"dense attn_bias must be 4-D with batch {batch}; got {tuple(attn_bias.shape)}")
    fits_node = attn_bias.shape[1] == nodes and attn_bias.shape[2] == nodes
    fits_graph = attn_bias.shape[2] == nodes and attn_bias.shape[3] == nodes
    if layout is None:
        if fits_node and fits_graph:
            raise ValueError(f"dense attn_bias {tuple(attn_bias.shape)} fits both [b, N, N, heads] and "
                             "[b, heads, N, N]; set dense_bias_layout ('node' or 'graph') on the module")
        layout = "node" if fits_node else "graph"
    if layout not in ("node", "graph"):
        raise ValueError("layout must be 'node', 'graph' or None")
    if layout == "node" and fits_node:
        e = attn_bias[src // nodes, src % nodes, dst % nodes, :]
    elif layout == "graph" and fits_graph:
        e = attn_bias[src // nodes, :, src % nodes, dst % nodes]
    else:
        raise ValueError(f"dense attn_bias {tuple(attn_bias.shape)} does not match {nodes} nodes in the "
                         f"'{layout}' form")
    if e.shape[1] not in (1, heads):
        raise ValueError(f"dense attn_bias carries {e.shape[1]} heads, the call has {heads}")
    return e


class CoreAttention(nn.Module):
    """``CoreAttention(hidden_size, attention_dropout_rate, num_heads[, attn_bias_dim | device])``.

    ``sparse_attention_bias`` takes (k, q, v, ...), the order of models/graphormer_dist_node_level.py:69,
    models/graphormer_dist_graph_level.py:238 and models/gt_dist_graph_level.py:83;
    :class:`CoreAttentionQKV` is the same module with the (q, k, v, ...) order of
    models/gt_dist_node_level.py:83 and models/gt_graph_level.py:83.  ``dense_bias_layout`` ("node",
    "graph" or None = told from the shape) names the form of a dense 4-D ``attn_bias``."""

    dense_bias_layout: Optional[str] = None

    def __init__(self, hidden_size: int, attention_dropout_rate: float, num_heads: int,
                 attn_bias_dim_or_device=None):
        super().__init__()
        world = get_sequence_parallel_world_size() if sequence_parallel_is_initialized() else 1
        self.hidden_size_per_partition = hidden_size // world
        self.hidden_size_per_attention_head = hidden_size // num_heads
        self.num_attention_heads_per_partition = num_heads // world
        self.scale = math.sqrt(self.hidden_size_per_attention_head)
        self.num_heads = num_heads
        self.attention_dropout_rate = attention_dropout_rate
        self.drop_out_rate = attention_dropout_rate
        # kept for attribute compatibility; the sparse branch of the reference applies no dropout
        self.att_dropout = nn.Dropout(attention_dropout_rate)

    # -- the op ---------------------------------------------------------------------------------------
    def _sparse(self, q, k, v, edge_index, attn_bias):
        batch, nodes = k.size(0), k.size(1)
        head_dim = self.hidden_size_per_attention_head
        if q.dim() == 4:
            heads = q.size(2)  # H/P in training under sequence parallelism, H otherwise
        else:
            heads = q.size(-1) // head_dim
        q3 = q.reshape(-1, heads, head_dim)
        k3 = k.reshape(-1, heads, head_dim)
        v3 = v.reshape(-1, heads, head_dim)
        bias = attn_bias
        if bias is not None and bias.dim() == 4:
            if isinstance(edge_index, SparseGraph):
                raise ValueError("a dense attn_bias needs the COO edge_index, not a SparseGraph")
            bias = edge_bias_from_dense(bias, edge_index, batch, nodes, heads, self.dense_bias_layout)
        return sparse_graph_attention(q3, k3, v3, edge_index, bias)

    def sparse_attention(self, q, k, v, edge_index, attn_bias=None):
        """attn_module.py:133-189: q, k, v [b, N, H, D] -> [b, N, H*D]."""
        batch, nodes = k.size(0), k.size(1)
        return self._sparse(q, k, v, edge_index, attn_bias).view(batch, nodes, -1)

    def sparse_attention_bias(self, k, q, v, edge_index, attn_bias=None):
        """models/graphormer_dist_node_level.py:69-127 (argument order k, q, v) -> [b*N, H, D].
        Code written against the (q, k, v) copies uses :class:`CoreAttentionQKV`."""
        return self._sparse(q, k, v, edge_index, attn_bias)

    def full_attention(self, *args, **kwargs):
        raise NotImplementedError("torchgt_b200 implements the sparse branch only; the dense 'full' "
                                  "baseline stays with the reference implementation")

    full_flash_attention = full_attention
    full_attention_hybrid = full_attention

    def forward(self, q, k, v, attn_bias=None, edge_index=None, attn_type=None, *args, **kwargs):
        """Model form ``forward(q, k, v, attn_bias=None, edge_index=None, attn_type=None)`` and the
        micro-benchmark form ``forward(q, k, v, edge_index, flash_attn=False, full=False, mask=None)``
        (attn_module.py:221-229).  Returns [b, s, H*D]."""
        batch, s_len = q.size(0), q.size(1)
        if _is_edge_argument(attn_bias):  # micro-benchmark form: 4th positional argument is the edge list
            flash = bool(edge_index) if edge_index is not None else kwargs.get("flash_attn", False)
            full = bool(attn_type) if attn_type is not None else kwargs.get("full", False)
            if flash or full:
                return self.full_attention()
            return self.sparse_attention(q, k, v, attn_bias)
        if attn_type != "sparse":
            return self.full_attention()
        if edge_index is None:
            raise ValueError("attn_type='sparse' needs edge_index")
        return self._sparse(q, k, v, edge_index, attn_bias).view(batch, s_len, -1)


class CoreAttentionQKV(CoreAttention):
    """The copies whose ``sparse_attention_bias`` takes (q, k, v, edge_index, attn_bias):
    models/gt_dist_node_level.py:83-142 and models/gt_graph_level.py:83-137.  Everything else is
    :class:`CoreAttention`."""

    def sparse_attention_bias(self, q, k, v, edge_index, attn_bias=None):
        return self._sparse(q, k, v, edge_index, attn_bias)
