"""Ulysses sequence-parallel attention layers without a global token (GT family).

Mirrors the reference's gt_sp/gt_layer.py: ``DistributedAttention`` (graph-level GT, always exchanges)
and ``DistributedAttentionNodeLevel`` (node-level GT, exchanges in training mode only).
"""
from __future__ import annotations

from typing import Any

from torch import Tensor

from .layer import _SeqAllToAll, _SeqGather, _SeqScatter, _UlyssesBase  # noqa: F401  (re-exported)


class DistributedAttention(_UlyssesBase):
    """gt_sp/gt_layer.py:142-206: q, k, v [b, s/p, H, D]; an optional dense bias [b, H, s/p, s] is
    exchanged with heads scattered (dim 1) and rows gathered (dim 2)."""

    exchanges_in_eval = True

    def forward(self, query: Tensor, key: Tensor, value: Tensor, attn_bias: Tensor, edge_index: Tensor,
                attn_type, *args: Any, pending=None) -> Tensor:
        out = self._single_node(query, key, value, attn_bias, edge_index, attn_type, alias=False, pending=pending)
        if out is not None:
            return out
        q, k, v = self._gather_sequence(query, key, value)
        bias = attn_bias
        if bias is not None:
            bias = _SeqAllToAll.apply(self.spg, bias, 1, 2)
        context = self.local_attn(q, k, v, bias, edge_index, attn_type, *args)
        return self._scatter_sequence(context)


class DistributedAttentionNodeLevel(DistributedAttention):
    """gt_sp/gt_layer.py:209-286: same exchange, bypassed in evaluation mode where rank 0 runs the
    whole sequence with all heads."""

    exchanges_in_eval = False

    def forward(self, query: Tensor, key: Tensor, value: Tensor, attn_bias: Tensor, edge_index: Tensor,
                attn_type, *args: Any, pending=None) -> Tensor:
        if not self.training:
            return self.local_attn(query, key, value, attn_bias, edge_index, attn_type, *args)
        return super().forward(query, key, value, attn_bias, edge_index, attn_type, *args, pending=pending)
