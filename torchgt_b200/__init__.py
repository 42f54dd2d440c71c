"""torchgt_b200 — B200-native sparse graph attention and its Ulysses exchange.

Public surface (mirrors the hot path of zxmeng98/torchgt):
  * :class:`CoreAttention` — drop-in module for the reference's sparse attention branch;
  * :func:`sparse_graph_attention`, :class:`SparseGraph` — the op and its reusable edge layout;
  * ``torchgt_b200.gt_sp`` — ``layer``/``gt_layer`` (``DistributedAttention*``, ``_SeqAllToAll``),
    ``initialize`` (sequence-parallel state) and ``utils`` (edge-index / global-token helpers);
  * :class:`LayerNorm`, :class:`Linear` — ``nn.LayerNorm`` / ``nn.Linear`` with the same parameters whose
    short-row normalisation and weight gradients run on this library's kernels (the two dense operations
    that dominate a training iteration at the models' width of 64).

All compute runs in hand-written CUDA kernels for sm_100a behind a C ABI (``include/torchgt_b200.h``)
loaded with ctypes; there is no CPU fallback.
"""
from .attn_module import CoreAttention
from .graph import SparseGraph, clear_graph_cache, graph_for, prepare_edges
from .layer_norm import LayerNorm
from .linear import Linear
from .sparse_attn import sparse_graph_attention

__all__ = ["CoreAttention", "SparseGraph", "sparse_graph_attention", "graph_for", "clear_graph_cache",
           "prepare_edges", "LayerNorm", "Linear"]
__version__ = "1.0"
