"""Graphormer shells (node-level and graph-level) around the sparse attention path.

Same constructor arguments, sub-module names and ``state_dict`` keys as the reference models
(models/graphormer_dist_node_level.py:226-395, models/graphormer_dist_graph_level.py:28-76,318-505),
so their checkpoints load with ``strict=True``.  The dense
layers are ordinary ``torch.nn`` modules (library GEMMs); the attention and its sequence-parallel
exchange are this library's kernels.  It exists so that end-to-end step and epoch times can be measured
without the reference's code; the dense-bias branch of the reference model (never taken on the sparse
path: every caller passes ``attn_bias=None``) is not reproduced.
"""
from __future__ import annotations

import math

import torch
from torch import nn
from torch.nn import functional as F

from .attn_module import CoreAttention
from .gt_sp.initialize import get_sequence_parallel_group, sequence_parallel_is_initialized
from .layer_norm import LayerNorm
from .linear import Linear
from .gt_sp.layer import DistributedAttentionNoMerge


def _init_params(module: nn.Module, n_layers: int) -> None:
    """models/graphormer_dist_node_level.py:18-25, models/graphormer_dist_graph_level.py:20-26:
    N(0, 0.02/sqrt(L)) linears, N(0, 0.02) embeddings."""
    if isinstance(module, nn.Linear):
        module.weight.data.normal_(mean=0.0, std=0.02 / math.sqrt(n_layers))
        if module.bias is not None:
            module.bias.data.zero_()
    elif isinstance(module, nn.Embedding):
        module.weight.data.normal_(mean=0.0, std=0.02)


class FeedForwardNetwork(nn.Module):
    def __init__(self, hidden_size: int, ffn_size: int, dropout_rate: float):
        super().__init__()
        self.layer1 = Linear(hidden_size, ffn_size)
        self.gelu = nn.GELU()
        self.layer2 = Linear(ffn_size, hidden_size)

    def forward(self, x):
        return self.layer2(self.gelu(self.layer1(x)))


class MultiHeadAttention(nn.Module):
    """Q/K/V projections, the Ulysses layer around the sparse attention, output projection
    (models/graphormer_dist_node_level.py:226-273)."""

    def __init__(self, hidden_size: int, attention_dropout_rate: float, num_heads: int, attn_bias_dim: int = 1):
        super().__init__()
        self.num_heads = num_heads
        self.att_size = hidden_size // num_heads
        self.linear_q = Linear(hidden_size, num_heads * self.att_size)
        self.linear_k = Linear(hidden_size, num_heads * self.att_size)
        self.linear_v = Linear(hidden_size, num_heads * self.att_size)
        core = CoreAttention(hidden_size, attention_dropout_rate, num_heads, attn_bias_dim)
        group = get_sequence_parallel_group() if sequence_parallel_is_initialized() else None
        self.dist_attn = DistributedAttentionNoMerge(core, group)
        self.output_layer = Linear(num_heads * self.att_size, hidden_size)
        # None: go through the sequence-parallel layer whenever a group exists; False: always attend
        # locally over the rows given (a single-GPU model inside a multi-rank job)
        self.sequence_parallel = None

    def forward(self, x, attn_bias=None, edge_index=None, attn_type=None, mask=None):
        b = x.size(0)
        use_sp = sequence_parallel_is_initialized() if self.sequence_parallel is None else self.sequence_parallel
        q = self.linear_q(x).view(b, -1, self.num_heads, self.att_size)
        # the exchange of q starts now and runs under the next two projections; k follows under v's
        pending = self.dist_attn.start_exchange(q, attn_bias, edge_index, attn_type) if use_sp else None
        k = self.linear_k(x).view(b, -1, self.num_heads, self.att_size)
        if pending is not None:
            pending.add(k)
        v = self.linear_v(x).view(b, -1, self.num_heads, self.att_size)
        if use_sp:
            ctx = self.dist_attn(q, k, v, attn_bias, edge_index, attn_type, pending=pending)
        else:  # single process without a sequence-parallel group: the layer would only pass through
            ctx = self.dist_attn.local_attn(q, k, v, attn_bias, edge_index, attn_type)
        return self.output_layer(ctx)


class EncoderLayer(nn.Module):
    """Pre-norm attention block + pre-norm feed-forward block (models/graphormer_dist_node_level.py:276-314)."""

    def __init__(self, hidden_size, ffn_size, dropout_rate, attention_dropout_rate, num_heads, attn_bias_dim=1):
        super().__init__()
        self.self_attention_norm = LayerNorm(hidden_size)
        self.self_attention = MultiHeadAttention(hidden_size, attention_dropout_rate, num_heads, attn_bias_dim)
        self.self_attention_dropout = nn.Dropout(dropout_rate)
        self.ffn_norm = LayerNorm(hidden_size)
        self.ffn = FeedForwardNetwork(hidden_size, ffn_size, dropout_rate)
        self.ffn_dropout = nn.Dropout(dropout_rate)

    def _fused_attention_half(self, x, attn_bias, edge_index, attn_type):
        """LayerNorm, projections, exchange, attention, exchange and output projection as one autograd
        node of two compute-and-move kernels around the attention kernels, when the call qualifies: training
        under sequence parallelism over peer memory, fp32, hidden size 64, sparse attention without a bias."""
        from .gt_sp import fused
        from .gt_sp.initialize import get_global_token_rows_on, get_last_batch_flag, get_sequence_parallel_world_size
        mha = self.self_attention
        if not (self.training and fused.fused_block_enabled() and mha.sequence_parallel is not False
                and sequence_parallel_is_initialized()):
            return None
        if not (x.is_cuda and x.dtype == torch.float32 and x.dim() == 3 and x.size(-1) == 64
                and mha.num_heads * mha.att_size == 64 and attn_bias is None and attn_type == "sparse"
                and edge_index is not None):
            return None
        world = get_sequence_parallel_world_size()
        if world < 2 or mha.num_heads % world != 0 or ((mha.num_heads // world) * mha.att_size) % 4 != 0:
            return None
        px = mha.dist_attn._peer_exchange(x.new_empty((1, 1, mha.num_heads, mha.att_size)), attn_bias, edge_index,
                                          attn_type)
        if px is None:
            return None
        rows = get_global_token_rows_on(x.device, get_last_batch_flag())
        return fused.attention_block(px, x, self.self_attention_norm, mha, edge_index, rows)

    def forward(self, x, attn_bias=None, edge_index=None, attn_type=None, mask=None):
        y = self._fused_attention_half(x, attn_bias, edge_index, attn_type)
        if y is None:
            y = self.self_attention(self.self_attention_norm(x), attn_bias, edge_index, attn_type=attn_type)
        x = x + self.self_attention_dropout(y)
        y = self.ffn(self.ffn_norm(x))
        return x + self.ffn_dropout(y)


class Graphormer(nn.Module):
    """``Graphormer(n_layers, num_heads, input_dim, hidden_dim, output_dim, attn_bias_dim, dropout_rate,
    input_dropout_rate, attention_dropout_rate, ffn_dim, num_global_node)`` — one node per token, the
    global token at local row 0 (models/graphormer_dist_node_level.py:317-395)."""

    def __init__(self, n_layers, num_heads, input_dim, hidden_dim, output_dim, attn_bias_dim, dropout_rate,
                 input_dropout_rate, attention_dropout_rate, ffn_dim, num_global_node):
        super().__init__()
        self.num_heads = num_heads
        self.node_encoder = Linear(input_dim, hidden_dim)
        self.input_dropout = nn.Dropout(input_dropout_rate)
        self.layers = nn.ModuleList(
            [EncoderLayer(hidden_dim, ffn_dim, dropout_rate, attention_dropout_rate, num_heads, attn_bias_dim)
             for _ in range(n_layers)])
        self.n_layers = n_layers
        self.final_ln = LayerNorm(hidden_dim)
        self.downstream_out_proj = Linear(hidden_dim, output_dim)
        self.hidden_dim = hidden_dim
        self.num_global_node = num_global_node
        self.graph_token = nn.Embedding(num_global_node, hidden_dim)
        self.graph_token_virtual_distance = nn.Embedding(num_global_node, attn_bias_dim)
        self.apply(lambda m: _init_params(m, n_layers))

    def forward(self, x, attn_bias, edge_index, perturb=None, attn_type=None):
        """x: this rank's [s/p, input_dim] features; edge_index: the batch's [2, E] edges (or a
        ``SparseGraph``) in the numbering of the gathered sequence; returns log-probabilities [s/p, C]."""
        if attn_bias is not None:
            raise NotImplementedError("the sparse path takes attn_bias=None (as every caller in the reference does)")
        h = self.node_encoder(x.unsqueeze(0))
        if perturb is not None:
            h = h + perturb
        token = self.graph_token.weight.unsqueeze(0).expand(h.size(0), -1, -1)
        h = self.input_dropout(torch.cat([token, h], dim=1))
        for layer in self.layers:
            h = layer(h, attn_bias=None, edge_index=edge_index, attn_type=attn_type)
        h = self.final_ln(h)
        return F.log_softmax(self.downstream_out_proj(h[0, 1:, :]), dim=1)


class GraphNodeFeature(nn.Module):
    """Summed atom embeddings + in/out-degree embeddings, graph token prepended at index 0
    (models/graphormer_dist_graph_level.py:28-71)."""

    def __init__(self, num_heads, num_atoms, num_in_degree, num_out_degree, hidden_dim):
        super().__init__()
        self.num_heads = num_heads
        self.num_atoms = num_atoms
        self.atom_encoder = nn.Embedding(num_atoms, hidden_dim, padding_idx=0)
        self.in_degree_encoder = nn.Embedding(num_in_degree, hidden_dim, padding_idx=0)
        self.out_degree_encoder = nn.Embedding(num_out_degree, hidden_dim, padding_idx=0)
        self.graph_token = nn.Embedding(1, hidden_dim)

    def forward(self, batched_data):
        x = batched_data.x
        h = (self.atom_encoder(x).sum(dim=-2) + self.in_degree_encoder(batched_data.in_degree) +
             self.out_degree_encoder(batched_data.out_degree))
        token = self.graph_token.weight.unsqueeze(0).expand(x.size(0), -1, -1)
        return torch.cat([token, h], dim=1)


# (atoms, in-degrees, out-degrees) table sizes per dataset family (models/graphormer_dist_graph_level.py:424-445)
_TABLES = {"ZINC": (64, 64, 64), "MalNet": (560000, 560000, 560000)}


class GraphormerGraphLevel(nn.Module):
    """``Graphormer(n_layers, num_heads, hidden_dim, dropout_rate, intput_dropout_rate, ffn_dim,
    dataset_name, edge_type, multi_hop_max_dist, attention_dropout_rate, output_dim)`` of
    models/graphormer_dist_graph_level.py:409-505: one padded graph per sequence, this rank's graph token
    at local index 0, prediction read from the token.  The reference builds no attention bias on this
    path (its ``GraphAttnBias`` is commented out), so none is built here."""

    def __init__(self, n_layers, num_heads, hidden_dim, dropout_rate, intput_dropout_rate, ffn_dim, dataset_name,
                 edge_type, multi_hop_max_dist, attention_dropout_rate, output_dim):
        super().__init__()
        atoms, in_deg, out_deg = _TABLES.get(dataset_name, (7000, 7000, 7000))
        self.graph_node_feature = GraphNodeFeature(num_heads, atoms, in_deg, out_deg, hidden_dim)
        self.input_dropout = nn.Dropout(intput_dropout_rate)
        self.layers = nn.ModuleList(
            [EncoderLayer(hidden_dim, ffn_dim, dropout_rate, attention_dropout_rate, num_heads)
             for _ in range(n_layers)])
        self.final_ln = LayerNorm(hidden_dim)
        if dataset_name == "PCQM4M-LSC":
            self.out_proj = Linear(hidden_dim, 1)
        else:
            self.downstream_out_proj = Linear(hidden_dim, output_dim)
        self.apply(lambda m: _init_params(m, n_layers))   # embeddings are drawn over their padding row too

    def forward(self, batched_data, perturb=None, attn_type=None):
        """batched_data: ``x`` int64 [b, s/p, F], ``in_degree`` / ``out_degree`` int64 [b, s/p], ``edge_index``
        [2, E] over the flattened rows of the gathered batch (or a ``SparseGraph``); returns [b, output_dim]."""
        h = self.input_dropout(self.graph_node_feature(batched_data))
        edge_index = batched_data.edge_index
        for layer in self.layers:
            h = layer(h, None, edge_index=edge_index, attn_type=attn_type)
        h = self.final_ln(h)
        head = self.out_proj if hasattr(self, "out_proj") else self.downstream_out_proj
        return head(h[:, 0, :])

