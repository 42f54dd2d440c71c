"""GT (graph transformer without a global token) shells around the sparse attention path.

``GTNodeLevel`` and ``GTGraphLevel`` take the constructor arguments of the reference's two ``GT``
classes (models/gt_dist_node_level.py:282-341, models/gt_dist_graph_level.py:279-365), use the same
sub-module names and so load the same ``state_dict``s with ``strict=True``.  The dense layers are
ordinary ``torch.nn`` modules; the attention and its sequence-parallel exchange are this library's
kernels.  Two properties of the reference's encoder block are kept because checkpoints and results
depend on them: the feed-forward branch reads the attention branch's output ``y`` (not the normalised
``x``), and ``self_attention_norm`` / ``downstream_out_proj`` exist as parameters but are never applied.
"""
from __future__ import annotations

import math

import torch
from torch import nn
from torch.nn import functional as F

from .attn_module import CoreAttentionQKV as CoreAttention  # (q, k, v) order, as models/gt_dist_node_level.py:83
from .gt_sp.gt_layer import DistributedAttention, DistributedAttentionNodeLevel, _SeqGather
from .gt_sp.initialize import get_sequence_parallel_group, sequence_parallel_is_initialized
from .layer_norm import LayerNorm
from .linear import Linear


def _init_params(module: nn.Module, n_layers: int) -> None:
    """models/gt_dist_node_level.py:21-27: N(0, 0.02/sqrt(L)) linears, N(0, 0.02) embeddings."""
    if isinstance(module, nn.Linear):
        module.weight.data.normal_(mean=0.0, std=0.02 / math.sqrt(n_layers))
        if module.bias is not None:
            module.bias.data.zero_()
    if isinstance(module, nn.Embedding):
        module.weight.data.normal_(mean=0.0, std=0.02)


class MultiHeadAttention(nn.Module):
    """Q/K/V projections and the Ulysses layer; the output projection is the block's ``O``
    (models/gt_dist_node_level.py:170-213, models/gt_dist_graph_level.py:165-208)."""

    def __init__(self, hidden_size: int, attention_dropout_rate: float, num_heads: int, node_level: bool):
        super().__init__()
        self.num_heads = num_heads
        self.att_size = hidden_size // num_heads
        self.linear_q = Linear(hidden_size, num_heads * self.att_size)
        self.linear_k = Linear(hidden_size, num_heads * self.att_size)
        self.linear_v = Linear(hidden_size, num_heads * self.att_size)
        core = CoreAttention(hidden_size, attention_dropout_rate, num_heads)
        group = get_sequence_parallel_group() if sequence_parallel_is_initialized() else None
        self.dist_attn = (DistributedAttentionNodeLevel if node_level else DistributedAttention)(core, group)

    def forward(self, x, attn_bias=None, mask=None, edge_index=None, attn_type=None):
        b = x.size(0)
        use_sp = sequence_parallel_is_initialized()
        q = self.linear_q(x).view(b, -1, self.num_heads, self.att_size)
        # the exchange of q starts now and runs under the next two projections; k follows under v's
        pending = self.dist_attn.start_exchange(q, attn_bias, edge_index, attn_type) if use_sp else None
        k = self.linear_k(x).view(b, -1, self.num_heads, self.att_size)
        if pending is not None:
            pending.add(k)
        v = self.linear_v(x).view(b, -1, self.num_heads, self.att_size)
        if use_sp:
            out = self.dist_attn(q, k, v, attn_bias, edge_index, attn_type, pending=pending)
        else:  # single process without a sequence-parallel group: the layer would only pass through
            out = self.dist_attn.local_attn(q, k, v, attn_bias, edge_index, attn_type)
        if out.size() != x.size():
            raise RuntimeError(f"attention returned {tuple(out.size())} for an input of {tuple(x.size())}")
        return out


class EncoderLayer(nn.Module):
    """Post-norm block (models/gt_dist_node_level.py:216-259)."""

    def __init__(self, hidden_size, ffn_size, dropout_rate, attention_dropout_rate, num_heads, node_level=True):
        super().__init__()
        self.self_attention_norm = LayerNorm(hidden_size)   # a parameter of the reference, never applied
        self.self_attention = MultiHeadAttention(hidden_size, attention_dropout_rate, num_heads, node_level)
        self.self_attention_dropout = nn.Dropout(dropout_rate)
        self.O = Linear(hidden_size, hidden_size)
        self.layer_norm1 = LayerNorm(hidden_size)
        self.FFN_layer1 = Linear(hidden_size, hidden_size * 2)
        self.FFN_layer2 = Linear(hidden_size * 2, hidden_size)
        self.layer_norm2 = LayerNorm(hidden_size)

    def forward(self, x, attn_bias=None, mask=None, edge_index=None, attn_type=None):
        y = self.self_attention(x, attn_bias, mask=mask, edge_index=edge_index, attn_type=attn_type)
        y = self.O(self.self_attention_dropout(y))
        x = self.layer_norm1(x + y)
        y = self.FFN_layer2(self.self_attention_dropout(F.relu(self.FFN_layer1(y))))
        return self.layer_norm2(x + y)


class MLPReadout(nn.Module):
    """hidden -> hidden/2 -> ... -> hidden/2^L -> output with ReLU in between
    (models/gt_dist_node_level.py:262-278)."""

    def __init__(self, input_dim: int, output_dim: int, L: int = 2):
        super().__init__()
        dims = [input_dim // 2 ** i for i in range(L + 1)]
        self.FC_layers = nn.ModuleList([Linear(a, b) for a, b in zip(dims[:-1], dims[1:])] +
                                       [Linear(dims[-1], output_dim)])
        self.L = L

    def forward(self, x):
        for layer in self.FC_layers[:-1]:
            x = F.relu(layer(x))
        return self.FC_layers[-1](x)


class GTNodeLevel(nn.Module):
    """``GT(n_layers, num_heads, input_dim, hidden_dim, output_dim, attn_bias_dim, dropout_rate,
    input_dropout_rate, attention_dropout_rate, ffn_dim, num_global_node)`` of
    models/gt_dist_node_level.py:282-341: one node per token, no global token."""

    def __init__(self, n_layers, num_heads, input_dim, hidden_dim, output_dim, attn_bias_dim, dropout_rate,
                 input_dropout_rate, attention_dropout_rate, ffn_dim, num_global_node):
        super().__init__()
        self.node_encoder = Linear(input_dim, hidden_dim)
        self.input_dropout = nn.Dropout(input_dropout_rate)
        self.layers = nn.ModuleList(
            [EncoderLayer(hidden_dim, ffn_dim, dropout_rate, attention_dropout_rate, num_heads, node_level=True)
             for _ in range(n_layers)])
        self.MLP_layer = MLPReadout(hidden_dim, output_dim)
        self.downstream_out_proj = Linear(hidden_dim, output_dim)   # a parameter of the reference, never applied
        self.apply(lambda m: _init_params(m, n_layers))

    def forward(self, x, attn_bias, edge_index, perturb=None, attn_type=None):
        """x: this rank's [s/p, input_dim] features; returns log-probabilities [s/p, C]."""
        h = self.input_dropout(self.node_encoder(x.unsqueeze(0)))
        for layer in self.layers:
            h = layer(h, edge_index=edge_index, attn_type=attn_type)
        return F.log_softmax(self.MLP_layer(h[0]), dim=1)


# embedding table sizes per dataset family (models/gt_dist_graph_level.py:300-320)
_NUM_ATOMS = {"ZINC": 64, "MalNet": 560000}


class GTGraphLevel(nn.Module):
    """``GT(n_layers, num_heads, hidden_dim, dropout_rate, intput_dropout_rate, ffn_dim, dataset_name,
    edge_type, multi_hop_max_dist, attention_dropout_rate, output_dim)`` of
    models/gt_dist_graph_level.py:279-365: one padded graph per sequence, integer node features summed
    over their embedding vectors, mean over the gathered sequence, MLP read-out."""

    def __init__(self, n_layers, num_heads, hidden_dim, dropout_rate, intput_dropout_rate, ffn_dim, dataset_name,
                 edge_type, multi_hop_max_dist, attention_dropout_rate, output_dim):
        super().__init__()
        self.embedding_h = nn.Embedding(_NUM_ATOMS.get(dataset_name, 7000), hidden_dim)
        self.graph_token = nn.Embedding(1, hidden_dim)   # a parameter of the reference, never applied
        self.input_dropout = nn.Dropout(intput_dropout_rate)
        self.layers = nn.ModuleList(
            [EncoderLayer(hidden_dim, ffn_dim, dropout_rate, attention_dropout_rate, num_heads, node_level=False)
             for _ in range(n_layers)])
        self.MLP_layer = MLPReadout(hidden_dim, output_dim)
        self.apply(lambda m: _init_params(m, n_layers))

    def forward(self, batched_data, perturb=None, attn_type=None):
        """batched_data.x: int64 [b, s/p, F]; batched_data.edge_index: [2, E] over the b * s flattened rows
        of the gathered batch (or a ``SparseGraph``); returns [b, output_dim]."""
        h = self.input_dropout(self.embedding_h(batched_data.x).sum(dim=-2))
        edge_index = batched_data.edge_index
        for layer in self.layers:
            h = layer(h, edge_index=edge_index, attn_type=attn_type)
        if sequence_parallel_is_initialized():
            h = _SeqGather.apply(h, 1)
        return self.MLP_layer(h.mean(dim=1))
