"""CPU restatement of the reference's sparse graph attention (test infrastructure, not product).

Two independent statements of the same arithmetic:

* :func:`sparse_attention_ops` — the reference's operation sequence, one PyTorch CPU op per line, in
  the order of ``CoreAttention.sparse_attention`` (attn_module.py:141-187; identical bodies at
  models/graphormer_dist_graph_level.py:243-292 and models/gt_dist_graph_level.py:88-137), with
  ``torch_scatter.scatter(src, index, dim=0, out=out, reduce='add')`` (torch-scatter 2.1.1, the
  reference's pinned dependency; call sites attn_module.py:180,185) restated as
  ``out.index_add_(0, index, src)``.  Differentiable, so autograd gives the reference gradients.
  Run in float32 it is also the timed CPU baseline.
* :func:`forward_closed_form` / :func:`backward_closed_form` — float64 numpy loops-free closed form
  of the forward and of the gradient the kernels implement, derived by hand from the same lines.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch


def sparse_attention_ops(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, edge_index: torch.Tensor,
                         bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q, k, v: [N, H, D]; edge_index: [2, E] int64 (row 0 source, row 1 destination);
    bias: per-edge [E] / [E, H] additive score bias or None.  Returns [N, H, D]."""
    n, heads, head_dim = q.shape
    scale = math.sqrt(head_dim)                                  # attn_module.py:94
    src_rows = edge_index[0].to(torch.long)
    dst_rows = edge_index[1].to(torch.long)
    src = k[src_rows]                                            # :146
    dest = q[dst_rows]                                           # :147
    score = torch.mul(src, dest)                                 # :148
    score = score / scale                                        # :151
    score = score.sum(-1, keepdim=True).clamp(-5, 5)             # :155
    if bias is not None:                                         # :158-164 (bias looked up per edge)
        b = bias if bias.dim() == 2 else bias.unsqueeze(1)
        score = score + b.to(score.dtype).unsqueeze(2)
    score = torch.exp(score)                                     # :168
    msg = v[src_rows] * score                                    # :173
    wv = torch.zeros_like(v)                                     # :179
    wv = wv.index_add(0, dst_rows, msg)                          # :180  scatter(reduce='add')
    z = score.new_zeros(n, heads, 1)                             # :184
    z = z.index_add(0, dst_rows, score)                          # :185
    return wv / (z + 1e-6)                                       # :187


def dense_bias_to_edges(attn_bias: torch.Tensor, edge_index: torch.Tensor) -> torch.Tensor:
    """Per-edge view of the reference's dense bias: ``attn_bias`` is [1, H, N, N] and the reference
    reads ``attn_bias.permute(0, 2, 3, 1)[0][src, dst, :]`` (models/graphormer_dist_graph_level.py:
    262-267).  Returns [E, H]."""
    b = attn_bias.permute(0, 2, 3, 1)[0]
    return b[edge_index[0].long(), edge_index[1].long(), :]


def _np64(t) -> np.ndarray:
    if isinstance(t, torch.Tensor):
        t = t.detach().to(torch.float64).cpu().numpy()
    return np.asarray(t, dtype=np.float64)


def _edge_terms(q, k, v, edge_index, bias):
    q, k, v = _np64(q), _np64(k), _np64(v)
    ei = edge_index.cpu().numpy() if isinstance(edge_index, torch.Tensor) else np.asarray(edge_index)
    s, d = ei[0].astype(np.int64), ei[1].astype(np.int64)
    n, heads, head_dim = q.shape
    raw = np.einsum("ehj,ehj->eh", k[s], q[d]) / math.sqrt(head_dim)
    t = np.clip(raw, -5.0, 5.0)
    if bias is not None:
        b = _np64(bias)
        t = t + (b if b.ndim == 2 else b[:, None])
    w = np.exp(t)
    return q, k, v, s, d, raw, w


def forward_closed_form(q, k, v, edge_index, bias=None) -> Tuple[np.ndarray, np.ndarray]:
    """float64 forward: returns (out [N, H, D], Z [N, H])."""
    q, k, v, s, d, raw, w = _edge_terms(q, k, v, edge_index, bias)
    n, heads, head_dim = q.shape
    z = np.zeros((n, heads))
    np.add.at(z, d, w)
    u = np.zeros((n, heads, head_dim))
    np.add.at(u, d, w[:, :, None] * v[s])
    return u / (z[:, :, None] + 1e-6), z


def backward_closed_form(q, k, v, edge_index, dout, bias=None):
    """float64 gradient of ``sum(out * dout)``: returns (dq, dk, dv, dbias_per_edge_and_head [E, H]).

    With G = dout, inv = 1/(Z + 1e-6):  dw = (G_d.V_s - G_d.O_d) inv_d;  dV_s += w inv_d G_d;
    dt = dw w;  da = dt [-5 <= raw <= 5];  dQ_d += da K_s / sqrt(D);  dK_s += da Q_d / sqrt(D)."""
    qn, kn, vn, s, d, raw, w = _edge_terms(q, k, v, edge_index, bias)
    g = _np64(dout)
    n, heads, head_dim = qn.shape
    out, z = forward_closed_form(q, k, v, edge_index, bias)
    inv = 1.0 / (z + 1e-6)
    delta = np.einsum("nhj,nhj->nh", g, out)
    dw = (np.einsum("ehj,ehj->eh", g[d], vn[s]) - delta[d]) * inv[d]
    dt = dw * w
    da = dt * ((raw >= -5.0) & (raw <= 5.0))
    scale = math.sqrt(head_dim)
    dq = np.zeros_like(qn)
    dk = np.zeros_like(kn)
    dv = np.zeros_like(vn)
    np.add.at(dq, d, da[:, :, None] * kn[s] / scale)
    np.add.at(dk, s, da[:, :, None] * qn[d] / scale)
    np.add.at(dv, s, (w * inv[d])[:, :, None] * g[d])
    return dq, dk, dv, dt
