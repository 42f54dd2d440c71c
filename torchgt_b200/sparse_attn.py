"""Autograd wrapper of the fused sparse graph-attention kernels.

``sparse_graph_attention(q, k, v, graph, bias)`` computes, for every edge e = (s -> d) and head h,

    w_e = exp(clamp(K[s,h] . Q[d,h] / sqrt(D), -5, 5) + bias_e),   out[d,h] = sum_e w_e V[s,h] / (sum_e w_e + 1e-6)

which is CoreAttention.sparse_attention of the reference (attn_module.py:133-189) without its
per-edge temporaries, and its gradient in two passes without floating-point atomics.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Union

import torch

from . import _cabi
from .graph import SparseGraph, graph_for

_DTYPES = {torch.float32: _cabi.TGT_F32, torch.bfloat16: _cabi.TGT_BF16}


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None or t.numel() == 0 else t.data_ptr()


def _scratch(graph: SparseGraph, heads: int, head_dim: int, dtype: int, phase: int, device) -> torch.Tensor:
    """Scratch of one call; its size is asked from the library once per (graph, shape, phase)."""
    key = (heads, head_dim, dtype, phase)
    nbytes = graph.scratch_bytes.get(key)
    if nbytes is None:
        lib = _cabi.load()
        n = ctypes.c_size_t()
        by_src = graph.by_src.byref() if phase == 1 else None
        _cabi.check(lib.tgt_sparse_attn_scratch_bytes(graph.by_dst.byref(), by_src, heads, head_dim, dtype, phase,
                                                      ctypes.byref(n)))
        nbytes = graph.scratch_bytes[key] = max(n.value, 16)
    return torch.empty(nbytes, dtype=torch.uint8, device=device)


class _SparseGraphAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, bias, graph: SparseGraph):
        lib = _cabi.load()
        n_rows, heads, head_dim = q.shape
        out = torch.empty_like(q)
        z = torch.empty((n_rows, heads), dtype=torch.float32, device=q.device)
        bias_heads = 0 if bias is None else (1 if bias.dim() == 1 else int(bias.shape[1]))
        scratch = _scratch(graph, heads, head_dim, _DTYPES[q.dtype], 0, q.device)
        _cabi.check(lib.tgt_sparse_attn_fwd(
            _ptr(q), _ptr(k), _ptr(v), _ptr(bias), bias_heads, graph.by_dst.byref(), _ptr(out), _ptr(z),
            heads, head_dim, _DTYPES[q.dtype], scratch.data_ptr(), scratch.numel(), _stream(q)))
        ctx.graph = graph
        ctx.bias_heads = bias_heads
        ctx.save_for_backward(q, k, v, bias, out, z)
        return out

    @staticmethod
    def backward(ctx, dout):
        lib = _cabi.load()
        q, k, v, bias, out, z = ctx.saved_tensors
        graph: SparseGraph = ctx.graph
        n_rows, heads, head_dim = q.shape
        dout = dout.contiguous()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dbias = None
        if bias is not None and ctx.needs_input_grad[3]:
            dbias = torch.empty_like(bias)
        scratch = _scratch(graph, heads, head_dim, _DTYPES[q.dtype], 1, q.device)
        _cabi.check(lib.tgt_sparse_attn_bwd(
            _ptr(dout), _ptr(q), _ptr(k), _ptr(v), _ptr(bias), ctx.bias_heads, _ptr(out), _ptr(z),
            graph.by_dst.byref(), graph.by_src.byref(), _ptr(dq), _ptr(dk), _ptr(dv), _ptr(dbias), heads,
            head_dim, _DTYPES[q.dtype], scratch.data_ptr(), scratch.numel(), _stream(q)))
        return dq, dk, dv, dbias, None


def _heads_fit_one_group(heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    row_bytes = heads * head_dim * (4 if dtype == torch.float32 else 2)
    return row_bytes <= 512 and (heads & (heads - 1)) == 0


def sparse_graph_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                           edge_index: Union[torch.Tensor, SparseGraph],
                           bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Sparse attention over the rows of ``q``/``k``/``v`` ([N, H, D], fp32 or bf16, CUDA).

    ``edge_index`` is the reference's [2, E] int64 COO list (row 0 = source, row 1 = destination) or a
    prebuilt :class:`SparseGraph`.  ``bias`` is an optional per-edge additive score bias in the order of
    ``edge_index`` columns, shape [E] (shared by all heads) or [E, H]; it is added after the clamp.
    Returns [N, H, D].  Raises if the tensors are not on a CUDA device: there is no CPU path.
    """
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("torchgt_b200.sparse_graph_attention needs CUDA tensors (no CPU fallback)")
    if q.dim() != 3 or q.shape != k.shape or q.shape != v.shape:
        raise ValueError(f"q, k, v must share the shape [N, H, D]; got {tuple(q.shape)}, "
                         f"{tuple(k.shape)}, {tuple(v.shape)}")
    if q.dtype not in _DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("q, k, v must all be float32 or all bfloat16")
    n_rows, heads, head_dim = q.shape
    graph = graph_for(edge_index, n_rows)
    graph.poll()   # a node id outside [0, N) found by the (asynchronous) layout build is raised here
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    if bias is not None:
        if bias.dim() == 2 and bias.shape[1] == 1 and heads != 1:
            bias = bias[:, 0]
        if bias.dim() not in (1, 2) or bias.shape[0] != graph.n_edges or \
                (bias.dim() == 2 and bias.shape[1] != heads):
            raise ValueError(f"bias must be [E] or [E, H] with E={graph.n_edges}, H={heads}; "
                             f"got {tuple(bias.shape)}")
        bias = bias.to(torch.float32)
        if bias.dim() == 1 and bias.requires_grad and not _heads_fit_one_group(heads, head_dim, q.dtype):
            # the kernels reduce a shared bias gradient inside one lane group only; let autograd sum heads
            bias = bias.unsqueeze(1).expand(-1, heads)
        bias = bias.contiguous()
        if graph.n_edges == 0:
            bias = None  # nothing to add the (empty) bias to
    return _SparseGraphAttention.apply(q, k, v, bias, graph)
