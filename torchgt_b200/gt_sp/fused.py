"""The Ulysses layer as ONE autograd node when the transport is peer memory: exchange, attention and
exchange back without any intermediate copy.

What the reference does per layer call (gt_sp/layer.py:502-550, gt_sp/gt_layer.py:153-206): three
``_SeqAllToAll`` on q, k, v (each: split, ``contiguous`` per chunk, all-to-all, ``cat``), the attention,
``copy_global_token0``, one more ``_SeqAllToAll``; and the same again, reversed, in backward.  Here:

  forward   push q, k, v straight into their final rows of the peers' slot -> barrier -> the attention
            kernel reads the slot in place and writes its output into this rank's own slot -> barrier
            -> every rank pulls its rows of all peers' outputs into an ordinary tensor (the global-token
            copy folded into the pull)
  backward  push dO -> barrier -> (global-token gradient folded into row 0) -> both backward passes read
            the two slots in place and write dQ, dK, dV into this rank's own slot -> barrier -> pull

The slot that holds q, k, v stays reserved from forward to backward; everything else is given back at
once (see ``p2p.PeerExchange`` for when a slot may be reused).
"""
from __future__ import annotations

import os
from typing import Optional

import torch
from torch import Tensor

from .. import _cabi, layer_norm, linear
from ..graph import SparseGraph, graph_for
from ..sparse_attn import _DTYPES, _scratch, _stream
from . import p2p


def fused_layer_enabled() -> bool:
    return os.environ.get("TGT_FUSED_LAYER", "1") != "0"


def eligible(query: Tensor, attn_bias, edge_index, attn_type, world: int) -> bool:
    """Can this call take the single-node path?  (CUDA fp32/bf16 [b, rows, H, D] tensors, sparse
    attention without a bias, heads divisible by the ranks, head slices that are whole 16-byte units.)"""
    if not fused_layer_enabled() or world < 2 or attn_type != "sparse" or attn_bias is not None:
        return False
    if not (isinstance(query, Tensor) and query.is_cuda and query.dim() == 4 and query.dtype in _DTYPES):
        return False
    if edge_index is None:
        return False
    heads, head_dim = query.shape[2], query.shape[3]
    if heads % world != 0 or query.numel() == 0:
        return False
    row_bytes = (heads // world) * head_dim * query.element_size()
    return row_bytes % 16 == 0 and (head_dim * query.element_size()) % 16 == 0


class PendingPush:
    """q, k and v on their way to the peers while the caller still computes the later ones.

    The reference computes the three projections and then exchanges them one after the other
    (models/graphormer_dist_node_level.py:254-264).  Here the landing slot is reserved when the first
    projection exists and each tensor is pushed on the exchange's side stream as soon as it has been
    computed, so its transfer runs under the next projection's GEMM; the layer's forward then only waits
    for the side stream before the barrier."""

    def __init__(self, px: "p2p.PeerExchange", first: Tensor):
        b, rows, heads, head_dim = first.shape
        self.px = px
        self.shape, self.dtype = tuple(first.shape), first.dtype
        self.row_bytes = (heads // px.world) * head_dim * first.element_size()
        self.tensor_bytes = b * px.world * rows * self.row_bytes
        px.check()
        self.slot = px.acquire(3 * self.tensor_bytes)
        self.sent = []                 # data_ptr of every tensor already on its way, in slot order
        self.keep = []
        self.add(first)

    def add(self, t: Tensor) -> None:
        if tuple(t.shape) != self.shape or t.dtype != self.dtype or len(self.sent) >= 3:
            raise ValueError("tensors pushed together must share shape and dtype (at most three)")
        t = t.detach().contiguous()
        px, side = self.px, self.px.side_stream
        side.wait_stream(torch.cuda.current_stream(t.device))      # t has been computed
        with torch.cuda.stream(side):
            b, rows = self.shape[0], self.shape[1]
            px.push([t], self.slot, b * rows, self.row_bytes, rows * self.row_bytes,
                    offset_bytes=len(self.sent) * self.tensor_bytes)
        t.record_stream(side)
        self.sent.append(t.data_ptr())
        self.keep.append(t)

    def finish(self, tensors) -> None:
        """Push what has not been pushed yet and make the current stream wait for all of it."""
        if [t.data_ptr() for t in tensors[:len(self.sent)]] != self.sent:
            raise RuntimeError("the tensors given to the layer are not the ones whose exchange was started")
        for t in tensors[len(self.sent):]:
            self.add(t)
        torch.cuda.current_stream(tensors[0].device).wait_stream(self.px.side_stream)
        self.keep = []


class _UlyssesSparseAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q: Tensor, k: Tensor, v: Tensor, graph: SparseGraph, px: "p2p.PeerExchange",
                alias_rows: Optional[Tensor], pending: Optional[PendingPush] = None):
        lib = _cabi.load()
        b, rows, heads, head_dim = q.shape
        world = px.world
        heads_l = heads // world
        row_bytes = heads_l * head_dim * q.element_size()
        n_rows = b * world * rows
        tensor_bytes = n_rows * row_bytes
        code = _DTYPES[q.dtype]
        # q, k, v -> peers: rank r' receives heads r' * heads_l .. of every row, at rows rank * rows + l
        if pending is not None:
            pending.finish([q, k, v])          # (some of) the pushes were started while k and v were computed
            qkv = pending.slot
        else:
            px.check()
            qkv = px.acquire(3 * tensor_bytes)
            px.push([q, k, v], qkv, b * rows, row_bytes, rows * row_bytes)
        px.mark("push q,k,v")
        px.barrier()
        px.mark("barrier")
        qg, kg, vg = (qkv.view(t * tensor_bytes, (n_rows, heads_l, head_dim), q.dtype) for t in range(3))
        landing = px.acquire(tensor_bytes, p2p.SOURCE)
        out_g = landing.view(0, (n_rows, heads_l, head_dim), q.dtype)
        z = torch.empty((n_rows, heads_l), dtype=torch.float32, device=q.device)
        scratch = _scratch(graph, heads_l, head_dim, code, 0, q.device)
        _cabi.check(lib.tgt_sparse_attn_fwd(qg.data_ptr(), kg.data_ptr(), vg.data_ptr(), None, 0,
                                            graph.by_dst.byref(), out_g.data_ptr(), z.data_ptr(), heads_l, head_dim,
                                            code, scratch.data_ptr(), scratch.numel(), _stream(q)))
        px.mark("attention forward")
        px.barrier()
        px.mark("barrier")
        out = torch.empty((b, rows, heads * head_dim), dtype=q.dtype, device=q.device)
        px.pull(landing, [out], b, rows, row_bytes, alias_rows)
        px.mark("pull out")
        px.release(landing)
        ctx.graph, ctx.px, ctx.qkv, ctx.alias_rows = graph, px, qkv, alias_rows
        ctx.dims = (b, rows, heads, head_dim, heads_l, row_bytes, n_rows, tensor_bytes, code)
        ctx.io_dtype = q.dtype
        ctx.save_for_backward(z)
        return out

    @staticmethod
    def backward(ctx, dout: Tensor):
        lib = _cabi.load()
        (z,) = ctx.saved_tensors
        px, graph, qkv = ctx.px, ctx.graph, ctx.qkv
        b, rows, heads, head_dim, heads_l, row_bytes, n_rows, tensor_bytes, code = ctx.dims
        dtype, dev = ctx.io_dtype, z.device
        world = px.world
        dout = dout.contiguous()
        if dout.dtype != dtype:
            dout = dout.to(dtype)
        px.check()
        landing = px.acquire(tensor_bytes)
        px.push([dout], landing, b * rows, row_bytes, rows * row_bytes)
        px.mark("push dO")
        px.barrier()
        px.mark("barrier")
        dog = landing.view(0, (n_rows, heads_l, head_dim), dtype)
        if ctx.alias_rows is not None:
            # gradient of "listed rows := row 0": row 0 collects the listed rows' gradients
            _cabi.check(lib.tgt_global_rows_reduce(dog.data_ptr(), ctx.alias_rows.data_ptr(), ctx.alias_rows.numel(),
                                                   b, world * rows, heads_l * head_dim, code, _stream(dog)))
        qg, kg, vg = (qkv.view(t * tensor_bytes, (n_rows, heads_l, head_dim), dtype) for t in range(3))
        grads = px.acquire(3 * tensor_bytes, p2p.SOURCE)
        dqg, dkg, dvg = (grads.view(t * tensor_bytes, (n_rows, heads_l, head_dim), dtype) for t in range(3))
        scratch = _scratch(graph, heads_l, head_dim, code, 1, dev)
        _cabi.check(lib.tgt_sparse_attn_bwd(
            dog.data_ptr(), qg.data_ptr(), kg.data_ptr(), vg.data_ptr(), None, 0, None, z.data_ptr(),
            graph.by_dst.byref(), graph.by_src.byref(), dqg.data_ptr(), dkg.data_ptr(), dvg.data_ptr(), None,
            heads_l, head_dim, code, scratch.data_ptr(), scratch.numel(), _stream(dog)))
        px.mark("attention backward")
        px.release(qkv)
        px.release(landing)
        ctx.qkv = None
        px.barrier()
        px.mark("barrier")
        dq, dk, dv = (torch.empty((b, rows, heads, head_dim), dtype=dtype, device=dev) for _ in range(3))
        px.pull(grads, [dq, dk, dv], b, rows, row_bytes)
        px.mark("pull dq,dk,dv")
        px.release(grads)
        px.check()
        return dq, dk, dv, None, None, None, None


def ulysses_sparse_attention(px: "p2p.PeerExchange", query: Tensor, key: Tensor, value: Tensor, edge_index,
                             alias_rows: Optional[Tensor] = None, pending: Optional[PendingPush] = None) -> Tensor:
    """[b, rows, H, D] x3 on every rank -> [b, rows, H*D]: sparse attention over the gathered sequence
    (``world * rows`` rows per batch entry, numbered rank-major) with the heads sharded over the ranks.
    ``alias_rows`` (device int32): rows of the gathered sequence whose output is row 0's output."""
    b, rows = query.shape[0], query.shape[1]
    graph = graph_for(edge_index, b * px.world * rows)
    graph.poll()
    q, k, v = query.contiguous(), key.contiguous(), value.contiguous()
    return _UlyssesSparseAttention.apply(q, k, v, graph, px, alias_rows, pending)


# ---- the attention half of an encoder layer as one node -----------------------------------------------
def fused_block_enabled() -> bool:
    """Whether the encoder layers take ``_UlyssesAttentionBlock`` (default; ``TGT_FUSED_BLOCK=0`` in the
    environment selects the layer node with library projections and the q and k pushes beside them instead).
    Whole training iteration on two GPUs, 64,000 nodes each: 3.36 ms with the block, 3.38 ms without when the
    library may use TF32 tensor cores; with fp32 library products the block is far ahead (its LayerNorm + three
    projections take 57 us in fp32 FMA including the stores, the library's fp32 path 190 us before any
    transfer)."""
    return os.environ.get("TGT_FUSED_BLOCK", "1") != "0"


class _UlyssesAttentionBlock(torch.autograd.Function):
    """``y = out_proj(attention(q_proj(LN(x)), k_proj(LN(x)), v_proj(LN(x))))`` with the Ulysses exchange
    inside, for fp32 and hidden size 64 (models/graphormer_dist_node_level.py:246-273,301 and
    gt_sp/layer.py:502-550 in one node).

    Forward: ``tgt_ln_qkv_push`` (LayerNorm, the three projections and the stores into the peers' slots
    in one kernel) -> barrier -> attention on the slot -> barrier -> ``tgt_pull_out_proj`` (gather over
    NVLink, global-token copy and output projection in one kernel).  No q, k, v tensor exists.
    Backward: the output projection's gradients, then push dO -> barrier -> both attention backward passes ->
    barrier -> pull dQ, dK, dV, then the gradients of the three projections and of the LayerNorm from the saved
    layer input (the normalised input is recomputed, not stored).  Input gradients are library GEMMs, weight
    and bias gradients csrc/linear_wgrad.cu, the LayerNorm csrc/layer_norm.cu."""

    @staticmethod
    def forward(ctx, x, gamma, beta, wq, bq, wk, bk, wv, bv, wo, bo, eps, heads, graph, px, alias_rows):
        lib = _cabi.load()
        b, rows, hidden = x.shape
        world = px.world
        head_dim = hidden // heads
        heads_l = heads // world
        row_bytes = heads_l * head_dim * 4
        n_rows = b * world * rows
        tensor_bytes = n_rows * row_bytes
        code = _cabi.TGT_F32
        px.check()
        x = x.contiguous()
        qkv = px.acquire(3 * tensor_bytes)
        _cabi.check(lib.tgt_ln_qkv_push(x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), float(eps), wq.data_ptr(),
                                        bq.data_ptr(), wk.data_ptr(), bk.data_ptr(), wv.data_ptr(), bv.data_ptr(),
                                        hidden, hidden, qkv.peers, qkv.nbytes, b, rows, world, px.rank, _stream(x)))
        px.mark("LayerNorm + q,k,v projections + push")
        px.barrier()
        px.mark("barrier")
        qg, kg, vg = (qkv.view(t * tensor_bytes, (n_rows, heads_l, head_dim), x.dtype) for t in range(3))
        landing = px.acquire(tensor_bytes, p2p.SOURCE)
        out_g = landing.view(0, (n_rows, heads_l, head_dim), x.dtype)
        z = torch.empty((n_rows, heads_l), dtype=torch.float32, device=x.device)
        scratch = _scratch(graph, heads_l, head_dim, code, 0, x.device)
        _cabi.check(lib.tgt_sparse_attn_fwd(qg.data_ptr(), kg.data_ptr(), vg.data_ptr(), None, 0,
                                            graph.by_dst.byref(), out_g.data_ptr(), z.data_ptr(), heads_l, head_dim,
                                            code, scratch.data_ptr(), scratch.numel(), _stream(x)))
        px.mark("attention forward")
        px.barrier()
        px.mark("barrier")
        attn = torch.empty((b, rows, hidden), dtype=x.dtype, device=x.device)
        y = torch.empty((b, rows, hidden), dtype=x.dtype, device=x.device)
        n_alias = 0 if alias_rows is None else int(alias_rows.numel())
        _cabi.check(lib.tgt_pull_out_proj(landing.peers, landing.nbytes, wo.data_ptr(), bo.data_ptr(), hidden, hidden,
                                          attn.data_ptr(), y.data_ptr(), b, rows, world, px.rank,
                                          alias_rows.data_ptr() if n_alias else None, n_alias, _stream(x)))
        px.mark("pull + output projection")
        px.release(landing)
        ctx.graph, ctx.px, ctx.qkv, ctx.alias_rows = graph, px, qkv, alias_rows
        ctx.dims = (b, rows, heads, head_dim, heads_l, row_bytes, n_rows, tensor_bytes, code, float(eps))
        ctx.save_for_backward(x, gamma, beta, wq, wk, wv, wo, attn, z)
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _cabi.load()
        x, gamma, beta, wq, wk, wv, wo, attn, z = ctx.saved_tensors
        px, graph, qkv = ctx.px, ctx.graph, ctx.qkv
        b, rows, heads, head_dim, heads_l, row_bytes, n_rows, tensor_bytes, code, eps = ctx.dims
        hidden = heads * head_dim
        world, dev = px.world, x.device
        dy2 = dy.contiguous().view(-1, hidden)
        # output projection
        d_wo, d_bo = linear.wgrad(dy2, attn.view(-1, hidden))
        dout = (dy2 @ wo).view(b, rows, hidden)
        px.check()
        landing = px.acquire(tensor_bytes)
        px.push([dout], landing, b * rows, row_bytes, rows * row_bytes)
        px.mark("push dO")
        px.barrier()
        px.mark("barrier")
        dog = landing.view(0, (n_rows, heads_l, head_dim), x.dtype)
        if ctx.alias_rows is not None:
            _cabi.check(lib.tgt_global_rows_reduce(dog.data_ptr(), ctx.alias_rows.data_ptr(), ctx.alias_rows.numel(),
                                                   b, world * rows, heads_l * head_dim, code, _stream(dog)))
        qg, kg, vg = (qkv.view(t * tensor_bytes, (n_rows, heads_l, head_dim), x.dtype) for t in range(3))
        grads = px.acquire(3 * tensor_bytes, p2p.SOURCE)
        dqg, dkg, dvg = (grads.view(t * tensor_bytes, (n_rows, heads_l, head_dim), x.dtype) for t in range(3))
        scratch = _scratch(graph, heads_l, head_dim, code, 1, dev)
        _cabi.check(lib.tgt_sparse_attn_bwd(
            dog.data_ptr(), qg.data_ptr(), kg.data_ptr(), vg.data_ptr(), None, 0, None, z.data_ptr(),
            graph.by_dst.byref(), graph.by_src.byref(), dqg.data_ptr(), dkg.data_ptr(), dvg.data_ptr(), None,
            heads_l, head_dim, code, scratch.data_ptr(), scratch.numel(), _stream(dog)))
        px.mark("attention backward")
        px.release(qkv)
        px.release(landing)
        ctx.qkv = None
        px.barrier()
        px.mark("barrier")
        dq, dk, dv = (torch.empty((b * rows, hidden), dtype=x.dtype, device=dev) for _ in range(3))
        px.pull(grads, [dq, dk, dv], b, rows, row_bytes)
        px.mark("pull dq,dk,dv")
        px.release(grads)
        px.check()
        # the three projections and the LayerNorm (its output recomputed from the saved layer input, not
        # stored).  Running the dO push and the three pulls on a side stream under these library GEMMs was
        # measured slower (5.67 against 5.57 ms per training iteration on two GPUs): the transfers are 20-50 us
        # each and the extra graph edges and the contention for SMs cost more than the overlap hides.
        xn, stats = layer_norm.forward_with_stats(x, gamma, beta, eps)
        xn2 = xn.view(-1, hidden)
        (d_wq, d_bq), (d_wk, d_bk), (d_wv, d_bv) = (linear.wgrad(g, xn2) for g in (dq, dk, dv))
        dxn = (dq @ wq).addmm_(dk, wk).addmm_(dv, wv).view(b, rows, hidden)
        dx, d_gamma, d_beta = layer_norm.backward(dxn, x, gamma, stats)
        return (dx, d_gamma, d_beta, d_wq, d_bq, d_wk, d_bk, d_wv, d_bv, d_wo, d_bo,
                None, None, None, None, None)


def attention_block(px, x, norm, mha, edge_index, alias_rows):
    """The fused attention half of a Graphormer encoder layer (see ``_UlyssesAttentionBlock``).  ``norm`` is the
    layer's LayerNorm, ``mha`` its MultiHeadAttention (linear_q/k/v, output_layer, num_heads)."""
    b, rows, _ = x.shape
    graph = graph_for(edge_index, b * px.world * rows)
    graph.poll()
    return _UlyssesAttentionBlock.apply(x, norm.weight, norm.bias, mha.linear_q.weight, mha.linear_q.bias,
                                        mha.linear_k.weight, mha.linear_k.bias, mha.linear_v.weight,
                                        mha.linear_v.bias, mha.output_layer.weight, mha.output_layer.bias, norm.eps,
                                        mha.num_heads, graph, px, alias_rows)
