"""Device-resident edge layouts (CSR by destination, CSC by source) for the sparse attention.

The reference consumes an unsorted COO ``edge_index`` ([2, E] int64; row 0 = source = K/V row,
row 1 = destination = Q/output row; attn_module.py:146-147) in every layer of every step.  Here the
edge list is sorted once per batch into two segment layouts that all layers and all epochs reuse.
"""
from __future__ import annotations

import ctypes
from collections import OrderedDict
from typing import Optional, Union

import torch

from . import _cabi

class EdgeLayout:
    """One orientation of the graph: edges sorted by destination (``group_by=1``) or source (0).

    ``perm`` is the stable argsort of the grouping endpoint, ``seg`` that endpoint in sorted order,
    ``other`` the opposite endpoint in sorted order, ``ptr`` the row pointers (all int32, on the GPU)."""

    def __init__(self, edge_index: torch.Tensor, n_rows: int, group_by: int, defer_check: bool = False):
        lib = _cabi.load()
        dev = edge_index.device
        n_edges = int(edge_index.shape[1])
        ws = ctypes.c_size_t()
        _cabi.check(lib.tgt_edge_layout_sizes(n_rows, n_edges, ctypes.byref(ws)))
        i32 = dict(dtype=torch.int32, device=dev)
        self.ptr = torch.empty(n_rows + 1, **i32)
        self.other = torch.empty(n_edges, **i32)
        self.perm = torch.empty(n_edges, **i32)
        self.seg = torch.empty(n_edges, **i32)
        workspace = torch.empty(max(ws.value, 16), dtype=torch.uint8, device=dev)
        stream = torch.cuda.current_stream(dev).cuda_stream
        nz = lambda t: t.data_ptr() if t.numel() else None
        # deferred check: the build does not synchronise; `bad_index` is read by SparseGraph.check()
        self.bad_index = torch.zeros(1, **i32) if defer_check else None
        _cabi.check(lib.tgt_edge_layout_build(
            nz(edge_index), n_edges, n_rows, group_by, self.ptr.data_ptr(), nz(self.other), nz(self.perm),
            nz(self.seg), workspace.data_ptr(), workspace.numel(),
            self.bad_index.data_ptr() if defer_check else None, stream))
        self.n_rows, self.n_edges, self.group_by = n_rows, n_edges, group_by
        self.c = _cabi.TgtLayout(n_rows=n_rows, n_edges=n_edges, ptr=self.ptr.data_ptr(), other=nz(self.other),
                                 perm=nz(self.perm), seg=nz(self.seg))

    def byref(self):
        return ctypes.byref(self.c)


class SparseGraph:
    """Handle holding both layouts of one batch graph.  Build once, pass in place of ``edge_index``."""

    def __init__(self, edge_index: torch.Tensor, n_rows: int, defer_check: bool = False):
        """``defer_check=True`` builds without synchronising the stream (for pipelined input loops): node
        ids outside [0, n_rows) are then not raised here but by a later :meth:`check` (they are replaced by
        0 in the layout, so kernels stay in bounds)."""
        if edge_index.dim() != 2 or edge_index.shape[0] != 2:
            raise ValueError("edge_index must be [2, E]")
        if not edge_index.is_cuda:
            raise RuntimeError("torchgt_b200 runs on CUDA only: edge_index must be a CUDA tensor")
        edge_index = edge_index.to(torch.int64).contiguous()
        self.n_rows = int(n_rows)
        self.n_edges = int(edge_index.shape[1])
        self.device = edge_index.device
        self._defer = bool(defer_check)
        self.by_dst = EdgeLayout(edge_index, self.n_rows, 1, self._defer)
        self._edge_index = edge_index  # kept until by_src is built
        self._by_src: Optional[EdgeLayout] = None

    @property
    def by_src(self) -> EdgeLayout:
        """Built on first backward (inference never needs it)."""
        if self._by_src is None:
            self._by_src = EdgeLayout(self._edge_index, self.n_rows, 0, self._defer)
            self._edge_index = None
        return self._by_src

    def check(self) -> None:
        """Raise if a deferred build saw a node id outside [0, n_rows) (synchronises)."""
        for lay in (self.by_dst, self._by_src):
            if lay is not None and lay.bad_index is not None and int(lay.bad_index.item()) != 0:
                raise _cabi.TgtError(_cabi.TGT_ERR_INDEX_RANGE, f"edge_index holds a node id outside [0, {self.n_rows})")


# ---- cache: the reference passes a raw edge_index tensor to every layer ---------------------------
_CACHE_CAPACITY = 16
_IDENTITY_CAPACITY = 4  # entries pin their edge_index tensor
_by_identity: "OrderedDict[tuple, tuple]" = OrderedDict()
_by_content: "OrderedDict[tuple, SparseGraph]" = OrderedDict()
_mixers = {}


def _fingerprint(edge_index: torch.Tensor) -> tuple:
    """Content hash computed on the device (wrapping int64 arithmetic), one small sync."""
    flat = edge_index.reshape(-1)
    key = (flat.device, )
    mix = _mixers.get(key)
    if mix is None:
        g = torch.Generator(device="cpu").manual_seed(0x7067)
        mix = (torch.randint(1, 2**62, (4099,), generator=g, dtype=torch.int64) * 2 + 1).to(flat.device)
        _mixers[key] = mix
    idx = torch.arange(flat.numel(), device=flat.device) % mix.numel()
    h = ((flat + 0x9E3779B1) * mix[idx]).sum()
    return (int(h.item()), int(flat.numel()))


def graph_for(edge_index: Union[torch.Tensor, SparseGraph], n_rows: int) -> SparseGraph:
    """Return the cached ``SparseGraph`` of ``edge_index`` (building it on first sight).

    Lookup is by tensor identity first (same object, unmodified: the 4 layers of one step), then by
    device-side content hash (the reference's loops upload a fresh copy of the same edges on every
    iteration, main_sp_sparse_node_level.py:178-182).
    """
    if isinstance(edge_index, SparseGraph):
        if edge_index.n_rows != n_rows:
            raise ValueError(f"graph has {edge_index.n_rows} rows, tensors have {n_rows}")
        return edge_index
    ident = (id(edge_index), edge_index.data_ptr(), edge_index._version, tuple(edge_index.shape), n_rows)
    hit = _by_identity.get(ident)
    if hit is not None and hit[0] is edge_index:
        _by_identity.move_to_end(ident)
        return hit[1]
    content = (_fingerprint(edge_index), n_rows, edge_index.device)
    graph = _by_content.get(content)
    if graph is None:
        graph = SparseGraph(edge_index, n_rows)
        _by_content[content] = graph
        while len(_by_content) > _CACHE_CAPACITY:
            _by_content.popitem(last=False)
    else:
        _by_content.move_to_end(content)
    _by_identity[ident] = (edge_index, graph)
    while len(_by_identity) > _IDENTITY_CAPACITY:
        _by_identity.popitem(last=False)
    return graph


def clear_graph_cache() -> None:
    _by_identity.clear()
    _by_content.clear()
