"""tgt_sparse_attn_fwd_noalloc: the forward for hosts that can hand the library no scratch memory
(their own arena owns the GPU, or they must stay clear of cudaMalloc).  It has to give what
tgt_sparse_attn_fwd gives, call after call, out of the scratch array built into the library.

Collected last on purpose: a failure here leaves every other test already run."""
import ctypes

import pytest
import torch

from helpers import TOL_BF16, TOL_F32, random_graph, rel_err
from oracle import sparse_attn_oracle as sao

pytestmark = pytest.mark.gpu


def _forward_both_ways(seed, n, heads, head_dim, with_bias, dtype=torch.float32):
    """Returns the results of both entry points and of the float64 oracle (evaluated on the inputs as the
    kernels see them, i.e. rounded to bf16 when that is the storage type)."""
    from torchgt_b200 import SparseGraph, _cabi
    lib = _cabi.load()
    code = _cabi.TGT_F32 if dtype == torch.float32 else _cabi.TGT_BF16
    gen = torch.Generator().manual_seed(seed)
    ei = random_graph(seed, n, 6.0)
    graph = SparseGraph(ei.cuda(), n)
    q, k, v = (torch.randn(n, heads, head_dim, generator=gen).to(dtype).cuda() for _ in range(3))
    bias = (torch.randn(ei.shape[1], generator=gen) * 0.2).cuda() if with_bias else None
    oracle_out, oracle_z = sao.forward_closed_form(q.float().cpu(), k.float().cpu(), v.float().cpu(), ei,
                                                   bias.cpu() if with_bias else None)
    bias_ptr, bias_heads = (bias.data_ptr(), 1) if with_bias else (None, 0)
    stream = torch.cuda.current_stream().cuda_stream

    # reference: the existing entry point with scratch allocated by the caller
    nbytes = ctypes.c_size_t()
    _cabi.check(lib.tgt_sparse_attn_scratch_bytes(graph.by_dst.byref(), None, heads, head_dim, code, 0,
                                                  ctypes.byref(nbytes)))
    scratch = torch.empty(max(nbytes.value, 16), dtype=torch.uint8, device="cuda")
    out_ref = torch.empty_like(q)
    z_ref = torch.empty(n, heads, device="cuda")
    _cabi.check(lib.tgt_sparse_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), bias_ptr, bias_heads,
                                        graph.by_dst.byref(), out_ref.data_ptr(), z_ref.data_ptr(), heads, head_dim,
                                        code, scratch.data_ptr(), scratch.numel(), stream))
    # the entry point under test: no scratch argument at all; outputs start as garbage
    out = torch.full_like(q, float("nan"))
    z = torch.full((n, heads), float("nan"), device="cuda")
    _cabi.check(lib.tgt_sparse_attn_fwd_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), bias_ptr, bias_heads,
                                                graph.by_dst.byref(), out.data_ptr(), z.data_ptr(), heads, head_dim,
                                                code, stream))
    torch.cuda.synchronize()
    return out, z, out_ref, z_ref, oracle_out, oracle_z


def test_two_calls_in_a_row_match_the_allocating_entry_point():
    from torchgt_b200 import _cabi
    lib = _cabi.load()
    lib.tgt_debug_set_tile_edges(8)        # many tiles, so rows do cross tiles and the scratch is used
    try:
        # second call: other sizes and values, so leftovers of the first call would show
        # The cases cover both ways rows that cross tiles are finished: inside the walk kernel (rows of more
        # than 64 bytes: arrival counters in the built-in array) and by a second kernel (rows of at most 64
        # bytes: 1 head x 8 and 2 heads x 8 in fp32), and both storage types.
        cases = ((1, 3000, 8, 8, True, torch.float32), (2, 1777, 4, 16, False, torch.float32),
                 (3, 2500, 1, 8, True, torch.float32), (4, 2100, 2, 8, False, torch.float32),
                 (5, 2800, 8, 8, True, torch.bfloat16), (6, 1900, 2, 8, True, torch.bfloat16))
        for seed, n, heads, head_dim, with_bias, dtype in cases:
            out, z, out_ref, z_ref, oracle_out, oracle_z = _forward_both_ways(seed, n, heads, head_dim, with_bias, dtype)
            tol = TOL_F32 if dtype == torch.float32 else TOL_BF16
            assert torch.isfinite(out.float()).all() and torch.isfinite(z).all()
            assert rel_err(out.float(), out_ref.float()) < tol          # the allocating entry point
            assert rel_err(z, z_ref) < tol
            assert rel_err(out.float(), oracle_out) < tol               # the float64 oracle
            assert rel_err(z, oracle_z) < tol
    finally:
        lib.tgt_debug_set_tile_edges(0)


def test_a_graph_beyond_the_built_in_scratch_is_refused_before_anything_runs():
    from torchgt_b200 import _cabi
    lib = _cabi.load()
    lib.tgt_debug_set_tile_edges(0)
    dummy = torch.zeros(64, dtype=torch.int32, device="cuda")
    # 200 million edges would need far more carry space than the library holds; the pointers are never used
    layout = _cabi.TgtLayout(n_rows=1000, n_edges=200_000_000, ptr=dummy.data_ptr(), other=dummy.data_ptr(),
                             perm=dummy.data_ptr(), seg=dummy.data_ptr())
    rc = lib.tgt_sparse_attn_fwd_noalloc(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), None, 0,
                                         ctypes.byref(layout), dummy.data_ptr(), dummy.data_ptr(), 8, 8,
                                         _cabi.TGT_F32, None)
    assert rc == 4                                       # TGT_ERR_WORKSPACE
    assert "built-in scratch" in _cabi.last_error()
    torch.cuda.synchronize()                             # the context is untouched
