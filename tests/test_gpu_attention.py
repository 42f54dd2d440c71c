"""The fused CUDA sparse attention against the CPU oracle and the reference's golden vectors."""
import numpy as np
import pytest
import torch

from helpers import TOL_BF16, TOL_F32, clustered_graph, load_golden, random_graph, rel_err
from oracle import sparse_attn_oracle as sao

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, params=[1, 2], ids=["lanes16", "lanes32"])
def _lane_widths(request):
    """Every test of this file runs with both lane widths of the walk kernels forced: 16 bytes, and 32
    bytes wherever they apply (fp32 heads of 32 to 128 bytes; other shapes fall back to 16).  The
    library's own choice per head size is one of the two; the other test files run with that choice."""
    from torchgt_b200 import _cabi
    _cabi.check(_cabi.load().tgt_debug_set_lane_mode(request.param))
    yield request.param
    _cabi.check(_cabi.load().tgt_debug_set_lane_mode(0))
    _cabi.check(_cabi.load().tgt_debug_set_tile_edges(0))


def _run_cuda(q, k, v, ei, dout, bias=None, dtype=torch.float32, tile_edges=0, bias_grad=True):
    """tile_edges > 0 forces that many edges per lane group, i.e. many small tiles."""
    from torchgt_b200 import SparseGraph, _cabi, sparse_graph_attention
    _cabi.check(_cabi.load().tgt_debug_set_tile_edges(tile_edges))
    dev = "cuda"
    qc, kc, vc = (torch.as_tensor(t).to(dev, dtype).requires_grad_() for t in (q, k, v))
    bc = None
    if bias is not None:
        bc = torch.as_tensor(bias).to(dev, torch.float32).requires_grad_(bias_grad)
    graph = SparseGraph(torch.as_tensor(ei).to(dev), qc.shape[0])
    out = sparse_graph_attention(qc, kc, vc, graph, bc)
    out.backward(torch.as_tensor(dout).to(dev, dtype))
    res = dict(out=out.detach(), dq=qc.grad, dk=kc.grad, dv=vc.grad)
    if bc is not None and bias_grad:
        res["dbias"] = bc.grad
    return res


def _check_against_closed_form(q, k, v, ei, dout, bias, res, tol, per_head_bias=True):
    out, _ = sao.forward_closed_form(q, k, v, ei, bias)
    dq, dk, dv, dt = sao.backward_closed_form(q, k, v, ei, dout, bias)
    assert rel_err(res["out"].float(), out) < tol
    assert rel_err(res["dq"].float(), dq) < tol
    assert rel_err(res["dk"].float(), dk) < tol
    assert rel_err(res["dv"].float(), dv) < tol
    if "dbias" in res:
        ref = dt if per_head_bias else dt.sum(axis=1)
        assert rel_err(res["dbias"], ref) < tol


@pytest.mark.parametrize("case", ["small_nobias", "clamped_nobias", "dense_bias", "one_head", "wide_head"])
def test_reference_golden_vectors(case):
    g = load_golden(f"attn_{case}.npz")
    bias = None
    if "attn_bias" in g:
        bias = sao.dense_bias_to_edges(torch.from_numpy(g["attn_bias"]), torch.from_numpy(g["edge_index"])).numpy()
    for tile_edges in (0, 4, 8):   # small tiles: most rows cross lane-group and tile boundaries
        res = _run_cuda(g["q"], g["k"], g["v"], g["edge_index"], g["dout"], bias, tile_edges=tile_edges)
        assert rel_err(res["out"], g["out"]) < TOL_F32
        assert rel_err(res["dq"], g["dq"]) < TOL_F32
        assert rel_err(res["dk"], g["dk"]) < TOL_F32
        assert rel_err(res["dv"], g["dv"]) < TOL_F32
        if bias is not None:
            n, h = g["q"].shape[0], g["q"].shape[1]
            dense = np.zeros((1, h, n, n))
            np.add.at(dense[0].transpose(1, 2, 0), (g["edge_index"][0], g["edge_index"][1]),
                      res["dbias"].double().cpu().numpy())
            assert rel_err(dense, g["dattn_bias"]) < TOL_F32
        deg = np.bincount(g["edge_index"][1], minlength=g["q"].shape[0])
        assert torch.all(res["out"][torch.from_numpy(deg == 0).cuda()] == 0)


SHAPES = [  # heads, head_dim  (fp32 lanes per row: heads*head_dim/4)
    (1, 8), (2, 8), (4, 8), (8, 8), (4, 16), (8, 16), (2, 32), (1, 64), (3, 8), (6, 16), (16, 8), (12, 8),
    (1, 4), (1, 128), (2, 128),
]


@pytest.mark.parametrize("heads,head_dim", SHAPES)
@pytest.mark.parametrize("bias_kind", ["none", "edge", "edge_head"])
def test_shapes_fp32(heads, head_dim, bias_kind):
    n = 300
    ei = random_graph(100 + heads * head_dim, n, 5.0)
    gen = torch.Generator().manual_seed(heads * 1000 + head_dim)
    q, k = (torch.randn(n, heads, head_dim, generator=gen) * 1.5 for _ in range(2))
    v, dout = (torch.randn(n, heads, head_dim, generator=gen) for _ in range(2))
    e = ei.shape[1]
    bias = {"none": None, "edge": torch.randn(e, generator=gen) * 0.3,
            "edge_head": torch.randn(e, heads, generator=gen) * 0.3}[bias_kind]
    for tile_edges in (0, 8):
        res = _run_cuda(q, k, v, ei, dout, bias, tile_edges=tile_edges)
        _check_against_closed_form(q, k, v, ei, dout, bias, res, TOL_F32, per_head_bias=bias_kind == "edge_head")


@pytest.mark.parametrize("heads,head_dim", [(1, 8), (2, 8), (8, 8), (4, 16), (8, 16), (2, 64), (3, 8)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_shapes_bf16(heads, head_dim, with_bias):
    n = 300
    ei = random_graph(200 + heads * head_dim, n, 5.0)
    gen = torch.Generator().manual_seed(heads * 77 + head_dim)
    # the oracle sees the bf16-rounded inputs
    q, k, v, dout = (torch.randn(n, heads, head_dim, generator=gen).bfloat16().float() for _ in range(4))
    bias = torch.randn(ei.shape[1], generator=gen) * 0.3 if with_bias else None
    res = _run_cuda(q, k, v, ei, dout, bias, dtype=torch.bfloat16, tile_edges=8)
    assert res["out"].dtype == torch.bfloat16 and res["dq"].dtype == torch.bfloat16
    _check_against_closed_form(q, k, v, ei, dout, bias, res, TOL_BF16, per_head_bias=False)


def test_edge_cases_empty_graph_single_row_and_self_loop_only():
    gen = torch.Generator().manual_seed(0)
    q, k, v, dout = (torch.randn(6, 8, 8, generator=gen) for _ in range(4))
    # no edges at all: output and all gradients are exactly zero (with or without an empty bias)
    res = _run_cuda(q, k, v, torch.zeros((2, 0), dtype=torch.long), dout)
    for t in res.values():
        assert torch.count_nonzero(t) == 0
    res = _run_cuda(q, k, v, torch.zeros((2, 0), dtype=torch.long), dout, bias=torch.zeros(0), bias_grad=False)
    assert torch.count_nonzero(res["out"]) == 0
    # one row, one self loop: out = v * w/(w + 1e-6)
    loop = torch.zeros((2, 1), dtype=torch.long)
    res = _run_cuda(q[:1], k[:1], v[:1], loop, dout[:1])
    ref_out, _ = sao.forward_closed_form(q[:1], k[:1], v[:1], loop)
    assert rel_err(res["out"], ref_out) < TOL_F32
    # with a single in-edge the softmax gradient cancels to ~1e-6 * |dO|: compare absolutely
    dq, dk, dv, _ = sao.backward_closed_form(q[:1], k[:1], v[:1], loop, dout[:1])
    assert np.abs(res["dq"].cpu().numpy() - dq).max() < 1e-5 and np.abs(res["dk"].cpu().numpy() - dk).max() < 1e-5
    assert rel_err(res["dv"], dv) < TOL_F32
    # duplicate edges count twice
    ei = torch.tensor([[1, 1, 2, 2, 2], [0, 0, 0, 3, 3]])
    res = _run_cuda(q, k, v, ei, dout)
    _check_against_closed_form(q, k, v, ei, dout, None, res, TOL_F32)


def test_clamp_boundaries_and_saturated_scores():
    n, heads, head_dim = 64, 8, 8
    gen = torch.Generator().manual_seed(3)
    ei = random_graph(9, n, 6.0)
    q, k = (torch.randn(n, heads, head_dim, generator=gen) * 4.0 for _ in range(2))   # most |raw| > 5
    v, dout = (torch.randn(n, heads, head_dim, generator=gen) for _ in range(2))
    res = _run_cuda(q, k, v, ei, dout)
    _check_against_closed_form(q, k, v, ei, dout, None, res, TOL_F32)
    # raw exactly +5 and -5 (head_dim 4 makes the scale an exact 1/2): the clamp passes the gradient
    # on both boundaries (inclusive mask, as torch.clamp's backward does)
    q2 = torch.zeros(2, 1, 4); k2 = torch.zeros(2, 1, 4)
    q2[0, 0, 0], k2[1, 0, 0] = 10.0, 1.0       # edge 1 -> 0 has raw = 5
    q2[1, 0, 0], k2[0, 0, 0] = -10.0, 1.0      # edge 0 -> 1 has raw = -5
    v2, d2 = torch.randn(2, 1, 4, generator=gen), torch.randn(2, 1, 4, generator=gen)
    ei2 = torch.tensor([[1, 0, 0, 1], [0, 1, 0, 1]])
    res = _run_cuda(q2, k2, v2, ei2, d2)
    ref_out, _ = sao.forward_closed_form(q2, k2, v2, ei2)
    assert rel_err(res["out"], ref_out) < TOL_F32
    # weights e^5 and e^-5 leave gradients of ~1e-5 from operands of ~10: compare absolutely, and
    # check that the boundary edges do carry a gradient (an exclusive mask would give exactly 0)
    dq, dk, dv, _ = sao.backward_closed_form(q2, k2, v2, ei2, d2)
    assert abs(dq[1, 0, 0]) > 1e-6
    for name, ref in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert np.abs(res[name].double().cpu().numpy() - ref).max() < 1e-6, name
    qr, kr, vr = (t.clone().requires_grad_() for t in (q2, k2, v2))
    sao.sparse_attention_ops(qr, kr, vr, ei2).backward(d2)
    assert (res["dq"].cpu() - qr.grad).abs().max() < 1e-6 and (res["dk"].cpu() - kr.grad).abs().max() < 1e-6


@pytest.mark.parametrize("heads", [8, 4, 2, 1])
def test_long_hub_row_and_column(heads):
    """A global-token-like row with in-degree and out-degree n (split into chunks and reduced)."""
    n = 5000
    gen = torch.Generator().manual_seed(heads)
    ei = random_graph(21, n, 2.0, hub=True)
    q, k, v, dout = (torch.randn(n, heads, 8, generator=gen) for _ in range(4))
    bias = torch.randn(ei.shape[1], generator=gen) * 0.1
    res = _run_cuda(q, k, v, ei, dout, bias)
    _check_against_closed_form(q, k, v, ei, dout, bias, res, TOL_F32, per_head_bias=False)


def test_every_row_is_written_even_when_buffers_hold_garbage():
    """Rows without edges, leading / trailing empty rows and gaps must be zero-filled by the kernels."""
    from torchgt_b200 import SparseGraph, _cabi
    import ctypes
    lib = _cabi.load()
    n, h, d = 500, 8, 8
    gen = torch.Generator().manual_seed(8)
    src = torch.randint(0, n, (900,), generator=gen)
    dst = torch.randint(100, 400, (900,), generator=gen)      # rows 0..99 and 400..499 have no in-edges
    dst = dst[(dst % 5) != 0]                                  # and every fifth row in between
    ei = torch.stack([src[: dst.numel()], dst])
    q, k, v, dout = (torch.randn(n, h, d, generator=gen) for _ in range(4))
    for tile_edges in (0, 4):
        res = _run_cuda(q, k, v, ei, dout, None, tile_edges=tile_edges)
        _check_against_closed_form(q, k, v, ei, dout, None, res, TOL_F32)
        for t in res.values():
            assert torch.isfinite(t).all()


def test_run_to_run_bitwise_determinism():
    ei, n = clustered_graph(7, 8000, 8, 40000, 0.17)
    gen = torch.Generator().manual_seed(1)
    q, k, v, dout = (torch.randn(n, 8, 8, generator=gen) for _ in range(4))
    bias = torch.randn(ei.shape[1], generator=gen) * 0.1
    a = _run_cuda(q, k, v, ei, dout, bias)
    b = _run_cuda(q, k, v, ei, dout, bias)
    for name in a:
        assert torch.equal(a[name], b[name]), name


def test_node_level_training_graph_4096_nodes_vs_ops_oracle():
    """4,096 nodes + global node, 8 random in-edges per node + self loops, through the reference's edge
    helpers; compared with the op-by-op fp32 restatement of the reference and its autograd."""
    from oracle import edge_layout_oracle as elo
    gen = torch.Generator().manual_seed(42)
    n = 4096
    dst = torch.arange(n).repeat_interleave(8)
    src = torch.randint(0, n, (n * 8,), generator=gen)
    raw = torch.cat([torch.stack([src, dst]), torch.stack([torch.arange(n), torch.arange(n)])], dim=1)
    ei = torch.from_numpy(elo.fix_edge_index(raw.numpy(), n))
    assert ei.shape[1] == 45056
    q, k, v, dout = (torch.randn(n + 1, 8, 8, generator=gen) for _ in range(4))
    res = _run_cuda(q, k, v, ei, dout)
    qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
    out = sao.sparse_attention_ops(qr, kr, vr, ei)
    out.backward(dout)
    assert rel_err(res["out"], out) < TOL_F32
    assert rel_err(res["dq"], qr.grad) < TOL_F32
    assert rel_err(res["dk"], kr.grad) < TOL_F32
    assert rel_err(res["dv"], vr.grad) < TOL_F32
    _check_against_closed_form(q, k, v, ei, dout, None, res, TOL_F32)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_F32), (torch.bfloat16, TOL_BF16)])
def test_benchmark_workload_64k_nodes(dtype, tol):
    """The 64K-node micro-benchmark shape: 64,001 rows, ~526K edges, 8 heads x 8, scalar edge bias."""
    ei, n = clustered_graph(1234, 64000, 8, 334000, 0.17)
    gen = torch.Generator().manual_seed(1234)
    q, k, v, dout = (torch.randn(n, 8, 8, generator=gen).to(dtype).float() for _ in range(4))
    bias = torch.randn(ei.shape[1], generator=gen) * 0.1
    res = _run_cuda(q, k, v, ei, dout, bias, dtype=dtype)
    _check_against_closed_form(q, k, v, ei, dout, bias, res, tol, per_head_bias=False)


def test_size_independent_properties_at_full_size():
    """Properties that need no oracle: out is linear in V; with V = 1 every output equals Z/(Z+1e-6);
    permuting the edge list leaves the result unchanged up to summation order."""
    from torchgt_b200 import SparseGraph, sparse_graph_attention
    ei, n = clustered_graph(99, 64000, 8, 334000, 0.17)
    gen = torch.Generator().manual_seed(5)
    q, k, v1, v2 = (torch.randn(n, 8, 8, generator=gen).cuda() for _ in range(4))
    graph = SparseGraph(ei.cuda(), n)
    o1 = sparse_graph_attention(q, k, v1, graph)
    o2 = sparse_graph_attention(q, k, v2, graph)
    o12 = sparse_graph_attention(q, k, 2.0 * v1 - 3.0 * v2, graph)
    assert rel_err(o12, 2.0 * o1 - 3.0 * o2) < TOL_F32
    ones = sparse_graph_attention(q, k, torch.ones_like(v1), graph)
    deg = torch.bincount(ei[1], minlength=n).cuda()
    assert torch.all(ones[deg == 0] == 0)
    assert torch.all((ones[deg > 0] > 0.99) & (ones[deg > 0] <= 1.0))
    shuffled = ei[:, torch.randperm(ei.shape[1], generator=gen)]
    o1s = sparse_graph_attention(q, k, v1, SparseGraph(shuffled.cuda(), n))
    assert rel_err(o1s, o1) < TOL_F32


def test_no_cpu_fallback_and_argument_errors():
    from torchgt_b200 import sparse_graph_attention
    from torchgt_b200._cabi import TgtError
    q = torch.randn(4, 8, 8)
    ei = torch.tensor([[0, 1], [1, 2]])
    with pytest.raises(RuntimeError, match="CUDA"):
        sparse_graph_attention(q, q, q, ei)
    qc = q.cuda()
    with pytest.raises(TgtError, match="UNSUPPORTED"):      # head_dim 12 is not a power of two
        sparse_graph_attention(torch.randn(4, 2, 12).cuda(), torch.randn(4, 2, 12).cuda(),
                               torch.randn(4, 2, 12).cuda(), ei.cuda())
    with pytest.raises(ValueError):
        sparse_graph_attention(qc, qc, qc, ei.cuda(), bias=torch.zeros(5).cuda())
    with pytest.raises(TypeError):
        sparse_graph_attention(qc.half(), qc.half(), qc.half(), ei.cuda())


def test_long_sequence_batch_870k_nodes_sampled_rows_against_the_oracle():
    """870,001 rows, 18.2 M power-law edges.  The CPU oracle cannot hold the whole problem, but every
    output row depends only on that row's in-edges (and every dK/dV row on its out-edges and the
    statistics of their destinations), so sampled rows are checked exactly against the fp64 oracle run
    on the sub-problem, plus full-size properties."""
    from torchgt_b200 import SparseGraph, sparse_graph_attention
    from torchgt_b200.synthetic import benchmark_870k
    ei, n = benchmark_870k()
    gen = torch.Generator().manual_seed(870)
    q, k, v, dout = (torch.randn(n, 8, 8, generator=gen) for _ in range(4))
    bias = torch.randn(ei.shape[1], generator=gen) * 0.1
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    bc = bias.cuda().requires_grad_()
    graph = SparseGraph(ei.cuda(), n)
    out = sparse_graph_attention(qc, kc, vc, graph, bc)
    out.backward(dout.cuda())
    out2 = sparse_graph_attention(qc.detach(), kc.detach(), vc.detach(), graph, bc.detach())
    assert torch.equal(out.detach(), out2)                                   # bitwise reproducible
    deg_in = torch.bincount(ei[1], minlength=n)
    assert torch.all(out.detach()[(deg_in == 0).cuda()] == 0)

    # ---- destination rows: out and dq from their in-edges only
    rows = torch.cat([torch.tensor([0]), torch.randint(1, n, (1500,), generator=gen)]).unique()
    is_sampled = torch.zeros(n, dtype=torch.bool); is_sampled[rows] = True
    sel = is_sampled[ei[1]]
    sub_ei, sub_bias = ei[:, sel], bias[sel]
    ref_out, _ = sao.forward_closed_form(q, k, v, sub_ei, sub_bias)
    dq, _, _, dt = sao.backward_closed_form(q, k, v, sub_ei, dout, sub_bias)
    assert rel_err(out.detach().cpu()[rows], ref_out[rows.numpy()]) < TOL_F32
    assert rel_err(qc.grad.cpu()[rows], dq[rows.numpy()]) < TOL_F32
    assert rel_err(bc.grad.cpu()[sel], dt.sum(axis=1)) < TOL_F32

    # ---- source rows: dk and dv from their out-edges; the destinations' statistics need all in-edges
    # of those destinations
    srcs = torch.randint(1, n, (300,), generator=gen).unique()
    is_src = torch.zeros(n, dtype=torch.bool); is_src[srcs] = True
    dests = ei[1][is_src[ei[0]]].unique()
    is_dest = torch.zeros(n, dtype=torch.bool); is_dest[dests] = True
    sel2 = is_dest[ei[1]]
    sub2, bias2 = ei[:, sel2], bias[sel2]
    _, dk, dv, _ = sao.backward_closed_form(q, k, v, sub2, dout, bias2)
    # rows in `srcs` have ALL their out-edges inside sub2 (every destination of theirs is in `dests`)
    assert rel_err(kc.grad.cpu()[srcs], dk[srcs.numpy()]) < TOL_F32
    assert rel_err(vc.grad.cpu()[srcs], dv[srcs.numpy()]) < TOL_F32


def test_many_small_random_graphs_with_forced_tile_sizes():
    """Randomised sweep over the segmented walk's corner cases: tiny tiles so that rows cross lane-group
    and tile boundaries everywhere, rows without edges at the start, in the middle and at the end, hubs,
    duplicates, every head split; forward and all gradients against the fp64 oracle."""
    rng = np.random.default_rng(2024)
    for trial in range(60):
        n = int(rng.integers(1, 70))
        e = int(rng.integers(0, 500))
        heads = int(rng.choice([1, 2, 3, 4, 8]))
        head_dim = int(rng.choice([4, 8, 16]))
        tile_edges = int(rng.choice([0, 4, 8, 12, 16, 20]))
        lo, hi = sorted(rng.integers(0, n, size=2).tolist())
        hi = max(hi, lo + 1) if n > 1 else 1
        dst = rng.integers(lo, hi, size=e)                       # leading / trailing rows without in-edges
        src = rng.integers(0, n, size=e)
        if e > 10 and rng.random() < 0.5:
            dst[: e // 2] = dst[0]                               # a hub row
        if e > 10 and rng.random() < 0.5:
            src[e // 3: 2 * e // 3] = src[-1]                    # a hub column
        ei = torch.from_numpy(np.stack([src, dst])).long()
        gen = torch.Generator().manual_seed(trial)
        scale = float(rng.choice([0.5, 1.5, 4.0]))
        q, k = (torch.randn(n, heads, head_dim, generator=gen) * scale for _ in range(2))
        v, dout = (torch.randn(n, heads, head_dim, generator=gen) for _ in range(2))
        kind = rng.choice(["none", "edge", "edge_head"])
        bias = {"none": None, "edge": torch.randn(e, generator=gen) * 0.3,
                "edge_head": torch.randn(e, heads, generator=gen) * 0.3}[str(kind)]
        res = _run_cuda(q, k, v, ei, dout, bias, tile_edges=tile_edges)
        ref_out, _ = sao.forward_closed_form(q, k, v, ei, bias)
        dq, dk, dv, dt = sao.backward_closed_form(q, k, v, ei, dout, bias)
        ctx = (trial, n, e, heads, head_dim, tile_edges, str(kind))
        # absolute floor: rows with a single in-edge have gradients that cancel to ~1e-7 of their operands
        floor = 1e-6 * max(1.0, scale * scale)
        for name, ref in (("out", ref_out), ("dq", dq), ("dk", dk), ("dv", dv)):
            err = np.abs(res[name].double().cpu().numpy() - ref).max() if ref.size else 0.0
            assert err < TOL_F32 * max(float(np.abs(ref).max()) if ref.size else 0.0, 0.0) + floor, (name, err, ctx)
        if bias is not None and e > 0:
            ref = dt if str(kind) == "edge_head" else dt.sum(axis=1)
            err = np.abs(res["dbias"].double().cpu().numpy() - ref).max()
            assert err < TOL_F32 * float(np.abs(ref).max()) + floor, ("dbias", err, ctx)


@pytest.mark.parametrize("heads,head_dim,dtype", [(1, 8, torch.float32), (2, 8, torch.float32), (8, 8, torch.float32),
                                                  (8, 8, torch.bfloat16), (4, 16, torch.float32)])
def test_strided_rows_k_and_v_side_by_side_give_the_same_bits(heads, head_dim, dtype):
    """tgt_sparse_attn_fwd_strided / _bwd_strided: q and dO with padded rows, K and V of a row stored side by
    side ([N, 2, H, D], what the woven push of the exchange delivers).  Only addresses change, so every
    result must equal the dense call bit for bit."""
    import ctypes
    from torchgt_b200 import SparseGraph, _cabi
    lib = _cabi.load()
    n = 700
    ei = random_graph(31 + heads, n, 6.0)
    graph = SparseGraph(ei.cuda(), n)
    gen = torch.Generator().manual_seed(heads + head_dim)
    q, k, v, dout = (torch.randn(n, heads, head_dim, generator=gen).to(dtype).cuda() for _ in range(4))
    bias = (torch.randn(ei.shape[1], generator=gen) * 0.2).cuda()
    code = _cabi.TGT_F32 if dtype == torch.float32 else _cabi.TGT_BF16
    es = q.element_size()
    row = heads * head_dim * es
    kv = torch.stack([k, v], dim=1).contiguous()                       # [n, 2, H, D]
    q_pad = torch.zeros(n, 2 * heads, head_dim, dtype=dtype, device="cuda"); q_pad[:, :heads] = q
    do_pad = torch.zeros(n, 3 * heads, head_dim, dtype=dtype, device="cuda"); do_pad[:, :heads] = dout
    stream = torch.cuda.current_stream().cuda_stream
    _cabi.check(lib.tgt_debug_set_tile_edges(8))
    nb = ctypes.c_size_t()
    results = []
    for (qq, q_row, kk, vv, kv_row, dd, d_row) in ((q, row, k, v, row, dout, row),
                                                   (q_pad, 2 * row, kv[:, 0], kv[:, 1], 2 * row, do_pad, 3 * row)):
        out, z = torch.empty_like(q), torch.empty(n, heads, device="cuda")
        dq, dk, dv, dbias = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q), torch.empty_like(bias)
        _cabi.check(lib.tgt_sparse_attn_scratch_bytes(graph.by_dst.byref(), graph.by_src.byref(), heads, head_dim,
                                                      code, 1, ctypes.byref(nb)))
        scratch = torch.empty(max(nb.value, 16), dtype=torch.uint8, device="cuda")
        _cabi.check(lib.tgt_sparse_attn_fwd_strided(qq.data_ptr(), q_row, kk.data_ptr(), vv.data_ptr(), kv_row,
                                                    bias.data_ptr(), 1, graph.by_dst.byref(), out.data_ptr(),
                                                    z.data_ptr(), heads, head_dim, code, scratch.data_ptr(),
                                                    scratch.numel(), stream))
        _cabi.check(lib.tgt_sparse_attn_bwd_strided(dd.data_ptr(), d_row, qq.data_ptr(), q_row, kk.data_ptr(),
                                                    vv.data_ptr(), kv_row, bias.data_ptr(), 1, out.data_ptr(),
                                                    z.data_ptr(), graph.by_dst.byref(), graph.by_src.byref(),
                                                    dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dbias.data_ptr(),
                                                    heads, head_dim, code, scratch.data_ptr(), scratch.numel(), stream,
                                                    0))
        torch.cuda.synchronize()
        results.append((out, z, dq, dk, dv, dbias))
    for a, b in zip(*results):
        assert torch.equal(a, b)
    # and they are right
    ref_out, _ = sao.forward_closed_form(q.float(), k.float(), v.float(), ei, bias)
    assert rel_err(results[1][0].float(), ref_out) < (TOL_F32 if dtype == torch.float32 else TOL_BF16)


@pytest.mark.parametrize("heads,head_dim,dtype", [(1, 8, torch.float32), (2, 8, torch.float32), (8, 8, torch.float32),
                                                  (8, 8, torch.bfloat16), (2, 64, torch.float32)])
@pytest.mark.parametrize("with_bias", [False, True])
def test_dependent_launches_change_no_bit(heads, head_dim, dtype, with_bias):
    """tgt_debug_set_dependent_launch: the kernels of a call chained with programmatic dependent launches in
    every combination of links, on a graph cut into many tiles, against the same call with ordinary launches;
    twice in a row each, so that a kernel that ran ahead of the one before it would show."""
    from torchgt_b200 import _cabi
    lib = _cabi.load()
    n = 3000
    ei = random_graph(77 + heads, n, 7.0)
    gen = torch.Generator().manual_seed(3 * heads + head_dim)
    q, k, v, dout = (torch.randn(n, heads, head_dim, generator=gen) for _ in range(4))
    bias = torch.randn(ei.shape[1], generator=gen) * 0.2 if with_bias else None
    results = {}
    try:
        for links in (0, 1, 2, 4, 5, 7):
            _cabi.check(lib.tgt_debug_set_dependent_launch(links))
            for _ in range(2):
                results.setdefault(links, []).append(_run_cuda(q, k, v, ei, dout, bias, dtype=dtype, tile_edges=8))
    finally:
        _cabi.check(lib.tgt_debug_set_dependent_launch(5))
    assert lib.tgt_debug_set_dependent_launch(8) != 0
    _cabi.check(lib.tgt_debug_set_dependent_launch(5))
    base = results[0][0]
    for links, runs in results.items():
        for res in runs:
            for name in base:
                assert torch.equal(res[name], base[name]), (links, name)
    _check_against_closed_form(q.to(dtype).float(), k.to(dtype).float(), v.to(dtype).float(), ei,
                               dout.to(dtype).float(), bias, {n_: t for n_, t in base.items() if n_ != "dbias"},
                               TOL_F32 if dtype == torch.float32 else TOL_BF16)
