"""The drop-in ``CoreAttention`` module through every call form the reference's models use."""
import pytest
import torch

from helpers import TOL_F32, random_graph, rel_err
from oracle import sparse_attn_oracle as sao

pytestmark = pytest.mark.gpu


def _inputs(b, n, h, d, seed=0):
    gen = torch.Generator().manual_seed(seed)
    return [torch.randn(b, n, h, d, generator=gen) for _ in range(3)]


def test_model_call_form_and_constructor_variants():
    from torchgt_b200 import CoreAttention
    n, h, d = 200, 8, 8
    q, k, v = _inputs(1, n, h, d)
    ei = random_graph(1, n, 4.0)
    ref = sao.sparse_attention_ops(q[0], k[0], v[0], ei).reshape(1, n, h * d)
    for ctor in ((h * d, 0.1, h, 1), (h * d, 0.1, h), (h * d, 0.1, h, "cuda")):
        core = CoreAttention(*ctor)
        assert core.hidden_size_per_attention_head == d and core.num_heads == h
        assert core.num_attention_heads_per_partition == h and abs(core.scale - d ** 0.5) < 1e-12
        assert len(list(core.state_dict())) == 0
        out = core(q.cuda(), k.cuda(), v.cuda(), None, ei.cuda(), "sparse")
        assert out.shape == (1, n, h * d)
        assert rel_err(out, ref) < TOL_F32
        out = core(q.cuda(), k.cuda(), v.cuda(), attn_bias=None, edge_index=ei.cuda(), attn_type="sparse")
        assert rel_err(out, ref) < TOL_F32
        # micro-benchmark form: forward(q, k, v, edge_index)
        assert rel_err(core(q.cuda(), k.cuda(), v.cuda(), ei.cuda()), ref) < TOL_F32
        assert rel_err(core.sparse_attention(q.cuda(), k.cuda(), v.cuda(), ei.cuda()), ref) < TOL_F32
        # Graphormer argument order (k, q, v)
        o3 = core.sparse_attention_bias(k.cuda(), q.cuda(), v.cuda(), ei.cuda(), None)
        assert o3.shape == (n, h, d) and rel_err(o3.reshape(1, n, -1), ref) < TOL_F32
    with pytest.raises(NotImplementedError):
        core(q.cuda(), k.cuda(), v.cuda(), None, ei.cuda(), "full")
    # GT argument order (q, k, v): models/gt_dist_node_level.py:83, models/gt_graph_level.py:83
    from torchgt_b200.attn_module import CoreAttentionQKV
    from torchgt_b200.gt import CoreAttention as GtCoreAttention
    assert GtCoreAttention is CoreAttentionQKV
    o4 = CoreAttentionQKV(h * d, 0.1, h).sparse_attention_bias(q.cuda(), k.cuda(), v.cuda(), ei.cuda(), None)
    assert o4.shape == (n, h, d) and rel_err(o4.reshape(1, n, -1), ref) < TOL_F32


def test_flattened_batch_with_dense_bias_graph_level_form():
    """Graph-level models flatten [b, N] rows and give a dense [b, H, N, N] bias
    (models/graphormer_dist_graph_level.py:243-267)."""
    from torchgt_b200 import CoreAttention
    from torchgt_b200.gt_sp.utils import flatten_edge_index_nopad
    b, n, h, d = 3, 40, 4, 8
    q, k, v = _inputs(b, n, h, d, seed=2)
    ei = flatten_edge_index_nopad([random_graph(10 + i, n, 3.0, duplicates=False) for i in range(b)], n)
    gen = torch.Generator().manual_seed(9)
    dense = (torch.randn(b, h, n, n, generator=gen) * 0.4)
    per_edge = dense[ei[0] // n, :, ei[0] % n, ei[1] % n]
    qr, kr, vr, br = (t.clone().requires_grad_() for t in (q, k, v, dense))
    ref = sao.sparse_attention_ops(qr.reshape(-1, h, d), kr.reshape(-1, h, d), vr.reshape(-1, h, d), ei,
                                   br[ei[0] // n, :, ei[0] % n, ei[1] % n])
    w = torch.randn(b * n, h, d, generator=gen)
    (ref * w).sum().backward()
    core = CoreAttention(h * d, 0.0, h)
    qc, kc, vc, bc = (t.clone().cuda().requires_grad_() for t in (q, k, v, dense))
    out = core(qc, kc, vc, bc, ei.cuda(), "sparse")
    assert out.shape == (b, n, h * d)
    (out.view(b * n, h, d) * w.cuda()).sum().backward()
    assert rel_err(out.reshape(-1), ref.reshape(-1)) < TOL_F32
    for mine, theirs in ((qc, qr), (kc, kr), (vc, vr), (bc, br)):
        assert rel_err(mine.grad, theirs.grad) < TOL_F32
    assert torch.equal(per_edge, dense[ei[0] // n, :, ei[0] % n, ei[1] % n])


def test_eval_mode_uses_all_heads_and_prebuilt_graph_is_accepted():
    from torchgt_b200 import CoreAttention, SparseGraph
    n, h, d = 128, 8, 8
    q, k, v = _inputs(1, n, h, d, seed=5)
    ei = random_graph(4, n, 4.0)
    core = CoreAttention(h * d, 0.0, h, 1).eval()
    graph = SparseGraph(ei.cuda(), n)
    out = core(q.cuda(), k.cuda(), v.cuda(), None, graph, "sparse")
    ref = sao.sparse_attention_ops(q[0], k[0], v[0], ei).reshape(1, n, h * d)
    assert rel_err(out, ref) < TOL_F32


def test_graph_level_batch_of_16_call_graphs():
    """The graph-level configuration: 16 sparse DAG-like graphs with 2,000-20,000 nodes (average degree
    about 2.5), padded to the largest and flattened to one block-diagonal edge list with per-graph offsets
    (data/collator_sp_sparse.py:126-133), run through the module as the GT models do ([b, N, H, D] in)."""
    from torchgt_b200 import CoreAttention
    from torchgt_b200.gt_sp.utils import flatten_edge_index_nopad
    gen = torch.Generator().manual_seed(16)
    sizes = torch.randint(2000, 20001, (16,), generator=gen).tolist()
    n_max = max(sizes)
    graphs = []
    for n in sizes:
        e = int(n * 2.5)
        src = torch.randint(0, n, (e,), generator=gen)
        dst = torch.minimum(src + 1 + torch.randint(0, 50, (e,), generator=gen), torch.tensor(n - 1))  # forward edges
        graphs.append(torch.stack([src, dst]))
    ei = flatten_edge_index_nopad(graphs, n_max)
    b, h, d = 16, 8, 8
    q, k, v = (torch.randn(b, n_max, h, d, generator=gen) for _ in range(3))
    w = torch.randn(b * n_max, h, d, generator=gen)
    qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
    ref = sao.sparse_attention_ops(qr.view(-1, h, d), kr.view(-1, h, d), vr.view(-1, h, d), ei)
    (ref * w).sum().backward()
    core = CoreAttention(h * d, 0.0, h)
    qc, kc, vc = (t.clone().cuda().requires_grad_() for t in (q, k, v))
    out = core(qc, kc, vc, None, ei.cuda(), "sparse")
    assert out.shape == (b, n_max, h * d)
    (out.view(b * n_max, h, d) * w.cuda()).sum().backward()
    assert rel_err(out.reshape(-1), ref.reshape(-1)) < TOL_F32
    for mine, theirs in ((qc, qr), (kc, kr), (vc, vr)):
        assert rel_err(mine.grad, theirs.grad) < TOL_F32
