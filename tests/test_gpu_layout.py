"""Edge layouts built on the GPU against the CPU oracle: bit-exact integer arrays."""
import numpy as np
import pytest
import torch

from helpers import random_graph
from oracle import edge_layout_oracle as elo

pytestmark = pytest.mark.gpu


def _check(ei_cpu: torch.Tensor, n_rows: int):
    from torchgt_b200.graph import SparseGraph
    graph = SparseGraph(ei_cpu.cuda(), n_rows)
    for group_by, lay in ((1, graph.by_dst), (0, graph.by_src)):
        ptr, other, perm = elo.segment_layout(ei_cpu.numpy(), n_rows, group_by)
        key = ei_cpu.numpy()[1 if group_by == 1 else 0]
        assert np.array_equal(lay.ptr.cpu().numpy().astype(np.int64), ptr)
        assert np.array_equal(lay.other.cpu().numpy().astype(np.int64), other)
        assert np.array_equal(lay.perm.cpu().numpy().astype(np.int64), perm)
        assert np.array_equal(lay.seg.cpu().numpy().astype(np.int64), key[perm])
    return graph


@pytest.mark.parametrize("n,deg", [(1, 0.0), (2, 1.0), (97, 4.0), (1000, 8.0), (5000, 3.0), (4097, 9.0)])
def test_random_graphs(n, deg):
    _check(random_graph(11 + n, n, deg), n)


def test_no_edges_and_single_edge():
    _check(torch.zeros((2, 0), dtype=torch.long), 5)
    _check(torch.tensor([[3], [1]]), 5)


def test_sorted_by_source_with_duplicates():
    ei = random_graph(5, 300, 6.0, duplicates=True)
    ei = ei[:, torch.argsort(ei[0])]            # the order reformat_graph leaves (gt_sp/utils.py:354-356)
    ei = torch.cat([ei, ei[:, :50]], dim=1)     # exact duplicates
    _check(ei, 300)


def test_benchmark_sized_graph():
    from torchgt_b200.synthetic import benchmark_64k
    ei, n_rows = benchmark_64k()
    assert ei.shape[1] == 526450 and n_rows == 64001
    _check(ei, n_rows)


def test_out_of_range_index_is_reported():
    from torchgt_b200._cabi import TgtError
    from torchgt_b200.graph import SparseGraph
    ei = torch.tensor([[0, 1, 9], [1, 2, 0]]).cuda()
    with pytest.raises(TgtError, match="INDEX_RANGE"):
        SparseGraph(ei, 5, defer_check=False)
    ei = torch.tensor([[0, 1, 2], [1, -1, 0]]).cuda()
    with pytest.raises(TgtError, match="INDEX_RANGE"):
        SparseGraph(ei, 5, defer_check=False)
    # the context is still usable afterwards
    SparseGraph(torch.tensor([[0, 1], [1, 2]]).cuda(), 5)


def test_deferred_range_check_does_not_raise_at_build_time_but_on_check():
    from torchgt_b200._cabi import TgtError
    from torchgt_b200.graph import SparseGraph
    good = SparseGraph(random_graph(2, 50, 3.0).cuda(), 50)     # the default build does not synchronise
    good.by_src
    good.check()
    bad = SparseGraph(torch.tensor([[0, 1, 9], [1, 2, 0]]).cuda(), 5)   # id 9 >= 5
    with pytest.raises(TgtError, match="INDEX_RANGE"):
        bad.check()
    with pytest.raises(TgtError, match="INDEX_RANGE"):
        bad.poll()                                                       # stays reported
    # the layout itself is in bounds (the bad id was replaced by 0), so using it cannot fault
    assert int(bad.by_dst.other.max()) < 5 and int(bad.by_dst.seg.max()) < 5


def test_graph_cache_hits_on_identity_and_on_content():
    from torchgt_b200.graph import clear_graph_cache, graph_for
    clear_graph_cache()
    ei = random_graph(3, 200, 4.0).cuda()
    g1 = graph_for(ei, 200)
    assert graph_for(ei, 200) is g1                 # same tensor object
    assert graph_for(ei.clone(), 200) is g1         # fresh upload of the same edges
    other = ei.clone()
    other[0, 0] = (other[0, 0] + 1) % 200
    assert graph_for(other, 200) is not g1
    ei[0, 0] = (ei[0, 0] + 1) % 200                 # in-place edit invalidates the identity entry
    assert graph_for(ei, 200) is not g1


def test_bad_graph_is_reported_by_the_first_use_that_finds_the_build_finished():
    from torchgt_b200 import sparse_graph_attention
    from torchgt_b200._cabi import TgtError
    from torchgt_b200.graph import SparseGraph
    bad = SparseGraph(torch.tensor([[0, 1, 9], [1, 2, 0]]).cuda(), 5)
    torch.cuda.synchronize()                     # the build has finished; nobody has looked at its result yet
    q = torch.randn(5, 2, 8, device="cuda")
    with pytest.raises(TgtError, match="INDEX_RANGE"):
        sparse_graph_attention(q, q, q, bad)


def test_graph_cache_compares_edge_lists_exactly():
    """Lists that differ only by the order of two columns, or by transposition, are different graphs
    (their perm differs, so per-edge biases would be applied to the wrong edges)."""
    from torchgt_b200.graph import clear_graph_cache, graph_for
    clear_graph_cache()
    n, e = 300, 2 * 4099
    gen = torch.Generator().manual_seed(9)
    ei = torch.randint(0, n, (2, e), generator=gen).cuda()
    g1 = graph_for(ei, n)
    swapped = ei.clone()
    swapped[:, [5, 5 + 4099]] = ei[:, [5 + 4099, 5]]
    assert not torch.equal(swapped, ei)
    g2 = graph_for(swapped, n)
    assert g2 is not g1
    g3 = graph_for(ei.flip(0).contiguous(), n)               # transposed graph
    assert g3 is not g1 and g3 is not g2
    assert graph_for(ei.clone(), n) is g1                    # all three stay cached side by side
    assert graph_for(swapped.clone(), n) is g2
    perm1, perm2 = g1.by_dst.perm.cpu(), g2.by_dst.perm.cpu()
    assert torch.equal(ei[1].cpu()[perm1.long()], g1.by_dst.seg.cpu().long())
    assert torch.equal(swapped[1].cpu()[perm2.long()], g2.by_dst.seg.cpu().long())


def test_int32_edge_lists_build_the_same_layouts():
    from torchgt_b200.graph import SparseGraph
    ei = random_graph(21, 700, 5.0)
    a, b = SparseGraph(ei.cuda(), 700), SparseGraph(ei.to(torch.int32).cuda(), 700)
    for la, lb in ((a.by_dst, b.by_dst), (a.by_src, b.by_src)):
        for name in ("ptr", "other", "perm", "seg"):
            assert torch.equal(getattr(la, name), getattr(lb, name)), name
    b.check()


@pytest.mark.parametrize("world", [1, 2, 4])
def test_device_side_batch_edges_equal_the_reference_helpers(world):
    """fix -> adjust -> flatten in one kernel against the CPU restatement of the three helpers
    (itself pinned to the reference's outputs in tests/golden/edges.npz)."""
    from torchgt_b200 import prepare_edges
    gen = torch.Generator().manual_seed(40 + world)
    nodes = [37, 64, 5, 120]
    raws = [torch.randint(0, n, (2, 3 * n + 1), generator=gen) for n in nodes]
    sub = -(-max(nodes) // world)                             # per-rank rows of the padded batch
    rows_per_graph = (sub + 1) * world
    fixed = [elo.fix_edge_index(r.numpy(), n) for r, n in zip(raws, nodes)]
    ref = elo.flatten_edge_index_nopad([elo.adjust_edge_index_nomerge(f, sub) for f in fixed], rows_per_graph)
    got = prepare_edges(torch.cat(raws, dim=1).cuda(), nodes, [r.shape[1] for r in raws], True, sub, rows_per_graph)
    assert got.dtype == torch.int32 and np.array_equal(got.cpu().numpy().astype(np.int64), ref)
    # single graph, no global token, no adjust: a plain narrowing copy
    plain = prepare_edges(raws[1].cuda(), nodes[1], None, False, 0, 0)
    assert np.array_equal(plain.cpu().numpy().astype(np.int64), raws[1].numpy())


def test_device_side_batch_edges_on_the_reference_golden_ring():
    from helpers import load_golden
    from torchgt_b200 import prepare_edges
    g = load_golden("edges.npz")
    got = prepare_edges(torch.from_numpy(g["ring"]).cuda(), 4, None, True, 2, 0)
    assert np.array_equal(got.cpu().numpy().astype(np.int64), g["ring_adjusted_L2"])
    for i in range(4):
        n, sub = int(g[f"rand{i}_n"]), int(g[f"rand{i}_sub"])
        got = prepare_edges(torch.from_numpy(g[f"rand{i}_in"]).cuda(), n, None, True, sub, 0)
        assert np.array_equal(got.cpu().numpy().astype(np.int64), g[f"rand{i}_adjusted"]), i
