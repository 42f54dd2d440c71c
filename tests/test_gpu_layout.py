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
        SparseGraph(ei, 5)
    ei = torch.tensor([[0, 1, 2], [1, -1, 0]]).cuda()
    with pytest.raises(TgtError, match="INDEX_RANGE"):
        SparseGraph(ei, 5)
    # the context is still usable afterwards
    SparseGraph(torch.tensor([[0, 1], [1, 2]]).cuda(), 5)


def test_deferred_range_check_does_not_raise_at_build_time_but_on_check():
    from torchgt_b200._cabi import TgtError
    from torchgt_b200.graph import SparseGraph
    good = SparseGraph(random_graph(2, 50, 3.0).cuda(), 50, defer_check=True)
    good.by_src
    good.check()
    bad = SparseGraph(torch.tensor([[0, 1, 9], [1, 2, 0]]).cuda(), 5, defer_check=True)   # id 9 >= 5
    with pytest.raises(TgtError, match="INDEX_RANGE"):
        bad.check()
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
