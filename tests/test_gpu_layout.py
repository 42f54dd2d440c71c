"""Edge layouts built on the GPU against the CPU oracle: bit-exact integer arrays."""
import numpy as np
import pytest
import torch

from helpers import clustered_graph, random_graph
from oracle import edge_layout_oracle as elo

pytestmark = pytest.mark.gpu


def _check(ei_cpu: torch.Tensor, n_rows: int, chunk_edges: int):
    from torchgt_b200.graph import SparseGraph
    graph = SparseGraph(ei_cpu.cuda(), n_rows, chunk_edges=chunk_edges)
    for group_by, lay in ((1, graph.by_dst), (0, graph.by_src)):
        ptr, other, perm = elo.segment_layout(ei_cpu.numpy(), n_rows, group_by)
        assert np.array_equal(lay.ptr.cpu().numpy().astype(np.int64), ptr)
        assert np.array_equal(lay.other.cpu().numpy().astype(np.int64), other)
        assert np.array_equal(lay.perm.cpu().numpy().astype(np.int64), perm)
        hub_row, hub_chunk_ptr, chunk_row, chunk_begin = elo.hub_chunks(ptr, chunk_edges)
        assert lay.n_hubs == len(hub_row) and lay.n_chunks == len(chunk_row)
        assert np.array_equal(lay.hub_row.cpu().numpy().astype(np.int64), hub_row)
        assert np.array_equal(lay.hub_chunk_ptr.cpu().numpy().astype(np.int64), hub_chunk_ptr)
        assert np.array_equal(lay.chunk_row.cpu().numpy().astype(np.int64), chunk_row)
        assert np.array_equal(lay.chunk_begin.cpu().numpy().astype(np.int64), chunk_begin)
    return graph


@pytest.mark.parametrize("n,deg,chunk", [(1, 0.0, 4), (2, 1.0, 1), (97, 4.0, 16), (1000, 8.0, 128),
                                         (5000, 3.0, 32), (4097, 9.0, 128)])
def test_random_graphs(n, deg, chunk):
    _check(random_graph(11 + n, n, deg), n, chunk)


def test_no_edges_and_single_edge():
    _check(torch.zeros((2, 0), dtype=torch.long), 5, 8)
    _check(torch.tensor([[3], [1]]), 5, 8)


def test_sorted_by_source_with_duplicates():
    ei = random_graph(5, 300, 6.0, duplicates=True)
    ei = ei[:, torch.argsort(ei[0])]            # the order reformat_graph leaves (gt_sp/utils.py:354-356)
    ei = torch.cat([ei, ei[:, :50]], dim=1)     # exact duplicates
    _check(ei, 300, 16)


def test_hub_row_lengths_around_the_chunk_size():
    for extra in (-1, 0, 1, 2):
        deg = 64 + extra
        ei = torch.stack([torch.arange(deg) % 7, torch.zeros(deg, dtype=torch.long)])
        _check(ei, 8, 64)
        _check(ei.flip(0), 8, 64)


def test_benchmark_sized_graph():
    ei, n_rows = clustered_graph(1234, 64000, 8, 334000, 0.17)
    graph = _check(ei, n_rows, 128)
    assert graph.by_dst.n_hubs >= 1 and graph.by_src.n_hubs >= 1


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
