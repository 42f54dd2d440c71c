"""Seeded synthetic graphs with the shapes of the reference's benchmark batches.

The reference measures on ogbn-arxiv / ogbn-products batches after its METIS reordering; those
datasets are not redistributable with this library, so the benchmarks and tests use generated graphs
with the same node counts, edge counts and cluster structure (README of the reference: 64,001 nodes /
526,450 edges / 17.5 % of edges cut by the 8-way partition for the 64K batch).
"""
from __future__ import annotations

import torch


def clustered_edges(seed: int, n_nodes: int, n_clusters: int, cluster_edges: int, cross_fraction: float,
                    zipf_exponent: float = 0.0):
    """Edges over node ids 1..n_nodes (id 0 is the global node): self loops, global-token edges in both
    directions, and ``cluster_edges`` random edges of which ``cross_fraction`` leave their cluster.
    With ``zipf_exponent`` > 1 the sources follow a power law (a few nodes with very many out-edges).
    Returns ([2, E] int64 on the CPU, n_rows = n_nodes + 1)."""
    gen = torch.Generator().manual_seed(seed)
    size = n_nodes // n_clusters
    nodes = torch.arange(1, n_nodes + 1)
    zeros = torch.zeros(n_nodes, dtype=torch.long)
    if zipf_exponent > 1.0:
        # inverse-CDF sampling of p(rank) ~ rank^(-1/(exponent-1)), ranks scattered over the node ids
        alpha = 1.0 / (zipf_exponent - 1.0)
        u = torch.rand(cluster_edges, generator=gen, dtype=torch.float64)
        ranks_ = (u * (float(n_nodes) ** (1.0 - alpha) - 1.0) + 1.0) ** (1.0 / (1.0 - alpha)) - 1.0
        src = torch.randperm(n_nodes, generator=gen)[ranks_.clamp_(0, n_nodes - 1).long()]
    else:
        src = torch.randint(0, n_nodes, (cluster_edges,), generator=gen)
    cross = torch.rand(cluster_edges, generator=gen) < cross_fraction
    same = (src // size) * size + torch.randint(0, size, (cluster_edges,), generator=gen)
    anywhere = torch.randint(0, n_nodes, (cluster_edges,), generator=gen)
    dst = torch.where(cross, anywhere, same)
    edge_index = torch.cat([torch.stack([nodes, nodes]), torch.stack([nodes, zeros]),
                            torch.stack([zeros, nodes]), torch.stack([src + 1, dst + 1])], dim=1)
    return edge_index.contiguous(), n_nodes + 1


def benchmark_64k(seed: int = 1234, ranks: int = 1):
    """The 64K-node attention micro-benchmark batch, scaled to ``ranks`` sequence-parallel ranks with
    64,000 nodes per rank: 8 clusters of 8,000 nodes per rank, about 526K directed edges per rank
    (average in-degree 8.2); 31.5 % of the random edges leave their cluster, i.e. 17.5 % of all edges
    are cut, the ratio the reference logs for this batch."""
    return clustered_edges(seed, 64000 * ranks, 8 * ranks, 334450 * ranks, 0.315)


def benchmark_870k(seed: int = 1234, zipf_exponent: float = 2.1):
    """The long-sequence batch: 870,000 nodes + global node, 18,214,272 directed edges (the sizes the
    reference logs for its 870K-token ogbn-products batch), power-law out-degrees (exponent 2.1), 8 clusters
    with 7.1 % of all edges cut.  ``zipf_exponent=0`` draws the sources uniformly instead (no hot rows)."""
    n = 870000
    random_edges = 18214272 - 3 * n
    return clustered_edges(seed, n, 8, random_edges, 1293861 / random_edges / 0.875, zipf_exponent=zipf_exponent)


def power_law_edges(seed: int, n_nodes: int, n_edges: int, exponent: float = 2.1):
    """Directed edges whose endpoints follow a Zipf-like popularity (a few very high-degree nodes),
    over node ids 0..n_nodes-1, plus one self loop per node.  Returns [2, E] int64 on the CPU."""
    gen = torch.Generator().manual_seed(seed)
    # inverse-CDF sampling of p(i) ~ (i + 1)^(-1/(exponent - 1)) over a random relabelling of the nodes
    alpha = 1.0 / (exponent - 1.0)
    def draw(count):
        u = torch.rand(count, generator=gen, dtype=torch.float64)
        ranks_ = (u * (float(n_nodes) ** (1.0 - alpha) - 1.0) + 1.0) ** (1.0 / (1.0 - alpha)) - 1.0
        return ranks_.clamp_(0, n_nodes - 1).long()
    relabel = torch.randperm(n_nodes, generator=gen)
    src = relabel[draw(n_edges)]
    dst = torch.randint(0, n_nodes, (n_edges,), generator=gen)
    loops = torch.arange(n_nodes)
    return torch.cat([torch.stack([src, dst]), torch.stack([loops, loops])], dim=1).contiguous()
