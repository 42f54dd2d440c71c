"""Batch construction of the node-level training loops: induced sub-graphs, the cluster-sparse block
generator and the per-rank batch slicing of the reference's gt_sp/utils.py.

Function names, argument order and results follow the reference (gt_sp/utils.py:61-82, 187-215,
218-305, 319-359, 409-520).  Everything is integer work on node ids and must be bit-exact; it runs on
whatever device its inputs live on (the reference runs it on the host for every batch).

Two third-party pieces of the reference are not available here and are restated from their published
behaviour: the three ``torch_geometric.utils`` calls inside ``gen_sub_edge_index``
(torch-geometric 2.0.0: ``remove_self_loops`` drops the columns with source == destination,
``add_self_loops`` appends (i, i) for i = 0..N-1 after the existing columns, ``subgraph`` with
``relabel_nodes=True`` keeps the columns whose two endpoints are in the subset and renumbers node
``subset[j]`` as ``j``), and the METIS partitioner behind ``reformat_graph`` (dgl 0.9.1), for which
a partitioner is passed in or set with :func:`set_partitioner`; the default cuts the node ids into
``k`` contiguous, equally long ranges.
"""
from __future__ import annotations

import random
from typing import Callable, Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist
from torch import Tensor

from .initialize import (get_sequence_parallel_group, get_sequence_parallel_rank, get_sequence_parallel_src_rank,
                         get_sequence_parallel_world_size, last_batch_flag, sequence_parallel_is_initialized)
from .utils import adjust_edge_index_nomerge, fix_edge_index


# ---- padding of the last, shorter batch (gt_sp/utils.py:61-82) ---------------------------------------
def pad_y(x: Tensor, padlen: int) -> Tensor:
    """Labels padded with -100 (ignored by nll_loss) up to ``padlen``."""
    if x.size(0) >= padlen:
        return x
    out = torch.full((padlen,), -100, dtype=x.dtype, device=x.device)
    out[:x.size(0)] = x
    return out


def pad_2d(x: Tensor, padlen: int) -> Tensor:
    """Feature rows padded with zeros up to ``padlen``."""
    if x.size(0) >= padlen:
        return x
    out = x.new_zeros([padlen, x.size(1)])
    out[:x.size(0)] = x
    return out


def random_split_idx(data_y, frac_train: float, frac_valid: float, frac_test: float, seed: int):
    """gt_sp/utils.py:187-199: shuffle 0..n-1 with Python's ``random`` seeded by ``seed`` and cut it
    into train / valid / test index tensors."""
    np.testing.assert_almost_equal(frac_train + frac_valid + frac_test, 1.0)
    random.seed(seed)
    n = data_y.shape[0]
    all_idx = np.arange(n)
    random.shuffle(all_idx)
    a, b = int(frac_train * n), int((frac_train + frac_valid) * n)
    return {"train": torch.tensor(all_idx[:a]), "valid": torch.tensor(all_idx[a:b]), "test": torch.tensor(all_idx[b:])}


# ---- induced sub-graph of a batch (gt_sp/utils.py:202-215) --------------------------------------------
def gen_sub_edge_index(edge_index: Tensor, idx_batch: Tensor, N: int) -> Tensor:
    """Edges among the nodes ``idx_batch`` of the whole graph, renumbered by position in ``idx_batch``:
    existing self loops are dropped, one self loop per node is added, and the kept columns keep their
    order (original edges first, then the self loops in node-id order)."""
    idx_batch = idx_batch.to(edge_index.device)
    src, dst = edge_index[0], edge_index[1]
    keep = src != dst                                              # remove_self_loops
    loops = torch.arange(N, dtype=edge_index.dtype, device=edge_index.device)
    adj = torch.cat([edge_index[:, keep], loops.unsqueeze(0).repeat(2, 1)], dim=1)   # add_self_loops
    member = torch.zeros(N, dtype=torch.bool, device=edge_index.device)
    member[idx_batch] = True
    new_id = torch.zeros(N, dtype=torch.long, device=edge_index.device)
    new_id[idx_batch] = torch.arange(idx_batch.size(0), device=edge_index.device)
    inside = member[adj[0]] & member[adj[1]]                      # subgraph(..., relabel_nodes=True)
    return new_id[adj[:, inside]]


# ---- cluster-sparse block generator (gt_sp/utils.py:218-305) ------------------------------------------
def create_pairs(N: int, M: int, off_N: int, off_M: int):
    """All pairs (a, b), a in [off_N, off_N + N), b in [off_M, off_M + M), a-major."""
    return [(a, b) for a in range(off_N, off_N + N) for b in range(off_M, off_M + M)]


def _expand_blocks(row0: Tensor, col0: Tensor, blocksize: int) -> Tensor:
    """[2, n_blocks * blocksize^2]: block i contributes create_pairs(blocksize, blocksize, row0[i], col0[i])."""
    within = torch.arange(blocksize * blocksize, device=row0.device)
    src = (row0.unsqueeze(1) + within // blocksize).reshape(-1)
    dst = (col0.unsqueeze(1) + within % blocksize).reshape(-1)
    return torch.stack([src, dst])


def generate_new_edges_optimized(edge_index, k: int, partition_ids, p: float, blocksize: int, new_id_mapping) -> Tensor:
    """Replace the edges between every pair of partitions by dense ``blocksize`` x ``blocksize`` blocks.

    For the partition pair (i, j) with E_ij edges and n_i, n_j nodes: density = E_ij / (n_i n_j); if it
    exceeds ``p`` the original edges are kept (renumbered); otherwise int(density * n_i * n_j /
    blocksize^2) + 1 blocks are placed at block coordinates drawn with numpy's legacy generator, seeded
    with the number of blocks placed so far, rows then columns alternating — the reference's draws,
    reproduced call for call, so the result is the same edge list column for column.  Two properties of
    the reference are kept because its results depend on them: the edge counts are stored per NON-EMPTY
    partition pair in sorted order and then read by the index i * k + j (so an empty pair shifts the
    counts of all later pairs), and pairs in which a partition has fewer than ``blocksize`` nodes get
    no edges at all.  Returns [2, E_new] int64 in the renumbered ids, on the device of ``edge_index``."""
    device = edge_index.device if isinstance(edge_index, Tensor) else torch.device("cpu")
    src, dst = (torch.as_tensor(t).cpu() for t in edge_index)
    part = torch.as_tensor(partition_ids).cpu().long()
    mapping = torch.as_tensor(np.asarray(new_id_mapping)).long()
    ps, pd = part[src.long()], part[dst.long()]
    # sorted by (partition of source, partition of destination, source, destination)
    order = np.lexsort((dst.numpy(), src.numpy(), pd.numpy(), ps.numpy()))
    s_sorted, d_sorted = src.numpy()[order], dst.numpy()[order]
    pair_sorted = (ps.numpy() * k + pd.numpy())[order]
    edge_count_list = np.zeros(k * k, dtype=np.int64)
    if pair_sorted.size:
        _, counts = np.unique(pair_sorted, return_counts=True)      # runs of equal pairs, in sorted order
        edge_count_list[:counts.size] = counts
    cumulative = np.concatenate([[0], np.cumsum(edge_count_list)])
    node_counts = np.bincount(part.numpy(), minlength=k).astype(np.int64)
    offsets = np.concatenate([[0], np.cumsum(node_counts)[:-1]]).astype(np.int64)

    pieces = []                          # the result piece by piece, in the reference's order
    keep_cnt = 0
    block_sq = blocksize * blocksize
    for i in range(k):
        for j in range(k):
            total = int(node_counts[i]) * int(node_counts[j])
            # numpy semantics of the reference (int64 / int64 -> float64; x / 0 -> inf or nan, no exception)
            with np.errstate(divide="ignore", invalid="ignore"):
                sparsity = np.float64(edge_count_list[i * k + j]) / np.float64(total)
            if sparsity > p:
                lo, hi = int(cumulative[i * k + j]), int(cumulative[i * k + j + 1])
                pieces.append(torch.stack([mapping[torch.from_numpy(s_sorted[lo:hi]).long()],
                                           mapping[torch.from_numpy(d_sorted[lo:hi]).long()]]))
                continue
            n_blocks = int(sparsity * total / block_sq) + 1
            rng = np.random.RandomState(keep_cnt)                   # np.random.seed(keep_cnt)
            if node_counts[i] >= blocksize and node_counts[j] >= blocksize:
                rows = np.empty(n_blocks, dtype=np.int64)
                cols = np.empty(n_blocks, dtype=np.int64)
                for b in range(n_blocks):
                    rows[b] = rng.randint(0, node_counts[i] // blocksize)
                    cols[b] = rng.randint(0, node_counts[j] // blocksize)
                keep_cnt += n_blocks
                # the block coordinates are a few numbers per partition pair; their expansion into
                # blocksize^2 edges each happens on the device of the edge list
                pieces.append(_expand_blocks(torch.from_numpy(rows * blocksize + offsets[i]).to(device),
                                             torch.from_numpy(cols * blocksize + offsets[j]).to(device), blocksize))
    if not pieces:
        return torch.zeros((2, 0), dtype=torch.long, device=device)
    return torch.cat([piece.to(device) for piece in pieces], dim=1)


_partitioner: Optional[Callable[[Tensor, int, int], Tensor]] = None


def set_partitioner(fn: Optional[Callable[[Tensor, int, int], Tensor]]) -> None:
    """``fn(edge_index, num_nodes, k) -> partition id per node`` used by :func:`reformat_graph` (the
    reference calls METIS through dgl there).  None restores the default: contiguous equal ranges."""
    global _partitioner
    _partitioner = fn


def contiguous_partition(edge_index: Tensor, num_nodes: int, k: int) -> Tensor:
    """Node ids cut into ``k`` contiguous ranges of (almost) equal length."""
    return (torch.arange(num_nodes) * k) // max(num_nodes, 1)


def reformat_graph(edge_index: Tensor, k: int, block_size: int, beta_coeffi="1", partition_ids=None) -> Tuple[Tensor, Tensor]:
    """gt_sp/utils.py:319-359: partition the batch graph into ``k`` clusters, renumber the nodes cluster
    by cluster, replace the edges by dense blocks (``generate_new_edges_optimized`` with p = 1, as the
    reference hard-codes) and sort the new edges by source.  Returns (edges [2, E_new], ``sorted_indices``
    = the old node id at every new position).  The order of edges with equal source is not specified
    (the reference uses a non-stable ``argsort``; a stable sort is used here)."""
    num_nodes = int(edge_index.max().item()) + 1 if edge_index.numel() else 0   # dgl.graph((src, dst)).num_nodes()
    if partition_ids is None:
        fn = _partitioner or contiguous_partition
        partition_ids = fn(edge_index, num_nodes, k)
    partition_ids = torch.as_tensor(partition_ids).cpu().long()
    new_id_mapping = np.empty(num_nodes, dtype=np.int64)
    current = 0
    part_np = partition_ids.numpy()
    for part_id in range(k):
        nodes = np.where(part_np == part_id)[0]
        new_id_mapping[nodes] = np.arange(current, current + len(nodes))
        current += len(nodes)
    new_edge_index = generate_new_edges_optimized(edge_index, k, partition_ids, 1, blocksize=block_size,
                                                  new_id_mapping=new_id_mapping)
    sorted_indices = torch.argsort(torch.from_numpy(new_id_mapping))
    by_source = torch.argsort(new_edge_index[0], stable=True)
    return new_edge_index[:, by_source], sorted_indices


# ---- one training batch of the node-level loops (gt_sp/utils.py:409-520) ------------------------------
def get_batch_reorder_blockize(args, x: Tensor, y: Tensor, idx_batch: Tensor, rest_split_sizes, device, edge_index: Tensor,
                               N: int, k: int, block_size: int, beta_coeffi="1"):
    """This rank's slice of one batch: features and labels of ``idx_batch`` (the last, shorter batch
    padded to equal per-rank length), and the batch's edge list — induced sub-graph, global token added
    and ids moved past the per-rank token slots for ``args.model == "graphormer"``, optionally reordered
    into cluster-sparse blocks (``args.reorder``; computed on the first rank of the group and broadcast,
    as the reference does).  Sets the last-batch flag the layers read.  Returns
    ``(x_i, y_i, edge_index_i, attn_bias)`` with ``attn_bias`` always None."""
    world = get_sequence_parallel_world_size() if sequence_parallel_is_initialized() else 1
    rank = get_sequence_parallel_rank() if sequence_parallel_is_initialized() else 0
    seq_length = args.seq_len
    x_i, y_i = x[idx_batch], y[idx_batch]
    edge_index_i = gen_sub_edge_index(edge_index, idx_batch, N)
    graphormer = args.model == "graphormer"
    if graphormer:
        edge_index_i = fix_edge_index(edge_index_i, idx_batch.shape[0])
    if getattr(args, "reorder", False):
        if world > 1:
            src_rank, group = get_sequence_parallel_src_rank(), get_sequence_parallel_group()
            if dist.get_rank() == src_rank:
                edge_index_i, sorted_indices = reformat_graph(edge_index_i, k, block_size, beta_coeffi)
                sizes = torch.tensor([edge_index_i.shape[1], sorted_indices.shape[0]], dtype=torch.int64, device=device)
            else:
                sizes = torch.empty(2, dtype=torch.int64, device=device)
            dist.broadcast(sizes, src_rank, group=group)
            n_edges, n_nodes = sizes.tolist()
            if dist.get_rank() == src_rank:
                edges_dev, order_dev = edge_index_i.to(device), sorted_indices.to(device)
            else:
                edges_dev = torch.empty((2, n_edges), dtype=torch.int64, device=device)
                order_dev = torch.empty(n_nodes, dtype=torch.int64, device=device)
            dist.broadcast(edges_dev, src_rank, group=group)
            dist.broadcast(order_dev, src_rank, group=group)
            edge_index_i, sorted_indices = edges_dev.to(x_i.device), order_dev.to(x_i.device)
        else:
            edge_index_i, sorted_indices = reformat_graph(edge_index_i, k, block_size, beta_coeffi)
        if graphormer:   # position 0 is the global token: not a row of x
            sorted_indices = sorted_indices[sorted_indices != 0] - 1
        x_i = torch.index_select(x_i, 0, sorted_indices.to(x_i.device))
        y_i = torch.index_select(y_i, 0, sorted_indices.to(y_i.device))
    if idx_batch.shape[0] < seq_length:
        if rest_split_sizes is None:
            raise ValueError("rest_split_sizes is needed for the last, shorter batch")
        per_rank = max(rest_split_sizes)
        x_i = pad_2d(x_i, per_rank * world)
        y_i = pad_y(y_i, per_rank * world)
        if graphormer:
            edge_index_i = adjust_edge_index_nomerge(edge_index_i, per_rank)
        last_batch_flag(True)
    else:
        if seq_length % world != 0:
            raise ValueError(f"seq_len {seq_length} is not divisible by {world} ranks")
        per_rank = seq_length // world
        if graphormer:
            edge_index_i = adjust_edge_index_nomerge(edge_index_i, per_rank)
        last_batch_flag(False)
    x_i = x_i[rank * per_rank:(rank + 1) * per_rank]
    y_i = y_i[rank * per_rank:(rank + 1) * per_rank]
    return x_i, y_i, edge_index_i, None
