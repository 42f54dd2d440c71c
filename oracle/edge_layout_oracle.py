"""CPU restatement of the integer side of the path (test infrastructure, not product): the edge
layouts the kernels walk and the reference's edge-index helpers.  All results are int64 numpy arrays
and are compared bit-for-bit."""
from __future__ import annotations

import numpy as np


def segment_layout(edge_index: np.ndarray, n_rows: int, group_by: int):
    """perm = stable argsort of the grouping endpoint; other = other endpoint[perm];
    ptr = exclusive prefix sum of bincount.  group_by = 1: by destination (row 1), 0: by source."""
    ei = np.asarray(edge_index, dtype=np.int64)
    key = ei[1] if group_by == 1 else ei[0]
    oth = ei[0] if group_by == 1 else ei[1]
    perm = np.argsort(key, kind="stable")
    ptr = np.zeros(n_rows + 1, dtype=np.int64)
    np.cumsum(np.bincount(key, minlength=n_rows), out=ptr[1:])
    return ptr, oth[perm], perm


def hub_chunks(ptr: np.ndarray, chunk_edges: int):
    """Rows with more than chunk_edges edges, cut into chunks of chunk_edges consecutive edges."""
    deg = np.diff(ptr)
    hub_row = np.nonzero(deg > chunk_edges)[0]
    chunk_row, chunk_begin, hub_chunk_ptr = [], [], [0]
    for r in hub_row:
        n = -(-int(deg[r]) // chunk_edges)
        chunk_row += [int(r)] * n
        chunk_begin += [int(ptr[r]) + i * chunk_edges for i in range(n)]
        hub_chunk_ptr.append(len(chunk_row))
    return (np.asarray(hub_row, dtype=np.int64), np.asarray(hub_chunk_ptr, dtype=np.int64),
            np.asarray(chunk_row, dtype=np.int64), np.asarray(chunk_begin, dtype=np.int64))


def fix_edge_index(x: np.ndarray, num_node: int) -> np.ndarray:
    """gt_sp/utils.py:34-50 (= data/collator_sp_sparse.py:107-123): shift every node id by one (row 0
    becomes the virtual node) and append the edges i -> 0 and 0 -> i for i = 1..num_node."""
    x = np.asarray(x, dtype=np.int64)
    nodes = np.arange(num_node, dtype=np.int64) + 1
    zeros = np.zeros(num_node, dtype=np.int64)
    to_virtual = np.stack([nodes, zeros])
    from_virtual = np.stack([zeros, nodes])
    return np.concatenate([x + 1, to_virtual, from_virtual], axis=1)


def adjust_edge_index_nomerge(edge_index: np.ndarray, sub_seq_len: int) -> np.ndarray:
    """gt_sp/utils.py:53-58: ids i > 0 move to i + (i - 1) // sub_seq_len (one slot per rank is
    reserved for that rank's copy of the virtual node); the reference takes the floor in float32."""
    e = np.asarray(edge_index, dtype=np.int64)
    shift = np.floor_divide(e.astype(np.float32) - np.float32(1), np.float32(sub_seq_len)).astype(np.int64)
    return np.where(e > 0, e + shift, e)


def flatten_edge_index_nopad(edge_indexes, batch_node_num: int) -> np.ndarray:
    """data/collator_sp_sparse.py:126-133: graph g of the batch gets offset g * batch_node_num."""
    parts = [np.asarray(x, dtype=np.int64) + g * batch_node_num for g, x in enumerate(edge_indexes)]
    return np.concatenate(parts, axis=1)
