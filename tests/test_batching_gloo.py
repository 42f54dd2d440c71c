"""Batch construction (gen_sub_edge_index, the cluster-sparse block generator, reformat_graph,
get_batch_reorder_blockize) against vectors the reference's own gt_sp/utils.py produced on two gloo
ranks (tests/golden/batching_P2.npz).  Integer work: every array must match bit for bit; edge lists that
the reference sorts with a non-stable argsort are compared as sorted multisets of columns."""
import os
import socket
import sys
import types
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden"
sys.path.insert(0, str(ROOT))

CASES = [("graphormer_blocks", "graphormer", 96), ("graphormer_blocks_last", "graphormer", 96),
         ("gt_blocks", "gt", 96), ("gt_blocks_last", "gt", 96)]


def _golden():
    with np.load(GOLDEN / "batching_P2.npz") as z:
        return {k: z[k] for k in z.files}


def _partition(edge_index, num_nodes, k):
    """The partitioner the goldens were made with (tests/golden/make_golden.py:golden_partition)."""
    return ((torch.arange(num_nodes) * 13) % num_nodes) * k // num_nodes


def _columns_sorted(ei: np.ndarray) -> np.ndarray:
    order = np.lexsort((ei[1], ei[0]))
    return ei[:, order]


def test_induced_subgraph_matches_the_reference():
    from torchgt_b200.gt_sp.utils import gen_sub_edge_index
    g = _golden()
    for name, _, _ in CASES:
        got = gen_sub_edge_index(torch.from_numpy(g[f"{name}/in_edge_index"]), torch.from_numpy(g[f"{name}/in_idx_batch"]),
                                 g[f"{name}/in_x"].shape[0])
        assert np.array_equal(got.numpy(), g[f"{name}/sub_edge_index"]), name


def test_block_generator_matches_the_reference_column_for_column():
    from torchgt_b200.gt_sp.utils import create_pairs, generate_new_edges_optimized, reformat_graph
    from torchgt_b200.gt_sp.batching import set_partitioner
    g = _golden()
    ei, part, mapping = (torch.from_numpy(g["blocks/edge_index"]), torch.from_numpy(g["blocks/partition"]), g["blocks/mapping"])
    assert np.array_equal(generate_new_edges_optimized(ei, 4, part, 1, 4, mapping).numpy(), g["blocks/p1"])
    assert np.array_equal(generate_new_edges_optimized(ei, 4, part, 0.02, 4, mapping).numpy(), g["blocks/p002"])
    assert create_pairs(2, 3, 5, 7) == [(5, 7), (5, 8), (5, 9), (6, 7), (6, 8), (6, 9)]
    set_partitioner(_partition)
    try:
        edges, order = reformat_graph(ei, 4, 4)
    finally:
        set_partitioner(None)
    assert np.array_equal(order.numpy(), g["blocks/reformat_order"])
    assert np.array_equal(edges[0].numpy(), g["blocks/reformat_edges"][0])        # sorted by source, as the reference's
    assert np.array_equal(_columns_sorted(edges.numpy()), _columns_sorted(g["blocks/reformat_edges"]))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import torchgt_b200.gt_sp.initialize as init
        from torchgt_b200.gt_sp.batching import set_partitioner
        from torchgt_b200.gt_sp.utils import get_batch_reorder_blockize
        g = _golden()
        init.set_global_token_num(1)
        init.initialize_sequence_parallel(96, 1, 1, world)
        set_partitioner(_partition)
        bad = []
        for name, model, seq_len in CASES:
            rest = g[f"{name}/in_rest"].tolist() or None
            args = types.SimpleNamespace(seq_len=seq_len, model=model, reorder=True, rank=rank)
            x_i, y_i, ei_i, bias = get_batch_reorder_blockize(
                args, torch.from_numpy(g[f"{name}/in_x"]), torch.from_numpy(g[f"{name}/in_y"]),
                torch.from_numpy(g[f"{name}/in_idx_batch"]), rest, "cpu", torch.from_numpy(g[f"{name}/in_edge_index"]),
                g[f"{name}/in_x"].shape[0], 3, 4)
            ok = (bias is None and np.array_equal(x_i.numpy(), g[f"{name}/r{rank}/x"])
                  and np.array_equal(y_i.numpy(), g[f"{name}/r{rank}/y"])
                  and np.array_equal(_columns_sorted(ei_i.numpy()), _columns_sorted(g[f"{name}/r{rank}/edge_index"]))
                  and int(init.get_last_batch_flag()) == int(g[f"{name}/r{rank}/last_batch"]))
            if not ok:
                bad.append(name)
        # without reordering (where the reference's own function stops on an unassigned variable): the
        # pieces it is made of, which are pinned one by one
        from torchgt_b200.gt_sp.utils import adjust_edge_index_nomerge, fix_edge_index, gen_sub_edge_index
        name = "graphormer_blocks"
        x, y = torch.from_numpy(g[f"{name}/in_x"]), torch.from_numpy(g[f"{name}/in_y"])
        idx, ei = torch.from_numpy(g[f"{name}/in_idx_batch"]), torch.from_numpy(g[f"{name}/in_edge_index"])
        args = types.SimpleNamespace(seq_len=96, model="graphormer", reorder=False, rank=rank)
        x_i, y_i, ei_i, _ = get_batch_reorder_blockize(args, x, y, idx, None, "cpu", ei, x.shape[0], 3, 4)
        want = adjust_edge_index_nomerge(fix_edge_index(gen_sub_edge_index(ei, idx, x.shape[0]), 96), 96 // world)
        if not (torch.equal(ei_i, want) and torch.equal(x_i, x[idx][rank * 48:(rank + 1) * 48])
                and torch.equal(y_i, y[idx][rank * 48:(rank + 1) * 48])):
            bad.append("no_reorder")
        ret[rank] = bad
    finally:
        dist.destroy_process_group()


def test_batches_match_the_reference_on_two_ranks():
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        ret = manager.dict()
        mp.spawn(_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
        for rank in range(2):
            assert list(ret[rank]) == [], (rank, list(ret[rank]))
