"""Generate the golden vectors under tests/golden/ by RUNNING THE REFERENCE ITSELF on CPU.

Run from the repository root on a machine that has the reference checkout:

    python tests/golden/make_golden.py --reference /path/to/torchgt

The reference imports torch_scatter / torch_sparse / torch_geometric / dgl, none of which are needed
by the code paths exercised here; they are replaced by minimal stand-ins
(``torch_scatter.scatter(src, index, dim=0, out=out, reduce='add')`` -> ``out.index_add_(0, index,
src)``, the documented semantics of torch-scatter 2.1.1).  gloo has no list all-to-all, so inside the
worker processes ``torch.distributed.all_to_all`` is routed through ``all_to_all_single``.

Outputs (all small .npz files, committed):
  attn_*.npz     CoreAttention.sparse_attention_bias forward + autograd gradients
  edges.npz      fix_edge_index / adjust_edge_index_nomerge / flatten_edge_index_nopad known answers
  ulysses_P*.npz _SeqAllToAll both directions and the DistributedAttentionNoMerge layer, P = 2, 4, 8 ranks
  layer_variants_P*.npz  the four Ulysses layer variants no reference model instantiates (global tokens
                 merged by mean), around a toy local attention: outputs and gradients, P ranks
  graphormer_node_level.npz  the reference's node-level Graphormer: parameters, log-probabilities, loss and
                 parameter gradients of one training step (3 layers, dropout 0, one rank), in fp32 and (keys
                 out64, loss64, grad64/...) with the model converted to fp64; the fp32 gradients differ by
                 about 1e-6 from run to run (multi-threaded index_add_ in the CPU backward)
  gt_node_level.npz   the same for the reference's node-level GT (3 layers, no global token, one rank)
  gt_graph_level.npz  the reference's graph-level GT on two ranks (3 padded graphs of 40 integer-featured
                 nodes): output, loss and the gradient of one copy of the loss
  graphormer_graph_level.npz  the reference's graph-level Graphormer, one rank (3 padded graphs of 40 nodes,
                 graph token at index 0 of each): output, loss, parameter gradients
  batching_P2.npz  get_batch_reorder_blockize on two ranks (full and last batches, Graphormer and GT, with and
                 without cluster-sparse blocks), gen_sub_edge_index, generate_new_edges_optimized, reformat_graph;
                 the three torch_geometric.utils calls and the METIS partitioner are stand-ins (see
                 install_batching_shims), everything else is the reference's own code
  graphormer_graph_level_P2.npz  the same model on two ranks (every rank's own graph token in front of its
                 20 nodes of each graph): per-rank outputs and per-rank parameter gradients
"""
from __future__ import annotations

import argparse
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

OUT_DIR = Path(__file__).resolve().parent


def install_shims():
    def scatter(src, index, dim=0, out=None, reduce="add"):
        assert dim == 0 and reduce == "add" and out is not None
        out.index_add_(0, index.to(torch.long), src)
        return out

    ts = types.ModuleType("torch_scatter"); ts.scatter = scatter
    tsp = types.ModuleType("torch_sparse"); tsp.SparseTensor = object; tsp.matmul = None
    tg = types.ModuleType("torch_geometric"); tgu = types.ModuleType("torch_geometric.utils")
    for name in ("degree", "to_undirected", "remove_self_loops", "add_self_loops", "subgraph"):
        setattr(tgu, name, None)
    tg.utils = tgu
    dgl = types.ModuleType("dgl")
    sys.modules.update({"torch_scatter": ts, "torch_sparse": tsp, "torch_geometric": tg,
                        "torch_geometric.utils": tgu, "dgl": dgl})


def random_graph(gen, n, avg_in_degree, hub=True, duplicates=False):
    """Directed edges [2, E]: random in-edges + self loops (+ a hub row 0 connected to everyone)."""
    e = int(n * avg_in_degree)
    src = torch.randint(0, n, (e,), generator=gen)
    dst = torch.randint(0, n, (e,), generator=gen)
    parts = [torch.stack([src, dst])]
    loops = torch.arange(n)
    parts.append(torch.stack([loops, loops]))
    if hub:
        others = torch.arange(1, n)
        zeros = torch.zeros(n - 1, dtype=torch.long)
        parts += [torch.stack([others, zeros]), torch.stack([zeros, others])]
    ei = torch.cat(parts, dim=1)
    if not duplicates:
        ei = torch.unique(ei, dim=1)
    ei = ei[:, torch.randperm(ei.shape[1], generator=gen)]
    # leave some rows without in-edges
    keep = ei[1] % 7 != 3
    return ei[:, keep].contiguous()


def make_attention_cases():
    from models.graphormer_dist_graph_level import CoreAttention as GraphLevelCore  # (k, q, v, ...)
    from models.gt_dist_node_level import CoreAttention as GtNodeCore               # (q, k, v, ...)

    cases = [
        # name, N, H, D, avg_deg, input scale, bias, duplicates
        ("small_nobias", 97, 8, 8, 4.0, 1.0, None, True),
        ("clamped_nobias", 64, 4, 16, 6.0, 3.0, None, True),
        ("dense_bias", 80, 8, 8, 5.0, 1.5, "dense", False),
        ("one_head", 50, 1, 8, 3.0, 2.0, "dense", False),
        ("wide_head", 40, 2, 32, 3.0, 1.0, None, True),
    ]
    for idx, (name, n, h, d, deg, scale, bias_kind, dup) in enumerate(cases):
        gen = torch.Generator().manual_seed(1000 + idx)
        ei = random_graph(gen, n, deg, hub=True, duplicates=dup)
        q = (torch.randn(1, n, h, d, generator=gen) * scale).requires_grad_()
        k = (torch.randn(1, n, h, d, generator=gen) * scale).requires_grad_()
        v = torch.randn(1, n, h, d, generator=gen).requires_grad_()
        dout = torch.randn(n, h, d, generator=gen)
        attn_bias = None
        if bias_kind == "dense":
            attn_bias = (torch.randn(1, h, n, n, generator=gen) * 0.5).requires_grad_()
        core = GraphLevelCore(h * d, 0.0, h)
        core.num_attention_heads_per_partition = h
        out = core.sparse_attention_bias(k, q, v, ei, attn_bias)       # [N, H, D]
        (out * dout).sum().backward()
        rec = dict(q=q.detach()[0].numpy(), k=k.detach()[0].numpy(), v=v.detach()[0].numpy(),
                   edge_index=ei.numpy(), dout=dout.numpy(), out=out.detach().numpy(),
                   dq=q.grad[0].numpy(), dk=k.grad[0].numpy(), dv=v.grad[0].numpy())
        if attn_bias is not None:
            rec["attn_bias"] = attn_bias.detach().numpy()
            rec["dattn_bias"] = attn_bias.grad.numpy()
        else:
            # same inputs through the GT node-level copy (argument order q, k, v): must agree exactly
            core2 = GtNodeCore(h * d, 0.0, h)
            core2.num_attention_heads_per_partition = h
            core2.train()
            out2 = core2.sparse_attention_bias(q.detach(), k.detach(), v.detach(), ei, None)
            assert torch.equal(out2, out.detach()), name
        np.savez_compressed(OUT_DIR / f"attn_{name}.npz", **rec)
        print("wrote", f"attn_{name}.npz", "N", n, "E", ei.shape[1])


def make_edge_cases():
    from data.collator_sp_sparse import (adjust_edge_index_nomerge, fix_edge_index,
                                         flatten_edge_index_nopad)
    import gt_sp.utils as ref_utils
    rec = {}
    ring = torch.tensor([[0, 1, 2, 3], [1, 2, 3, 0]])
    fixed = fix_edge_index(ring, 4)
    assert torch.equal(fixed, ref_utils.fix_edge_index(ring, 4))
    adj = adjust_edge_index_nomerge(fixed, 2)
    assert torch.equal(adj, ref_utils.adjust_edge_index_nomerge(fixed, 2))
    rec["ring"], rec["ring_fixed"], rec["ring_adjusted_L2"] = ring.numpy(), fixed.numpy(), adj.numpy()
    rec["ring_flat_6"] = flatten_edge_index_nopad([adj, adj[:, :3]], 6).numpy()
    gen = torch.Generator().manual_seed(7)
    for i, (n, e, sub) in enumerate([(12, 30, 3), (64, 300, 16), (1000, 5000, 125), (4096, 9000, 512)]):
        x = torch.randint(0, n, (2, e), generator=gen)
        fixed = fix_edge_index(x, n)
        adj = adjust_edge_index_nomerge(fixed, sub)
        rec[f"rand{i}_in"], rec[f"rand{i}_n"], rec[f"rand{i}_sub"] = x.numpy(), np.int64(n), np.int64(sub)
        rec[f"rand{i}_fixed"], rec[f"rand{i}_adjusted"] = fixed.numpy(), adj.numpy()
    g0 = torch.randint(0, 9, (2, 20), generator=gen)
    g1 = torch.randint(0, 9, (2, 11), generator=gen)
    g2 = torch.randint(0, 9, (2, 17), generator=gen)
    rec["flat_in0"], rec["flat_in1"], rec["flat_in2"] = g0.numpy(), g1.numpy(), g2.numpy()
    rec["flat_out_10"] = flatten_edge_index_nopad([g0, g1, g2], 10).numpy()
    np.savez_compressed(OUT_DIR / "edges.npz", **rec)
    print("wrote edges.npz")


def _ulysses_worker(rank, world, ref_path, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, ref_path)
    install_shims()
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)

    def all_to_all_via_single(output_list, input_list, group=None):
        out = torch.empty_like(torch.stack(input_list))
        dist.all_to_all_single(out, torch.stack(input_list).contiguous(), group=group)
        for o, chunk in zip(output_list, out):
            o.copy_(chunk)
    dist.all_to_all = all_to_all_via_single
    torch.distributed.all_to_all = all_to_all_via_single

    import gt_sp.initialize as init
    L, H, D = 6, 8, 8
    S = L * world
    init._GLOBAL_TOKEN_NUM = 1
    init.initialize_sequence_parallel(S, 1, 1, world)
    init.set_global_token_indices(list(range(0, world * (L + 1), L + 1)))
    from gt_sp.layer import DistributedAttentionNoMerge, _SeqAllToAll
    from models.graphormer_dist_node_level import CoreAttention
    from gt_sp.utils import adjust_edge_index_nomerge, fix_edge_index

    gen = torch.Generator().manual_seed(500 + rank)
    q = torch.randn(1, L + 1, H, D, generator=gen).requires_grad_()
    k = torch.randn(1, L + 1, H, D, generator=gen).requires_grad_()
    v = torch.randn(1, L + 1, H, D, generator=gen).requires_grad_()
    dout = torch.randn(1, L + 1, H * D, generator=gen)
    group = init.get_sequence_parallel_group()
    a2a_21 = _SeqAllToAll.apply(group, q.detach(), 2, 1)
    ctx_like = torch.randn(1, world * (L + 1), (H // world) * D, generator=gen)
    a2a_12 = _SeqAllToAll.apply(group, ctx_like, 1, 2)

    ggen = torch.Generator().manual_seed(77)      # same graph on every rank
    raw = torch.randint(0, S, (2, 5 * S), generator=ggen)
    ei = adjust_edge_index_nomerge(fix_edge_index(raw, S), L)
    core = CoreAttention(H * D, 0.0, H, 1)
    layer = DistributedAttentionNoMerge(core, group)
    layer.train()
    out = layer(q, k, v, None, ei, "sparse")
    (out * dout).sum().backward()
    rec = dict(q=q.detach().numpy(), k=k.detach().numpy(), v=v.detach().numpy(), dout=dout.numpy(),
               a2a_21=a2a_21.numpy(), ctx_like=ctx_like.numpy(), a2a_12=a2a_12.numpy(),
               edge_index=ei.numpy(), out=out.detach().numpy(), dq=q.grad.numpy(), dk=k.grad.numpy(),
               dv=v.grad.numpy())
    gathered = [None] * world
    dist.all_gather_object(gathered, rec)
    if rank == 0:
        flat = {f"r{r}_{name}": val for r, g in enumerate(gathered) for name, val in g.items()}
        flat["L"], flat["H"], flat["D"] = np.int64(L), np.int64(H), np.int64(D)
        np.savez_compressed(out_path, **flat)
        print("wrote", out_path)
    dist.destroy_process_group()


class ToyAttention(torch.nn.Module):
    """Stand-in local attention for the layer variants nothing in the reference instantiates: an
    elementwise mix of q, k, v plus a per-row bias term, so that only the layers' own exchange /
    merge / extend logic is under test.  tests/test_ulysses_gloo.py carries an identical copy."""

    def forward(self, q, k, v, attn_bias=None, *args):
        b, s = q.size(0), q.size(1)
        out = (0.5 * q + 0.25 * k * k - v).reshape(b, s, -1)
        if attn_bias is not None:
            sq = attn_bias * attn_bias                    # (a dense gradient, not a broadcast one)
            if attn_bias.size(1) == s:                    # [b, s, x, y]
                out = out + sq.sum(dim=(2, 3)).unsqueeze(-1)
            else:                                         # [b, heads, s, y]
                out = out + sq.sum(dim=(1, 3)).unsqueeze(-1)
        return out


def _variants_worker(rank, world, ref_path, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, ref_path)
    install_shims()
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)

    def all_to_all_via_single(output_list, input_list, group=None):
        out = torch.empty_like(torch.stack(input_list))
        dist.all_to_all_single(out, torch.stack(input_list).contiguous(), group=group)
        for o, chunk in zip(output_list, out):
            o.copy_(chunk)
    dist.all_to_all = all_to_all_via_single
    torch.distributed.all_to_all = all_to_all_via_single
    import gt_sp.initialize as init
    L, H, D = 5, 8, 4
    S = L * world
    init._GLOBAL_TOKEN_NUM = 1
    init.initialize_sequence_parallel(S, 1, 1, world)
    init.set_global_token_indices(list(range(0, world * (L + 1), L + 1)))
    import gt_sp.layer as ref_layer
    group = init.get_sequence_parallel_group()
    gen = torch.Generator().manual_seed(900 + rank)
    rec = {}
    cases = {
        "DistributedAttention": lambda: torch.randn(1, L + 1, S + 1, 2, generator=gen),
        "DistributedAttentionGlobal0": lambda: torch.randn(1, L + 1, S + 1, 2, generator=gen),
        "DistributedAttentionLocalBias": lambda: torch.randn(1, H, S + 1, S + 1, generator=torch.Generator().manual_seed(5)),
        "DistributedAttentionAll2all": lambda: torch.randn(1, H, L + 1, S + 1, generator=gen),
    }
    for name, make_bias in cases.items():
        q, k, v = (torch.randn(1, L + 1, H, D, generator=gen).requires_grad_() for _ in range(3))
        bias = make_bias().requires_grad_()
        dout = torch.randn(1, L + 1, H * D, generator=gen)
        layer = getattr(ref_layer, name)(ToyAttention(), group).train()
        if name == "DistributedAttention":
            out = layer(q, k, v, bias)
        else:
            out = layer(q, k, v, bias, None)
        (out * dout).sum().backward()
        for key, val in (("q", q), ("k", k), ("v", v), ("bias", bias), ("dout", dout), ("out", out),
                         ("dq", q.grad), ("dk", k.grad), ("dv", v.grad), ("dbias", bias.grad)):
            rec[f"{name}/{key}"] = val.detach().numpy()
    gathered = [None] * world
    dist.all_gather_object(gathered, rec)
    if rank == 0:
        flat = {f"r{r}/{name}": val for r, g in enumerate(gathered) for name, val in g.items()}
        flat["L"], flat["H"], flat["D"] = np.int64(L), np.int64(H), np.int64(D)
        np.savez_compressed(out_path, **flat)
        print("wrote", out_path)
    dist.destroy_process_group()


def make_variant_cases(ref_path, worlds=(2, 4, 8)):
    import torch.multiprocessing as mp
    for world in worlds:
        mp.spawn(_variants_worker, args=(world, ref_path, 29631 + world, str(OUT_DIR / f"layer_variants_P{world}.npz")),
                 nprocs=world, join=True)


def _model_worker(rank, world, ref_path, port, out_path):
    """Reference node-level Graphormer, one rank (the exchange degenerates to a copy), dropout 0."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, ref_path)
    install_shims()
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)

    def all_to_all_copy(output_list, input_list, group=None):
        for o, i in zip(output_list, input_list):
            o.copy_(i)
    dist.all_to_all = all_to_all_copy
    torch.distributed.all_to_all = all_to_all_copy
    import gt_sp.initialize as init
    n = 300
    init._GLOBAL_TOKEN_NUM = 1
    init.initialize_sequence_parallel(n, 1, 1, 1)
    init.set_global_token_indices([0])
    from models.graphormer_dist_node_level import Graphormer
    from gt_sp.utils import adjust_edge_index_nomerge, fix_edge_index
    torch.manual_seed(11)
    model = Graphormer(3, 8, 24, 64, 7, 1, 0.0, 0.0, 0.0, 64, 1)
    # the reference initialises with std 0.02/sqrt(L): scale up so that attention scores are not all ~0
    with torch.no_grad():
        for p_ in model.parameters():
            p_.mul_(8.0)
    gen = torch.Generator().manual_seed(12)
    x = torch.randn(n, 24, generator=gen)
    y = torch.randint(0, 7, (n,), generator=gen)
    raw = torch.cat([torch.randint(0, n, (2, 6 * n), generator=gen), torch.arange(n).repeat(2, 1)], dim=1)
    ei = adjust_edge_index_nomerge(fix_edge_index(raw, n), n)
    model.train()
    out = model(x, None, ei, attn_type="sparse")
    loss = torch.nn.functional.nll_loss(out, y)
    loss.backward()
    rec = {"x": x.numpy(), "y": y.numpy(), "edge_index": ei.numpy(), "out": out.detach().numpy(),
           "loss": np.float64(loss.item())}
    for name, p_ in model.state_dict().items():
        rec["param/" + name] = p_.numpy()
    for name, p_ in model.named_parameters():
        if p_.grad is not None:
            rec["grad/" + name] = p_.grad.numpy()
    # the same step of the same model in fp64: what both fp32 evaluations (the reference's above and the
    # CUDA path's) approximate; gradients that are sums of cancelling terms are compared with this one
    model64 = model.double()          # in place: the fp32 parameters and gradients are recorded above
    model64.zero_grad(set_to_none=True)
    out64 = model64(x.double(), None, ei, attn_type="sparse")
    loss64 = torch.nn.functional.nll_loss(out64, y)
    loss64.backward()
    rec["out64"] = out64.detach().numpy()
    rec["loss64"] = np.float64(loss64.item())
    for name, p_ in model64.named_parameters():
        if p_.grad is not None:
            rec["grad64/" + name] = p_.grad.numpy()
    n_params = sum(p_.numel() for p_ in Graphormer(4, 8, 128, 64, 40, 1, 0.0, 0.0, 0.0, 64, 1).parameters())
    rec["params_of_the_readme_model"] = np.int64(n_params)     # the reference's README logs 111913
    np.savez_compressed(out_path, **rec)
    print("wrote", out_path, "loss", loss.item(), "params(4L/64/8h/128->40)", n_params)
    dist.destroy_process_group()


def make_model_case(ref_path):
    import torch.multiprocessing as mp
    mp.spawn(_model_worker, args=(1, ref_path, 29621, str(OUT_DIR / "graphormer_node_level.npz")), nprocs=1, join=True)


def make_ulysses_cases(ref_path, worlds=(2, 4, 8)):
    import torch.multiprocessing as mp
    for world in worlds:
        mp.spawn(_ulysses_worker, args=(world, ref_path, 29611 + world, str(OUT_DIR / f"ulysses_P{world}.npz")),
                 nprocs=world, join=True)


def _gt_node_worker(rank, world, ref_path, port, out_path):
    """Reference node-level GT (no global token), one rank, dropout 0, training mode (so the layer
    goes through its exchange, which is a copy with one rank)."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, ref_path)
    install_shims()
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)

    def all_to_all_copy(output_list, input_list, group=None):
        for o, i in zip(output_list, input_list):
            o.copy_(i)
    dist.all_to_all = all_to_all_copy
    torch.distributed.all_to_all = all_to_all_copy
    import gt_sp.initialize as init
    n = 260
    init.initialize_sequence_parallel(n, 1, 1, 1)
    from models.gt_dist_node_level import GT
    torch.manual_seed(21)
    model = GT(3, 8, 20, 64, 6, 1, 0.0, 0.0, 0.0, 64, 0)
    with torch.no_grad():                      # std 0.02/sqrt(L) would leave all attention scores ~0
        for p_ in model.parameters():
            p_.mul_(8.0)
    gen = torch.Generator().manual_seed(22)
    x = torch.randn(n, 20, generator=gen)
    y = torch.randint(0, 6, (n,), generator=gen)
    ei = torch.cat([torch.randint(0, n, (2, 5 * n), generator=gen), torch.arange(n).repeat(2, 1)], dim=1)
    model.train()
    out = model(x, None, ei, attn_type="sparse")
    loss = torch.nn.functional.nll_loss(out, y)
    loss.backward()
    rec = {"x": x.numpy(), "y": y.numpy(), "edge_index": ei.numpy(), "out": out.detach().numpy(),
           "loss": np.float64(loss.item())}
    for name, p_ in model.state_dict().items():
        rec["param/" + name] = p_.numpy()
    for name, p_ in model.named_parameters():
        if p_.grad is not None:
            rec["grad/" + name] = p_.grad.numpy()
    np.savez_compressed(out_path, **rec)
    print("wrote", out_path, "loss", loss.item())
    dist.destroy_process_group()


class _Batch:
    """The two attributes of the collated batch that the graph-level models read."""

    def __init__(self, x, edge_index):
        self.x, self.edge_index = x, edge_index


def _gt_graph_worker(rank, world, ref_path, port, out_path):
    """Reference graph-level GT on `world` gloo ranks (its backward does not run with one rank), dropout 0.
    Recorded: the full inputs, the output (identical on all ranks) and the gradient of ONE copy of the
    loss: encoder and embedding gradients summed over the ranks (each rank holds the part that flows
    through its slice of the sequence), read-out gradients from rank 0 (every rank holds all of it)."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, ref_path)
    install_shims()
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)

    def all_to_all_via_single(output_list, input_list, group=None):
        out = torch.empty_like(torch.stack(input_list))
        dist.all_to_all_single(out, torch.stack(input_list).contiguous(), group=group)
        for o, chunk in zip(output_list, out):
            o.copy_(chunk)
    dist.all_to_all = all_to_all_via_single
    torch.distributed.all_to_all = all_to_all_via_single
    import gt_sp.initialize as init
    b, s, feats, classes = 3, 40, 5, 5
    L = s // world
    init.initialize_sequence_parallel(s, 1, 1, world)
    from models.gt_dist_graph_level import GT
    torch.manual_seed(31)
    model = GT(2, 8, 64, 0.0, 0.0, 64, "ZINC", "multi_hop", 5, 0.0, classes)
    with torch.no_grad():
        for p_ in model.parameters():
            p_.mul_(8.0)
    gen = torch.Generator().manual_seed(32)
    x = torch.randint(0, 64, (b, s, feats), generator=gen)
    y = torch.randint(0, classes, (b,), generator=gen)
    # edges inside each graph, numbered over the b * s flattened rows of the gathered batch
    per_graph = []
    for g in range(b):
        e = torch.cat([torch.randint(0, s, (2, 4 * s), generator=gen), torch.arange(s).repeat(2, 1)], dim=1)
        per_graph.append(e + g * s)
    ei = torch.cat(per_graph, dim=1)
    model.train()
    out = model(_Batch(x[:, rank * L:(rank + 1) * L].contiguous(), ei), attn_type="sparse")
    loss = torch.nn.functional.cross_entropy(out, y)
    loss.backward()
    grads = {}
    for name, p_ in model.named_parameters():
        if p_.grad is None:
            continue
        g = p_.grad.clone()
        if not name.startswith("MLP_layer"):
            dist.all_reduce(g)
        grads[name] = g
    if rank == 0:
        rec = {"x": x.numpy(), "y": y.numpy(), "edge_index": ei.numpy(), "out": out.detach().numpy(),
               "loss": np.float64(loss.item()), "world": np.int64(world)}
        for name, p_ in model.state_dict().items():
            rec["param/" + name] = p_.numpy()
        for name, g in grads.items():
            rec["grad/" + name] = g.numpy()
        np.savez_compressed(out_path, **rec)
        print("wrote", out_path, "loss", loss.item())
    dist.destroy_process_group()


def _graphormer_graph_worker(rank, world, ref_path, port, out_path):
    """Reference graph-level Graphormer, one rank, dropout 0: 3 padded graphs of 40 nodes, one graph token
    each at local index 0, edges over the 3 * 41 flattened rows."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, ref_path)
    install_shims()
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)

    def all_to_all_copy(output_list, input_list, group=None):
        for o, i in zip(output_list, input_list):
            o.copy_(i)
    dist.all_to_all = all_to_all_copy
    torch.distributed.all_to_all = all_to_all_copy
    import gt_sp.initialize as init
    b, s, feats, classes = 3, 40, 2, 5
    init._GLOBAL_TOKEN_NUM = 1
    init.initialize_sequence_parallel(s, 1, 1, 1)
    init.set_global_token_indices([0])
    from models.graphormer_dist_graph_level import Graphormer
    torch.manual_seed(41)
    model = Graphormer(2, 8, 64, 0.0, 0.0, 64, "ZINC", "multi_hop", 5, 0.0, classes)
    with torch.no_grad():
        for p_ in model.parameters():
            p_.mul_(8.0)
    gen = torch.Generator().manual_seed(42)
    batch = _Batch(torch.randint(0, 64, (b, s, feats), generator=gen), None)
    batch.in_degree = torch.randint(0, 64, (b, s), generator=gen)
    batch.out_degree = torch.randint(0, 64, (b, s), generator=gen)
    y = torch.randint(0, classes, (b,), generator=gen)
    rows = s + 1
    per_graph = []
    for g in range(b):
        nodes = torch.arange(1, rows)
        e = torch.cat([torch.randint(1, rows, (2, 4 * s), generator=gen), torch.arange(rows).repeat(2, 1),
                       torch.stack([nodes, torch.zeros_like(nodes)]), torch.stack([torch.zeros_like(nodes), nodes])],
                      dim=1)
        per_graph.append(e + g * rows)
    batch.edge_index = torch.cat(per_graph, dim=1)
    rec = {"x": batch.x.numpy(), "in_degree": batch.in_degree.numpy(), "out_degree": batch.out_degree.numpy(),
           "y": y.numpy(), "edge_index": batch.edge_index.numpy()}
    model.train()
    out = model(batch, attn_type="sparse")
    loss = torch.nn.functional.cross_entropy(out, y)
    loss.backward()
    rec["out"], rec["loss"] = out.detach().numpy(), np.float64(loss.item())
    for name, p_ in model.state_dict().items():
        rec["param/" + name] = p_.numpy()
    for name, p_ in model.named_parameters():
        if p_.grad is not None:
            rec["grad/" + name] = p_.grad.numpy()
    np.savez_compressed(out_path, **rec)
    print("wrote", out_path, "loss", loss.item())
    dist.destroy_process_group()


def _graphormer_graph_p2_worker(rank, world, ref_path, port, out_path):
    """Reference graph-level Graphormer on `world` gloo ranks, dropout 0, batch of 3 graphs: every rank
    holds s/world nodes of each graph behind its own copy of the graph token (local index 0), the
    gathered sequence has world * (s/world + 1) rows per graph.  Recorded per rank: its input slice, its
    output (read from its token row), and its parameter gradients before any all-reduce."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, ref_path)
    install_shims()
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)

    def all_to_all_via_single(output_list, input_list, group=None):
        out = torch.empty_like(torch.stack(input_list))
        dist.all_to_all_single(out, torch.stack(input_list).contiguous(), group=group)
        for o, chunk in zip(output_list, out):
            o.copy_(chunk)
    dist.all_to_all = all_to_all_via_single
    torch.distributed.all_to_all = all_to_all_via_single
    import gt_sp.initialize as init
    b, s, feats, classes = 3, 40, 2, 5
    L = s // world
    rows = world * (L + 1)                       # rows per graph in the gathered sequence
    init._GLOBAL_TOKEN_NUM = 1
    init.initialize_sequence_parallel(s, 1, 1, world)
    init.set_global_token_indices(list(range(0, rows, L + 1)))
    from models.graphormer_dist_graph_level import Graphormer
    torch.manual_seed(51)
    model = Graphormer(2, 8, 64, 0.0, 0.0, 64, "ZINC", "multi_hop", 5, 0.0, classes)
    with torch.no_grad():
        for p_ in model.parameters():
            p_.mul_(8.0)
    gen = torch.Generator().manual_seed(52)
    x = torch.randint(0, 64, (b, s, feats), generator=gen)
    in_deg = torch.randint(0, 64, (b, s), generator=gen)
    out_deg = torch.randint(0, 64, (b, s), generator=gen)
    y = torch.randint(0, classes, (b,), generator=gen)
    per_graph = []
    for g in range(b):
        e = torch.cat([torch.randint(0, rows, (2, 4 * rows), generator=gen), torch.arange(rows).repeat(2, 1)], dim=1)
        per_graph.append(e + g * rows)
    ei = torch.cat(per_graph, dim=1)
    sl = slice(rank * L, (rank + 1) * L)
    batch = _Batch(x[:, sl].contiguous(), ei)
    batch.in_degree, batch.out_degree = in_deg[:, sl].contiguous(), out_deg[:, sl].contiguous()
    model.train()
    out = model(batch, attn_type="sparse")
    loss = torch.nn.functional.cross_entropy(out, y)
    loss.backward()
    rec = {"out": out.detach().numpy(), "loss": np.float64(loss.item())}
    for name, p_ in model.named_parameters():
        if p_.grad is not None:
            rec["grad/" + name] = p_.grad.numpy()
    gathered = [None] * world
    dist.all_gather_object(gathered, rec)
    if rank == 0:
        flat = {f"r{r}/{name}": val for r, g in enumerate(gathered) for name, val in g.items()}
        flat.update({"x": x.numpy(), "in_degree": in_deg.numpy(), "out_degree": out_deg.numpy(), "y": y.numpy(),
                     "edge_index": ei.numpy(), "world": np.int64(world)})
        for name, p_ in model.state_dict().items():
            flat["param/" + name] = p_.numpy()
        np.savez_compressed(out_path, **flat)
        print("wrote", out_path, "losses", [float(g["loss"]) for g in gathered])
    dist.destroy_process_group()


def make_gt_cases(ref_path):
    import torch.multiprocessing as mp
    mp.spawn(_gt_node_worker, args=(1, ref_path, 29641, str(OUT_DIR / "gt_node_level.npz")), nprocs=1, join=True)
    mp.spawn(_gt_graph_worker, args=(2, ref_path, 29642, str(OUT_DIR / "gt_graph_level.npz")), nprocs=2, join=True)
    mp.spawn(_graphormer_graph_worker, args=(1, ref_path, 29643, str(OUT_DIR / "graphormer_graph_level.npz")),
             nprocs=1, join=True)
    mp.spawn(_graphormer_graph_p2_worker, args=(2, ref_path, 29644, str(OUT_DIR / "graphormer_graph_level_P2.npz")),
             nprocs=2, join=True)


def install_batching_shims(k_hint=None):
    """Working stand-ins for what gt_sp/utils.py needs to build a batch: the three torch_geometric.utils
    calls (torch-geometric 2.0.0 behaviour, restated) and a deterministic partitioner in place of dgl's
    METIS (node i of an n-node graph goes to partition ((13 i) mod n) * k // n)."""
    install_shims()
    tgu = sys.modules["torch_geometric.utils"]

    def remove_self_loops(edge_index, edge_attr=None):
        mask = edge_index[0] != edge_index[1]
        return edge_index[:, mask], None

    def add_self_loops(edge_index, edge_attr=None, fill_value=None, num_nodes=None):
        loops = torch.arange(num_nodes, dtype=torch.long).unsqueeze(0).repeat(2, 1)
        return torch.cat([edge_index, loops], dim=1), None

    def subgraph(subset, edge_index, edge_attr=None, relabel_nodes=False, num_nodes=None):
        n_mask = torch.zeros(num_nodes, dtype=torch.bool)
        n_mask[subset] = 1
        mask = n_mask[edge_index[0]] & n_mask[edge_index[1]]
        edge_index = edge_index[:, mask]
        if relabel_nodes:
            n_idx = torch.zeros(num_nodes, dtype=torch.long)
            n_idx[subset] = torch.arange(subset.size(0))
            edge_index = n_idx[edge_index]
        return edge_index, None

    tgu.remove_self_loops, tgu.add_self_loops, tgu.subgraph = remove_self_loops, add_self_loops, subgraph
    dgl = sys.modules["dgl"]

    class _Graph:
        def __init__(self, pair):
            self.n = int(max(int(pair[0].max()), int(pair[1].max()))) + 1

        def num_nodes(self):
            return self.n

    dgl.graph = lambda pair: _Graph(pair)
    dgl.metis_partition_assignment = lambda g, k: ((torch.arange(g.n) * 13) % g.n) * k // g.n


def golden_partition(edge_index, num_nodes, k):
    """The partitioner the batching goldens were made with (see install_batching_shims)."""
    return ((torch.arange(num_nodes) * 13) % num_nodes) * k // num_nodes


BATCH_CASES = [
    # name, model, nodes of the whole graph, seq_len, batch size (== seq_len: full batch; smaller: last batch).
    # All with args.reorder = True: without it the reference's function stops on an unassigned variable
    # (gt_sp/utils.py:511 reads attn_bias, which only the reorder branch sets).
    ("graphormer_blocks", "graphormer", 200, 96, 96),
    ("graphormer_blocks_last", "graphormer", 200, 96, 71),
    ("gt_blocks", "gt", 200, 96, 96),
    ("gt_blocks_last", "gt", 200, 96, 70),
]


def _batch_worker(rank, world, ref_path, port, out_path):
    """get_batch_reorder_blockize of the reference on `world` gloo ranks: per case and rank the feature and
    label slice, the edge list and the last-batch flag; plus gen_sub_edge_index and reformat_graph on their own."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, ref_path)
    install_batching_shims()
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import gt_sp.initialize as init
    import gt_sp.utils as ref
    init._GLOBAL_TOKEN_NUM = 1
    init.initialize_sequence_parallel(96, 1, 1, world)
    rec = {}
    for name, model, n_all, seq_len, batch in BATCH_CASES:
        gen = torch.Generator().manual_seed(sum(map(ord, name)))
        edge_index = torch.randint(0, n_all, (2, 6 * n_all), generator=gen)
        x = torch.randn(n_all, 5, generator=gen)
        y = torch.randint(0, 7, (n_all,), generator=gen)
        idx_batch = torch.randperm(n_all, generator=gen)[:batch]
        rest = None
        if batch < seq_len:
            base, extra = divmod(batch, world)
            rest = [base + (1 if r < extra else 0) for r in range(world)]
        args = types.SimpleNamespace(seq_len=seq_len, model=model, reorder=True, rank=rank)
        x_i, y_i, ei_i, bias = ref.get_batch_reorder_blockize(args, x, y, idx_batch, rest, "cpu", edge_index, n_all, 3, 4)
        assert bias is None
        rec.update({f"{name}/in_edge_index": edge_index.numpy(), f"{name}/in_x": x.numpy(), f"{name}/in_y": y.numpy(),
                    f"{name}/in_idx_batch": idx_batch.numpy(),
                    f"{name}/in_rest": np.asarray(rest if rest is not None else [], dtype=np.int64),
                    f"{name}/r{rank}/x": x_i.numpy(), f"{name}/r{rank}/y": y_i.numpy(),
                    f"{name}/r{rank}/edge_index": ei_i.numpy(),
                    f"{name}/r{rank}/last_batch": np.int64(int(init.get_last_batch_flag()))})
        if rank == 0:
            rec[f"{name}/sub_edge_index"] = ref.gen_sub_edge_index(edge_index, idx_batch, n_all).numpy()
    if rank == 0:   # the block generator on its own, both of its branches
        gen = torch.Generator().manual_seed(77)
        n, k, bs = 300, 4, 4
        ei = torch.randint(0, n, (2, 2500), generator=gen)
        part = ((torch.arange(n) * 13) % n) * k // n
        mapping = np.empty(n, dtype=np.int64)
        cur = 0
        for pid in range(k):
            nodes = np.where(part.numpy() == pid)[0]
            mapping[nodes] = np.arange(cur, cur + len(nodes))
            cur += len(nodes)
        rec["blocks/edge_index"], rec["blocks/partition"], rec["blocks/mapping"] = ei.numpy(), part.numpy(), mapping
        rec["blocks/p1"] = ref.generate_new_edges_optimized(ei, k, part, 1, bs, mapping).numpy()
        rec["blocks/p002"] = ref.generate_new_edges_optimized(ei, k, part, 0.02, bs, mapping).numpy()
        new_edges, order = ref.reformat_graph(ei, k, bs)
        rec["blocks/reformat_edges"], rec["blocks/reformat_order"] = new_edges.numpy(), order.numpy()
    gathered = [None] * world
    dist.all_gather_object(gathered, rec)
    if rank == 0:
        flat = {}
        for g in gathered:
            flat.update(g)
        np.savez_compressed(out_path, **flat)
        print("wrote", out_path)
    dist.destroy_process_group()


def make_batch_cases(ref_path):
    import torch.multiprocessing as mp
    mp.spawn(_batch_worker, args=(2, ref_path, 29651, str(OUT_DIR / "batching_P2.npz")), nprocs=2, join=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of zxmeng98/torchgt")
    ap.add_argument("--only", default="", help="'gt' regenerates the GT and graph-level model files only, "
                                               "'p8' the eight-rank exchange and layer files only, 'batching' the batch-construction file only, "
                                               "'model' the node-level Graphormer file only")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    install_shims()
    torch.set_num_threads(1)
    if args.only == "gt":
        make_gt_cases(args.reference)
        return
    if args.only == "model":
        make_model_case(args.reference)
        return
    if args.only == "batching":
        make_batch_cases(args.reference)
        return
    if args.only == "p8":
        make_ulysses_cases(args.reference, worlds=(8,))
        make_variant_cases(args.reference, worlds=(8,))
        return
    make_attention_cases()
    make_edge_cases()
    make_ulysses_cases(args.reference)
    make_model_case(args.reference)
    make_variant_cases(args.reference)
    make_gt_cases(args.reference)
    make_batch_cases(args.reference)


if __name__ == "__main__":
    main()
