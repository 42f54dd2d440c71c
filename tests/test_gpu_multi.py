"""The Ulysses layer on real GPUs over NCCL (needs at least two devices; skipped otherwise): the full
drop-in stack — DistributedAttentionNoMerge around CoreAttention with the CUDA kernels — against the
vectors the reference's own layer produced."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden"

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, transport, ret):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TGT_EXCHANGE=transport.split("-")[0], TGT_P2P_SPIN_LIMIT="4000000",
                      TGT_FUSED_LAYER="0" if transport.endswith("-unfused") else "1")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import torchgt_b200.gt_sp.initialize as init
        from torchgt_b200 import CoreAttention
        from torchgt_b200.gt_sp.layer import DistributedAttentionNoMerge, _SeqAllToAll
        with np.load(GOLDEN / f"ulysses_P{world}.npz") as z:
            g = {k: z[k] for k in z.files}
        L, H, D = int(g["L"]), int(g["H"]), int(g["D"])
        init.set_global_token_num(1)
        init.initialize_sequence_parallel(L * world, 1, 1, world)
        init.set_global_token_indices(list(range(0, world * (L + 1), L + 1)))
        group = init.get_sequence_parallel_group()
        t = lambda name: torch.from_numpy(g[f"r{rank}_{name}"]).to(dev)
        errs = {}
        errs["a2a_21"] = float((_SeqAllToAll.apply(group, t("q"), 2, 1) - t("a2a_21")).abs().max())
        errs["a2a_12"] = float((_SeqAllToAll.apply(group, t("ctx_like"), 1, 2) - t("a2a_12")).abs().max())
        q, k, v = (t(n).clone().requires_grad_() for n in "qkv")
        layer = DistributedAttentionNoMerge(CoreAttention(H * D, 0.0, H, 1), group).train()
        out = layer(q, k, v, None, torch.from_numpy(g["r0_edge_index"]).to(dev), "sparse")
        (out * t("dout")).sum().backward()
        for name, mine in (("out", out.detach()), ("dq", q.grad), ("dk", k.grad), ("dv", v.grad)):
            ref = t(name)
            errs[name] = float((mine - ref).abs().max() / ref.abs().max())
        # a second step through the same slots (their reuse is the delicate part of the transport)
        q2, k2, v2 = (t(n).clone().requires_grad_() for n in "qkv")
        out2 = layer(q2, k2, v2, None, torch.from_numpy(g["r0_edge_index"]).to(dev), "sparse")
        (out2 * t("dout")).sum().backward()
        errs["out_again"] = float((out2.detach() - t("out")).abs().max() / t("out").abs().max())
        errs["dk_again"] = float((k2.grad - t("dk")).abs().max() / t("dk").abs().max())
        torch.cuda.synchronize()
        from torchgt_b200.gt_sp import p2p
        px = p2p.peer_exchange_for(group, dev)
        errs["used_peer_memory"] = px is not None
        p2p.check_peer_exchanges()
        ret[rank] = errs
    finally:
        from torchgt_b200.gt_sp import p2p
        p2p.reset_peer_exchanges()
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("transport", ["p2p", "p2p-unfused", "nccl"])
def test_nomerge_layer_on_real_gpus(world, transport):
    """transport = p2p: the library's own NVLink peer-memory exchange with the layer as one autograd node
    (attention reads the landed q, k, v in place); p2p-unfused: the same transport behind the general
    _SeqAllToAll; nccl: one all_to_all_single."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        ret = manager.dict()
        mp.spawn(_worker, args=(world, _free_port(), transport, ret), nprocs=world, join=True)
        for rank in range(world):
            errs = dict(ret[rank])
            assert errs.pop("used_peer_memory") == transport.startswith("p2p")
            assert errs["a2a_21"] == 0.0 and errs["a2a_12"] == 0.0, (rank, errs)
            assert max(errs.values()) < 1e-5, (rank, errs)


class _Batch:
    def __init__(self, x, edge_index):
        self.x, self.edge_index = x, edge_index


def _gt_worker(rank, world, port, ret):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TGT_P2P_SPIN_LIMIT="4000000")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import torchgt_b200.gt_sp.initialize as init
        from torchgt_b200.gt import GTGraphLevel
        with np.load(GOLDEN / "gt_graph_level.npz") as z:
            g = {k: z[k] for k in z.files}
        s_len = g["x"].shape[1]
        L = s_len // world
        init.initialize_sequence_parallel(s_len, 1, 1, world)
        model = GTGraphLevel(2, 8, 64, 0.0, 0.0, 64, "ZINC", "multi_hop", 5, 0.0, 5)
        model.load_state_dict({k[len("param/"):]: torch.from_numpy(v) for k, v in g.items() if k.startswith("param/")},
                              strict=True)
        model = model.to(dev).train()
        x = torch.from_numpy(g["x"][:, rank * L:(rank + 1) * L]).contiguous().to(dev)
        out = model(_Batch(x, torch.from_numpy(g["edge_index"]).to(dev)), attn_type="sparse")
        loss = torch.nn.functional.cross_entropy(out, torch.from_numpy(g["y"]).to(dev))
        loss.backward()
        ref = torch.from_numpy(g["out"]).to(dev)
        errs = {"out": float((out.detach() - ref).abs().max() / ref.abs().max())}
        worst = 0.0
        for name, p in model.named_parameters():
            if "grad/" + name not in g:
                continue
            grad = p.grad.clone()
            if not name.startswith("MLP_layer"):       # each rank holds the part through its slice of the sequence
                dist.all_reduce(grad)
            gref = torch.from_numpy(g["grad/" + name]).to(dev)
            if float(gref.abs().max()) < 1e-7:
                continue
            worst = max(worst, float((grad - gref).abs().max() / gref.abs().max()))
        errs["grads"] = worst
        torch.cuda.synchronize()
        ret[rank] = errs
    finally:
        from torchgt_b200.gt_sp import p2p
        p2p.reset_peer_exchanges()
        dist.destroy_process_group()


def test_gt_graph_level_model_on_two_gpus_matches_the_reference_on_two_ranks():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        ret = manager.dict()
        mp.spawn(_gt_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
        for rank in range(2):
            assert ret[rank]["out"] < 1e-4 and ret[rank]["grads"] < 1e-4, (rank, dict(ret[rank]))


def _graphormer_graph_worker(rank, world, port, fused_block, ret):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TGT_P2P_SPIN_LIMIT="4000000", TGT_FUSED_BLOCK=fused_block)
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import torchgt_b200.gt_sp.initialize as init
        from torchgt_b200.graphormer import GraphormerGraphLevel
        with np.load(GOLDEN / "graphormer_graph_level_P2.npz") as z:
            g = {k: z[k] for k in z.files}
        s_len = g["x"].shape[1]
        L = s_len // world
        init.set_global_token_num(1)
        init.initialize_sequence_parallel(s_len, 1, 1, world)
        init.set_global_token_indices(list(range(0, world * (L + 1), L + 1)))
        model = GraphormerGraphLevel(2, 8, 64, 0.0, 0.0, 64, "ZINC", "multi_hop", 5, 0.0, 5)
        model.load_state_dict({k[len("param/"):]: torch.from_numpy(v) for k, v in g.items() if k.startswith("param/")},
                              strict=True)
        model = model.to(dev).train()
        sl = slice(rank * L, (rank + 1) * L)
        batch = _Batch(torch.from_numpy(g["x"][:, sl]).contiguous().to(dev), torch.from_numpy(g["edge_index"]).to(dev))
        batch.in_degree = torch.from_numpy(g["in_degree"][:, sl]).contiguous().to(dev)
        batch.out_degree = torch.from_numpy(g["out_degree"][:, sl]).contiguous().to(dev)
        out = model(batch, attn_type="sparse")
        loss = torch.nn.functional.cross_entropy(out, torch.from_numpy(g["y"]).to(dev))
        loss.backward()
        ref = torch.from_numpy(g[f"r{rank}/out"]).to(dev)
        errs = {"out": float((out.detach() - ref).abs().max() / ref.abs().max())}
        worst, checked = 0.0, 0
        for name, p in model.named_parameters():
            key = f"r{rank}/grad/{name}"
            if key not in g or float(np.abs(g[key]).max()) < 1e-7:
                continue
            gref = torch.from_numpy(g[key]).to(dev)
            worst = max(worst, float((p.grad - gref).abs().max() / gref.abs().max()))
            checked += 1
        errs["grads"], errs["checked"] = worst, checked
        torch.cuda.synchronize()
        ret[rank] = errs
    finally:
        from torchgt_b200.gt_sp import p2p
        p2p.reset_peer_exchanges()
        dist.destroy_process_group()


@pytest.mark.parametrize("fused_block", ["1", "0"], ids=["fused-block", "layer-node"])
def test_graphormer_graph_level_model_on_two_gpus_matches_the_reference_rank_by_rank(fused_block):
    """Batch of three graphs, every rank's own graph token in front of its slice: exercises the exchange and
    the global-token copy with a batch dimension.  fused-block: LayerNorm, projections and exchange in the
    kernels of csrc/fused_projection.cu; layer-node: library projections with the pushes started beside them."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        ret = manager.dict()
        mp.spawn(_graphormer_graph_worker, args=(2, _free_port(), fused_block, ret), nprocs=2, join=True)
        for rank in range(2):
            errs = dict(ret[rank])
            assert errs["out"] < 1e-4 and errs["grads"] < 1e-4 and errs["checked"] >= 35, (rank, errs)
