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
                      TGT_EXCHANGE=transport, TGT_P2P_SPIN_LIMIT="4000000")
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
        torch.cuda.synchronize()
        from torchgt_b200.gt_sp import p2p
        px = p2p.peer_exchange_for(group, dev)
        errs["used_peer_memory"] = px is not None
        if px is not None:
            px.check()
        ret[rank] = errs
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("transport", ["p2p", "nccl"])
def test_nomerge_layer_on_real_gpus(world, transport):
    """transport = p2p: the library's own NVLink peer-memory exchange; nccl: one all_to_all_single."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        ret = manager.dict()
        mp.spawn(_worker, args=(world, _free_port(), transport, ret), nprocs=world, join=True)
        for rank in range(world):
            errs = dict(ret[rank])
            assert errs.pop("used_peer_memory") == (transport == "p2p")
            assert errs["a2a_21"] == 0.0 and errs["a2a_12"] == 0.0, (rank, errs)
            assert max(errs.values()) < 1e-5, (rank, errs)
