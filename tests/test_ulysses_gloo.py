"""The Ulysses layers on CPU ranks (gloo, world size 2, 4 and 8): exchange index maps, global-token
handling and autograd, against vectors produced by the reference's own layers.  The attention inside
is the CPU oracle (passed in as ``local_attention``), so these tests cover the multi-rank host logic."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden"


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class OracleAttention(torch.nn.Module):
    """local_attention stand-in for CPU ranks: the reference's op sequence from oracle/."""

    def forward(self, q, k, v, attn_bias=None, edge_index=None, attn_type=None):
        from oracle.sparse_attn_oracle import sparse_attention_ops
        b, s = q.size(0), q.size(1)
        h, d = q.size(2), q.size(3)
        out = sparse_attention_ops(q.reshape(-1, h, d), k.reshape(-1, h, d), v.reshape(-1, h, d), edge_index,
                                   attn_bias)
        return out.view(b, s, -1)


class ToyAttention(torch.nn.Module):
    """Identical copy of the stand-in local attention in tests/golden/make_golden.py."""

    def forward(self, q, k, v, attn_bias=None, *args):
        b, s = q.size(0), q.size(1)
        out = (0.5 * q + 0.25 * k * k - v).reshape(b, s, -1)
        if attn_bias is not None:
            sq = attn_bias * attn_bias
            if attn_bias.size(1) == s:
                out = out + sq.sum(dim=(2, 3)).unsqueeze(-1)
            else:
                out = out + sq.sum(dim=(1, 3)).unsqueeze(-1)
        return out


VARIANTS = ["DistributedAttention", "DistributedAttentionGlobal0", "DistributedAttentionLocalBias",
            "DistributedAttentionAll2all"]


def _worker(rank, world, port, case, ret):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import torchgt_b200.gt_sp.initialize as init
        from torchgt_b200.gt_sp import gt_layer, layer
        golden_file = f"layer_variants_P{world}.npz" if case == "variants" else f"ulysses_P{world}.npz"
        with np.load(GOLDEN / golden_file) as z:
            g = {k: z[k] for k in z.files}
        L, H, D = int(g["L"]), int(g["H"]), int(g["D"])
        init.set_global_token_num(1)
        init.initialize_sequence_parallel(L * world, 1, 1, world)
        init.set_global_token_indices(list(range(0, world * (L + 1), L + 1)))
        group = init.get_sequence_parallel_group()
        t = lambda name: torch.from_numpy(g[f"r{rank}_{name}"])
        errs = {}
        if case == "maps":
            errs["a2a_21"] = float((layer._SeqAllToAll.apply(group, t("q"), 2, 1) - t("a2a_21")).abs().max())
            errs["a2a_12"] = float((layer._SeqAllToAll.apply(group, t("ctx_like"), 1, 2) - t("a2a_12")).abs().max())
            # backward of one direction is the other direction
            x = t("q").clone().requires_grad_()
            y = layer._SeqAllToAll.apply(group, x, 2, 1)
            y.backward(t("a2a_21"))
            errs["a2a_roundtrip"] = float((x.grad - t("q")).abs().max())
            # gather / scatter helpers
            part = torch.full((1, 3, 2), float(rank)).requires_grad_()
            full = layer._SeqGather.apply(part, 1)
            assert full.shape == (1, 3 * world, 2)
            errs["gather"] = float((full[:, 3 * rank:3 * rank + 3] - rank).abs().max() +
                                   (full[:, 0:3] - 0).abs().max())
            full.backward(torch.arange(3 * world, dtype=torch.float32).view(1, -1, 1).expand(1, -1, 2).contiguous())
            errs["gather_bwd"] = float((part.grad[0, :, 0] - torch.arange(3 * rank, 3 * rank + 3)).abs().max())
            heads = torch.arange(2 * world, dtype=torch.float32).view(1, -1, 1, 1).repeat(1, 1, 2, 2).requires_grad_()
            mine = layer._SeqScatter.apply(heads)
            errs["scatter"] = float((mine[0, :, 0, 0] - torch.arange(2 * rank, 2 * rank + 2)).abs().max())
            mine.sum().backward()
            errs["scatter_bwd"] = float((heads.grad - 1).abs().max())
        elif case == "nomerge":
            q, k, v = (t(n).clone().requires_grad_() for n in "qkv")
            lay = layer.DistributedAttentionNoMerge(OracleAttention(), group).train()
            out = lay(q, k, v, None, torch.from_numpy(g["r0_edge_index"]), "sparse")
            (out * t("dout")).sum().backward()
            for name, mine in (("out", out.detach()), ("dq", q.grad), ("dk", k.grad), ("dv", v.grad)):
                ref = t(name)
                errs[name] = float((mine - ref).abs().max() / ref.abs().max())
            # evaluation mode bypasses the exchange
            lay.eval()
            ev = lay(q.detach(), k.detach(), v.detach(), None, torch.tensor([[0], [0]]), "sparse")
            assert ev.shape == (1, L + 1, H * D)
        elif case == "variants":
            for name in VARIANTS:
                tv = lambda key: torch.from_numpy(g[f"r{rank}/{name}/{key}"])
                q, k, v, bias = (tv(n).clone().requires_grad_() for n in ("q", "k", "v", "bias"))
                lay = getattr(layer, name)(ToyAttention(), group).train()
                out = lay(q, k, v, bias) if name == "DistributedAttention" else lay(q, k, v, bias, None)
                (out * tv("dout")).sum().backward()
                for key, mine in (("out", out.detach()), ("dq", q.grad), ("dk", k.grad), ("dv", v.grad),
                                  ("dbias", bias.grad)):
                    ref = tv(key)
                    errs[f"{name}/{key}"] = float((mine - ref).abs().max() / max(float(ref.abs().max()), 1e-30))
        elif case == "gt":
            # GT layers: no global token.  Every rank checks against a single-process evaluation of the
            # whole sequence with all heads.
            from oracle.sparse_attn_oracle import sparse_attention_ops
            gen = torch.Generator().manual_seed(5)
            S = (L + 1) * world
            qf, kf, vf, wf = (torch.randn(1, S, H, D, generator=gen) for _ in range(4))
            ei = torch.randint(0, S, (2, 6 * S), generator=gen)
            sl = slice(rank * (L + 1), (rank + 1) * (L + 1))
            q, k, v = (x[:, sl].clone().requires_grad_() for x in (qf, kf, vf))
            for cls in (gt_layer.DistributedAttention, gt_layer.DistributedAttentionNodeLevel):
                lay = cls(OracleAttention(), group).train()
                out = lay(q, k, v, None, ei, "sparse")
                q.grad = k.grad = v.grad = None
                (out * wf[:, sl].reshape(1, L + 1, -1)).sum().backward()
                qr, kr, vr = (x[0].clone().requires_grad_() for x in (qf, kf, vf))
                ref = sparse_attention_ops(qr, kr, vr, ei)
                (ref * wf[0]).sum().backward()
                errs[cls.__name__ + "_out"] = float((out[0] - ref[sl].reshape(L + 1, -1)).abs().max())
                errs[cls.__name__ + "_dq"] = float((q.grad[0] - qr.grad[sl]).abs().max())
                errs[cls.__name__ + "_dk"] = float((k.grad[0] - kr.grad[sl]).abs().max())
                errs[cls.__name__ + "_dv"] = float((v.grad[0] - vr.grad[sl]).abs().max())
        ret[rank] = errs
    finally:
        dist.destroy_process_group()


def _run(world, case):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        ret = manager.dict()
        mp.spawn(_worker, args=(world, _free_port(), case, ret), nprocs=world, join=True)
        return {r: dict(ret[r]) for r in range(world)}


@pytest.mark.parametrize("world", [2, 4, 8])
def test_exchange_maps_and_gather_scatter(world):
    for rank, errs in _run(world, "maps").items():
        assert all(v == 0.0 for v in errs.values()), (rank, errs)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_nomerge_layer_matches_reference_outputs_and_gradients(world):
    for rank, errs in _run(world, "nomerge").items():
        assert max(errs.values()) < 1e-5, (rank, errs)


@pytest.mark.parametrize("world", [2])
def test_gt_layers_match_single_process_attention(world):
    for rank, errs in _run(world, "gt").items():
        assert max(errs.values()) < 1e-5, (rank, errs)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_layer_variants_with_merged_global_tokens_match_the_reference(world):
    """DistributedAttention, ...Global0, ...LocalBias, ...All2all of the reference (no model uses them):
    same outputs and gradients around the same toy local attention, bias paths included."""
    for rank, errs in _run(world, "variants").items():
        assert len(errs) == 20
        assert max(errs.values()) < 1e-6, (rank, errs)
