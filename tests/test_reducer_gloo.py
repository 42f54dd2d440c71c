"""The flat-bucket gradient averager on CPU ranks (gloo, 2 and 4 ranks) against the reference's
per-parameter loop (main_sp_sparse_node_level.py:204-208: ``grad.div_(P); all_reduce(grad)`` for every
parameter that has a gradient)."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _Net(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.a = torch.nn.Linear(5, 7)
        self.b = torch.nn.Linear(7, 3)
        self.unused = torch.nn.Embedding(2, 4)      # never receives a gradient (like graph_token_virtual_distance)
        self.c = torch.nn.LayerNorm(3)

    def forward(self, x):
        return self.c(self.b(torch.tanh(self.a(x))))


def _worker(rank, world, port, ret):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import torchgt_b200.gt_sp.initialize as init
        from torchgt_b200.gt_sp.reducer import Reducer, sync_params_and_buffers
        init.initialize_sequence_parallel(8 * world, 1, 1, world)
        torch.manual_seed(100 + rank)               # different weights per rank until they are synchronised
        model = _Net()
        sync_params_and_buffers(model)
        reference = _Net()
        reference.load_state_dict(model.state_dict())
        gathered = [torch.empty_like(model.a.weight) for _ in range(world)]
        dist.all_gather(gathered, model.a.weight.data)
        errs = {"synced": max(float((g - gathered[0]).abs().max()) for g in gathered)}
        reducer = Reducer().init(model)
        worst, none_kept = 0.0, True
        for step in range(3):                       # step 0 learns which parameters get gradients
            x = torch.randn(6, 5, generator=torch.Generator().manual_seed(10 * step + rank))
            # reference loop
            reference.zero_grad(set_to_none=True)
            reference(x).square().sum().backward()
            for p in reference.parameters():
                if p.requires_grad and p.grad is not None:
                    p.grad.div_(world)
                    dist.all_reduce(p.grad, op=dist.ReduceOp.SUM, group=init.get_sequence_parallel_group())
            # flat bucket
            reducer.prepare()
            model(x).square().sum().backward()
            reducer.synchronize()
            for (name, p), pr in zip(model.named_parameters(), reference.parameters()):
                if pr.grad is None:
                    none_kept = none_kept and p.grad is None
                else:
                    worst = max(worst, float((p.grad - pr.grad).abs().max() / pr.grad.abs().max().clamp_min(1e-30)))
                    assert p.grad.data_ptr() >= reducer.flat_gradients.data_ptr()   # a view of the flat buffer
        errs["grads"], errs["none_kept"] = worst, none_kept
        ret[rank] = errs
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_flat_bucket_average_equals_the_per_parameter_loop(world):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        ret = manager.dict()
        mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
        for rank in range(world):
            errs = dict(ret[rank])
            assert errs["synced"] == 0.0 and errs["none_kept"], (rank, errs)
            # the flat buffer is summed over the ranks in another order than 80 small tensors are: fp32 rounding
            assert errs["grads"] < 1e-5, (rank, errs)
