"""The two compute-and-move kernels around the exchange (tgt_ln_qkv_push, tgt_pull_out_proj) on one GPU:
every rank's slot is an ordinary local buffer and the ranks run one after the other, against plain PyTorch
fp32 (LayerNorm, nn.Linear) followed by the exchange's index maps (oracle/ulysses_oracle.py)."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import ulysses_oracle as uo

pytestmark = pytest.mark.gpu

HIDDEN, HEADS = 64, 8


def _peer_table(areas):
    return (ctypes.c_void_p * len(areas))(*[a.data_ptr() for a in areas])


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("batch,rows", [(1, 70), (2, 33), (1, 1000)])
@pytest.mark.parametrize("with_norm", [True, False])
def test_layernorm_projections_and_push_land_where_the_all_to_all_puts_them(world, batch, rows, with_norm):
    from torchgt_b200 import _cabi
    lib = _cabi.load()
    gen = torch.Generator().manual_seed(17 * world + rows)
    norm = torch.nn.LayerNorm(HIDDEN)
    lin = [torch.nn.Linear(HIDDEN, HIDDEN) for _ in range(3)]
    with torch.no_grad():
        norm.weight.copy_(torch.randn(HIDDEN, generator=gen) * 0.3 + 1.0)
        norm.bias.copy_(torch.randn(HIDDEN, generator=gen) * 0.2)
    xs = [torch.randn(batch, rows, HIDDEN, generator=gen) * 2.0 + 0.5 for _ in range(world)]
    tensor_bytes = batch * world * rows * (HIDDEN // world) * 4
    slots = [torch.zeros(3 * tensor_bytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    table = _peer_table(slots)
    dev = lambda t: t.detach().cuda().contiguous()
    g, b = (dev(norm.weight), dev(norm.bias)) if with_norm else (None, None)
    w = [dev(l.weight) for l in lin]
    bias = [dev(l.bias) for l in lin]
    stream = torch.cuda.current_stream().cuda_stream
    for r in range(world):
        x = xs[r].cuda()
        _cabi.check(lib.tgt_ln_qkv_push(x.data_ptr(), g.data_ptr() if with_norm else None,
                                        b.data_ptr() if with_norm else None, norm.eps, w[0].data_ptr(), bias[0].data_ptr(),
                                        w[1].data_ptr(), bias[1].data_ptr(), w[2].data_ptr(), bias[2].data_ptr(), HIDDEN,
                                        HIDDEN, table, slots[0].numel(), batch, rows, world, r, stream))
    torch.cuda.synchronize()
    with torch.no_grad():
        ref = [[l(norm(x) if with_norm else x).view(batch, rows, HEADS, HIDDEN // HEADS).numpy() for x in xs] for l in lin]
    for t in range(3):
        want = uo.seq_all_to_all(ref[t], 2, 1)                       # [b, world * rows, H / world, D] per rank
        for r in range(world):
            got = slots[r][t * tensor_bytes:(t + 1) * tensor_bytes].view(torch.float32)
            got = got.view(batch, world * rows, HEADS // world, HIDDEN // HEADS).cpu().numpy()
            err = np.abs(got - want[r]).max() / np.abs(want[r]).max()
            assert err < 1e-5, (t, r, err)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("batch,rows,alias", [(1, 70, False), (2, 33, True), (1, 1000, True)])
def test_pull_and_output_projection_match_all_to_all_then_linear(world, batch, rows, alias):
    from torchgt_b200 import _cabi
    lib = _cabi.load()
    gen = torch.Generator().manual_seed(29 * world + rows)
    lin = torch.nn.Linear(HIDDEN, HIDDEN)
    width = HIDDEN // world
    held = [torch.randn(batch, world * rows, width, generator=gen) for _ in range(world)]   # every rank's attention output
    slots = [h.cuda().contiguous() for h in held]
    table = _peer_table(slots)
    alias_list = list(range(0, world * rows, rows))
    rows_dev = torch.tensor(alias_list, dtype=torch.int32, device="cuda") if alias else None
    w, b = lin.weight.detach().cuda().contiguous(), lin.bias.detach().cuda().contiguous()
    stream = torch.cuda.current_stream().cuda_stream
    srcs = [uo.copy_global_token0(h.numpy(), alias_list) if alias else h.numpy() for h in held]
    want_ctx = uo.seq_all_to_all(srcs, 1, 2)                          # [b, rows, HIDDEN] per rank
    for r in range(world):
        ctx = torch.full((batch, rows, HIDDEN), float("nan"), device="cuda")
        y = torch.full((batch, rows, HIDDEN), float("nan"), device="cuda")
        _cabi.check(lib.tgt_pull_out_proj(table, slots[0].numel() * 4, w.data_ptr(), b.data_ptr(), HIDDEN, HIDDEN,
                                          ctx.data_ptr(), y.data_ptr(), batch, rows, world, r,
                                          rows_dev.data_ptr() if alias else None, len(alias_list) if alias else 0, stream))
        torch.cuda.synchronize()
        assert np.array_equal(ctx.cpu().numpy(), want_ctx[r]), r
        with torch.no_grad():
            want_y = lin(torch.from_numpy(want_ctx[r])).numpy()
        err = np.abs(y.cpu().numpy() - want_y).max() / np.abs(want_y).max()
        assert err < 1e-5, (r, err)


def test_sizes_that_are_not_built_are_refused_before_anything_runs():
    from torchgt_b200 import _cabi
    lib = _cabi.load()
    d = torch.zeros(4096, device="cuda")
    table = _peer_table([d])
    p = d.data_ptr()
    rc = lib.tgt_ln_qkv_push(p, None, None, 1e-5, p, p, p, p, p, p, 96, 96, table, d.numel() * 4, 1, 4, 1, 0, None)
    assert rc == 3 and "64" in _cabi.last_error()
    rc = lib.tgt_pull_out_proj(table, d.numel() * 4, p, p, 64, 128, p, p, 1, 4, 1, 0, None, 0, None)
    assert rc == 3
    torch.cuda.synchronize()
