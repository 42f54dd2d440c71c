"""Re-layout kernels of the Ulysses exchange on one GPU: all ranks' buffers are processed in turn and the
collective itself is emulated by indexing, then compared with the CPU restatement of _SeqAllToAll."""
import ctypes

import numpy as np
import pytest
import torch

from helpers import load_golden
from oracle import ulysses_oracle as uo

pytestmark = pytest.mark.gpu


def _emulated_exchange(xs_per_rank, s, g, world):
    """xs_per_rank[r] = list of tensors of rank r.  Runs pack (per rank) -> all-to-all by indexing ->
    unpack (per rank) through the C ABI, exactly as torchgt_b200.gt_sp.exchange does with NCCL."""
    import math
    from torchgt_b200 import _cabi
    from torchgt_b200.gt_sp.utils import _elem
    lib = _cabi.load()
    n_t = len(xs_per_rank[0])
    x0 = xs_per_rank[0][0]
    shape = list(x0.shape)
    chunk = shape.copy(); chunk[s] //= world
    per_peer = math.prod(chunk)
    outer_s, width_s = math.prod(shape[:s]), chunk[s] * math.prod(shape[s + 1:])
    out_shape = chunk.copy(); out_shape[g] *= world
    outer_g, width_g = math.prod(chunk[:g]), math.prod(chunk[g:])
    dtype, mult = _elem(x0)
    stream = torch.cuda.current_stream().cuda_stream
    sends = []
    for xs in xs_per_rank:
        send = torch.empty((world, n_t * per_peer), dtype=x0.dtype, device="cuda")
        ptrs = [t.data_ptr() for t in xs] + [None] * (3 - n_t)
        _cabi.check(lib.tgt_a2a_pack_heads(ptrs[0], ptrs[1], ptrs[2], n_t, send.data_ptr(), 1, outer_s,
                                           width_s * mult, world, dtype, stream))
        sends.append(send)
    outs_per_rank = []
    for r in range(world):
        recv = torch.stack([sends[src][r] for src in range(world)]).contiguous()
        outs = [torch.empty(out_shape, dtype=x0.dtype, device="cuda") for _ in range(n_t)]
        optrs = [t.data_ptr() for t in outs] + [None] * (3 - n_t)
        _cabi.check(lib.tgt_a2a_unpack_heads(recv.data_ptr(), n_t, optrs[0], optrs[1], optrs[2], 1, outer_g,
                                             width_g * mult, world, dtype, stream))
        outs_per_rank.append(outs)
    return outs_per_rank


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,s,g,n_t", [((1, 7, 8, 8), 2, 1, 3), ((2, 5, 8, 8), 2, 1, 3), ((1, 16, 64), 1, 2, 1),
                                           ((3, 8, 24), 1, 2, 2), ((1, 8, 6, 9, 8), 3, 1, 1), ((2, 8, 16, 5), 1, 2, 1)])
def test_relayout_kernels_match_all_to_all_semantics(world, dtype, shape, s, g, n_t):
    if shape[s] % world != 0:
        pytest.skip("scatter axis not divisible")
    gen = torch.Generator().manual_seed(world * 31 + n_t)
    xs_per_rank = [[torch.randn(shape, generator=gen).to(dtype).cuda() for _ in range(n_t)] for _ in range(world)]
    outs = _emulated_exchange(xs_per_rank, s, g, world)
    for t in range(n_t):
        ref = uo.seq_all_to_all([xs_per_rank[r][t].float().cpu().numpy() for r in range(world)], s, g)
        for r in range(world):
            assert np.array_equal(outs[r][t].float().cpu().numpy(), ref[r])


def test_named_entry_points_for_the_two_directions():
    """tgt_a2a_pack_heads/unpack_seq (q, k, v direction) and tgt_a2a_pack_seq/unpack_heads (context
    direction) with their natural [batch, seq, width] arguments, against the reference's golden maps."""
    from torchgt_b200 import _cabi
    lib = _cabi.load()
    stream = torch.cuda.current_stream().cuda_stream
    for world in (2, 4, 8):
        g = load_golden(f"ulysses_P{world}.npz")
        L1, H, D = int(g["L"]) + 1, int(g["H"]), int(g["D"])
        W = (H // world) * D
        sends = []
        for r in range(world):
            q = torch.from_numpy(g[f"r{r}_q"]).cuda()
            send = torch.empty(world * L1 * W, device="cuda")
            _cabi.check(lib.tgt_a2a_pack_heads(q.data_ptr(), None, None, 1, send.data_ptr(), 1, L1, W, world,
                                               _cabi.TGT_F32, stream))
            sends.append(send.view(world, -1))
        for r in range(world):
            recv = torch.stack([sends[src][r] for src in range(world)]).contiguous()
            y = torch.empty(1, world * L1, H // world, D, device="cuda")
            _cabi.check(lib.tgt_a2a_unpack_seq(recv.data_ptr(), 1, y.data_ptr(), None, None, 1, L1, W, world,
                                               _cabi.TGT_F32, stream))
            assert np.array_equal(y.cpu().numpy(), g[f"r{r}_a2a_21"])
        sends = []
        for r in range(world):
            c = torch.from_numpy(g[f"r{r}_ctx_like"]).cuda()
            send = torch.empty(world * L1 * W, device="cuda")
            _cabi.check(lib.tgt_a2a_pack_seq(c.data_ptr(), None, None, 1, send.data_ptr(), 1, L1, W, world,
                                             _cabi.TGT_F32, stream))
            sends.append(send.view(world, -1))
        for r in range(world):
            recv = torch.stack([sends[src][r] for src in range(world)]).contiguous()
            y = torch.empty(1, L1, H * D, device="cuda")
            _cabi.check(lib.tgt_a2a_unpack_heads(recv.data_ptr(), 1, y.data_ptr(), None, None, 1, L1, W, world,
                                                 _cabi.TGT_F32, stream))
            assert np.array_equal(y.cpu().numpy(), g[f"r{r}_a2a_12"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_global_rows_broadcast_and_its_backward(dtype):
    import torchgt_b200.gt_sp.initialize as init
    from torchgt_b200.gt_sp.utils import copy_global_token0
    init.destroy_sequence_parallel()
    init._state.group, init._state.world_size, init._state.rank = object(), 4, 0
    rows = [0, 6, 12, 18]
    init.set_global_token_indices(rows)
    try:
        gen = torch.Generator().manual_seed(4)
        x = torch.randn(2, 24, 16, generator=gen).to(dtype)
        xc = x.cuda().requires_grad_()
        y = copy_global_token0(xc * 1.0, 1)
        ref = uo.copy_global_token0(x.float().numpy(), rows)
        assert np.array_equal(y.detach().float().cpu().numpy(), ref)
        w = torch.randn(2, 24, 16, generator=gen).to(dtype)
        (y * w.cuda()).sum().backward()
        xr = x.float().clone().requires_grad_()
        yr = xr * 1.0
        yr[:, rows, :] = yr[:, 0:1, :].expand(-1, 4, -1)
        (yr * w.float()).sum().backward()
        tol = 1e-6 if dtype == torch.float32 else 2e-2
        assert torch.allclose(xc.grad.float().cpu(), xr.grad, rtol=tol, atol=tol)
    finally:
        init.destroy_sequence_parallel()


def test_relayout_argument_errors():
    from torchgt_b200 import _cabi
    lib = _cabi.load()
    x = torch.zeros(64, device="cuda")
    assert lib.tgt_a2a_pack_heads(x.data_ptr(), None, None, 2, x.data_ptr(), 1, 4, 4, 2, 0, None) == 1
    assert "n_tensors" in _cabi.last_error()
    assert lib.tgt_a2a_pack_heads(x.data_ptr(), None, None, 1, x.data_ptr(), 1, 4, 4, 2, 7, None) == 1
    assert lib.tgt_a2a_pack_heads(x.data_ptr() + 4, None, None, 1, x.data_ptr(), 1, 4, 4, 2, 0, None) == 1
    assert "aligned" in _cabi.last_error()


def _peer_table(areas):
    return (ctypes.c_void_p * len(areas))(*[a.data_ptr() for a in areas])


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("staged", [0, 1])
@pytest.mark.parametrize("shape,s,g,n_t,alias", [((1, 9, 8, 8), 2, 1, 3, False), ((2, 6, 8, 8), 2, 1, 2, False),
                                                 ((1, 32, 64), 1, 2, 1, False), ((2, 16, 32), 1, 2, 1, True),
                                                 ((1, 64, 8), 1, 2, 3, False)])
def test_peer_push_and_fetch_match_all_to_all_semantics(world, staged, shape, s, g, n_t, alias):
    """The peer-memory transport on one GPU: every rank's slot is an ordinary local buffer and the ranks
    push one after the other (a real multi-rank barrier needs one GPU per rank and is covered by the
    multi-GPU tests)."""
    import math
    from torchgt_b200 import _cabi
    lib = _cabi.load()
    if shape[s] % world != 0:
        pytest.skip("scatter axis not divisible")
    gen = torch.Generator().manual_seed(world + n_t)
    xs = [[torch.randn(shape, generator=gen).cuda() for _ in range(n_t)] for _ in range(world)]
    nbytes = xs[0][0].numel() * 4
    slot_bytes = ((n_t * nbytes + 255) // 256) * 256
    slots = [torch.zeros(slot_bytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    table = _peer_table(slots)
    stream = torch.cuda.current_stream().cuda_stream
    chunk = list(shape); chunk[s] //= world
    out_shape = list(chunk); out_shape[g] *= world
    outer_s = math.prod(shape[:s])
    ws_bytes = chunk[s] * math.prod(shape[s + 1:]) * 4
    wg_bytes = math.prod(chunk[g:]) * 4
    rows = torch.tensor([0, 4, 12], dtype=torch.int32, device="cuda") if alias else None
    for step in range(2):          # the slot is reused
        for r in range(world):
            ptrs = [t.data_ptr() for t in xs[r]] + [None] * (3 - n_t)
            _cabi.check(lib.tgt_p2p_push(ptrs[0], ptrs[1], ptrs[2], n_t, table, slot_bytes, outer_s, ws_bytes, wg_bytes,
                                         world, r, rows.data_ptr() if alias else None, 3 if alias else 0,
                                         shape[-1] * 4 if alias else 0, staged, stream))
        outs = []
        for r in range(world):
            ys = [torch.empty(out_shape, device="cuda") for _ in range(n_t)]
            optrs = [t.data_ptr() for t in ys] + [None] * (3 - n_t)
            _cabi.check(lib.tgt_p2p_fetch(slots[r].data_ptr(), slot_bytes, n_t, optrs[0], optrs[1], optrs[2], nbytes,
                                          staged, world, wg_bytes, stream))
            outs.append(ys)
        torch.cuda.synchronize()
        for t in range(n_t):
            srcs = [xs[r][t].cpu().numpy() for r in range(world)]
            if alias:
                srcs = [uo.copy_global_token0(x, [0, 4, 12]) for x in srcs]
            ref = uo.seq_all_to_all(srcs, s, g)
            for r in range(world):
                got = outs[r][t].cpu().numpy()
                assert np.array_equal(got, ref[r]), (step, t, r)
                if not staged:       # final-position pushes can be read in place, without the fetch
                    in_place = slots[r][t * nbytes:(t + 1) * nbytes].view(torch.float32).view(*out_shape)
                    assert np.array_equal(in_place.cpu().numpy(), ref[r]), (step, t, r)
        xs = [[x + 1.0 for x in row] for row in xs]      # new values for the next exchange


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("batch,rows_local", [(1, 9), (2, 5), (1, 301)])
def test_woven_push_puts_k_and_v_of_a_row_side_by_side(world, batch, rows_local):
    """TGT_PUSH_WOVEN: the tensors pushed together arrive as one tensor [b, P * rows, n_t, H_l * D]."""
    from torchgt_b200 import _cabi
    lib = _cabi.load()
    H, D = 8, 8
    gen = torch.Generator().manual_seed(3 * world + rows_local)
    xs = [[torch.randn(batch, rows_local, H, D, generator=gen).cuda() for _ in range(2)] for _ in range(world)]
    nbytes = xs[0][0].numel() * 4
    slots = [torch.zeros(2 * nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    table = _peer_table(slots)
    stream = torch.cuda.current_stream().cuda_stream
    row_bytes = (H // world) * D * 4
    for r in range(world):
        _cabi.check(lib.tgt_p2p_push(xs[r][0].data_ptr(), xs[r][1].data_ptr(), None, 2, table, 2 * nbytes,
                                     batch * rows_local, row_bytes, rows_local * row_bytes, world, r, None, 0, 0,
                                     _cabi.TGT_PUSH_WOVEN, stream))
    torch.cuda.synchronize()
    refs = [uo.seq_all_to_all([xs[r][t].cpu().numpy() for r in range(world)], 2, 1) for t in range(2)]
    for r in range(world):
        woven = slots[r].view(torch.float32).view(batch, world * rows_local, 2, H // world, D).cpu().numpy()
        for t in range(2):
            assert np.array_equal(woven[:, :, t], refs[t][r]), (r, t)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("batch,rows_local,n_t,alias", [(1, 9, 1, False), (2, 5, 3, False), (1, 301, 1, True),
                                                        (3, 4, 1, True)])
def test_peer_pull_matches_all_to_all_semantics(world, batch, rows_local, n_t, alias):
    """Heads -> sequence by reading the peers' slots: y[b, l, r * W + c] = slot_r[b, rank * rows + l, c]
    (gt_sp/layer.py:30-49 with scatter_idx=1, gather_idx=2), global-token rows taken from row 0."""
    from torchgt_b200 import _cabi
    lib = _cabi.load()
    H, D = 8, 8
    W = (H // world) * D
    gen = torch.Generator().manual_seed(7 * world + n_t)
    # rank r holds n_t tensors [b, world * rows, W] back to back in its slot
    held = [[torch.randn(batch, world * rows_local, W, generator=gen) for _ in range(n_t)] for _ in range(world)]
    slots = [torch.cat([t.reshape(-1) for t in held[r]]).cuda() for r in range(world)]
    table = _peer_table(slots)
    slot_bytes = slots[0].numel() * 4
    stream = torch.cuda.current_stream().cuda_stream
    alias_list = list(range(0, world * rows_local, rows_local))
    rows_dev = torch.tensor(alias_list, dtype=torch.int32, device="cuda") if alias else None
    for r in range(world):
        ys = [torch.full((batch, rows_local, world * W), float("nan"), device="cuda") for _ in range(n_t)]
        ptrs = [t.data_ptr() for t in ys] + [None] * (3 - n_t)
        _cabi.check(lib.tgt_p2p_pull(table, slot_bytes, n_t, ptrs[0], ptrs[1], ptrs[2], batch, rows_local, W * 4,
                                     world, r, rows_dev.data_ptr() if alias else None, len(alias_list) if alias else 0,
                                     stream))
        torch.cuda.synchronize()
        for t in range(n_t):
            srcs = [held[p][t].numpy() for p in range(world)]
            if alias:
                srcs = [uo.copy_global_token0(x, alias_list) for x in srcs]
            ref = uo.seq_all_to_all(srcs, 1, 2)
            assert np.array_equal(ys[t].cpu().numpy(), ref[r]), (r, t)


def test_peer_barrier_gives_up_after_its_poll_limit_and_reports_the_rank():
    """A peer that never signals: the barrier must return after spin_limit polls, name the rank it waited
    for in the status word, and leave the context usable."""
    from torchgt_b200 import _cabi
    lib = _cabi.load()
    ctl = int(lib.tgt_p2p_control_bytes())
    areas = [torch.zeros(ctl, dtype=torch.uint8, device="cuda") for _ in range(3)]
    status = torch.zeros(1, dtype=torch.int32).pin_memory()
    stream = torch.cuda.current_stream().cuda_stream
    _cabi.check(lib.tgt_p2p_barrier(_peer_table(areas), 3, 1, 2000, status.data_ptr(), stream))
    torch.cuda.synchronize()
    assert int(status[0]) in (1, 3)            # 1 + rank 0 or 1 + rank 2, whichever lane gave up last
    assert float(torch.ones(4, device="cuda").sum()) == 4.0
    # argument errors are reported before any launch
    assert lib.tgt_p2p_barrier(_peer_table(areas), 3, 5, 10, status.data_ptr(), stream) == 1
    assert lib.tgt_p2p_barrier(_peer_table(areas), 3, 1, 10, None, stream) == 1
    assert lib.tgt_p2p_push(areas[0].data_ptr(), None, None, 1, _peer_table(areas), 32, 1, 16, 16, 3, 0, None, 0, 0,
                            0, stream) == 1   # 48 bytes do not fit a 32-byte slot
