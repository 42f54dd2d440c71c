"""The short-row LayerNorm kernels (forward, backward) against torch.nn.functional.layer_norm in fp64."""
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-5   # relative to the largest reference value, fp32


def _reference(x, w, b, dy, eps):
    xd, wd, bd = (t.detach().double().cpu().requires_grad_() for t in (x, w, b))
    y = torch.nn.functional.layer_norm(xd, (xd.shape[-1],), wd, bd, eps)
    y.backward(dy.double().cpu())
    return y.detach(), xd.grad, wd.grad, bd.grad


def _close(got, ref, tol=TOL):
    scale = float(ref.abs().max()) if ref.numel() else 0.0
    err = float((got.double().cpu() - ref).abs().max()) if ref.numel() else 0.0
    return err <= tol * max(scale, 1e-30), (err, scale)


@pytest.mark.parametrize("hidden", [4, 8, 24, 32, 64, 80, 128, 256, 512])
@pytest.mark.parametrize("rows", [1, 5, 257, 4099])
def test_layer_norm_forward_and_backward_match_torch(rows, hidden):
    from torchgt_b200.layer_norm import LayerNorm
    gen = torch.Generator().manual_seed(rows * 1000 + hidden)
    x = (torch.randn(rows, hidden, generator=gen) * 2 + 0.5).cuda().requires_grad_()
    dy = torch.randn(rows, hidden, generator=gen).cuda()
    mod = LayerNorm(hidden).cuda()
    with torch.no_grad():
        mod.weight.copy_(torch.randn(hidden, generator=gen).cuda())
        mod.bias.copy_(torch.randn(hidden, generator=gen).cuda())
    y = mod(x)
    y.backward(dy)
    ref_y, ref_dx, ref_dw, ref_db = _reference(x, mod.weight, mod.bias, dy, mod.eps)
    for got, ref in ((y, ref_y), (x.grad, ref_dx), (mod.weight.grad, ref_dw), (mod.bias.grad, ref_db)):
        ok, info = _close(got, ref)
        assert ok, info


def test_layer_norm_benchmark_shape_three_dimensional_input_and_reproducibility():
    """[1, 64001, 64] as the encoder layers see it; two runs give the same bits (no atomics)."""
    from torchgt_b200.layer_norm import LayerNorm
    gen = torch.Generator().manual_seed(11)
    x0 = torch.randn(1, 64001, 64, generator=gen).cuda()
    dy = torch.randn(1, 64001, 64, generator=gen).cuda()
    mod = LayerNorm(64).cuda()
    with torch.no_grad():
        mod.weight.copy_(torch.rand(64, generator=gen).cuda() + 0.5)
        mod.bias.copy_(torch.randn(64, generator=gen).cuda())
    runs = []
    for _ in range(2):
        x = x0.clone().requires_grad_()
        mod.zero_grad()
        y = mod(x)
        y.backward(dy)
        runs.append((y.detach().clone(), x.grad.clone(), mod.weight.grad.clone(), mod.bias.grad.clone()))
    for a, b in zip(*runs):
        assert torch.equal(a, b)
    ref = _reference(x0, mod.weight, mod.bias, dy, mod.eps)
    for got, want in zip(runs[0], ref):
        ok, info = _close(got, want.view_as(got.cpu()))
        assert ok, info


def test_layer_norm_falls_back_to_torch_for_what_the_kernels_do_not_cover():
    from torchgt_b200.layer_norm import LayerNorm
    for mod, x in ((LayerNorm(6).cuda(), torch.randn(3, 6).cuda()),                       # not a multiple of 4
                   (LayerNorm(64).cuda().double(), torch.randn(3, 64).cuda().double()),   # fp64
                   (LayerNorm(64, elementwise_affine=False).cuda(), torch.randn(3, 64).cuda()),
                   (LayerNorm((2, 32)).cuda(), torch.randn(3, 2, 32).cuda())):
        ref = torch.nn.functional.layer_norm(x, mod.normalized_shape, mod.weight, mod.bias, mod.eps)
        assert torch.equal(mod(x), ref)


def test_layer_norm_argument_errors_come_back_as_codes():
    import ctypes
    from torchgt_b200 import _cabi
    lib = _cabi.load()
    x = torch.randn(4, 64).cuda()
    nb = ctypes.c_size_t()
    assert lib.tgt_layer_norm_bwd_scratch_bytes(4, 6, ctypes.byref(nb)) == 3
    assert lib.tgt_layer_norm_fwd(x.data_ptr(), None, None, 1e-5, 4, 64, x.data_ptr(), None, None) == 1
    assert lib.tgt_layer_norm_fwd(x.data_ptr(), x.data_ptr(), x.data_ptr(), 1e-5, 4, 1024, x.data_ptr(), None,
                                  None) == 3
    assert lib.tgt_layer_norm_bwd(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), 4, 64, x.data_ptr(),
                                  x.data_ptr(), x.data_ptr(), None, 0, None) == 4


def test_layer_norm_and_linear_accept_views_that_start_off_a_16_byte_boundary():
    """A contiguous view four bytes into its storage cannot be read 16 bytes at a time: the modules copy it."""
    from torchgt_b200.layer_norm import LayerNorm
    from torchgt_b200.linear import Linear
    torch.manual_seed(9)
    rows = 300
    flat = torch.randn(rows * 64 + 1, device="cuda")
    x = flat[1:].view(rows, 64)
    assert x.data_ptr() % 16 != 0 and x.is_contiguous()
    ln, lin = LayerNorm(64).cuda(), Linear(64, 64).cuda()
    xa = x.detach().requires_grad_()
    y = lin(ln(xa))
    gflat = torch.randn(rows * 64 + 1, device="cuda")
    y.backward(gflat[1:].view(rows, 64))
    xd = x.detach().double().requires_grad_()
    ref = torch.nn.functional.linear(
        torch.nn.functional.layer_norm(xd, (64,), ln.weight.double(), ln.bias.double(), ln.eps),
        lin.weight.double(), lin.bias.double())
    ref.backward(gflat[1:].view(rows, 64).double())
    tol = 2e-3 if torch.backends.cuda.matmul.allow_tf32 else 1e-5
    assert _close(y, ref.detach().cpu(), tol)[0]
    assert _close(xa.grad, xd.grad.cpu(), tol)[0]
