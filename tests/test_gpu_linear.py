"""The weight/bias-gradient kernel of the narrow linear layers against fp64 products."""
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 1e-5   # relative to the largest reference value; fp32 FMA sums over the rows


def _err(got, ref):
    ref = ref.double().cpu()
    return float((got.double().cpu() - ref).abs().max() / ref.abs().max().clamp_min(1e-30))


@pytest.mark.parametrize("in_features,out_features", [(64, 64), (128, 64), (64, 128), (192, 64), (64, 40), (128, 4),
                                                      (64, 100)])
@pytest.mark.parametrize("rows", [1, 31, 33, 4099, 64001])
def test_weight_and_bias_gradients_match_fp64(rows, in_features, out_features):
    from torchgt_b200.linear import wgrad
    gen = torch.Generator().manual_seed(rows + in_features * 7 + out_features)
    dy = torch.randn(rows, out_features, generator=gen).cuda()
    x = torch.randn(rows, in_features, generator=gen).cuda()
    dw, db = wgrad(dy, x)
    dw2, db2 = wgrad(dy, x)
    assert torch.equal(dw, dw2) and torch.equal(db, db2)          # fixed summation order
    assert _err(dw, dy.double().t() @ x.double()) < TOL
    assert _err(db, dy.double().sum(0)) < TOL
    dw3, none = wgrad(dy, x, with_bias=False)
    assert none is None and torch.equal(dw3, dw)


def test_linear_module_matches_nn_linear_and_keeps_its_state_dict():
    from torchgt_b200.linear import Linear
    torch.manual_seed(3)
    ours, ref = Linear(64, 128).cuda(), torch.nn.Linear(64, 128).cuda().double()
    assert set(ours.state_dict()) == set(ref.state_dict())
    ref.load_state_dict({k: v.double() for k, v in ours.state_dict().items()})
    x = torch.randn(1, 5000, 64, device="cuda")
    dy = torch.randn(1, 5000, 128, device="cuda")
    xa, xb = x.clone().requires_grad_(), x.double().requires_grad_()
    ya, yb = ours(xa), ref(xb)
    ya.backward(dy)
    yb.backward(dy.double())
    tf32 = torch.backends.cuda.matmul.allow_tf32
    tol = 2e-3 if tf32 else 1e-5        # the forward product and the input gradient are library GEMMs
    assert _err(ya, yb) < tol and _err(xa.grad, xb.grad) < tol
    assert _err(ours.weight.grad, ref.weight.grad) < TOL and _err(ours.bias.grad, ref.bias.grad) < TOL


def test_linear_falls_back_to_torch_for_what_the_kernel_does_not_cover():
    from torchgt_b200.linear import Linear
    torch.manual_seed(4)
    for mod, x in ((Linear(64, 42).cuda(), torch.randn(9, 64).cuda()),               # 42 outputs
                   (Linear(24, 64).cuda(), torch.randn(9, 24).cuda()),               # 24 inputs
                   (Linear(64, 64).cuda().double(), torch.randn(9, 64).cuda().double()),
                   (Linear(64, 64, bias=False).cuda(), torch.randn(9, 64).cuda())):
        x = x.requires_grad_()
        y = mod(x)
        y.sum().backward()
        ref = torch.nn.functional.linear(x, mod.weight, mod.bias)
        assert torch.equal(y, ref)
        assert mod.weight.grad is not None and x.grad is not None


def test_linear_wgrad_argument_errors_come_back_as_codes():
    import ctypes
    from torchgt_b200 import _cabi
    lib = _cabi.load()
    t = torch.randn(8, 64).cuda()
    nb = ctypes.c_size_t()
    assert lib.tgt_linear_wgrad_scratch_bytes(8, 40, 64, ctypes.byref(nb)) == 3       # TGT_ERR_UNSUPPORTED
    assert lib.tgt_linear_wgrad_scratch_bytes(8, 64, 42, ctypes.byref(nb)) == 3
    assert lib.tgt_linear_wgrad(t.data_ptr(), t.data_ptr(), 8, 64, 64, None, None, None, 0, None) == 1   # INVALID
    assert lib.tgt_linear_wgrad(t.data_ptr(), t.data_ptr(), 8, 64, 64, t.data_ptr(), None, None, 0, None) == 4   # WORKSPACE
