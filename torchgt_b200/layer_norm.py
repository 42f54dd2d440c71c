"""``LayerNorm``: ``torch.nn.LayerNorm`` with the same parameters and ``state_dict`` keys whose CUDA fp32
path runs the short-row kernels of ``csrc/layer_norm.cu`` (models/graphormer_dist_node_level.py:301,306,395
are ``nn.LayerNorm(64)`` over 64,000 to 870,000 rows).  Anything else — CPU tensors, other dtypes, a hidden
size the kernels do not cover, no affine parameters — is ``torch.nn.LayerNorm`` itself."""
from __future__ import annotations

import ctypes

import torch

from . import _cabi


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def supported(x: torch.Tensor, hidden: int) -> bool:
    return x.is_cuda and x.dtype == torch.float32 and hidden % 4 == 0 and 4 <= hidden <= 512 and x.shape[-1] == hidden


_scratch_bytes: dict = {}


def _bwd_scratch(rows: int, hidden: int, device) -> torch.Tensor:
    key = (rows, hidden)
    if key not in _scratch_bytes:
        nb = ctypes.c_size_t()
        _cabi.check(_cabi.load().tgt_layer_norm_bwd_scratch_bytes(rows, hidden, ctypes.byref(nb)))
        _scratch_bytes[key] = nb.value
    return torch.empty(max(_scratch_bytes[key], 16), dtype=torch.uint8, device=device)


def forward_with_stats(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float):
    """y and the [rows, 2] (mean, 1/sqrt(var+eps)) the backward needs; x contiguous fp32 on a GPU."""
    hidden = x.shape[-1]
    rows = x.numel() // hidden
    y = torch.empty_like(x)
    stats = torch.empty((rows, 2), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        _cabi.check(_cabi.load().tgt_layer_norm_fwd(x.data_ptr(), weight.data_ptr(), bias.data_ptr(), float(eps), rows,
                                                    hidden, y.data_ptr(), stats.data_ptr(), _stream(x)))
    return y, stats


def backward(dy: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, stats: torch.Tensor):
    """dx, dgamma, dbeta from the upstream gradient, the saved input and the forward's statistics."""
    hidden = x.shape[-1]
    rows = x.numel() // hidden
    dx = torch.empty_like(x)
    dgamma = torch.empty(hidden, dtype=torch.float32, device=x.device)
    dbeta = torch.empty(hidden, dtype=torch.float32, device=x.device)
    scratch = _bwd_scratch(rows, hidden, x.device)
    with torch.cuda.device(x.device):
        _cabi.check(_cabi.load().tgt_layer_norm_bwd(dy.data_ptr(), x.data_ptr(), weight.data_ptr(), stats.data_ptr(),
                                                    rows, hidden, dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(),
                                                    scratch.data_ptr(), scratch.numel(), _stream(x)))
    return dx, dgamma, dbeta


def _aligned(t: torch.Tensor) -> torch.Tensor:
    """Contiguous ``t``, copied when it is a view that starts off a 16-byte boundary (the kernels move 16 bytes
    at a time)."""
    t = t.contiguous()
    return t if t.data_ptr() % 16 == 0 else t.clone()


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        x, weight, bias = _aligned(x), _aligned(weight), _aligned(bias)
        y, stats = forward_with_stats(x, weight, bias, eps)
        ctx.save_for_backward(x, weight, stats)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, stats = ctx.saved_tensors
        dx, dgamma, dbeta = backward(_aligned(dy), x, weight, stats)
        return dx, dgamma, dbeta, None


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """``F.layer_norm(x, (hidden,), weight, bias, eps)`` over the last dimension."""
    if weight is not None and bias is not None and supported(x, weight.numel()):
        return _LayerNormFn.apply(x, weight, bias, eps)
    return torch.nn.functional.layer_norm(x, (x.shape[-1],), weight, bias, eps)


class LayerNorm(torch.nn.LayerNorm):
    """Drop-in for ``nn.LayerNorm(hidden)``: same constructor, parameters and ``state_dict``."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if len(self.normalized_shape) == 1 and self.elementwise_affine and self.bias is not None:
            return layer_norm(x, self.weight, self.bias, self.eps)
        return super().forward(x)
