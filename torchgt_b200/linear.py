"""``Linear``: ``torch.nn.Linear`` with the same parameters and ``state_dict`` keys whose backward takes the
weight and bias gradients from ``csrc/linear_wgrad.cu`` when the layer is narrow and the rows are many (the
models' 64 x 64 projections and FFN layers over 64,000 to 870,000 rows: a product with a 64 x 64 result and a
reduction over every row, which a library GEMM runs on a few CTAs).  The forward product and the input
gradient stay library GEMMs; CPU tensors, other dtypes, inputs that are not a multiple of 64 wide and outputs
that are not a multiple of 4 wide take ``torch.nn.functional.linear`` end to end."""
from __future__ import annotations

import ctypes

import torch
from torch.nn import functional as F

from . import _cabi

_scratch_bytes: dict = {}


def supported(x: torch.Tensor, in_features: int, out_features: int) -> bool:
    return (x.is_cuda and x.dtype == torch.float32 and in_features % 64 == 0 and out_features % 4 == 0 and
            64 <= in_features <= 1024 and 4 <= out_features <= 1024)


def _aligned(t: torch.Tensor) -> torch.Tensor:
    """``t`` itself, or a copy when it is a view that starts off a 16-byte boundary (the kernels load 16 bytes
    at a time)."""
    return t if t.data_ptr() % 16 == 0 else t.clone()


def wgrad(dy: torch.Tensor, x: torch.Tensor, with_bias: bool = True):
    """``dy.t() @ x`` and ``dy.sum(0)`` for contiguous fp32 ``dy`` [rows, out] and ``x`` [rows, in] on a GPU."""
    dy, x = _aligned(dy), _aligned(x)
    rows, out_features = dy.shape
    in_features = x.shape[1]
    key = (rows, in_features, out_features)
    if key not in _scratch_bytes:
        nb = ctypes.c_size_t()
        _cabi.check(_cabi.load().tgt_linear_wgrad_scratch_bytes(rows, in_features, out_features, ctypes.byref(nb)))
        _scratch_bytes[key] = nb.value
    scratch = torch.empty(max(_scratch_bytes[key], 16), dtype=torch.uint8, device=dy.device)
    dw = torch.empty((out_features, in_features), dtype=torch.float32, device=dy.device)
    db = torch.empty(out_features, dtype=torch.float32, device=dy.device) if with_bias else None
    with torch.cuda.device(dy.device):
        _cabi.check(_cabi.load().tgt_linear_wgrad(dy.data_ptr(), x.data_ptr(), rows, in_features, out_features,
                                                  dw.data_ptr(), db.data_ptr() if with_bias else None,
                                                  scratch.data_ptr(), scratch.numel(),
                                                  torch.cuda.current_stream(dy.device).cuda_stream))
    return dw, db


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        return F.linear(x, weight, bias)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy2 = dy.contiguous().view(-1, weight.shape[0])
        dx = (dy2 @ weight).view(x.shape) if ctx.needs_input_grad[0] else None
        dw = db = None
        if ctx.needs_input_grad[1] or (ctx.has_bias and ctx.needs_input_grad[2]):
            dw, db = wgrad(dy2, x.contiguous().view(-1, weight.shape[1]), ctx.has_bias)
        return dx, dw, db


def linear(x: torch.Tensor, weight: torch.Tensor, bias) -> torch.Tensor:
    """``F.linear(x, weight, bias)``."""
    if supported(x, weight.shape[1], weight.shape[0]) and torch.is_grad_enabled() and (
            weight.requires_grad or x.requires_grad):
        return _LinearFn.apply(x, weight, bias)
    return F.linear(x, weight, bias)


class Linear(torch.nn.Linear):
    """Drop-in for ``nn.Linear``: same constructor, parameters and ``state_dict``."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return linear(x, self.weight, self.bias)
