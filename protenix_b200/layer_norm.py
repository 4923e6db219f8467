"""LayerNorm modules backed by ``px_layer_norm_fwd``.

Same constructor, parameter names and forward as the reference's ``FusedLayerNorm``
(protenix/model/layer_norm/layer_norm.py:199-233) and its ``LayerNorm`` factory
(protenix/model/triangular/layers.py:246-256).  Under ``torch.no_grad()`` (the inference path) the forward is one
kernel launch; when gradients are wanted the op runs as an autograd function whose backward is
``px_layer_norm_bwd`` (the reference's ``FusedLayerNormAffineFunction``, layer_norm.py:69-196).
"""
from __future__ import annotations

import numbers
from typing import Optional, Union

import torch
from torch.nn.parameter import Parameter

from . import ops


class _LayerNormFunction(torch.autograd.Function):
    """y = LayerNorm(x) with optional scale and offset; saves x and the fp32 row statistics for the backward."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        d = x.dtype
        w = weight.detach().to(d) if weight is not None else None
        b = bias.detach().to(d) if bias is not None else None
        xc = x.contiguous()
        y, mean, invvar = ops.layer_norm(xc, w, b, eps, return_stats=True)
        ctx.save_for_backward(xc, w, mean, invvar)
        ctx.has_bias = bias is not None
        ctx.param_dtypes = (None if weight is None else weight.dtype, None if bias is None else bias.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, w, mean, invvar = ctx.saved_tensors
        want_w = w is not None and ctx.needs_input_grad[1]
        want_b = ctx.has_bias and ctx.needs_input_grad[2]
        dx, dw, db = ops.layer_norm_bwd(dy.contiguous(), xc, mean, invvar, w, want_w, want_b)
        wd, bd = ctx.param_dtypes
        return (dx if ctx.needs_input_grad[0] else None, None if dw is None else dw.to(wd),
                None if db is None else db.to(bd), None)


class FusedLayerNorm(torch.nn.Module):
    def __init__(self, normalized_shape: Union[int, list, torch.Size], create_scale: bool = True,
                 create_offset: bool = True, eps: float = 1e-5) -> None:
        super().__init__()
        if isinstance(normalized_shape, numbers.Integral):
            normalized_shape = (normalized_shape,)
        self.normalized_shape = torch.Size(normalized_shape)
        if len(self.normalized_shape) != 1:
            raise RuntimeError("FusedLayerNorm normalises over the last axis only")
        self.eps = eps
        self.weight = Parameter(torch.ones(*normalized_shape)) if create_scale else None
        self.bias = Parameter(torch.zeros(*normalized_shape)) if create_offset else None

    def reset_parameters(self) -> None:
        if self.weight is not None:
            torch.nn.init.ones_(self.weight)
        if self.bias is not None:
            torch.nn.init.zeros_(self.bias)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        if input.shape[-1] != self.normalized_shape[0]:
            raise RuntimeError(
                f"Expected input with last dimension {self.normalized_shape[0]}, got {tuple(input.shape)}")
        if torch.is_grad_enabled() and (input.requires_grad or (self.weight is not None and self.weight.requires_grad)
                                        or (self.bias is not None and self.bias.requires_grad)):
            return _LayerNormFunction.apply(input, self.weight, self.bias, self.eps)
        x = input.contiguous()
        d = x.dtype
        w = self.weight.detach().to(d) if self.weight is not None else None
        b = self.bias.detach().to(d) if self.bias is not None else None
        return ops.layer_norm(x, w, b, self.eps)


def LayerNorm(c_in: int, create_scale: bool = True, create_offset: bool = True, eps: float = 1e-5) -> torch.nn.Module:
    return FusedLayerNorm(c_in, create_scale=create_scale, create_offset=create_offset, eps=eps)
