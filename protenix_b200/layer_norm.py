"""LayerNorm modules backed by ``px_layer_norm_fwd``.

Same constructor, parameter names and forward as the reference's ``FusedLayerNorm``
(protenix/model/layer_norm/layer_norm.py:199-233) and its ``LayerNorm`` factory
(protenix/model/triangular/layers.py:246-256).  Forward only (inference path).
"""
from __future__ import annotations

import numbers
from typing import Optional, Union

import torch
from torch.nn.parameter import Parameter

from . import ops


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
        x = input.contiguous()
        d = x.dtype
        w = self.weight.detach().to(d) if self.weight is not None else None
        b = self.bias.detach().to(d) if self.bias is not None else None
        return ops.layer_norm(x, w, b, self.eps)


def LayerNorm(c_in: int, create_scale: bool = True, create_offset: bool = True, eps: float = 1e-5) -> torch.nn.Module:
    return FusedLayerNorm(c_in, create_scale=create_scale, create_offset=create_offset, eps=eps)
