"""Linear containers and the SwiGLU ``Transition``.

Mirrors protenix/model/modules/primitives.py:33-101 (``Linear`` / ``LinearNoBias``) and
:166-230 (``Transition``): same constructor arguments, parameter names and initialisers
(truncated-normal fan-in scaling; the reference draws from scipy's truncnorm, here torch's
``trunc_normal_`` gives the same distribution).  The pair transition (c_in = 128, n = 4) runs
as one fused kernel; the single-representation transition is a few tiny GEMMs left to torch.
"""
from __future__ import annotations

import math
from functools import partial
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .layer_norm import LayerNorm

_TRUNC_STD = 0.87962566103423978  # std of a unit normal truncated to [-2, 2]


def trunc_normal_init_(weight: torch.Tensor, scale: float = 1.0) -> None:
    fan_in = weight.shape[1]
    std = math.sqrt(scale / max(1, fan_in)) / _TRUNC_STD
    with torch.no_grad():
        nn.init.trunc_normal_(weight, mean=0.0, std=std, a=-2.0 * std, b=2.0 * std)


class Linear(nn.Linear):
    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None,
                 precision: Optional[torch.dtype] = None, initializer: str = "default") -> None:
        self.use_bias = bias
        self.precision = precision
        self.initializer = initializer
        super().__init__(in_features, out_features, bias=bias, device=device, dtype=dtype)
        self._init_params()

    @torch.no_grad()
    def _init_params(self) -> None:
        if self.use_bias:
            nn.init.zeros_(self.bias)
        if self.initializer == "default":
            trunc_normal_init_(self.weight, scale=1.0)
        elif self.initializer == "relu":
            trunc_normal_init_(self.weight, scale=2.0)
        elif self.initializer == "zeros":
            nn.init.zeros_(self.weight)
        else:
            raise ValueError(f"Invalid initializer: {self.initializer}.")

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        if self.precision is not None:
            d = input.dtype
            b = self.bias.to(self.precision) if self.bias is not None else None
            return F.linear(input.to(self.precision), self.weight.to(self.precision), b).to(d)
        return F.linear(input, self.weight, self.bias)


LinearNoBias = partial(Linear, bias=False)


class Transition(nn.Module):
    """x -> W_o(silu(W_a LN(x)) * (W_b LN(x))); returns the update (no residual)."""

    def __init__(self, c_in: int, n: int) -> None:
        super().__init__()
        self.n = n
        self.c_in = c_in
        self.layernorm1 = LayerNorm(c_in)
        self.linear_no_bias_a = LinearNoBias(in_features=c_in, out_features=n * c_in, initializer="relu")
        self.linear_no_bias_b = LinearNoBias(in_features=c_in, out_features=n * c_in, initializer="relu")
        self.linear_no_bias = LinearNoBias(in_features=n * c_in, out_features=c_in, initializer="zeros")

    def _fused_ok(self, x: torch.Tensor) -> bool:
        return self.c_in == ops.C_Z and self.n == 4 and x.dtype in (torch.float32, torch.bfloat16)

    def _weights(self):
        return (self.layernorm1.weight.detach().float(), self.layernorm1.bias.detach().float(),
                self.linear_no_bias_a.weight, self.linear_no_bias_b.weight,
                self.linear_no_bias.weight)

    def forward_residual_(self, x: torch.Tensor) -> torch.Tensor:
        """x += Transition(x) in place (pair path of the Pairformer block)."""
        ops.transition(x, x, *self._weights(), add_residual=True)
        return x

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("Transition: CUDA tensors only (no CPU path)")
        if self._fused_ok(x):
            xc = x.contiguous()
            return ops.transition(xc, torch.empty_like(xc), *self._weights(), add_residual=False)
        # small widths (single representation, c_in = 384): LayerNorm kernel + library GEMMs, fp32 arithmetic whatever
        # the storage type of x and of the parameters
        y = self.layernorm1(x.float().contiguous())
        a = F.silu(F.linear(y, self.linear_no_bias_a.weight.float()))
        b = F.linear(y, self.linear_no_bias_b.weight.float())
        return F.linear(a * b, self.linear_no_bias.weight.float()).to(x.dtype)
