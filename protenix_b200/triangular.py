"""Triangle multiplication and triangle attention modules over the sm_100a kernels.

Class names, constructor arguments, forward signatures and parameter names follow
protenix/model/triangular/triangular.py:93-727 and protenix/model/triangular/layers.py:104-473
so that reference checkpoints load unchanged.  The reference's back-end switches
(``triangle_multiplicative``, ``triangle_attention``), ``inplace_safe``, ``chunk_size`` and
``_inplace_chunk_size`` are accepted and ignored: there is a single fused path whose memory use
does not depend on them.
"""
from __future__ import annotations

import math
from functools import partialmethod
from typing import List, Optional

import torch
import torch.nn as nn

from . import ops
from .layer_norm import LayerNorm
from .primitives import trunc_normal_init_


class OpenfoldLinear(nn.Linear):
    """nn.Linear with the AlphaFold initialisers (protenix/model/triangular/layers.py:104-197)."""

    def __init__(self, in_dim: int, out_dim: int, bias: bool = True, init: str = "default", init_fn=None,
                 precision: Optional[torch.dtype] = None) -> None:
        super().__init__(in_dim, out_dim, bias=bias)
        with torch.no_grad():
            if bias:
                self.bias.fill_(0)
            if init_fn is not None:
                init_fn(self.weight, self.bias)
            elif init == "default":
                trunc_normal_init_(self.weight, scale=1.0)
            elif init == "relu":
                trunc_normal_init_(self.weight, scale=2.0)
            elif init == "glorot":
                nn.init.xavier_uniform_(self.weight, gain=1)
            elif init == "gating":
                self.weight.fill_(0.0)
                if bias:
                    self.bias.fill_(1.0)
            elif init == "normal":
                nn.init.kaiming_normal_(self.weight, nonlinearity="linear")
            elif init == "final":
                self.weight.fill_(0.0)
            else:
                raise ValueError("Invalid init string.")
        self.precision = precision


def _pair_input(z: torch.Tensor, mask: Optional[torch.Tensor]):
    """Accept [N,N,C] or [1,N,N,C] CUDA tensors; return (3-D contiguous view, fp32 mask, had_batch)."""
    if not z.is_cuda:
        raise RuntimeError("pair tensor must live on a CUDA device: this package has no CPU path")
    batch = z.dim() == 4
    if batch:
        if z.shape[0] != 1:
            raise RuntimeError("leading batch dimensions other than 1 are not supported")
        z = z[0]
    if z.dim() != 3:
        raise RuntimeError(f"expected [N, N, C] or [1, N, N, C], got {tuple(z.shape)}")
    if mask is not None:
        if mask.dim() == 3:
            mask = mask[0]
        mask = mask.to(device=z.device, dtype=torch.float32).contiguous()
    return z.contiguous(), mask, batch


class BaseTriangleMultiplicativeUpdate(nn.Module):
    def __init__(self, c_z: int, c_hidden: int, _outgoing: bool) -> None:
        super().__init__()
        self.c_z = c_z
        self.c_hidden = c_hidden
        self._outgoing = _outgoing
        self.linear_g = OpenfoldLinear(c_z, c_z, bias=False, init="gating")
        self.linear_z = OpenfoldLinear(c_hidden, c_z, bias=False, init="final")
        self.layer_norm_in = LayerNorm(c_z)
        self.layer_norm_out = LayerNorm(c_hidden)
        self.sigmoid = nn.Sigmoid()


class TriangleMultiplicativeUpdate(BaseTriangleMultiplicativeUpdate):
    """Algorithms 11 / 12.  ``forward`` returns the update, or z + update with ``_add_with_inplace``."""

    def __init__(self, c_z: int, c_hidden: int, _outgoing: bool = True) -> None:
        super().__init__(c_z=c_z, c_hidden=c_hidden, _outgoing=_outgoing)
        self.linear_a_p = OpenfoldLinear(c_z, c_hidden, bias=False)
        self.linear_a_g = OpenfoldLinear(c_z, c_hidden, bias=False, init="gating")
        self.linear_b_p = OpenfoldLinear(c_z, c_hidden, bias=False)
        self.linear_b_g = OpenfoldLinear(c_z, c_hidden, bias=False, init="gating")

    def _kernel_args(self):
        if self.c_z != ops.C_Z or self.c_hidden != ops.C_Z:
            raise RuntimeError(
                f"TriangleMultiplication kernels are specialised for c_z = c_hidden = {ops.C_Z}; "
                f"got c_z={self.c_z}, c_hidden={self.c_hidden} (no fallback path)")
        f = lambda p: p.detach().float()
        return (f(self.layer_norm_in.weight), f(self.layer_norm_in.bias), f(self.layer_norm_out.weight),
                f(self.layer_norm_out.bias), self.linear_a_p.weight, self.linear_a_g.weight,
                self.linear_b_p.weight, self.linear_b_g.weight, self.linear_z.weight,
                self.linear_g.weight)

    def apply_(self, z: torch.Tensor, mask: Optional[torch.Tensor], zn: Optional[torch.Tensor] = None) -> torch.Tensor:
        """z += update, in place, on a contiguous [N,N,128] tensor (used by the block).  ``zn``: the standardised
        fp16 copy of an fp32 z, if the caller has it."""
        ops.triangle_multiplication(z, z, mask, *self._kernel_args(), incoming=not self._outgoing,
                                    add_residual=True, eps=self.layer_norm_in.eps, zn=zn)
        return z

    def forward(self, z: torch.Tensor, mask: Optional[torch.Tensor] = None, inplace_safe: bool = False,
                _add_with_inplace: bool = False, _inplace_chunk_size: Optional[int] = 256,
                triangle_multiplicative: str = "torch") -> torch.Tensor:
        zc, mask, batch = _pair_input(z, mask)
        add = bool(inplace_safe and _add_with_inplace)
        out = zc if (add and zc.data_ptr() == z.data_ptr()) else torch.empty_like(zc)
        ops.triangle_multiplication(zc, out, mask, *self._kernel_args(), incoming=not self._outgoing,
                                    add_residual=add, eps=self.layer_norm_in.eps)
        return out[None] if batch else out


class TriangleMultiplicationOutgoing(TriangleMultiplicativeUpdate):
    __init__ = partialmethod(TriangleMultiplicativeUpdate.__init__, _outgoing=True)


class TriangleMultiplicationIncoming(TriangleMultiplicativeUpdate):
    __init__ = partialmethod(TriangleMultiplicativeUpdate.__init__, _outgoing=False)


class Attention(nn.Module):
    """Parameter container of the gated multi-head attention used by triangle attention
    (protenix/model/triangular/layers.py:299-359); the arithmetic runs in the fused kernels."""

    def __init__(self, c_q: int, c_k: int, c_v: int, c_hidden: int, no_heads: int, gating: bool = True) -> None:
        super().__init__()
        self.c_q, self.c_k, self.c_v = c_q, c_k, c_v
        self.c_hidden = c_hidden
        self.no_heads = no_heads
        self.gating = gating
        self.linear_q = OpenfoldLinear(c_q, c_hidden * no_heads, bias=False)
        self.linear_k = OpenfoldLinear(c_k, c_hidden * no_heads, bias=False)
        self.linear_v = OpenfoldLinear(c_v, c_hidden * no_heads, bias=False)
        self.linear_o = OpenfoldLinear(c_hidden * no_heads, c_q, bias=False, init="final")
        self.linear_g = OpenfoldLinear(c_q, c_hidden * no_heads, bias=False, init="gating") if gating else None
        self.sigmoid = nn.Sigmoid()


class TriangleAttention(nn.Module):
    """Algorithms 13 / 14.  ``forward`` returns the update (no residual), like the reference."""

    def __init__(self, c_in: int, c_hidden: int, no_heads: int, starting: bool = True, inf: float = 1e9) -> None:
        super().__init__()
        self.c_in = c_in
        self.c_hidden = c_hidden
        self.no_heads = no_heads
        self.starting = starting
        self.inf = inf
        self.layer_norm = LayerNorm(c_in)
        self.linear = OpenfoldLinear(c_in, no_heads, bias=False)
        self.mha = Attention(c_in, c_in, c_in, c_hidden, no_heads)

    def _kernel_args(self):
        if (self.c_in, self.c_hidden, self.no_heads) != (ops.C_Z, ops.D_HEAD_PAIR, ops.N_HEAD_PAIR):
            raise RuntimeError(
                f"TriangleAttention kernels are specialised for c_in={ops.C_Z}, {ops.N_HEAD_PAIR} heads x "
                f"{ops.D_HEAD_PAIR}; got c_in={self.c_in}, {self.no_heads} heads x {self.c_hidden} (no fallback path)")
        m = self.mha
        return (self.layer_norm.weight.detach().float(), self.layer_norm.bias.detach().float(),
                self.linear.weight, m.linear_q.weight, m.linear_k.weight,
                m.linear_v.weight, m.linear_g.weight, m.linear_o.weight)

    def apply_(self, z: torch.Tensor, mask: Optional[torch.Tensor], ending: bool,
               zn: Optional[torch.Tensor] = None) -> torch.Tensor:
        """z += update in place; ``ending`` selects attention along columns of the *untransposed* z,
        which equals the reference's transpose / starting-node / transpose sequence
        (protenix/model/modules/pairformer.py:160-168)."""
        ops.triangle_attention(z, z, mask, *self._kernel_args(), ending=ending, add_residual=True,
                               eps=self.layer_norm.eps, inf=self.inf, zn=zn)
        return z

    def forward(self, x: torch.Tensor, mask: Optional[torch.Tensor] = None, chunk_size: Optional[int] = None,
                triangle_attention: str = "torch", inplace_safe: bool = False) -> torch.Tensor:
        xc, mask, batch = _pair_input(x, mask)
        out = torch.empty_like(xc)
        ops.triangle_attention(xc, out, mask, *self._kernel_args(), ending=not self.starting, add_residual=False,
                               eps=self.layer_norm.eps, inf=self.inf)
        return out[None] if batch else out


TriangleAttentionStartingNode = TriangleAttention


class TriangleAttentionEndingNode(TriangleAttention):
    __init__ = partialmethod(TriangleAttention.__init__, starting=False)
