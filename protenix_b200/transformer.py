"""Single-representation attention with pair bias (Algorithm 24, ``has_s=False`` form).

Parameter names follow protenix/model/modules/transformer.py:40-254 and
protenix/model/modules/primitives.py:680-760.  The O(N^2 c_z) part -- LayerNorm(z) and the
128 -> n_heads projection that produces the bias -- runs in ``px_pair_bias_proj``; what is
left is attention over an [N, c_a] matrix (about 0.2 % of a block's FLOPs), computed in fp32
with torch's scaled-dot-product attention.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .layer_norm import LayerNorm
from .primitives import Linear, LinearNoBias


class _SingleAttention(nn.Module):
    """Parameter container: linear_q (with bias), linear_k/v/o/g (no bias)."""

    def __init__(self, c_q: int, c_hidden: int, num_heads: int, zero_init: bool) -> None:
        super().__init__()
        self.c_hidden = c_hidden
        self.num_heads = num_heads
        self.linear_q = Linear(in_features=c_q, out_features=c_hidden * num_heads)
        self.linear_k = LinearNoBias(c_q, c_hidden * num_heads)
        self.linear_v = LinearNoBias(c_q, c_hidden * num_heads)
        self.linear_o = LinearNoBias(c_hidden * num_heads, c_q)
        self.linear_g = LinearNoBias(c_q, c_hidden * num_heads, initializer="zeros")
        if zero_init:
            nn.init.zeros_(self.linear_o.weight)


class AttentionPairBias(nn.Module):
    def __init__(self, has_s: bool = True, create_offset_ln_z: bool = False, n_heads: int = 16, c_a: int = 768,
                 c_s: int = 384, c_z: int = 128, biasinit: float = -2.0, cross_attention_mode: bool = False) -> None:
        super().__init__()
        if has_s or cross_attention_mode:
            raise RuntimeError("only the has_s=False form used by PairformerBlock is implemented")
        assert c_a % n_heads == 0
        self.n_heads = n_heads
        self.has_s = has_s
        self.create_offset_ln_z = create_offset_ln_z
        self.layernorm_a = LayerNorm(c_a)
        self.attention = _SingleAttention(c_q=c_a, c_hidden=c_a // n_heads, num_heads=n_heads, zero_init=True)
        self.layernorm_z = LayerNorm(c_z, create_offset=create_offset_ln_z)
        self.linear_nobias_z = LinearNoBias(in_features=c_z, out_features=n_heads)

    def pair_bias(self, z: torch.Tensor, zn: Optional[torch.Tensor] = None) -> torch.Tensor:
        """[H, N, N] fp32 = Linear(LayerNorm(z)): the only thing this module takes from the pair representation.
        ``zn``: the standardised fp16 copy of a contiguous fp32 z, when the caller has it."""
        if z.dim() == 4:
            z = z[0]
        ln_b = self.layernorm_z.bias
        return ops.pair_bias_proj(z.contiguous(), self.layernorm_z.weight.detach().float(),
                                  ln_b.detach().float() if ln_b is not None else None,
                                  self.linear_nobias_z.weight, eps=self.layernorm_z.eps, zn=zn)

    def forward(self, a: torch.Tensor, s: Optional[torch.Tensor], z: Optional[torch.Tensor],
                bias: Optional[torch.Tensor] = None, **_unused) -> torch.Tensor:
        """``bias`` = a pair bias computed earlier with ``pair_bias(z)`` (z may then be None)."""
        dt = a.dtype
        att = self.attention
        if bias is None:
            bias = self.pair_bias(z)
        x = self.layernorm_a(a.float().contiguous())
        lead = x.shape[:-2]
        n, h, d = x.shape[-2], self.n_heads, att.c_hidden
        # fp32 arithmetic whatever the storage type of a and of the parameters (a module cast with .bfloat16() included)
        f = lambda p: p.float()
        q = F.linear(x, f(att.linear_q.weight), f(att.linear_q.bias)).view(*lead, n, h, d).transpose(-2, -3)
        k = F.linear(x, f(att.linear_k.weight)).view(*lead, n, h, d).transpose(-2, -3)
        v = F.linear(x, f(att.linear_v.weight)).view(*lead, n, h, d).transpose(-2, -3)
        o = F.scaled_dot_product_attention(q / math.sqrt(d), k, v, attn_mask=bias, scale=1.0)
        o = o.transpose(-2, -3).reshape(*lead, n, h * d)
        o = o * torch.sigmoid(F.linear(x, f(att.linear_g.weight)))
        return F.linear(o, f(att.linear_o.weight)).to(dt)
