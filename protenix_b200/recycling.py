"""The recycling loop of the trunk around the Pairformer stack.

Mirrors the part of ``Protenix.get_pairformer_output`` that feeds the hot path
(protenix/model/protenix.py:230-296, parameters :157-168): every cycle

    z = z_init + linear_no_bias_z_cycle(layernorm_z_cycle(z))
    s = s_init + linear_no_bias_s(layernorm_s(s))
    s, z = pairformer_stack(s, z, pair_mask)

starting from z = 0 and s = 0.  Between the two updates the reference calls the template embedder
(not part of this class) and the MSA module (``msa_n_blocks > 0`` builds it here under the
reference's name ``msa_module``; protenix/model/protenix.py:258-267).  Parameter names are the
reference's, so the matching entries of a reference checkpoint load directly.

The pair update is one kernel (``ops.recycle_update``: LayerNorm folded into the 128x128
weight, residual added in the epilogue); the single update is [N, 384] and uses torch.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .layer_norm import LayerNorm
from .pairformer import PairformerStack
from .primitives import LinearNoBias
from .triangular import _pair_input


class RecyclingTrunk(nn.Module):
    def __init__(self, n_blocks: int = 48, n_heads: int = 16, c_z: int = 128, c_s: int = 384,
                 dropout: float = 0.25, N_cycle: int = 4, msa_n_blocks: int = 0, c_s_inputs: int = 449,
                 msa_configs: Optional[dict] = None) -> None:
        super().__init__()
        self.N_cycle = N_cycle
        self.c_z = c_z
        self.c_s = c_s
        self.linear_no_bias_z_cycle = LinearNoBias(in_features=c_z, out_features=c_z)
        self.linear_no_bias_s = LinearNoBias(in_features=c_s, out_features=c_s)
        self.layernorm_z_cycle = LayerNorm(c_z)
        self.layernorm_s = LayerNorm(c_s)
        # protenix/model/protenix.py:167-168: both recycling projections start at zero
        nn.init.zeros_(self.linear_no_bias_z_cycle.weight)
        nn.init.zeros_(self.linear_no_bias_s.weight)
        self.pairformer_stack = PairformerStack(n_blocks=n_blocks, n_heads=n_heads, c_z=c_z, c_s=c_s, dropout=dropout)
        if msa_n_blocks > 0:
            from .msa import MSAModule

            self.msa_module = MSAModule(n_blocks=msa_n_blocks, c_z=c_z, c_s_inputs=c_s_inputs, msa_configs=msa_configs)
        else:
            self.msa_module = None

    def update_pair(self, z: Optional[torch.Tensor], z_init: torch.Tensor, out: Optional[torch.Tensor] = None
                    ) -> torch.Tensor:
        """z_init + W LN(z); ``z`` None stands for the zeros of the first cycle.  ``out`` may be ``z``."""
        ln = self.layernorm_z_cycle
        if z is None:
            z = torch.zeros_like(z_init)
        return ops.recycle_update(z, z_init, ln.weight.detach().float(),
                                  ln.bias.detach().float() if ln.bias is not None else None,
                                  self.linear_no_bias_z_cycle.weight, eps=ln.eps, out=out)

    def update_single(self, s: torch.Tensor, s_init: torch.Tensor) -> torch.Tensor:
        x = self.layernorm_s(s.float().contiguous())
        return (s_init.float() + F.linear(x, self.linear_no_bias_s.weight)).to(s_init.dtype)

    @torch.no_grad()
    def forward(self, s_init: torch.Tensor, z_init: torch.Tensor, pair_mask: Optional[torch.Tensor] = None,
                N_cycle: Optional[int] = None, input_feature_dict: Optional[dict] = None,
                s_inputs: Optional[torch.Tensor] = None, **stack_kwargs) -> Tuple[torch.Tensor, torch.Tensor]:
        """``input_feature_dict`` (MSA features) and ``s_inputs`` feed the MSA module when the trunk has one."""
        n_cycle = self.N_cycle if N_cycle is None else N_cycle
        zi, mask, batch = _pair_input(z_init, pair_mask)
        zi = zi.contiguous()
        stack_kwargs.pop("inplace_safe", None)
        z: Optional[torch.Tensor] = None
        s = torch.zeros_like(s_init)
        for _ in range(n_cycle):
            z = self.update_pair(z, zi, out=z)            # the previous z is dead after this: updated in place
            if self.msa_module is not None and input_feature_dict is not None:
                z = self.msa_module(input_feature_dict, z, s_inputs, mask, inplace_safe=True)
            s = self.update_single(s, s_init)
            s, z = self.pairformer_stack(s, z, mask, inplace_safe=True, **stack_kwargs)
        if z is None:
            z = torch.zeros_like(zi)
        return s, (z[None] if batch else z)
