"""The pair-representation side of the MSA module: OuterProductMean.

Mirror of ``OuterProductMean`` in protenix/model/triangular/layers.py:657-780 (constructor arguments, forward
signature, ``state_dict`` keys).  The work that scales with N^2 -- the outer product summed over the MSA rows
(2 * 1024 * S FLOP per pair element) and the 1024 -> 128 output projection with bias, normalisation and the
residual -- runs in the tcgen05 kernels behind ``px_opm_outer`` / ``px_opm_out``.  What scales with S * N (the
LayerNorm of the MSA embedding, the two c_m -> 32 projections, the mask and the normalisation counts: a thousandth of
the FLOPs) is prepared here with the LayerNorm kernel and library GEMMs.  CUDA only; c_hidden = 32 and c_z = 128 are
the compiled shapes, N <= 1024.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from . import ops
from .layer_norm import LayerNorm
from .triangular import OpenfoldLinear


class OuterProductMean(nn.Module):
    def __init__(self, c_m: int, c_z: int, c_hidden: int, eps: float = 1e-3) -> None:
        super().__init__()
        self.c_m, self.c_z, self.c_hidden, self.eps = c_m, c_z, c_hidden, eps
        self.layer_norm = LayerNorm(c_m)
        self.linear_1 = OpenfoldLinear(c_m, c_hidden, bias=False)
        self.linear_2 = OpenfoldLinear(c_m, c_hidden, bias=False)
        self.linear_out = OpenfoldLinear(c_hidden ** 2, c_z, init="final")

    def _run(self, m: torch.Tensor, mask: Optional[torch.Tensor], z_in: Optional[torch.Tensor],
             z_out: torch.Tensor) -> torch.Tensor:
        ln_b = self.layer_norm.bias
        return ops.outer_product_mean(z_in, z_out, m, mask, self.layer_norm.weight, ln_b, self.linear_1.weight,
                                      self.linear_2.weight, self.linear_out.weight, self.linear_out.bias,
                                      eps=self.eps, ln_eps=self.layer_norm.eps)

    @staticmethod
    def _msa_input(m: torch.Tensor, mask: Optional[torch.Tensor]):
        if not m.is_cuda:
            raise RuntimeError("the MSA embedding must live on a CUDA device: this package has no CPU path")
        batch = m.dim() == 4
        if batch:
            if m.shape[0] != 1:
                raise RuntimeError("leading batch dimensions other than 1 are not supported")
            m = m[0]
            mask = None if mask is None else mask[0]
        if m.dim() != 3:
            raise RuntimeError(f"expected [N_seq, N_res, c_m] or [1, N_seq, N_res, c_m], got {tuple(m.shape)}")
        return m.contiguous(), mask, batch

    @torch.no_grad()
    def forward(self, m: torch.Tensor, mask: Optional[torch.Tensor] = None, chunk_size: Optional[int] = None,
                inplace_safe: bool = False) -> torch.Tensor:
        """[*, N_res, N_res, c_z] update from m [*, N_seq, N_res, c_m] and mask [*, N_seq, N_res] (None: all ones).
        ``chunk_size`` and ``inplace_safe`` are accepted and have nothing to choose between here."""
        m, mask, batch = self._msa_input(m, mask)
        n = m.shape[1]
        out = torch.empty(n, n, self.c_z, dtype=torch.bfloat16 if m.dtype == torch.bfloat16 else torch.float32,
                          device=m.device)
        self._run(m, mask, None, out)
        return out[None] if batch else out

    @torch.no_grad()
    def apply_(self, z: torch.Tensor, m: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        """z += OuterProductMean(m) in place on a contiguous [N, N, c_z] pair tensor (how MSABlock uses the module)."""
        m, mask, _ = self._msa_input(m, mask)
        return self._run(m, mask, z, z)
