"""The pair-representation side of the MSA module: OuterProductMean.

Mirror of ``OuterProductMean`` in protenix/model/triangular/layers.py:657-780 (constructor arguments, forward
signature, ``state_dict`` keys).  The work that scales with N^2 -- the outer product summed over the MSA rows
(2 * 1024 * S FLOP per pair element) and the 1024 -> 128 output projection with bias, normalisation and the
residual -- runs in the tcgen05 kernels behind ``px_opm_outer`` / ``px_opm_out``.  What scales with S * N (the
LayerNorm of the MSA embedding, the two c_m -> 32 projections, the mask and the normalisation counts: a thousandth of
the FLOPs) is prepared here with the LayerNorm kernel and library GEMMs.  CUDA only; c_hidden = 32 and c_z = 128 are
the compiled shapes; the outer products are formed for blocks of token rows so that their buffer stays within 2 GiB.
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


class MSAPairWeightedAveraging(nn.Module):
    """Mirror of protenix/model/modules/pairformer.py:343-422.  The pair bias Linear(LayerNorm(z)) (n_heads values per
    pair element, the only N^2-sized step) runs in ``px_pair_bias_proj``; the rest is S*N-sized work on the LayerNorm
    kernel and library GEMMs."""

    def __init__(self, c_m: int = 64, c: int = 32, c_z: int = 128, n_heads: int = 8) -> None:
        super().__init__()
        from .primitives import LinearNoBias

        self.c_m, self.c, self.n_heads, self.c_z = c_m, c, n_heads, c_z
        self.layernorm_m = LayerNorm(c_m)
        self.linear_no_bias_mv = LinearNoBias(in_features=c_m, out_features=c * n_heads)
        self.layernorm_z = LayerNorm(c_z)
        self.linear_no_bias_z = LinearNoBias(in_features=c_z, out_features=n_heads)
        self.linear_no_bias_mg = LinearNoBias(in_features=c_m, out_features=c * n_heads, initializer="zeros")
        self.linear_no_bias_out = LinearNoBias(in_features=c * n_heads, out_features=c_m, initializer="zeros")

    def pair_weights(self, z: torch.Tensor) -> torch.Tensor:
        """w [n_heads, N, N] = softmax over the second token index of Linear(LayerNorm(z)), fp32."""
        ln_b = self.layernorm_z.bias
        b = ops.pair_bias_proj(z.contiguous(), self.layernorm_z.weight.detach().float(),
                               None if ln_b is None else ln_b.detach().float(), self.linear_no_bias_z.weight,
                               eps=self.layernorm_z.eps)
        return torch.softmax(b, dim=-1)

    @torch.no_grad()
    def forward(self, m: torch.Tensor, z: torch.Tensor, w: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The update of m [S, N, c_m] (not added).  ``w``: pair weights computed earlier with ``pair_weights(z)``."""
        if w is None:
            w = self.pair_weights(z)
        s_rows, n, _ = m.shape
        mn = self.layernorm_m(m)
        v = self.linear_no_bias_mv(mn).view(s_rows, n, self.n_heads, self.c)
        g = torch.sigmoid(self.linear_no_bias_mg(mn)).view(s_rows, n, self.n_heads, self.c)
        # wv[s, i, h, :] = sum_j w[h, i, j] v[s, j, h, :]: one [N x N] . [N x S c] product per head
        vh = v.permute(2, 1, 0, 3).reshape(self.n_heads, n, s_rows * self.c)
        wv = torch.bmm(w.to(vh.dtype), vh).view(self.n_heads, n, s_rows, self.c).permute(2, 1, 0, 3)
        o = (g * wv).reshape(s_rows, n, self.n_heads * self.c)
        return self.linear_no_bias_out(o)


class MSAStack(nn.Module):
    """Mirror of protenix/model/modules/pairformer.py:425-572 (eval path: ``inference_forward``)."""

    def __init__(self, c_m: int = 64, c_z: int = 128, c: int = 8, dropout: float = 0.15,
                 msa_chunk_size: Optional[int] = 2048, msa_max_size: Optional[int] = 16384) -> None:
        super().__init__()
        from .primitives import Transition

        self.c = c
        self.msa_pair_weighted_averaging = MSAPairWeightedAveraging(c_m=c_m, c=c, c_z=c_z)
        self.p_drop = dropout
        self.transition_m = Transition(c_in=c_m, n=4)
        self.msa_chunk_size, self.msa_max_size = msa_chunk_size, msa_max_size

    @torch.no_grad()
    def forward(self, m: torch.Tensor, z: torch.Tensor) -> torch.Tensor:
        """m += PairWeightedAveraging(m, z); m += Transition(m), in place over chunks of MSA rows."""
        if self.training and self.p_drop > 0:
            raise RuntimeError("MSAStack: training-mode dropout is not implemented; call .eval()")
        w = self.msa_pair_weighted_averaging.pair_weights(z)      # the same for every chunk
        chunk = self.msa_chunk_size or m.shape[0]
        for start in range(0, m.shape[0], chunk):
            part = m[start:start + chunk]
            part += self.msa_pair_weighted_averaging(part, z, w)
            part += self.transition_m(part)
        return m


class MSABlock(nn.Module):
    """Mirror of protenix/model/modules/pairformer.py:575-678: outer product mean into z, the MSA stack (unless this
    is the last block), then a pair-only Pairformer block."""

    def __init__(self, c_m: int = 64, c_z: int = 128, c_hidden: int = 32, is_last_block: bool = False,
                 msa_dropout: float = 0.15, pair_dropout: float = 0.25, msa_chunk_size: Optional[int] = 2048,
                 msa_max_size: Optional[int] = 16384, hidden_scale_up: bool = False) -> None:
        super().__init__()
        from .pairformer import PairformerBlock

        self.c_m, self.c_z, self.c_hidden, self.is_last_block = c_m, c_z, c_hidden, is_last_block
        self.outer_product_mean_msa = OuterProductMean(c_m=c_m, c_z=c_z, c_hidden=c_hidden)
        if not is_last_block:
            self.msa_stack = MSAStack(c_m=c_m, c_z=c_z, dropout=msa_dropout, msa_chunk_size=msa_chunk_size,
                                      msa_max_size=msa_max_size)
        self.pair_stack = PairformerBlock(c_z=c_z, c_s=0, dropout=pair_dropout, hidden_scale_up=hidden_scale_up)

    @torch.no_grad()
    def forward(self, m: torch.Tensor, z: torch.Tensor, pair_mask, triangle_multiplicative: str = "torch",
                triangle_attention: str = "torch", inplace_safe: bool = False, chunk_size: Optional[int] = None):
        """(m, z) -> (m or None, z).  m [S, N, c_m], z [N, N, c_z] (a leading batch of 1 is accepted for z).  m is
        updated in place, as the reference's eval path does; z is copied first unless ``inplace_safe``."""
        batch = z.dim() == 4
        zc = z[0] if batch else z
        if not zc.is_cuda or not m.is_cuda:
            raise RuntimeError("MSABlock: CUDA tensors only (no CPU path)")
        zc = zc.contiguous()
        if not inplace_safe and zc.data_ptr() == z.data_ptr():
            zc = zc.clone()
        mm = m[0] if m.dim() == 4 else m
        self.outer_product_mean_msa.apply_(zc, mm)
        if not self.is_last_block:
            mm = self.msa_stack(mm, zc)
        _, zc = self.pair_stack(None, zc, pair_mask, inplace_safe=True)
        return (None if self.is_last_block else m), (zc[None] if batch else zc)


def sample_msa_indices(n: int, device, lower_bound: int = 1, strategy: str = "random") -> torch.Tensor:
    """How many and which MSA rows a forward pass uses (protenix/model/utils.py:290-311): a size drawn uniformly from
    [min(lower_bound, n), n], then a random subset or the first rows."""
    if strategy not in ("random", "topk"):
        raise ValueError("strategy must be 'random' or 'topk'")
    size = int(torch.randint(low=min(lower_bound, n), high=n + 1, size=(1,)).item())
    return torch.randperm(n, device=device)[:size] if strategy == "random" else torch.arange(size, device=device)


class MSAModule(nn.Module):
    """Mirror of protenix/model/modules/pairformer.py:682-911 (Algorithm 8): MSA features -> m, then ``n_blocks``
    MSABlocks that write into the pair representation.  Eval only."""

    def __init__(self, n_blocks: int = 4, c_m: int = 64, c_z: int = 128, c_s_inputs: int = 449,
                 msa_dropout: float = 0.15, pair_dropout: float = 0.25, blocks_per_ckpt: Optional[int] = 1,
                 msa_chunk_size: Optional[int] = 2048, msa_max_size: Optional[int] = 16384,
                 msa_configs: Optional[dict] = None, hidden_scale_up: bool = False) -> None:
        super().__init__()
        from .primitives import LinearNoBias

        msa_configs = msa_configs or {}
        self.n_blocks, self.c_m, self.c_s_inputs, self.blocks_per_ckpt = n_blocks, c_m, c_s_inputs, blocks_per_ckpt
        self.msa_chunk_size, self.msa_max_size = msa_chunk_size, msa_max_size
        self.input_feature = {"msa": 32, "has_deletion": 1, "deletion_value": 1}
        self.msa_configs = {"enable": msa_configs.get("enable", False), "strategy": msa_configs.get("strategy", "random"),
                            "train_cutoff": 512, "test_cutoff": 16384, "train_lowerb": 1, "test_lowerb": 1}
        if "sample_cutoff" in msa_configs:
            self.msa_configs["train_cutoff"] = msa_configs["sample_cutoff"].get("train", 512)
            self.msa_configs["test_cutoff"] = msa_configs["sample_cutoff"].get("test", 16384)
            self.msa_max_size = self.msa_configs["train_cutoff"]
        if "min_size" in msa_configs:
            self.msa_configs["train_lowerb"] = msa_configs["min_size"].get("train", 1)
            self.msa_configs["test_lowerb"] = msa_configs["min_size"].get("test", 1)
        self.linear_no_bias_m = LinearNoBias(in_features=32 + 1 + 1, out_features=c_m)
        self.linear_no_bias_s = LinearNoBias(in_features=c_s_inputs, out_features=c_m)
        self.blocks = nn.ModuleList(
            MSABlock(c_m=c_m, c_z=c_z, is_last_block=(i + 1 == n_blocks), msa_dropout=msa_dropout,
                     pair_dropout=pair_dropout, msa_chunk_size=self.msa_chunk_size, msa_max_size=self.msa_max_size,
                     hidden_scale_up=hidden_scale_up) for i in range(n_blocks))

    @torch.no_grad()
    def forward(self, input_feature_dict: dict, z: torch.Tensor, s_inputs: torch.Tensor, pair_mask: torch.Tensor,
                triangle_multiplicative: str = "torch", triangle_attention: str = "torch",
                inplace_safe: bool = False, chunk_size: Optional[int] = None) -> torch.Tensor:
        """z [N, N, c_z] (or [1, N, N, c_z]) -> updated z.  ``input_feature_dict``: "msa" [N_msa, N] int64 classes,
        "has_deletion" and "deletion_value" [N_msa, N]."""
        if self.n_blocks < 1 or "msa" not in input_feature_dict or input_feature_dict["msa"].dim() < 2:
            return z
        if self.training:
            raise RuntimeError("MSAModule: eval mode only")
        msa = input_feature_dict["msa"]
        idx = sample_msa_indices(msa.shape[-2], msa.device, self.msa_configs["test_lowerb"], self.msa_configs["strategy"])
        if self.msa_configs["test_cutoff"] > 0:
            idx = idx[:self.msa_configs["test_cutoff"]]
        feat = {k: torch.index_select(input_feature_dict[k], -2, idx) for k in self.input_feature}
        onehot = torch.zeros(*feat["msa"].shape, 32, dtype=torch.float32, device=msa.device)
        onehot.scatter_(feat["msa"].dim(), feat["msa"].unsqueeze(-1), 1)
        sample = torch.cat([onehot, feat["has_deletion"].reshape(*onehot.shape[:-1], 1).float(),
                            feat["deletion_value"].reshape(*onehot.shape[:-1], 1).float()], dim=-1)
        m = self.linear_no_bias_m(sample) + self.linear_no_bias_s(s_inputs.float())
        if m.dim() == 4:
            m = m[0]
        m = m.contiguous()
        first = True
        for block in self.blocks:
            m, z = block(m, z, pair_mask, inplace_safe=inplace_safe or not first, chunk_size=chunk_size)
            first = False               # every later block works on the copy the first one made
        return z
