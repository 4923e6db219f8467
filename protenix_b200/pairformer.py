"""``PairformerBlock`` / ``PairformerStack`` drop-ins over the sm_100a kernels.

Constructor arguments, forward signature, return values and ``state_dict`` keys are those of
protenix/model/modules/pairformer.py:42-340.  A block is eight kernel families on the pair
tensor (triangle multiplication out/in: projection, contraction, output stage; triangle
attention start/end: projection, flash attention, output stage; transition) plus the small
single-representation branch.  z is updated in place on a private copy (or on the caller's
tensor with ``inplace_safe=True``); the two transposed copies of z the reference makes around
the ending-node attention do not exist here -- the ending-node kernels index z transposed.

Inference only: dropout is the identity (eval mode), gradients are not produced.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch
import torch.nn as nn

from . import ops
from .primitives import Transition
from .transformer import AttentionPairBias
from .triangular import (TriangleAttention, TriangleMultiplicationIncoming, TriangleMultiplicationOutgoing,
                         _pair_input)


class PairformerBlock(nn.Module):
    def __init__(self, n_heads: int = 16, c_z: int = 128, c_s: int = 384, c_hidden_mul: int = 128,
                 c_hidden_pair_att: int = 32, no_heads_pair: int = 4, num_intermediate_factor: int = 4,
                 dropout: float = 0.25, hidden_scale_up: bool = False) -> None:
        super().__init__()
        self.n_heads = n_heads
        if hidden_scale_up:
            no_heads_pair = c_z // c_hidden_pair_att
            c_hidden_mul = c_z
        self.tri_mul_out = TriangleMultiplicationOutgoing(c_z=c_z, c_hidden=c_hidden_mul)
        self.tri_mul_in = TriangleMultiplicationIncoming(c_z=c_z, c_hidden=c_hidden_mul)
        self.tri_att_start = TriangleAttention(c_in=c_z, c_hidden=c_hidden_pair_att, no_heads=no_heads_pair)
        self.tri_att_end = TriangleAttention(c_in=c_z, c_hidden=c_hidden_pair_att, no_heads=no_heads_pair)
        self.p_drop = dropout
        self.pair_transition = Transition(c_in=c_z, n=num_intermediate_factor)
        self.c_s = c_s
        if self.c_s > 0:
            self.attention_pair_bias = AttentionPairBias(has_s=False, create_offset_ln_z=True, n_heads=n_heads,
                                                         c_a=c_s, c_z=c_z)
            self.single_transition = Transition(c_in=c_s, n=4)

    def pair_path_(self, zc: torch.Tensor, mask: Optional[torch.Tensor], zn: Optional[torch.Tensor] = None) -> None:
        """The five pair updates of the block, in place.  ``zn``: the standardised fp16 copy of an fp32 zc as passed
        in, when the caller has it (the first triangle update then skips its standardising pass)."""
        self.tri_mul_out.apply_(zc, mask, zn=zn)
        self.tri_mul_in.apply_(zc, mask)
        self.tri_att_start.apply_(zc, mask, ending=False)
        self.tri_att_end.apply_(zc, mask, ending=True)
        self.pair_transition.forward_residual_(zc)

    def single_path(self, s: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
        """The single-representation update, given the pair bias of the block's final z.  It needs nothing else from
        z, and the pair path never reads s: a stack can run it beside the pair path of the next block."""
        s = s + self.attention_pair_bias(a=s, s=None, z=None, bias=bias)
        return s + self.single_transition(s)

    @torch.no_grad()
    def forward(self, s: Optional[torch.Tensor], z: torch.Tensor, pair_mask: Optional[torch.Tensor],
                triangle_multiplicative: str = "torch", triangle_attention: str = "torch",
                inplace_safe: bool = False, chunk_size: Optional[int] = None
                ) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
        if self.training and self.p_drop > 0:
            raise RuntimeError("PairformerBlock: training-mode dropout is not implemented; call .eval()")
        zc, mask, batch = _pair_input(z, pair_mask)
        if not inplace_safe and zc.data_ptr() == z.data_ptr():
            zc = zc.clone()
        self.pair_path_(zc, mask)
        if self.c_s > 0:
            s = self.single_path(s, self.attention_pair_bias.pair_bias(zc))
        return s, (zc[None] if batch else zc)


class PairformerStack(nn.Module):
    def __init__(self, n_blocks: int = 48, n_heads: int = 16, c_z: int = 128, c_s: int = 384,
                 num_intermediate_factor: int = 4, dropout: float = 0.25, blocks_per_ckpt: Optional[int] = None,
                 hidden_scale_up: bool = False) -> None:
        super().__init__()
        self.n_blocks = n_blocks
        self.n_heads = n_heads
        self.blocks_per_ckpt = blocks_per_ckpt
        self.blocks = nn.ModuleList(
            PairformerBlock(n_heads=n_heads, c_z=c_z, c_s=c_s, num_intermediate_factor=num_intermediate_factor,
                            dropout=dropout, hidden_scale_up=hidden_scale_up) for _ in range(n_blocks))

    @torch.no_grad()
    def forward(self, s: torch.Tensor, z: torch.Tensor, pair_mask: Optional[torch.Tensor],
                triangle_multiplicative: str = "torch", triangle_attention: str = "torch",
                inplace_safe: bool = False, chunk_size: Optional[int] = None
                ) -> Tuple[torch.Tensor, torch.Tensor]:
        zc, mask, batch = _pair_input(z, pair_mask)
        if not inplace_safe and zc.data_ptr() == z.data_ptr():
            zc = zc.clone()
        # The pair path does not depend on s, and the single path takes only the pair bias from z: the single path of
        # block b runs on a side stream beside the pair path of block b + 1.
        main = torch.cuda.current_stream(zc.device)
        side = _side_stream(zc.device)
        side.wait_stream(main)
        # fp32 z: the standardised copy made for a block's pair bias (its final z) also serves the first triangle
        # update of the next block, which normalises the same rows with the same eps
        zn_buf = torch.empty_like(zc, dtype=torch.float16) if zc.dtype == torch.float32 and s is not None else None
        zn, zn_eps = None, None
        for block in self.blocks:
            if block.training and block.p_drop > 0:
                raise RuntimeError("PairformerBlock: training-mode dropout is not implemented; call .eval()")
            block.pair_path_(zc, mask, zn if zn is not None and zn_eps == block.tri_mul_out.layer_norm_in.eps else None)
            zn = None
            if block.c_s > 0 and s is not None:
                if zn_buf is not None:
                    zn = ops.standardise_rows(zc, block.attention_pair_bias.layernorm_z.eps, out=zn_buf)
                    zn_eps = block.attention_pair_bias.layernorm_z.eps
                bias = block.attention_pair_bias.pair_bias(zc, zn)   # reads the block's final z, on the main stream
                bias.record_stream(side)
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    s = block.single_path(s, bias)
        main.wait_stream(side)
        if s is not None:
            s.record_stream(main)
        if os.environ.get("PX_CHECK_DEVICE_ERRORS", "0") == "1":    # synchronises: off unless asked for
            ops.device_error_flags(zc.device)
        return s, (zc[None] if batch else zc)


_SIDE_STREAMS = {}


def _side_stream(device: torch.device) -> "torch.cuda.Stream":
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = torch.cuda.Stream(device=device)
    return _SIDE_STREAMS[key]
