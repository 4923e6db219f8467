"""B200-native (sm_100a) Pairformer pair-representation forward path behind the module API of
bytedance/Protenix.  One code path: hand-written CUDA kernels reached through a C ABI
(``include/px_b200.h``); nothing falls back to the CPU or to another back-end."""
from .layer_norm import FusedLayerNorm, LayerNorm
from .msa import OuterProductMean
from .pairformer import PairformerBlock, PairformerStack
from .primitives import Linear, LinearNoBias, Transition
from .recycling import RecyclingTrunk
from .transformer import AttentionPairBias
from .triangular import (OpenfoldLinear, TriangleAttention, TriangleAttentionEndingNode,
                         TriangleAttentionStartingNode, TriangleMultiplicationIncoming,
                         TriangleMultiplicationOutgoing, TriangleMultiplicativeUpdate)
from .fused_ops import dropout_add_rowwise

__all__ = [
    "FusedLayerNorm", "LayerNorm", "PairformerBlock", "PairformerStack", "Linear", "LinearNoBias", "Transition",
    "AttentionPairBias", "OpenfoldLinear", "TriangleAttention", "TriangleAttentionEndingNode",
    "TriangleAttentionStartingNode", "TriangleMultiplicationIncoming", "TriangleMultiplicationOutgoing",
    "TriangleMultiplicativeUpdate", "dropout_add_rowwise", "RecyclingTrunk", "OuterProductMean",
]
__version__ = "0.1.0"
