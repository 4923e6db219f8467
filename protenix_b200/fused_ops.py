"""``dropout_add_rowwise`` for the inference path.

In eval mode (or p = 0) the reference's op is ``residual + x``
(protenix/model/modules/fused_ops.py:190-224, branch :213-214).  The fused kernels of this
package fold that add into their epilogues; this function exists for API compatibility.
"""
import torch


def dropout_add_rowwise(residual: torch.Tensor, x: torch.Tensor, p: float, training: bool) -> torch.Tensor:
    if training and p > 0.0:
        raise RuntimeError("row-wise dropout (training) is outside the scope of this package")
    return residual + x
