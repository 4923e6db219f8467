"""``dropout_add_rowwise``: residual + dropout(x) with the dropout mask shared along axis -3.

Mirror of protenix/model/modules/fused_ops.py:190-224.  In eval mode (or p = 0) the op is ``residual + x`` (:213-214);
the fused kernels of this package fold that add into their epilogues, and this function exists for API compatibility.
In training mode the mask of shape [..., 1, C, D] is drawn exactly as the reference's own fallback draws it
(``dropout`` of a tensor of ones, :219-223), so the same seed gives the same mask, and the scaled product and the add
run in one kernel (``px_scale_add_rowwise``), forward and backward.  CUDA tensors only.
"""
import torch

from . import ops


class _DropoutAddRowwise(torch.autograd.Function):
    @staticmethod
    def forward(ctx, residual, x, mask):
        ctx.save_for_backward(mask)
        return ops.scale_add_rowwise(residual, x, mask)

    @staticmethod
    def backward(ctx, grad):
        (mask,) = ctx.saved_tensors
        gx = ops.scale_add_rowwise(None, grad.contiguous(), mask) if ctx.needs_input_grad[1] else None
        return (grad if ctx.needs_input_grad[0] else None), gx, None


def dropout_add_rowwise(residual: torch.Tensor, x: torch.Tensor, p_drop: float, training: bool) -> torch.Tensor:
    if not training or p_drop == 0.0:
        return residual + x
    if not x.is_cuda:
        raise RuntimeError("dropout_add_rowwise (training): CUDA tensors only, this package has no CPU path")
    shape = list(x.shape)
    shape[-3] = 1
    mask = torch.nn.functional.dropout(x.new_ones(shape), p=p_drop, training=True)
    return _DropoutAddRowwise.apply(residual, x, mask)
