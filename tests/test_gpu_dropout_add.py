"""dropout_add_rowwise on the GPU, after the reference's own tests of the op (tests/test_fused_dropout_add.py:20-140:
no-drop exactness, the mask shared along axis -3, gradients) plus identity to the bit with the reference's torch
formula for the same seed."""
import pytest
import torch

import protenix_b200 as px

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _reference_formula(residual, x, p):
    """protenix/model/modules/fused_ops.py:219-223 (the reference's fallback path)."""
    shape = list(x.shape)
    shape[-3] = 1
    mask = torch.nn.functional.dropout(x.new_ones(shape), p=p, training=True)
    return residual + x * mask


def test_no_dropout_is_exactly_the_sum():
    torch.manual_seed(42)
    residual, x = torch.randn(2, 4, 8, 16, device=DEV), torch.randn(2, 4, 8, 16, device=DEV)
    assert torch.equal(px.dropout_add_rowwise(residual, x, 0.0, True), residual + x)
    assert torch.equal(px.dropout_add_rowwise(residual, x, 0.5, False), residual + x)


def test_mask_is_shared_along_the_row_axis():
    torch.manual_seed(42)
    r_dim, c, d = 4, 2, 8
    residual = torch.zeros(1, r_dim, c, d, device=DEV)
    x = torch.ones(1, r_dim, c, d, device=DEV)
    out = px.dropout_add_rowwise(residual, x, 0.5, True)
    assert set(out.unique().tolist()) <= {0.0, 2.0} and 0.0 < float(out.mean()) < 2.0
    for r in range(1, r_dim):
        assert torch.equal(out[0, 0], out[0, r])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(2, 3, 4, 8), (1, 37, 20, 128), (5, 7, 3), (3, 2, 5, 7, 9)])
def test_same_seed_gives_the_reference_formula_to_the_bit(shape, dtype):
    g = torch.Generator().manual_seed(sum(shape))
    residual, x = torch.randn(shape, generator=g).to(dtype).to(DEV), torch.randn(shape, generator=g).to(dtype).to(DEV)
    torch.manual_seed(7)
    want = _reference_formula(residual, x, 0.25)
    torch.manual_seed(7)
    got = px.dropout_add_rowwise(residual, x, 0.25, True)
    assert got.dtype == dtype and torch.equal(got, want)


def test_gradients():
    residual = torch.randn(2, 3, 4, 8, device=DEV, requires_grad=True)
    x = torch.randn(2, 3, 4, 8, device=DEV, requires_grad=True)
    torch.manual_seed(3)
    px.dropout_add_rowwise(residual, x, 0.3, True).sum().backward()
    assert torch.equal(residual.grad, torch.ones_like(residual))
    torch.manual_seed(3)
    mask = torch.nn.functional.dropout(torch.ones(2, 1, 4, 8, device=DEV), p=0.3, training=True)
    assert torch.equal(x.grad, mask.expand_as(x)) and float(x.grad.abs().sum()) > 0
    r0 = torch.randn(2, 3, 4, 8, device=DEV, requires_grad=True)
    x0 = torch.randn(2, 3, 4, 8, device=DEV, requires_grad=True)
    px.dropout_add_rowwise(r0, x0, 0.0, True).sum().backward()
    assert torch.equal(r0.grad, torch.ones_like(r0)) and torch.equal(x0.grad, torch.ones_like(x0))
