"""The recycling update z = z_init + W LN(z) and the recycling loop around the stack: CUDA path against the CPU
oracle and against the vector produced by the reference's own layers.

Tolerances (relative Frobenius error against fp32 ground truth): one update with bf16 operands <= 1e-2 of the
update term and <= 4e-3 of the result; the three-cycle, two-block trunk <= 3e-2 (the stack bound).
"""
import pytest
import torch

import protenix_b200 as px
from protenix_b200 import ops
from golden_cases import CASES, make_inputs
from helpers import build_module, golden, params_of, relf
from oracle import pairformer_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _weights(seed):
    g = torch.Generator().manual_seed(seed)
    return {"ln.weight": 1 + 0.1 * torch.randn(128, generator=g), "ln.bias": 0.1 * torch.randn(128, generator=g),
            "lin.weight": torch.randn(128, 128, generator=g) / 128 ** 0.5}


@pytest.mark.parametrize("zdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [1, 127, 128, 129, 1000, 148 * 128 * 2 + 77])
def test_recycle_update_ragged_rows(rows, zdtype):
    p = _weights(rows)
    g = torch.Generator().manual_seed(rows + 1)
    z = (torch.randn(rows, 128, generator=g) * 2 + 0.5).to(zdtype)
    zi = torch.randn(rows, 128, generator=g).to(zdtype)
    out = ops.recycle_update(z.to(DEV), zi.to(DEV), p["ln.weight"].to(DEV), p["ln.bias"].to(DEV),
                             p["lin.weight"].to(DEV).bfloat16())
    assert out.dtype == zdtype and out.shape == z.shape
    ref = O.recycle_update(z.double(), zi.double(), {k: v.double() for k, v in p.items()}, "ln", "lin")
    upd = ref - zi.double()
    assert relf(out.double().cpu() - zi.double(), upd) < 1e-2
    assert relf(out, ref) < 4e-3


def test_recycle_update_of_zeros_is_the_projected_offset_and_bias_may_be_absent():
    p = _weights(3)
    zi = torch.randn(300, 128)
    z = torch.zeros(300, 128)
    out = ops.recycle_update(z.to(DEV), zi.to(DEV), p["ln.weight"].to(DEV), p["ln.bias"].to(DEV),
                             p["lin.weight"].to(DEV).bfloat16())
    ref = zi + (p["lin.weight"] @ p["ln.bias"])[None]
    assert relf(out, ref) < 2e-3
    out = ops.recycle_update(z.to(DEV), zi.to(DEV), p["ln.weight"].to(DEV), None, p["lin.weight"].to(DEV).bfloat16())
    assert torch.equal(out.cpu(), zi)


@pytest.mark.parametrize("alias", ["z", "z_init"])
def test_recycle_update_in_place_gives_the_same_bits(alias):
    p = _weights(5)
    g = torch.Generator().manual_seed(6)
    z = torch.randn(40, 50, 128, generator=g).bfloat16().to(DEV)
    zi = torch.randn(40, 50, 128, generator=g).bfloat16().to(DEV)
    args = (p["ln.weight"].to(DEV), p["ln.bias"].to(DEV), p["lin.weight"].to(DEV).bfloat16())
    ref = ops.recycle_update(z, zi, *args)
    z2, zi2 = z.clone(), zi.clone()
    out = ops.recycle_update(z2, zi2, *args, out=z2 if alias == "z" else zi2)
    assert torch.equal(out, ref)


def test_recycle_update_rejects_bad_arguments():
    p = _weights(7)
    args = (p["ln.weight"].to(DEV), p["ln.bias"].to(DEV), p["lin.weight"].to(DEV).bfloat16())
    z = torch.zeros(4, 128, device=DEV)
    with pytest.raises(RuntimeError):
        ops.recycle_update(z, torch.zeros(5, 128, device=DEV), *args)
    with pytest.raises(RuntimeError):
        ops.recycle_update(z, z.bfloat16(), *args)
    with pytest.raises(RuntimeError):
        ops.recycle_update(z.cpu(), z.cpu(), *args)
    assert ops.recycle_update(z[:0], z[:0], *args).shape == (0, 128)


@pytest.mark.parametrize("zdtype", [torch.float32, torch.bfloat16])
def test_recycling_trunk_against_reference_vector(zdtype):
    case = CASES["recycle_n16"]
    m = build_module("recycle", case).to(DEV)
    inp = make_inputs(case)
    s, z = m(inp["s"].to(DEV), inp["z"].to(DEV).to(zdtype), inp["mask"].to(DEV))
    g = golden()
    assert z.dtype == zdtype
    assert relf(z, g["recycle_n16.z"]) < 3e-2 and relf(s, g["recycle_n16.s"]) < 3e-2


def test_recycling_trunk_with_reference_init_returns_the_inputs():
    """Both recycling projections and every residual branch of the stack start at zero (protenix/model/protenix.py:167-168)."""
    torch.manual_seed(0)
    m = px.RecyclingTrunk(n_blocks=1, N_cycle=2).eval().to(DEV)
    z = torch.randn(12, 12, 128, device=DEV)
    s = torch.randn(12, 384, device=DEV)
    s2, z2 = m(s, z)
    assert relf(z2, z) < 1e-6 and relf(s2, s) < 1e-6
    assert sorted(k for k in m.state_dict() if not k.startswith("pairformer_stack.")) == [
        "layernorm_s.bias", "layernorm_s.weight", "layernorm_z_cycle.bias", "layernorm_z_cycle.weight",
        "linear_no_bias_s.weight", "linear_no_bias_z_cycle.weight"]
