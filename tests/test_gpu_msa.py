"""OuterProductMean (the MSA module's update of the pair representation) on the GPU against the reference's own
vectors and against the CPU oracle.  Tolerance: relative Frobenius error <= 1e-2 against fp32 ground truth (fp16
operands, fp32 accumulation: measured values are around 1e-3)."""
import pytest
import torch

import protenix_b200 as px
from golden_cases import CASES, make_inputs
from helpers import build_module, golden, params_of, relf
from oracle import pairformer_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 1e-2


@pytest.mark.parametrize("name", ["opm_n24", "opm_n40_nomask"])
def test_outer_product_mean_against_reference_vectors(name):
    case = CASES[name]
    inp = make_inputs(case)
    mod = build_module("opm", case).to(DEV)
    mask = None if inp["msa_mask"] is None else inp["msa_mask"].to(DEV)
    y = mod(inp["m"].to(DEV), mask=mask)
    assert y.dtype == torch.float32 and torch.isfinite(y).all()
    assert relf(y, golden()[name + ".y"]) < TOL
    y1 = mod(inp["m"].to(DEV)[None], mask=None if mask is None else mask[None])      # a batch of one, as the reference allows
    assert y1.shape == (1,) + tuple(y.shape) and torch.equal(y1[0], y)
    px.ops.device_error_flags()


@pytest.mark.parametrize("n,s_rows,p_drop,zdtype", [(1, 1, 0.0, torch.float32), (37, 5, 0.3, torch.float32),
                                                    (100, 37, 0.2, torch.bfloat16), (128, 64, 0.0, torch.float32),
                                                    (130, 200, 0.5, torch.float32), (256, 128, 0.1, torch.bfloat16),
                                                    (384, 256, 0.2, torch.float32)])
def test_outer_product_mean_added_to_z_vs_oracle(n, s_rows, p_drop, zdtype):
    """z += OuterProductMean(m), as MSABlock applies it: ragged N and N_seq, random MSA masks (columns that no MSA
    row covers divide by eps alone), both storage types of z."""
    g = torch.Generator().manual_seed(1000 * n + s_rows)
    m = torch.randn(s_rows, n, 64, generator=g)
    mask = (torch.rand(s_rows, n, generator=g) > p_drop).float() if p_drop > 0 else None
    z = torch.randn(n, n, 128, generator=g).to(zdtype)
    mod = build_module("opm", dict(wseed=n + 7)).to(DEV)
    ref_upd = O.outer_product_mean(m, mask, params_of(mod))
    zc = z.to(DEV).clone()
    mod.apply_(zc, m.to(DEV), None if mask is None else mask.to(DEV))
    want = z.float() + ref_upd
    assert torch.isfinite(zc.float()).all()
    tol = TOL if zdtype == torch.float32 else 1.2e-2          # bf16 storage rounds the sum once more
    assert relf(zc, want) < tol, (n, s_rows, relf(zc, want))
    upd = mod(m.to(DEV), mask=None if mask is None else mask.to(DEV))
    assert relf(upd, ref_upd) < TOL, (n, s_rows, relf(upd, ref_upd))
    px.ops.device_error_flags()


def test_outer_product_mean_is_bilinear_in_the_two_projections():
    """A size-independent property at a size the CPU oracle would not finish quickly: doubling linear_1 doubles the
    update minus the bias term; swapping linear_1 and linear_2 transposes (i, j) and (c, e)."""
    n, s_rows = 512, 384
    g = torch.Generator().manual_seed(3)
    m = torch.randn(s_rows, n, 64, generator=g).to(DEV)
    mod = build_module("opm", dict(wseed=5)).to(DEV)
    with torch.no_grad():
        mod.linear_out.bias.zero_()
    y = mod(m)
    with torch.no_grad():
        mod.linear_1.weight.mul_(2.0)
    y2 = mod(m)
    assert relf(y2, 2.0 * y) < 2e-3
    with torch.no_grad():
        mod.linear_1.weight.mul_(0.5)
        w1, w2 = mod.linear_1.weight.clone(), mod.linear_2.weight.clone()
        mod.linear_1.weight.copy_(w2)
        mod.linear_2.weight.copy_(w1)
        wo = mod.linear_out.weight.view(128, 32, 32).transpose(1, 2).reshape(128, 1024).clone()
        mod.linear_out.weight.copy_(wo)
    y3 = mod(m)
    assert relf(y3, y.transpose(0, 1)) < 2e-3
    px.ops.device_error_flags()


def test_outer_product_mean_rejects_what_it_was_not_built_for():
    mod = build_module("opm", dict(wseed=1)).to(DEV)
    with pytest.raises(RuntimeError):
        mod(torch.randn(4, 8, 64))                                   # CPU tensor
    other = px.OuterProductMean(c_m=64, c_z=128, c_hidden=16).to(DEV)
    with pytest.raises(RuntimeError):
        other(torch.randn(4, 8, 64, device=DEV))                     # c_hidden other than 32


@pytest.mark.parametrize("name", ["msa_block_n20", "msa_block_last_n16"])
@pytest.mark.parametrize("zdtype", [torch.float32, torch.bfloat16])
def test_msa_block_against_reference_vectors(name, zdtype):
    """One block of the MSA module against what the reference itself returned: z through the outer product mean and
    the pair-only Pairformer block, m through pair-weighted averaging and its transition."""
    case = CASES[name]
    inp = make_inputs(case)
    mod = build_module("msa_block", case).to(DEV)
    m_in = inp["m"].to(DEV)
    m, z = mod(m_in.clone(), inp["z"].to(zdtype).to(DEV), inp["mask"].to(DEV))
    g = golden()
    assert relf(z, g[name + ".z"]) < (TOL if zdtype == torch.float32 else 1.5e-2)
    if case["last"]:
        assert m is None
    else:
        assert relf(m, g[name + ".m"]) < TOL
    px.ops.device_error_flags()


def test_msa_block_vs_oracle_ragged_sizes_and_chunked_msa_rows():
    n, s_rows = 100, 33
    g = torch.Generator().manual_seed(9)
    m = torch.randn(s_rows, n, 64, generator=g)
    z = torch.randn(n, n, 128, generator=g)
    t = torch.ones(n)
    t[n - 7:] = 0
    mask = t[:, None] * t[None, :]
    from protenix_b200.msa import MSABlock
    from protenix_b200.init_utils import randomize_parameters_

    mod = randomize_parameters_(MSABlock(msa_chunk_size=10), 21).eval().to(DEV)      # four chunks of MSA rows
    m_ref, z_ref = O.msa_block(m, z, mask, params_of(mod))
    m_out, z_out = mod(m.to(DEV).clone(), z.to(DEV), mask.to(DEV))
    assert relf(z_out, z_ref) < TOL and relf(m_out, m_ref) < TOL
    # the input z is left alone unless the caller allows in-place work; m is updated in place like the reference's
    zin = z.to(DEV)
    mod(m.to(DEV).clone(), zin, mask.to(DEV))
    assert torch.equal(zin.cpu(), z)
    px.ops.device_error_flags()


def test_outer_product_mean_in_blocks_of_rows_is_the_same_to_the_bit(monkeypatch):
    """The outer products are formed for blocks of token rows to bound their buffer; the block size changes no bit."""
    n, s_rows = 150, 40
    g = torch.Generator().manual_seed(17)
    m = torch.randn(s_rows, n, 64, generator=g).to(DEV)
    mask = (torch.rand(s_rows, n, generator=g) > 0.2).float().to(DEV)
    z = torch.randn(n, n, 128, generator=g).to(DEV)
    mod = build_module("opm", dict(wseed=2)).to(DEV)
    whole = mod.apply_(z.clone(), m, mask)
    monkeypatch.setattr(px.ops, "OPM_X_BYTES", 2048 * n * 37)       # blocks of 37 rows: 37, 37, 37, 37, 2
    parts = mod.apply_(z.clone(), m, mask)
    assert torch.equal(whole, parts)
    ref = z.cpu() + O.outer_product_mean(m.cpu(), mask.cpu(), params_of(mod))
    assert relf(parts, ref) < TOL
    px.ops.device_error_flags()


@pytest.mark.parametrize("zdtype", [torch.float32, torch.bfloat16])
def test_msa_module_against_reference_vector(zdtype):
    """The whole MSA module (feature embedding, three blocks) against the reference's own output; and with the
    reference's default random sampling of MSA rows the module still runs and returns a finite z of the same shape."""
    name = "msa_module_n18"
    case = CASES[name]
    inp = make_inputs(case)
    mod = build_module("msa_module", case).to(DEV)
    feat = {k: inp[k].to(DEV) for k in ("msa", "has_deletion", "deletion_value")}
    z_in = inp["z"].to(zdtype).to(DEV)
    z = mod(feat, z_in, inp["s_inputs"].to(DEV), inp["mask"].to(DEV))
    assert relf(z, golden()[name + ".z"]) < (1.5e-2 if zdtype == torch.float32 else 2.5e-2)   # three blocks deep
    assert torch.equal(z_in.cpu(), inp["z"].to(zdtype))                  # the caller's z is not written
    from protenix_b200.msa import MSAModule
    from protenix_b200.init_utils import randomize_parameters_

    torch.manual_seed(0)
    rnd = randomize_parameters_(MSAModule(n_blocks=2, msa_configs={"enable": True, "strategy": "random"}), 4).eval().to(DEV)
    z2 = rnd(feat, z_in, inp["s_inputs"].to(DEV), inp["mask"].to(DEV))
    assert z2.shape == z_in.shape and torch.isfinite(z2.float()).all()
    assert rnd({}, z_in, inp["s_inputs"].to(DEV), inp["mask"].to(DEV)) is z_in      # no MSA features: z comes back as it is
    px.ops.device_error_flags()


def test_recycling_trunk_with_msa_module_against_reference_vector():
    """Two recycling cycles of (pair update, MSA module, single update, Pairformer stack) against the reference's own
    loop (protenix/model/protenix.py:230-296 without the template embedder)."""
    name = "trunk_msa_n16"
    case = CASES[name]
    inp = make_inputs(case)
    mod = build_module("trunk_msa", case).to(DEV)
    feat = {k: inp[k].to(DEV) for k in ("msa", "has_deletion", "deletion_value")}
    s, z = mod(inp["s"].to(DEV), inp["z"].to(DEV), inp["mask"].to(DEV), input_feature_dict=feat,
               s_inputs=inp["s_inputs"].to(DEV))
    g = golden()
    assert relf(z, g[name + ".z"]) < 2e-2 and relf(s, g[name + ".s"]) < 2e-2        # eight blocks deep
    px.ops.device_error_flags()
