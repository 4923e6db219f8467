"""The CPU oracle against vectors produced by the reference itself (tests/golden/make_golden.py)."""
import pytest
import torch

from golden_cases import CASES, make_inputs
from helpers import build_module, golden, params_of, relf
from oracle import pairformer_oracle as O

TOL = 2e-5  # fp32 reference vs fp32 restatement: different summation orders only


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_matches_reference_vectors(name):
    case = CASES[name]
    kind = case["kind"]
    g = golden()
    inp = make_inputs(case)
    p = params_of(build_module(kind, case))
    if kind == "block":
        s, z = O.pairformer_block(inp["s"], inp["z"], inp["mask"], p)
        assert relf(z, g[name + ".z"]) < TOL
        if s is not None:
            assert relf(s, g[name + ".s"]) < TOL
    elif kind == "stack":
        s, z = O.pairformer_stack(inp["s"], inp["z"], inp["mask"], p, n_blocks=case["n_blocks"])
        assert relf(z, g[name + ".z"]) < TOL and relf(s, g[name + ".s"]) < TOL
    elif kind in ("tri_mul_out", "tri_mul_in"):
        y = O.triangle_multiplication(inp["z"], inp["mask"], p, outgoing=(kind == "tri_mul_out"))
        assert relf(y, g[name + ".y"]) < TOL
    elif kind in ("tri_att_start", "tri_att_end"):
        y = O.triangle_attention(inp["z"], inp["mask"], p, starting=(kind == "tri_att_start"))
        assert relf(y, g[name + ".y"]) < TOL
        y2 = O.triangle_attention(inp["z"], inp["mask"], p, starting=(kind == "tri_att_start"), row_chunk=7)
        assert relf(y2, y) < 1e-6
    elif kind == "transition":
        assert relf(O.transition(inp["x"], p), g[name + ".y"]) < TOL
    elif kind == "layer_norm":
        assert relf(O.layer_norm(inp["x"], p.get("weight"), p.get("bias")), g[name + ".y"]) < TOL
    elif kind == "recycle":
        s, z = O.recycling_trunk(inp["s"], inp["z"], inp["mask"], p, n_blocks=case["n_blocks"], n_cycle=case["n_cycle"])
        assert relf(z, g[name + ".z"]) < TOL and relf(s, g[name + ".s"]) < TOL
    elif kind == "opm":
        assert relf(O.outer_product_mean(inp["m"], inp["msa_mask"], p), g[name + ".y"]) < TOL
    elif kind == "msa_block":
        m, z = O.msa_block(inp["m"], inp["z"], inp["mask"], p, is_last_block=case["last"])
        assert relf(z, g[name + ".z"]) < TOL
        assert (m is None) == case["last"]
        if m is not None:
            assert relf(m, g[name + ".m"]) < TOL
    elif kind == "msa_module":
        z = O.msa_module(inp["msa"], inp["has_deletion"], inp["deletion_value"], inp["z"], inp["s_inputs"], inp["mask"], p,
                         n_blocks=case["n_blocks"])
        assert relf(z, g[name + ".z"]) < TOL
    elif kind == "trunk_msa":
        msa = {k: inp[k] for k in ("msa", "has_deletion", "deletion_value", "s_inputs")}
        s, z = O.recycling_trunk(inp["s"], inp["z"], inp["mask"], p, n_blocks=case["n_blocks"], n_cycle=case["n_cycle"],
                                 msa=msa, msa_n_blocks=case["msa_n_blocks"])
        assert relf(z, g[name + ".z"]) < TOL and relf(s, g[name + ".s"]) < TOL
    else:
        raise AssertionError(kind)


def test_oracle_fp64_agrees_with_fp32():
    case = CASES["block_pair_n20"]
    inp = make_inputs(case)
    m = build_module("block", case)
    _, z32 = O.pairformer_block(None, inp["z"], None, params_of(m))
    _, z64 = O.pairformer_block(None, inp["z"].double(), None, params_of(m, torch.float64))
    assert relf(z32, z64) < 1e-5


def test_reference_init_block_is_identity():
    """With the reference's own initialisers every residual branch ends in a zero projection."""
    import protenix_b200 as px

    torch.manual_seed(0)
    blk = px.PairformerBlock().eval()
    z = torch.randn(12, 12, 128)
    s = torch.randn(12, 384)
    s2, z2 = O.pairformer_block(s, z, None, params_of(blk))
    assert torch.equal(z2, z) and torch.equal(s2, s)


def test_mask_independence_is_bit_exact_in_oracle():
    """Perturbing z at padded positions changes no bit of tri-mul / tri-att outputs in the valid region."""
    from golden_cases import padding_mask

    n, pad = 18, 4
    g = torch.Generator().manual_seed(5)
    z = torch.randn(n, n, 128, generator=g)
    mask = padding_mask(n, pad)
    z2 = z.clone()
    z2[n - pad:, :, :] += torch.randn(pad, n, 128, generator=g)
    z2[:, n - pad:, :] += torch.randn(n, pad, 128, generator=g)
    v = n - pad
    for kind in ("tri_mul_out", "tri_mul_in"):
        p = params_of(build_module(kind, dict(wseed=3)))
        a = O.triangle_multiplication(z, mask, p, outgoing=(kind == "tri_mul_out"))
        b = O.triangle_multiplication(z2, mask, p, outgoing=(kind == "tri_mul_out"))
        assert torch.equal(a[:v, :v], b[:v, :v])
    for kind in ("tri_att_start", "tri_att_end"):
        p = params_of(build_module(kind, dict(wseed=4)))
        a = O.triangle_attention(z, mask, p, starting=(kind == "tri_att_start"))
        b = O.triangle_attention(z2, mask, p, starting=(kind == "tri_att_start"))
        assert torch.equal(a[:v, :v], b[:v, :v])


def test_row_slab_timing_sample_equals_the_full_updates():
    """The CPU-baseline sample computes exactly a row slab of each of the five pair updates."""
    from golden_cases import random_mask

    n, r0, r1 = 40, 8, 20
    p = params_of(build_module("block", dict(c_s=0, wseed=3)))
    z = torch.randn(n, n, 128, generator=torch.Generator().manual_seed(1))
    mask = random_mask(n, 1)
    slab, shared = O.pair_path_row_slab(z, mask, p, r0, r1)
    slab2, _ = O.pair_path_row_slab(z, mask, p, r0, r1, shared)
    full = {
        "tri_mul_out": O.triangle_multiplication(z, mask, O._sub(p, "tri_mul_out"), True)[r0:r1],
        "tri_mul_in": O.triangle_multiplication(z, mask, O._sub(p, "tri_mul_in"), False)[r0:r1],
        "tri_att_start": O.triangle_attention(z, mask, O._sub(p, "tri_att_start"), True)[r0:r1],
        "tri_att_end": O.triangle_attention(z, mask, O._sub(p, "tri_att_end"), False).transpose(0, 1)[r0:r1],
        "pair_transition": O.transition(z, O._sub(p, "pair_transition"))[r0:r1],
    }
    for k, v in full.items():
        assert relf(slab[k], v) < 1e-5, k
        assert torch.equal(slab[k], slab2[k])
