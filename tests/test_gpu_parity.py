"""Parity of the CUDA path (through the module API -> ctypes -> C ABI) with the CPU oracle and
with the vectors produced by the reference itself.

Tolerances (relative Frobenius error against fp32 ground truth):
  * bf16-operand kernels, per op and per block: <= 1e-2 (the reference's own bf16 noise floor
    for one block is 0.6-0.95e-2);  after a multi-block stack: <= 3e-2
  * LayerNorm op in fp32: <= 1e-5; in bf16/fp16: bounded by output rounding
  * mask / padding handling: bit-exact
"""
import math

import pytest
import torch

import protenix_b200 as px
from golden_cases import CASES, make_inputs, padding_mask, random_mask
from helpers import build_module, golden, params_of, relf
from oracle import pairformer_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL_OP = 1e-2
TOL_BLOCK = 1e-2
TOL_STACK = 3e-2


def cuda(t):
    return None if t is None else t.to(DEV)


# ------------------------------------------------------------------------------- LayerNorm
@pytest.mark.parametrize("name", [k for k in sorted(CASES) if CASES[k]["kind"] == "layer_norm"])
def test_layer_norm_golden_fp32(name):
    case = CASES[name]
    m = build_module("layer_norm", case).to(DEV)
    y = m(cuda(make_inputs(case)["x"]))
    assert relf(y, golden()[name + ".y"]) < 1e-5


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("cols", [128, 384, 64, 16, 833, 768, 256, 2050, 9000])
def test_layer_norm_widths_dtypes_and_stats(dtype, cols):
    from protenix_b200 import ops

    g = torch.Generator().manual_seed(cols)
    x = (torch.randn(37, cols, generator=g) * 2 + 0.5).to(dtype)
    w = (1 + 0.1 * torch.randn(cols, generator=g)).to(dtype)
    b = (0.1 * torch.randn(cols, generator=g)).to(dtype)
    for ww, bb in ((w, b), (w, None), (None, b), (None, None)):
        y, mean, invvar = ops.layer_norm(cuda(x), cuda(ww), cuda(bb), 1e-5, return_stats=True)
        ref = O.layer_norm(x.double(), None if ww is None else ww.double(), None if bb is None else bb.double())
        tol = 1e-5 if dtype == torch.float32 else (6e-3 if dtype == torch.bfloat16 else 8e-4)
        assert y.dtype == dtype and relf(y, ref) < tol
        mu, iv = O.layer_norm_stats(x.double())
        assert relf(mean, mu) < 1e-5 and relf(invvar, iv) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,cols,scale,offset", [(200, 128, True, True), (64, 384, True, True), (33, 833, True, False),
                                                    (77, 64, False, False), (1000, 128, True, True), (5, 9000, True, True),
                                                    (1, 16, False, True)])
def test_layer_norm_backward_against_autograd_of_the_oracle(rows, cols, scale, offset, dtype):
    """dx, dweight, dbias of the LayerNorm op (the reference's extension has the matching backward_* functions,
    layer_norm_cuda.cpp:162-179) against torch autograd through the fp64 oracle on the same (rounded) inputs."""
    g = torch.Generator().manual_seed(rows * 7 + cols)
    x = (torch.randn(rows, cols, generator=g) * 2 + 3).to(dtype)
    dy = torch.randn(rows, cols, generator=g).to(dtype)
    mod = px.LayerNorm(cols, create_scale=scale, create_offset=offset).to(DEV)
    with torch.no_grad():
        if scale:
            mod.weight.copy_(1 + 0.2 * torch.randn(cols, generator=g))
        if offset:
            mod.bias.copy_(0.2 * torch.randn(cols, generator=g))
    xg = x.to(DEV).requires_grad_(True)
    y = mod(xg)
    y.backward(dy.to(DEV))
    x64 = x.double().requires_grad_(True)
    w64 = mod.weight.detach().cpu().to(dtype).double().requires_grad_(True) if scale else None
    b64 = mod.bias.detach().cpu().to(dtype).double().requires_grad_(True) if offset else None
    O.layer_norm(x64, w64, b64).backward(dy.double())
    tol = 2e-5 if dtype == torch.float32 else (6e-3 if dtype == torch.bfloat16 else 1e-3)
    assert relf(xg.grad, x64.grad) < tol
    if scale:
        assert mod.weight.grad.dtype == mod.weight.dtype and relf(mod.weight.grad, w64.grad) < tol
    if offset:
        assert relf(mod.bias.grad, b64.grad) < tol
    with torch.no_grad():                                   # the inference path is the plain kernel, same values
        assert torch.equal(mod(x.to(DEV)), y.detach())


def test_layer_norm_leading_dims_and_empty():
    m = px.LayerNorm(128).to(DEV)
    x = torch.randn(3, 5, 7, 128, device=DEV)
    assert m(x).shape == x.shape
    assert m(torch.empty(0, 128, device=DEV)).shape == (0, 128)
    with pytest.raises(RuntimeError):
        m(torch.randn(4, 64, device=DEV))


# --------------------------------------------------------------------- per-op golden vectors
@pytest.mark.parametrize("zdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["tri_mul_out_n20", "tri_mul_in_n20", "tri_att_start_n20", "tri_att_end_n20",
                                  "transition_pair"])
def test_ops_against_reference_vectors(name, zdtype):
    case = CASES[name]
    m = build_module(case["kind"], case).to(DEV)
    inp = make_inputs(case)
    if case["kind"] == "transition":
        y = m(cuda(inp["x"]).to(zdtype))
    else:
        y = m(cuda(inp["z"]).to(zdtype), mask=cuda(inp["mask"]))
    assert y.dtype == zdtype
    assert relf(y, golden()[name + ".y"]) < TOL_OP


def test_transition_single_width_matches_reference_vector():
    case = CASES["transition_single"]
    m = build_module("transition", case).to(DEV)
    assert relf(m(cuda(make_inputs(case)["x"])), golden()["transition_single.y"]) < 1e-4


# ------------------------------------------------------------------ per-op, ragged sizes, masks
def _mask(kind, n, seed):
    if kind == "none":
        return None
    if kind == "pad":
        return padding_mask(n, max(1, n // 10))
    return random_mask(n, seed)


@pytest.mark.parametrize("n,mask_kind,zdtype", [
    (1, "none", torch.float32), (7, "rand", torch.bfloat16), (17, "pad", torch.float32),
    (64, "none", torch.bfloat16), (100, "rand", torch.bfloat16), (128, "pad", torch.bfloat16),
    (136, "rand", torch.float32), (200, "pad", torch.bfloat16), (257, "rand", torch.bfloat16)])
@pytest.mark.parametrize("kind", ["tri_mul_out", "tri_mul_in", "tri_att_start", "tri_att_end"])
def test_triangle_ops_vs_oracle(kind, n, mask_kind, zdtype):
    g = torch.Generator().manual_seed(100 + n)
    z = torch.randn(n, n, 128, generator=g)
    mask = _mask(mask_kind, n, n)
    m = build_module(kind, dict(wseed=n + 1)).to(DEV)
    zq = z.to(zdtype)
    y = m(cuda(zq), mask=cuda(mask))
    p = params_of(m)
    if kind.startswith("tri_mul"):
        ref = O.triangle_multiplication(zq.float(), mask, p, outgoing=(kind == "tri_mul_out"))
    else:
        ref = O.triangle_attention(zq.float(), mask, p, starting=(kind == "tri_att_start"), row_chunk=64)
    assert torch.isfinite(y.float()).all()
    assert relf(y, ref) < TOL_OP, (kind, n, mask_kind)


@pytest.mark.parametrize("zdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", ["tri_mul_out", "tri_mul_in", "tri_att_start", "tri_att_end"])
def test_layer_norm_of_rows_far_from_zero_mean(kind, zdtype):
    """The projection kernels fold LayerNorm into the weights and take the row statistics from E[x^2] - mean^2:
    rows whose mean is 30 deviations away from zero (far beyond what a pair representation holds) must still
    come out within the tolerance."""
    n = 72
    g = torch.Generator().manual_seed(5)
    z = torch.randn(n, n, 128, generator=g) + 30.0 * torch.randn(n, n, 1, generator=g) + 3.0 * torch.randn(1, 1, 128, generator=g)
    mask = _mask("rand", n, n)
    m = build_module(kind, dict(wseed=9)).to(DEV)
    zq = z.to(zdtype)
    y = m(cuda(zq), mask=cuda(mask))
    p = params_of(m)
    if kind.startswith("tri_mul"):
        ref = O.triangle_multiplication(zq.float(), mask, p, outgoing=(kind == "tri_mul_out"))
    else:
        ref = O.triangle_attention(zq.float(), mask, p, starting=(kind == "tri_att_start"), row_chunk=64)
    assert torch.isfinite(y.float()).all()
    assert relf(y, ref) < TOL_OP, (kind, zdtype)


@pytest.mark.parametrize("rows", [1, 100, 128, 129, 1000])
def test_transition_ragged_rows(rows):
    m = build_module("transition", dict(c=128, n=4, wseed=77)).to(DEV)
    x = torch.randn(rows, 128, generator=torch.Generator().manual_seed(rows))
    for dt in (torch.float32, torch.bfloat16):
        xq = x.to(dt)
        assert relf(m(cuda(xq)), O.transition(xq.float(), params_of(m))) < TOL_OP


# ----------------------------------------------------------------------- mask semantics (exact)
@pytest.mark.parametrize("kind", ["tri_mul_out", "tri_mul_in", "tri_att_start", "tri_att_end"])
def test_padded_positions_do_not_change_a_bit_of_the_valid_region(kind):
    n, pad = 150, 20
    g = torch.Generator().manual_seed(9)
    z = torch.randn(n, n, 128, generator=g)
    z2 = z.clone()
    z2[n - pad:] += torch.randn(pad, n, 128, generator=g)
    z2[:, n - pad:] += torch.randn(n, pad, 128, generator=g)
    mask = cuda(padding_mask(n, pad))
    m = build_module(kind, dict(wseed=12)).to(DEV)
    v = n - pad
    for dt in (torch.float32, torch.bfloat16):
        a = m(cuda(z).to(dt), mask=mask)
        b = m(cuda(z2).to(dt), mask=mask)
        assert torch.equal(a[:v, :v], b[:v, :v])


def test_fully_masked_rows_give_the_uniform_average_like_the_reference():
    n = 40
    g = torch.Generator().manual_seed(3)
    z = torch.randn(n, n, 128, generator=g)
    mask = torch.ones(n, n)
    mask[5, :] = 0          # starting node: every key of row 5 is masked
    m = build_module("tri_att_start", dict(wseed=8)).to(DEV)
    y = m(cuda(z), mask=cuda(mask))
    ref = O.triangle_attention(z, mask, params_of(m), starting=True)
    assert torch.isfinite(y).all() and relf(y[5], ref[5]) < TOL_OP and relf(y, ref) < TOL_OP


def test_mask_none_equals_all_ones():
    n = 48
    z = cuda(torch.randn(n, n, 128, generator=torch.Generator().manual_seed(4)))
    for kind in ("tri_mul_in", "tri_att_end"):
        m = build_module(kind, dict(wseed=5)).to(DEV)
        assert torch.equal(m(z, mask=None), m(z, mask=torch.ones(n, n, device=DEV)))


# ------------------------------------------------------------------------------ block and stack
@pytest.mark.parametrize("zdtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["block_n24", "block_pair_n20"])
def test_block_against_reference_vectors(name, zdtype):
    case = CASES[name]
    m = build_module("block", case).to(DEV)
    inp = make_inputs(case)
    s, z = m(cuda(inp["s"]), cuda(inp["z"]).to(zdtype), cuda(inp["mask"]))
    g = golden()
    assert relf(z, g[name + ".z"]) < TOL_BLOCK
    if s is not None:
        assert relf(s, g[name + ".s"]) < TOL_BLOCK


def test_stack_against_reference_vectors():
    case = CASES["stack2_n16"]
    m = build_module("stack", case).to(DEV)
    inp = make_inputs(case)
    s, z = m(cuda(inp["s"]), cuda(inp["z"]), cuda(inp["mask"]))
    g = golden()
    assert relf(z, g["stack2_n16.z"]) < TOL_STACK and relf(s, g["stack2_n16.s"]) < TOL_STACK


@pytest.mark.parametrize("zdtype", [torch.float32, torch.bfloat16])
def test_block_config1_n128(zdtype):
    """Single block, N=128, c_z=128, c_s=384, all-ones mask, z,s ~ N(0,1) (re-drawn weights)."""
    n = 128
    torch.manual_seed(0)
    z, s = torch.randn(n, n, 128), torch.randn(n, 384)
    m = build_module("block", dict(c_s=384, wseed=1)).to(DEV)
    s1, z1 = m(cuda(s), cuda(z).to(zdtype), torch.ones(n, n, device=DEV))
    s0, z0 = O.pairformer_block(s, z, torch.ones(n, n), params_of(m))
    assert relf(z1, z0) < TOL_BLOCK and relf(s1, s0) < TOL_BLOCK
    # update-only error: the residual does not hide it
    assert relf(z1.float().cpu() - z.to(zdtype).float(), z0 - z) < 2e-2


def test_stack_error_growth_stays_in_budget():
    n, nb = 64, 6
    g = torch.Generator().manual_seed(21)
    z, s = torch.randn(n, n, 128, generator=g), torch.randn(n, 384, generator=g)
    mask = padding_mask(n, 5)
    m = build_module("stack", dict(n_blocks=nb, c_s=384, wseed=31)).to(DEV)
    s0, z0 = O.pairformer_stack(s, z, mask, params_of(m), n_blocks=nb)
    for dt in (torch.float32, torch.bfloat16):
        s1, z1 = m(cuda(s), cuda(z).to(dt), cuda(mask))
        assert relf(z1, z0) < TOL_STACK and relf(s1, s0) < TOL_STACK


def test_confidence_head_stack_in_the_fp32_residual_path():
    """The confidence head runs a 4-block PairformerStack on an fp32 pair tensor outside autocast
    (protenix/model/modules/confidence.py:99-106, 307-315).  The fp32-residual path (fp16 operands of standardised
    rows, fp32 accumulation, statistics and residuals) keeps that stack within 2e-3 of the fp64 oracle -- the level of
    TF32 arithmetic, five times tighter than the per-block bound of the 16-bit path."""
    n, nb = 96, 4
    g = torch.Generator().manual_seed(77)
    z, s = torch.randn(n, n, 128, generator=g), torch.randn(n, 384, generator=g)
    mask = padding_mask(n, 9)
    m = build_module("stack", dict(n_blocks=nb, c_s=384, wseed=41)).to(DEV)
    # the fp32 oracle: in fully masked rows the reference's fp32 sum -1e9 + logit drops the logit (a uniform average),
    # which is the behaviour to match; an fp64 oracle keeps it and differs there by construction
    s0, z0 = O.pairformer_stack(s, z, mask, params_of(m), n_blocks=nb)
    s1, z1 = m(cuda(s), cuda(z), cuda(mask))
    assert z1.dtype == torch.float32
    assert relf(z1, z0) < 2e-3 and relf(s1, s0) < 2e-3, (relf(z1, z0), relf(s1, s0))
    v = n - 9                                        # and against fp64 where the mask leaves something to attend to
    _, z64 = O.pairformer_stack(s.double(), z.double(), mask.double(), params_of(m, torch.float64), n_blocks=nb)
    assert relf(z1[:v, :v], z64[:v, :v]) < 2e-3


def test_block_api_contract():
    n = 33
    g = torch.Generator().manual_seed(2)
    z = cuda(torch.randn(n, n, 128, generator=g))
    s = cuda(torch.randn(n, 384, generator=g))
    mask = cuda(padding_mask(n, 3))
    m = build_module("block", dict(c_s=384, wseed=6)).to(DEV)
    z_keep = z.clone()
    s1, z1 = m(s, z, mask, triangle_multiplicative="cuequivariance", triangle_attention="triattention", chunk_size=64)
    assert torch.equal(z, z_keep) and z1.data_ptr() != z.data_ptr()          # functional by default
    zi = z.clone()
    s2, z2 = m(s, zi, mask, inplace_safe=True)
    assert z2.data_ptr() == zi.data_ptr() and torch.equal(z2, z1) and torch.equal(s2, s1)   # in-place == functional
    s3, z3 = m(s, z, mask)
    assert torch.equal(z3, z1) and torch.equal(s3, s1)                         # run-to-run determinism
    s4, z4 = m(s, z[None], mask[None])                                         # batch of one, as the reference's test
    assert z4.shape == (1, n, n, 128) and torch.equal(z4[0], z1)
    sp, zp = build_module("block", dict(c_s=0, wseed=6)).to(DEV)(None, z, mask)
    assert sp is None and zp.shape == z.shape
    with pytest.raises(RuntimeError):
        m(s, z[:, :, :64].contiguous(), mask)


def test_stacked_blocks_with_half_precision_modules_like_the_reference_regression_test():
    """After the reference's TestPairformerCueqContiguity (tests/test_fused_dropout_add.py:140-221): three blocks
    whose parameters were cast to bf16, bf16 inputs with a leading batch of one (z, s and the mask), the
    cuEquivariance back-end names in the kwargs, in place; z must come back contiguous and finite, and equal to what
    fp32 parameters of the same values give."""
    n = 128
    g = torch.Generator().manual_seed(5)
    blocks = [build_module("block", dict(c_s=384, wseed=50 + i)).to(DEV).bfloat16() for i in range(3)]
    z = torch.randn(1, n, n, 128, generator=g).to(torch.bfloat16).to(DEV)
    s = torch.randn(1, n, 384, generator=g).to(torch.bfloat16).to(DEV)
    mask = torch.ones(1, n, n, dtype=torch.bfloat16, device=DEV)
    z_run, s_run = z.clone(), s.clone()
    for blk in blocks:
        s_run, z_run = blk(s_run, z_run, mask, triangle_multiplicative="cuequivariance",
                           triangle_attention="cuequivariance", inplace_safe=True)
        assert z_run.is_contiguous() and z_run.shape == z.shape and z_run.dtype == torch.bfloat16
        assert s_run.shape == s.shape
    assert torch.isfinite(z_run.float()).all() and torch.isfinite(s_run.float()).all()
    z_ref, s_ref = z.clone(), s.clone()
    for blk in blocks:
        s_ref, z_ref = blk.float()(s_ref, z_ref, mask.float(), inplace_safe=True)
    assert relf(z_run, z_ref) < 2e-2


def test_tri_mul_add_with_inplace_returns_sum():
    n = 40
    z = cuda(torch.randn(n, n, 128, generator=torch.Generator().manual_seed(8)))
    m = build_module("tri_mul_out", dict(wseed=2)).to(DEV)
    upd = m(z)
    zi = z.clone()
    out = m(zi, inplace_safe=True, _add_with_inplace=True)
    assert out.data_ptr() == zi.data_ptr() and relf(out, z + upd) < 1e-6


def test_state_dict_round_trip_changes_results():
    n = 24
    z = cuda(torch.randn(n, n, 128, generator=torch.Generator().manual_seed(1)))
    a = build_module("block", dict(c_s=0, wseed=1)).to(DEV)
    b = build_module("block", dict(c_s=0, wseed=2)).to(DEV)
    za = a(None, z, None)[1]
    assert not torch.equal(za, b(None, z, None)[1])
    b.load_state_dict(a.state_dict(), strict=True)
    assert torch.equal(za, b(None, z, None)[1])


# ------------------------------------------------------------- stage-level: tcgen05 contraction
@pytest.mark.parametrize("n", [1, 20, 100, 128, 136, 200, 257, 520])
def test_contraction_stage_through_c_abi(n):
    """px_trimul_contract (TMA + tcgen05 + TMEM) against an fp32 einsum of the same fp16 operands, scaled by
    PX_TRIMUL_X_SCALE: only the fp16 rounding of the output separates them.  Ragged sizes exercise the TMA zero fill."""
    import ctypes

    from protenix_b200 import _lib, ops

    lib = _lib.load()
    ldn = ops.ld(n)
    g = torch.Generator().manual_seed(n)
    a = torch.zeros(128, n, ldn, dtype=torch.float16)
    b = torch.zeros_like(a)
    a[:, :, :n] = torch.randn(128, n, n, generator=g).to(torch.float16)
    b[:, :, :n] = torch.randn(128, n, n, generator=g).to(torch.float16)
    a, b = a.cuda(), b.cuda()
    x = torch.full((128, n, ldn), float("nan"), dtype=torch.float16, device=DEV)
    rc = lib.px_trimul_contract(a.data_ptr(), b.data_ptr(), x.data_ptr(), 128, n, ldn,
                                torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    flags = ctypes.c_uint32(99)
    assert lib.px_device_error_flags(ctypes.byref(flags)) == 0 and flags.value == 0   # no bounded wait ran out
    ref = torch.einsum("cik,cjk->cij", a.float()[:, :, :n], b.float()[:, :, :n]) * ops.X_SCALE
    got = x[:, :, :n].float()
    assert torch.isfinite(got).all()
    assert relf(got, ref) < 5e-4
    assert torch.equal(got, ref.to(torch.float16).float()) or relf(got, ref.to(torch.float16).float()) < 3e-4
