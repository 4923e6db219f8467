"""CPU oracle for the Pairformer pair-representation forward path.

TEST INFRASTRUCTURE ONLY.  This file is the checker, never the product: it may be imported
by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline leg of ``bench.py``;
nothing under ``protenix_b200/`` imports it.

It is an independent restatement, in plain torch tensor algebra, of what the reference
(bytedance/Protenix v2.0.0, torch back-end, eval mode) computes.  Every function names the
reference lines it follows.  Parity of this restatement with the reference itself is pinned
by ``tests/golden/`` (vectors produced by importing the reference, see
``tests/golden/make_golden.py``) and checked by ``tests/test_oracle_golden.py``.

All functions take plain tensors plus a flat ``dict`` of parameters whose keys are the
reference's ``state_dict`` keys relative to the module (e.g. ``"tri_mul_out.linear_g.weight"``).
Arithmetic runs in the dtype of the inputs (fp32 by default, fp64 for tighter checks).
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F

Params = Dict[str, torch.Tensor]


def _sub(p: Params, prefix: str) -> Params:
    """Parameters below ``prefix.`` with the prefix stripped."""
    n = len(prefix) + 1
    return {k[n:]: v for k, v in p.items() if k.startswith(prefix + ".")}


def layer_norm(x: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor],
               eps: float = 1e-5) -> torch.Tensor:
    """y = (x - mean) * rsqrt(var_biased + eps) * weight + bias over the last axis.

    Follows protenix/model/triangular/layers.py:200-243 (OpenFoldLayerNorm) and the CUDA op
    protenix/model/layer_norm/kernel/layer_norm_cuda_kernel.cu:145-229 (biased variance,
    optional scale / offset).
    """
    mu = x.mean(dim=-1, keepdim=True)
    xc = x - mu
    var = (xc * xc).mean(dim=-1, keepdim=True)
    y = xc * torch.rsqrt(var + eps)
    if weight is not None:
        y = y * weight
    if bias is not None:
        y = y + bias
    return y


def layer_norm_stats(x: torch.Tensor, eps: float = 1e-5) -> Tuple[torch.Tensor, torch.Tensor]:
    """(mean, invvar) per row as the reference op returns them for its backward
    (protenix/model/layer_norm/kernel/layer_norm_cuda.cpp:73-90)."""
    mu = x.mean(dim=-1)
    var = ((x - mu[..., None]) ** 2).mean(dim=-1)
    return mu, torch.rsqrt(var + eps)


def transition(x: torch.Tensor, p: Params) -> torch.Tensor:
    """SwiGLU transition: W_o( silu(W_a LN(x)) * (W_b LN(x)) ), no residual.

    Follows protenix/model/modules/primitives.py:190-230.
    """
    y = layer_norm(x, p["layernorm1.weight"], p["layernorm1.bias"])
    a = y @ p["linear_no_bias_a.weight"].T
    b = y @ p["linear_no_bias_b.weight"].T
    return (F.silu(a) * b) @ p["linear_no_bias.weight"].T


def _contract(a: torch.Tensor, b: torch.Tensor, outgoing: bool) -> torch.Tensor:
    """Channel-batched product as the reference forms it (protenix/model/triangular/triangular.py:123-150):
    channels first, one matmul per channel, channels last again.  a: [I, K, C] (outgoing) or [K, I, C]."""
    if outgoing:
        x = torch.matmul(a.permute(2, 0, 1), b.permute(2, 1, 0))
    else:
        x = torch.matmul(a.permute(2, 1, 0), b.permute(2, 0, 1))
    return x.permute(1, 2, 0)


def _attend(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """softmax(q k^T + bias) v for q,k,v [I, N, H, D] and bias broadcastable to [I, H, Q, K]; returns
    [I, Q, H, D] (protenix/model/triangular/layers.py:276-296)."""
    q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)      # [I, H, N, D]
    w = torch.softmax(torch.matmul(q, k.transpose(-1, -2)) + bias, dim=-1)
    return torch.matmul(w, v).transpose(1, 2)


def triangle_multiplication(z: torch.Tensor, mask: Optional[torch.Tensor], p: Params,
                            outgoing: bool) -> torch.Tensor:
    """Triangle multiplicative update (returns the update, without the residual).

    Follows protenix/model/triangular/triangular.py:519-566 (functional branch) and
    :123-150 (_combine_projections): outgoing x[i,j,c] = sum_k a[i,k,c] b[j,k,c],
    incoming x[i,j,c] = sum_k a[k,i,c] b[k,j,c]; the mask multiplies a and b after gating.
    """
    if mask is None:
        mask = z.new_ones(z.shape[:-1])
    m = mask[..., None]
    zn = layer_norm(z, p["layer_norm_in.weight"], p["layer_norm_in.bias"])
    a = m * torch.sigmoid(zn @ p["linear_a_g.weight"].T) * (zn @ p["linear_a_p.weight"].T)
    b = m * torch.sigmoid(zn @ p["linear_b_g.weight"].T) * (zn @ p["linear_b_p.weight"].T)
    x = _contract(a, b, outgoing)
    x = layer_norm(x, p["layer_norm_out.weight"], p["layer_norm_out.bias"])
    x = x @ p["linear_z.weight"].T
    g = torch.sigmoid(zn @ p["linear_g.weight"].T)
    return x * g


def triangle_attention(x: torch.Tensor, mask: Optional[torch.Tensor], p: Params,
                       starting: bool = True, inf: float = 1e9,
                       row_chunk: Optional[int] = None) -> torch.Tensor:
    """Triangle attention around the starting node (``starting=False``: ending node, i.e.
    the same thing on the transposed pair tensor).  Returns the update, no residual.

    Follows protenix/model/triangular/triangular.py:657-715 and the torch attention of
    protenix/model/triangular/layers.py:276-296, :361-398:
    L[i,h,q,k] = (q[i,q,h]/sqrt(d)) . k[i,k,h] + inf*(mask[i,k]-1) + (W_b LN(x))[q,k,h],
    softmax over k, o = P v, out = W_o(o * sigmoid(W_g LN(x))).
    ``row_chunk`` only bounds memory (rows i are independent).
    """
    if mask is None:
        mask = x.new_ones(x.shape[:-1])
    if not starting:
        x = x.transpose(0, 1)
        mask = mask.transpose(0, 1)
    n = x.shape[0]
    h = p["linear.weight"].shape[0]
    xn = layer_norm(x, p["layer_norm.weight"], p["layer_norm.bias"])
    tri_bias = (xn @ p["linear.weight"].T).permute(2, 0, 1)          # [H, Q, K]
    d = p["mha.linear_q.weight"].shape[0] // h
    out = torch.empty_like(xn)
    step = n if row_chunk is None else row_chunk
    for r0 in range(0, n, step):
        xr = xn[r0:r0 + step]
        q = (xr @ p["mha.linear_q.weight"].T).view(-1, n, h, d) / math.sqrt(d)
        k = (xr @ p["mha.linear_k.weight"].T).view(-1, n, h, d)
        v = (xr @ p["mha.linear_v.weight"].T).view(-1, n, h, d)
        o = _attend(q, k, v, (inf * (mask[r0:r0 + step] - 1))[:, None, None, :] + tri_bias[None])
        g = torch.sigmoid(xr @ p["mha.linear_g.weight"].T).view(-1, n, h, d)
        out[r0:r0 + step] = (o * g).reshape(-1, n, h * d) @ p["mha.linear_o.weight"].T
    if not starting:
        out = out.transpose(0, 1)
    return out


def attention_pair_bias(s: torch.Tensor, z: torch.Tensor, p: Params, n_heads: int) -> torch.Tensor:
    """Single-representation attention with pair bias, has_s=False variant (no residual).

    Follows protenix/model/modules/transformer.py:159-254 (standard_multihead_attention)
    and protenix/model/modules/primitives.py:233-291, :782-879: q has a bias term, logits are
    q.k/sqrt(d) + W_z LN(z), gate sigmoid(W_g a) applied before the output projection.
    """
    a = layer_norm(s, p["layernorm_a.weight"], p["layernorm_a.bias"])
    bias = layer_norm(z, p["layernorm_z.weight"], p.get("layernorm_z.bias")) @ p["linear_nobias_z.weight"].T
    bias = bias.permute(2, 0, 1)                                      # [H, N, N]
    n, c = a.shape
    d = c // n_heads
    q = (a @ p["attention.linear_q.weight"].T + p["attention.linear_q.bias"]).view(n, n_heads, d)
    k = (a @ p["attention.linear_k.weight"].T).view(n, n_heads, d)
    v = (a @ p["attention.linear_v.weight"].T).view(n, n_heads, d)
    logits = torch.einsum("qhd,khd->hqk", q / math.sqrt(d), k) + bias
    w = torch.softmax(logits, dim=-1)
    o = torch.einsum("hqk,khd->qhd", w, v).reshape(n, c)
    g = torch.sigmoid(a @ p["attention.linear_g.weight"].T)
    return (o * g) @ p["attention.linear_o.weight"].T


def pairformer_block(s: Optional[torch.Tensor], z: torch.Tensor, pair_mask: Optional[torch.Tensor],
                     p: Params, n_heads: int = 16, row_chunk: Optional[int] = None
                     ) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
    """One Pairformer block in eval mode (dropout is the identity).

    Follows protenix/model/modules/pairformer.py:103-224.  The reference transposes z,
    runs a starting-node module on it and transposes back (:160-168); here the ending-node
    form of ``triangle_attention`` does the same arithmetic.
    """
    z = z + triangle_multiplication(z, pair_mask, _sub(p, "tri_mul_out"), outgoing=True)
    z = z + triangle_multiplication(z, pair_mask, _sub(p, "tri_mul_in"), outgoing=False)
    z = z + triangle_attention(z, pair_mask, _sub(p, "tri_att_start"), starting=True, row_chunk=row_chunk)
    z = z + triangle_attention(z, pair_mask, _sub(p, "tri_att_end"), starting=False, row_chunk=row_chunk)
    z = z + transition(z, _sub(p, "pair_transition"))
    if s is not None and any(k.startswith("attention_pair_bias.") for k in p):
        s = s + attention_pair_bias(s, z, _sub(p, "attention_pair_bias"), n_heads)
        s = s + transition(s, _sub(p, "single_transition"))
    return s, z


def pairformer_stack(s: Optional[torch.Tensor], z: torch.Tensor, pair_mask: Optional[torch.Tensor],
                     p: Params, n_blocks: int, n_heads: int = 16, row_chunk: Optional[int] = None
                     ) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
    """``n_blocks`` blocks in sequence; parameter keys are ``blocks.{i}.<block key>``.

    Follows protenix/model/modules/pairformer.py:291-340 (no-grad path of checkpoint_blocks,
    protenix/model/utils.py:865-866: a plain loop).
    """
    for i in range(n_blocks):
        s, z = pairformer_block(s, z, pair_mask, _sub(p, f"blocks.{i}"), n_heads, row_chunk)
    return s, z


def recycle_update(x: torch.Tensor, x_init: torch.Tensor, p: Params, ln: str, lin: str) -> torch.Tensor:
    """x_init + W LN(x): one recycling update (protenix/model/protenix.py:246 for z, :287 for s)."""
    return x_init + layer_norm(x, p[ln + ".weight"], p.get(ln + ".bias")) @ p[lin + ".weight"].t()


def recycling_trunk(s_init: torch.Tensor, z_init: torch.Tensor, pair_mask: Optional[torch.Tensor], p: Params,
                    n_blocks: int, n_cycle: int, n_heads: int = 16, msa: Optional[dict] = None,
                    msa_n_blocks: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """The recycling loop around the Pairformer stack, without template embedder and MSA module.

    Follows protenix/model/protenix.py:230-296: z and s start at zero (:230-231); every cycle
    z = z_init + linear_no_bias_z_cycle(layernorm_z_cycle(z)) (:246),
    s = s_init + linear_no_bias_s(layernorm_s(s)) (:287), then the stack (:288-296).
    """
    z = torch.zeros_like(z_init)
    s = torch.zeros_like(s_init)
    for _ in range(n_cycle):
        z = recycle_update(z, z_init, p, "layernorm_z_cycle", "linear_no_bias_z_cycle")
        if msa is not None and msa_n_blocks > 0:        # protenix/model/protenix.py:258-267, between the two updates
            z = msa_module(msa["msa"], msa["has_deletion"], msa["deletion_value"], z, msa["s_inputs"], pair_mask,
                           _sub(p, "msa_module"), msa_n_blocks)
        s = recycle_update(s, s_init, p, "layernorm_s", "linear_no_bias_s")
        s, z = pairformer_stack(s, z, pair_mask, _sub(p, "pairformer_stack"), n_blocks, n_heads)
    return s, z


def outer_product_mean(m: torch.Tensor, msa_mask: Optional[torch.Tensor], p: Params, eps: float = 1e-3) -> torch.Tensor:
    """The pair update of the MSA module's OuterProductMean: [N, N, c_z] from an MSA embedding m [S, N, c_m] and an
    MSA mask [S, N] (None: all ones).

    Follows protenix/model/triangular/layers.py:657-780: ln = LayerNorm(m) (:749); a = linear_1(ln) * mask,
    b = linear_2(ln) * mask (:752-757); outer[i, j, c, e] = sum_s a[s, i, c] * b[s, j, e] (einsum at :687, after the
    transposes at :761-762), flattened with c slow and e fast (:690); linear_out with its bias (:693); divided by
    norm[i, j] + eps with norm = sum_s mask[s, i] * mask[s, j] (:770-771, :775-777).  The caller adds the result to z
    (protenix/model/modules/pairformer.py, MSABlock.forward).
    """
    if msa_mask is None:
        msa_mask = m.new_ones(m.shape[:-1])
    ln = layer_norm(m, p["layer_norm.weight"], p.get("layer_norm.bias"))
    a = (ln @ p["linear_1.weight"].t()) * msa_mask[..., None]            # [S, N, C]
    b = (ln @ p["linear_2.weight"].t()) * msa_mask[..., None]
    n, c = a.shape[1], a.shape[2]
    outer = torch.einsum("sic,sje->ijce", a, b).reshape(n, n, c * c)
    out = outer @ p["linear_out.weight"].t() + p["linear_out.bias"]
    norm = torch.einsum("si,sj->ij", msa_mask, msa_mask)[..., None] + eps
    return out / norm


def msa_pair_weighted_averaging(m: torch.Tensor, z: torch.Tensor, p: Params, n_heads: int = 8) -> torch.Tensor:
    """The update of the MSA embedding m [S, N, c_m] weighted by the pair representation (not added).

    Follows protenix/model/modules/pairformer.py:385-422: v = linear_no_bias_mv(LN(m)) split into heads (:398-402),
    b = linear_no_bias_z(LN(z)) (:403-405), g = sigmoid(linear_no_bias_mg(LN(m))) (:406-411), w = softmax of b over
    the second token index (dim -2 of [i, j, h], :412), wv[s, i, h, :] = sum_j w[i, j, h] v[s, j, h, :] (:413-415),
    linear_no_bias_out(g * wv) (:416-420).
    """
    mn = layer_norm(m, p["layernorm_m.weight"], p.get("layernorm_m.bias"))
    s_rows, n, _ = m.shape
    v = (mn @ p["linear_no_bias_mv.weight"].t()).view(s_rows, n, n_heads, -1)
    g = torch.sigmoid(mn @ p["linear_no_bias_mg.weight"].t()).view(s_rows, n, n_heads, -1)
    b = layer_norm(z, p["layernorm_z.weight"], p.get("layernorm_z.bias")) @ p["linear_no_bias_z.weight"].t()
    w = torch.softmax(b, dim=-2)
    wv = torch.einsum("ijh,sjhc->sihc", w, v)
    return (g * wv).reshape(s_rows, n, -1) @ p["linear_no_bias_out.weight"].t()


def msa_stack(m: torch.Tensor, z: torch.Tensor, p: Params) -> torch.Tensor:
    """m + pair-weighted averaging, then + transition (protenix/model/modules/pairformer.py:551-572, the eval path;
    its chunking over MSA rows changes nothing in the result)."""
    m = m + msa_pair_weighted_averaging(m, z, _sub(p, "msa_pair_weighted_averaging"))
    return m + transition(m, _sub(p, "transition_m"))


def msa_block(m: torch.Tensor, z: torch.Tensor, pair_mask: Optional[torch.Tensor], p: Params,
              is_last_block: bool = False) -> Tuple[Optional[torch.Tensor], torch.Tensor]:
    """One block of the MSA module (protenix/model/modules/pairformer.py:658-678): z += OuterProductMean(m) without an
    MSA mask (:659-661), m = MSAStack(m, z) unless this is the last block (:662-664), then the pair-only Pairformer
    block (:666-674); the last block returns no m (:675-678)."""
    z = z + outer_product_mean(m, None, _sub(p, "outer_product_mean_msa"))
    if not is_last_block:
        m = msa_stack(m, z, _sub(p, "msa_stack"))
    _, z = pairformer_block(None, z, pair_mask, _sub(p, "pair_stack"))
    return (None if is_last_block else m), z


def msa_module(msa: torch.Tensor, has_deletion: torch.Tensor, deletion_value: torch.Tensor, z: torch.Tensor,
               s_inputs: torch.Tensor, pair_mask: Optional[torch.Tensor], p: Params, n_blocks: int) -> torch.Tensor:
    """The MSA module on MSA rows that are already sampled (protenix/model/modules/pairformer.py:872-911): the
    features one_hot(msa, 32) | has_deletion | deletion_value (:872-889) through linear_no_bias_m (:895), plus
    linear_no_bias_s(s_inputs) broadcast over the rows (:898), then the blocks (:899-910); the last block returns no m
    (:675-678)."""
    feat = torch.cat([F.one_hot(msa, 32).to(z.dtype), has_deletion[..., None].to(z.dtype),
                      deletion_value[..., None].to(z.dtype)], dim=-1)
    m = feat @ p["linear_no_bias_m.weight"].t() + s_inputs @ p["linear_no_bias_s.weight"].t()
    for i in range(n_blocks):
        m, z = msa_block(m, z, pair_mask, _sub(p, f"blocks.{i}"), is_last_block=(i + 1 == n_blocks))
    return z


def rel_frobenius(a: torch.Tensor, b: torch.Tensor) -> float:
    """||a - b||_F / ||b||_F in fp64."""
    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def pair_path_row_slab(z: torch.Tensor, pair_mask: Optional[torch.Tensor], p: Params, r0: int, r1: int,
                       shared: Optional[dict] = None, only: Optional[Tuple[str, ...]] = None
                       ) -> Tuple[Dict[str, torch.Tensor], dict]:
    """Timing sample of one block's pair path: the five pair updates for output rows [r0, r1) only.

    Every update is computed from the same input z (the sequential dependence between the five
    sub-modules is dropped: values do not change the cost).  All row-wise work -- LayerNorms, every
    projection including both a and b of the two multiplications and the pair-bias projection,
    gates, output projections, the transition -- is done for the slab's (r1 - r0) * N pair elements,
    and the O(N^3) products are done for the slab's output rows, so the arithmetic volume is
    exactly (r1 - r0) / N of one block's pair path.  The operands of the other token axis that a
    slab needs in full (b over all rows for the outgoing product, a and b for the incoming one,
    the [H, N, N] pair bias) come from ``shared``: computed here by the same formulas when it is
    None (so that the slabs equal the full updates; the tests use this), or supplied by a caller
    that only wants the timing and passes stand-in tensors of the right shapes.  Returns the five
    update slabs by sub-module name; the ending-node slab is indexed by column (rows [r0, r1) of
    the transposed update).  ``only`` restricts the work to the named sub-modules (parity tests at sizes where the
    full update does not fit).  Used by the CPU-baseline leg of the benchmark and by tests.
    """
    want = lambda name: only is None or name in only
    n = z.shape[0]
    mask = pair_mask if pair_mask is not None else z.new_ones(n, n)

    def gated(zn, q, which, m):
        return m[..., None] * torch.sigmoid(zn @ q[f"linear_{which}_g.weight"].T) * (zn @ q[f"linear_{which}_p.weight"].T)

    if shared is None:
        shared = {}
        for name in ("tri_mul_out", "tri_mul_in"):
            if not want(name):
                continue
            q = _sub(p, name)
            zn = layer_norm(z, q["layer_norm_in.weight"], q["layer_norm_in.bias"])
            shared[name + ".a"] = gated(zn, q, "a", mask)
            shared[name + ".b"] = gated(zn, q, "b", mask)
        for name, tr in (("tri_att_start", False), ("tri_att_end", True)):
            if not want(name):
                continue
            q = _sub(p, name)
            x = z.transpose(0, 1) if tr else z
            xn = layer_norm(x, q["layer_norm.weight"], q["layer_norm.bias"])
            shared[name + ".bias"] = (xn @ q["linear.weight"].T).permute(2, 0, 1).contiguous()
    rows = slice(r0, r1)
    out: Dict[str, torch.Tensor] = {}
    for name in ("tri_mul_out", "tri_mul_in"):
        if not want(name):
            continue
        q = _sub(p, name)
        zn = layer_norm(z[rows], q["layer_norm_in.weight"], q["layer_norm_in.bias"])
        a_slab = gated(zn, q, "a", mask[rows])
        b_slab = gated(zn, q, "b", mask[rows])      # this slab's share of the other operand's projection
        if name == "tri_mul_out":
            x = _contract(a_slab, shared[name + ".b"], True)
        else:
            x = _contract(shared[name + ".a"][:, rows], shared[name + ".b"], False)
        del b_slab
        x = layer_norm(x, q["layer_norm_out.weight"], q["layer_norm_out.bias"]) @ q["linear_z.weight"].T
        out[name] = x * torch.sigmoid(zn @ q["linear_g.weight"].T)
    for name, tr in (("tri_att_start", False), ("tri_att_end", True)):
        if not want(name):
            continue
        q = _sub(p, name)
        x = (z.transpose(0, 1) if tr else z)[rows]
        m = (mask.transpose(0, 1) if tr else mask)[rows]
        h = q["linear.weight"].shape[0]
        d = q["mha.linear_q.weight"].shape[0] // h
        xn = layer_norm(x, q["layer_norm.weight"], q["layer_norm.bias"])
        bias_slab = xn @ q["linear.weight"].T        # this slab's share of the pair-bias projection
        del bias_slab
        qq = (xn @ q["mha.linear_q.weight"].T).view(-1, n, h, d) / math.sqrt(d)
        kk = (xn @ q["mha.linear_k.weight"].T).view(-1, n, h, d)
        vv = (xn @ q["mha.linear_v.weight"].T).view(-1, n, h, d)
        o = _attend(qq, kk, vv, (1e9 * (m - 1))[:, None, None, :] + shared[name + ".bias"][None])
        g = torch.sigmoid(xn @ q["mha.linear_g.weight"].T).view(-1, n, h, d)
        out[name] = (o * g).reshape(-1, n, h * d) @ q["mha.linear_o.weight"].T
    if want("pair_transition"):
        out["pair_transition"] = transition(z[rows], _sub(p, "pair_transition"))
    return out, shared
