"""Plain-torch (CPU, fp32) implementation of the stage interface of ``protenix_b200.sharded``.

Test infrastructure: it produces tensors in exactly the layouts the CUDA stages use (channel-major
a/b/x with zero pad columns, q/k/v per attended row, padded pair bias and mask bias), so that the
distributed choreography can run on CPU ranks (gloo) and be compared with the oracle.
"""
import math

import torch
import torch.nn.functional as F

LOG2E = math.log2(math.e)


def _ln(x, m):
    return F.layer_norm(x, (x.shape[-1],), m.weight, m.bias, m.eps)


def _pad_last(t, to, value=0.0):
    return F.pad(t, (0, to - t.shape[-1]), value=value) if to != t.shape[-1] else t.contiguous()


def _ld(n, m=8):
    return (n + m - 1) // m * m


class TorchStages:
    def standardised(self, z, eps):
        return None                                        # the fp32 stand-in normalises inside every stage

    def trimul_in_proj(self, mod, z, mask, incoming, zn=None):
        zn = _ln(z, mod.layer_norm_in)
        m = (mask if mask is not None else z.new_ones(z.shape[:2]))[..., None]
        a = m * torch.sigmoid(zn @ mod.linear_a_g.weight.T) * (zn @ mod.linear_a_p.weight.T)
        b = m * torch.sigmoid(zn @ mod.linear_b_g.weight.T) * (zn @ mod.linear_b_p.weight.T)
        perm = (2, 1, 0) if incoming else (2, 0, 1)        # -> [c][u][t]
        a, b = a.permute(*perm), b.permute(*perm)
        return _pad_last(a, _ld(a.shape[-1])), _pad_last(b, _ld(b.shape[-1]))

    def trimul_contract(self, a, b):
        n = a.shape[1]
        x = torch.einsum("cik,cjk->cij", a, b)
        return _pad_last(x, _ld(n))

    def trimul_out(self, mod, x, z, zn=None):
        n_j = z.shape[1]
        xin = x[:, :, :n_j].permute(1, 2, 0)
        zn = _ln(z, mod.layer_norm_in)
        z += (_ln(xin, mod.layer_norm_out) @ mod.linear_z.weight.T) * torch.sigmoid(zn @ mod.linear_g.weight.T)
        return z

    def triatt_in_proj(self, mod, z, mask, ending=False, zn=None):
        n_u, n_t, _ = z.shape
        xn = _ln(z, mod.layer_norm)
        h, d = mod.no_heads, mod.c_hidden
        sh = lambda t: t.view(n_u, n_t, h, d).permute(0, 2, 1, 3).contiguous()
        q = sh(xn @ mod.mha.linear_q.weight.T) * (LOG2E / math.sqrt(d))
        k = sh(xn @ mod.mha.linear_k.weight.T)
        v = _pad_last(sh(xn @ mod.mha.linear_v.weight.T).transpose(2, 3), _ld(n_t))   # [u][h][d][ld(t)]
        ldm = _ld(n_t, 128)
        bias = _pad_last(((xn @ mod.linear.weight.T) * LOG2E).permute(2, 0, 1), ldm)
        m = mask if mask is not None else z.new_ones(n_u, n_t)
        mb = _pad_last((m - 1) * mod.inf * LOG2E, ldm, float("-inf"))
        return q, k, v, bias, mb

    def triatt_flash(self, q, k, v, bias_full, mb):
        n_u, h, n, d = q.shape
        logits = torch.einsum("uhqd,uhkd->uhqk", q, k) + bias_full[None, :, :, :n] + mb[:, None, None, :n]
        w = torch.softmax(logits * math.log(2.0), dim=-1)
        return torch.einsum("uhqk,uhdk->uqhd", w, v[..., :n]).reshape(n_u, n, h * d)

    def triatt_out(self, mod, o, z, ending=False, zn=None):
        xn = _ln(z, mod.layer_norm)
        z += (o * torch.sigmoid(xn @ mod.mha.linear_g.weight.T)) @ mod.mha.linear_o.weight.T
        return z

    def transition(self, mod, z, out=None):
        y = _ln(z, mod.layernorm1)
        upd = (F.silu(y @ mod.linear_no_bias_a.weight.T) * (y @ mod.linear_no_bias_b.weight.T)) @ mod.linear_no_bias.weight.T
        if out is None:
            z += upd
            return z
        out.copy_(z + upd)
        return out

    def pair_bias(self, mod, z, zn=None):
        return (_ln(z, mod.layernorm_z) @ mod.linear_nobias_z.weight.T).permute(2, 0, 1).contiguous()

    def single_layer_norm(self, ln, x):
        return _ln(x, ln)

    def recycle_update(self, ln, lin, z, z_init, out):
        out.copy_(z_init + _ln(z, ln) @ lin.weight.T)
        return out
