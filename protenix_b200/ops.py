"""Tensor-level wrappers over the C ABI (``include/px_b200.h``).

Each function validates its tensors on the host (device, dtype, contiguity, shape), passes raw
pointers plus the current CUDA stream to the library and raises ``RuntimeError`` on a non-zero
status.  torch is used for memory and streams only.
"""
from __future__ import annotations

import os
from typing import Dict, Optional, Tuple

import torch

from . import _lib
from ._lib import PX_BF16, PX_F16, PX_F32
from .weights import w16_of

_DTYPE = {torch.float32: PX_F32, torch.bfloat16: PX_BF16, torch.float16: PX_F16}
C_Z = 128
X_SCALE = 1.0 / 64      # PX_TRIMUL_X_SCALE: the contraction stores x scaled so that it stays inside the fp16 range
N_HEAD_PAIR = 4
D_HEAD_PAIR = 32


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _need_cuda(t: torch.Tensor, name: str) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: this package has no CPU path")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def _pair_dtype(z: torch.Tensor) -> int:
    if z.dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError(f"pair tensor must be float32 or bfloat16, got {z.dtype}")
    return _DTYPE[z.dtype]


def _check_pair(z: torch.Tensor, name: str = "z") -> int:
    _need_cuda(z, name)
    if z.dim() != 3 or z.shape[0] != z.shape[1] or z.shape[2] != C_Z:
        raise RuntimeError(f"{name} must have shape [N, N, {C_Z}], got {tuple(z.shape)}")
    return z.shape[0]


F16 = torch.float16


def _zfmt(z: torch.Tensor) -> torch.dtype:
    """Format of the weights that multiply rows of z: bf16 rows are multiplied as stored, fp32 rows as fp16."""
    return torch.bfloat16 if z.dtype == torch.bfloat16 else torch.float16


def _w(w: torch.Tensor, fmt: torch.dtype, shape: Tuple[int, ...], name: str) -> torch.Tensor:
    """A weight matrix (an fp32 parameter or an already converted tensor) in the 16-bit format the kernel wants;
    the conversion is cached per parameter version."""
    if not isinstance(w, torch.Tensor) or not w.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: this package has no CPU path")
    if tuple(w.shape) != shape or not w.is_floating_point():
        raise RuntimeError(f"{name} must be a floating-point tensor of shape {shape}, got {w.dtype} {tuple(w.shape)}")
    return w16_of(w, fmt)


def _check_v(v: torch.Tensor, n: int, name: str) -> None:
    _need_cuda(v, name)
    if v.dtype != torch.float32 or tuple(v.shape) != (n,):
        raise RuntimeError(f"{name} must be float32 ({n},), got {v.dtype} {tuple(v.shape)}")


def _check_mask(mask: Optional[torch.Tensor], n: int) -> Optional[torch.Tensor]:
    if mask is None:
        return None
    _need_cuda(mask, "mask")
    if mask.dtype != torch.float32 or tuple(mask.shape) != (n, n):
        raise RuntimeError(f"mask must be float32 ({n},{n}), got {mask.dtype} {tuple(mask.shape)}")
    return mask


# ---------------------------------------------------------------------------------------------
class StageTimer:
    """Optional per-kernel CUDA-event timing on the launching stream (used by bench.py)."""

    def __init__(self) -> None:
        self.events = []          # (name, start, stop)

    def summary(self) -> Dict[str, Tuple[int, float]]:
        """name -> (launches, total milliseconds); call after a device synchronize."""
        out: Dict[str, Tuple[int, float]] = {}
        for name, a, b in self.events:
            c, t = out.get(name, (0, 0.0))
            out[name] = (c + 1, t + a.elapsed_time(b))
        return out


_timer: Optional[StageTimer] = None
launch_count = 0     # kernels of this library launched since import (or since reset_launch_count)


def set_stage_timer(t: Optional[StageTimer]) -> None:
    global _timer
    _timer = t


def reset_launch_count() -> int:
    global launch_count
    n, launch_count = launch_count, 0
    return n


def _launch(name: str, fn, *args) -> None:
    """Call one C-ABI launcher, optionally bracketed by CUDA events (one kernel per launcher, except
    ``px_triatt_flash``, which runs its small tile-flag kernel first: its stage time covers both)."""
    global launch_count
    if _timer is not None:
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record()
        st = fn(*args)
        b.record()
        _timer.events.append((name, a, b))
    else:
        st = fn(*args)
    launch_count += 1
    _lib.check(st, name)


KERNEL_FAMILIES = ("trimul_contract", "triatt_flash", "transition", "trimul_in_proj", "trimul_out", "triatt_in_proj",
                   "triatt_out", "pair_bias_proj", "recycle_update", "selftest", "peer_barrier",
                   "outer_product_mean")   # bit order of px_device_error_flags


def device_error_flags(device=None, raise_on_error: bool = True) -> int:
    """Synchronise the device and read (and clear) the record of device-side waits that ran out.

    Every wait inside the kernels is bounded; one that gives up makes its kernel return early and leaves a flag.
    Returns the flag word (bit f = ``KERNEL_FAMILIES[f]``); raises ``RuntimeError`` on a non-zero word unless
    ``raise_on_error`` is false.  It synchronises, so call it after a forward pass, not between kernels.
    """
    import ctypes

    flags = ctypes.c_uint32(0)
    detail = (ctypes.c_uint32 * len(KERNEL_FAMILIES))()
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        _lib.check(_lib.load().px_device_error_detail(ctypes.byref(flags), detail), "px_device_error_detail")
    if flags.value and raise_on_error:
        what = ", ".join(f"{KERNEL_FAMILIES[f]} (wait codes 0x{detail[f]:x})" for f in range(len(KERNEL_FAMILIES))
                         if flags.value >> f & 1)
        raise RuntimeError(f"a bounded device-side wait ran out in: {what}; the outputs of those kernels are not valid")
    return int(flags.value)


_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}


def workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """A per-(device, stream) scratch buffer, grown on demand and reused between calls."""
    dev = torch.device(device)
    key = (dev.index if dev.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(dev).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        _workspaces.pop(key, None)
        buf = None
        buf = torch.empty(int(nbytes), dtype=torch.uint8, device=dev)
        _workspaces[key] = buf
    return buf


def release_workspaces() -> None:
    _workspaces.clear()


def ld(n: int) -> int:
    return int(_lib.load().px_ld(n))


# ---------------------------------------------------------------------------------------------
def layer_norm(x: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor], eps: float = 1e-5,
               return_stats: bool = False):
    """LayerNorm over the last axis.  Returns y, or (y, mean, invvar) with fp32 statistics."""
    _need_cuda(x, "input")
    if x.dtype not in _DTYPE:
        raise RuntimeError(f"layer_norm supports float32/bfloat16/float16, got {x.dtype}")
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    for t, nm in ((weight, "weight"), (bias, "bias")):
        if t is not None:
            _need_cuda(t, nm)
            if t.dtype != x.dtype or t.numel() != cols:
                raise RuntimeError(f"{nm} must be {x.dtype} with {cols} elements")
    y = torch.empty_like(x)
    mean = invvar = None
    if return_stats:
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        invvar = torch.empty(rows, dtype=torch.float32, device=x.device)
    _launch("px_layer_norm_fwd", _lib.load().px_layer_norm_fwd, _ptr(x), _ptr(weight), _ptr(bias), _ptr(y),
            _ptr(mean), _ptr(invvar), rows, cols, float(eps), _DTYPE[x.dtype], _stream(x))
    return (y, mean, invvar) if return_stats else y


def layer_norm_bwd(dy: torch.Tensor, x: torch.Tensor, mean: torch.Tensor, invvar: torch.Tensor,
                   weight: Optional[torch.Tensor], want_weight: bool, want_bias: bool):
    """Gradients of layer_norm: (dx, dweight or None, dbias or None) from the upstream gradient dy, the input x and the
    fp32 statistics the forward returned."""
    _need_cuda(dy, "dy")
    _need_cuda(x, "x")
    if dy.shape != x.shape or dy.dtype != x.dtype or x.dtype not in _DTYPE:
        raise RuntimeError("dy must match x (float32 / bfloat16 / float16)")
    cols = x.shape[-1]
    rows = x.numel() // cols if cols else 0
    if mean.numel() != rows or invvar.numel() != rows or mean.dtype != torch.float32 or invvar.dtype != torch.float32:
        raise RuntimeError("mean and invvar must be the float32 [rows] statistics of the forward")
    if weight is not None and (weight.dtype != x.dtype or weight.numel() != cols):
        raise RuntimeError(f"weight must be {x.dtype} with {cols} elements")
    dy, x = dy.contiguous(), x.contiguous()
    dx = torch.empty_like(x)
    dw = torch.empty(cols, dtype=x.dtype, device=x.device) if want_weight else None
    db = torch.empty(cols, dtype=x.dtype, device=x.device) if want_bias else None
    scratch = torch.empty(2 * cols, dtype=torch.float32, device=x.device) if (want_weight or want_bias) else None
    _launch("px_layer_norm_bwd", _lib.load().px_layer_norm_bwd, _ptr(dy), _ptr(x), _ptr(mean), _ptr(invvar), _ptr(weight),
            _ptr(dx), _ptr(dw), _ptr(db), _ptr(scratch), rows, cols, _DTYPE[x.dtype], _stream(x))
    return dx, dw, db


def scale_add_rowwise(residual: Optional[torch.Tensor], x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """residual + x * mask with mask [..., 1, C, D] shared over axis -3 of x [..., R, C, D] (residual None: x * mask)."""
    _need_cuda(x, "x")
    _need_cuda(mask, "mask")
    if x.dim() < 3 or x.dtype not in _DTYPE or mask.dtype != x.dtype:
        raise RuntimeError("x must be [..., R, C, D] in float32 / bfloat16 / float16 and the mask of the same type")
    want = list(x.shape)
    want[-3] = 1
    if list(mask.shape) != want:
        raise RuntimeError(f"mask must have shape {want}")
    if residual is not None and (residual.shape != x.shape or residual.dtype != x.dtype or not residual.is_cuda):
        raise RuntimeError("residual must match x")
    x = x.contiguous()
    residual = None if residual is None else residual.contiguous()
    mask = mask.contiguous()
    out = torch.empty_like(x)
    rows, cd = x.shape[-3], x.shape[-2] * x.shape[-1]
    batches = x.numel() // (rows * cd) if rows * cd else 0
    _launch("px_scale_add_rowwise", _lib.load().px_scale_add_rowwise, _ptr(residual), _ptr(x), _ptr(mask), _ptr(out),
            batches, rows, cd, _DTYPE[x.dtype], _stream(x))
    return out


def standardise_rows(z: torch.Tensor, eps: float = 1e-5, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """zn = fp16((z - mean) * rstd) over rows of 128 channels of an fp32 tensor: the rows the tensor core multiplies
    when the pair tensor is stored as fp32.  One copy serves every stage that normalises the same z."""
    _need_cuda(z, "z")
    if z.dtype != torch.float32 or z.shape[-1] != C_Z:
        raise RuntimeError("standardise_rows takes a float32 tensor [..., 128]")
    if out is None:
        out = torch.empty(z.shape, dtype=torch.float16, device=z.device)
    rows = z.numel() // C_Z
    _launch("px_standardise_rows", _lib.load().px_standardise_rows, _ptr(z), _ptr(out), rows, float(eps), _stream(z))
    return out


def add_update_rows(z: torch.Tensor, upd: torch.Tensor) -> torch.Tensor:
    """z += upd in place for an fp32 tensor [..., 128] and an fp16 update of the same shape."""
    _need_cuda(z, "z")
    _need_cuda(upd, "upd")
    if z.dtype != torch.float32 or upd.dtype != torch.float16 or z.shape != upd.shape or z.shape[-1] != C_Z:
        raise RuntimeError("add_update_rows takes a float32 tensor [..., 128] and a float16 update of the same shape")
    _launch("px_add_update_rows", _lib.load().px_add_update_rows, _ptr(z), _ptr(upd), z.numel() // C_Z, _stream(z))
    return z


def _zn_arg(z: torch.Tensor, zn: Optional[torch.Tensor]) -> Optional[int]:
    """Raw pointer of an optional standardised copy of z that the caller hands in."""
    if zn is None:
        return None
    if z.dtype != torch.float32:
        raise RuntimeError("zn goes with a float32 pair tensor")
    if zn.dtype != torch.float16 or zn.shape != z.shape or zn.device != z.device or not zn.is_contiguous():
        raise RuntimeError("zn must be a contiguous float16 tensor of the shape of z")
    return zn.data_ptr()


def _rows_of(z: torch.Tensor, zn: Optional[torch.Tensor], eps: float) -> Tuple[torch.Tensor, int]:
    """The rows a stage multiplies and their dtype code: bf16 z itself, or the standardised fp16 copy of an fp32 z
    (made here unless the caller already holds one; a float16 ``z`` is taken to be that copy)."""
    if z.dtype == torch.bfloat16:
        return z, PX_BF16
    if z.dtype == torch.float16:
        return z, PX_F16
    if z.dtype != torch.float32:
        raise RuntimeError(f"pair tensor must be float32 or bfloat16, got {z.dtype}")
    if zn is None:
        zn = standardise_rows(z, eps)
    elif zn.dtype != torch.float16 or zn.shape != z.shape or not zn.is_cuda or not zn.is_contiguous():
        raise RuntimeError("zn must be the contiguous float16 standardised copy of z")
    return zn, PX_F16


def triangle_multiplication(z_in: torch.Tensor, z_out: torch.Tensor, mask: Optional[torch.Tensor],
                            ln_in_w, ln_in_b, ln_out_w, ln_out_b, w_ap, w_ag, w_bp, w_bg, w_z, w_g,
                            incoming: bool, add_residual: bool, eps: float = 1e-5,
                            zn: Optional[torch.Tensor] = None) -> torch.Tensor:
    """zn: the standardised fp16 copy of an fp32 z_in when the caller already has it (same eps)."""
    n = _check_pair(z_in, "z_in")
    if _check_pair(z_out, "z_out") != n or z_out.dtype != z_in.dtype:
        raise RuntimeError("z_out must match z_in in shape and dtype")
    mask = _check_mask(mask, n)
    for v, nm in ((ln_in_w, "ln_in_w"), (ln_in_b, "ln_in_b"), (ln_out_w, "ln_out_w"), (ln_out_b, "ln_out_b")):
        _check_v(v, C_Z, nm)
    zf = _zfmt(z_in)
    w_ap, w_ag, w_bp, w_bg, w_g = (_w(w, zf, (C_Z, C_Z), nm) for w, nm in
                                   ((w_ap, "w_ap"), (w_ag, "w_ag"), (w_bp, "w_bp"), (w_bg, "w_bg"), (w_g, "w_g")))
    w_z = _w(w_z, F16, (C_Z, C_Z), "w_z")
    lib = _lib.load()
    ws = workspace(z_in.device, lib.px_trimul_workspace_bytes(n))
    ldn = lib.px_ld(n)
    per = C_Z * n * ldn * 2                      # bytes of one channel-major [128][N][ld] fp16 tensor
    a, b, x = ws.data_ptr(), ws.data_ptr() + per, ws.data_ptr() + 2 * per
    dt, st, eps = _pair_dtype(z_in), _stream(z_in), float(eps)
    rows, rows_dt = _ptr(z_in), dt
    zn = _zn_arg(z_in, zn)
    if dt == PX_F32:            # the projection and the output stage normalise the same z: one standardised copy
        if zn is None:
            zn = ws.data_ptr() + 3 * per
            _launch("px_standardise_rows", lib.px_standardise_rows, _ptr(z_in), zn, n * n, eps, st)
        rows, rows_dt = zn, PX_F16
    _launch("px_trimul_in_proj", lib.px_trimul_in_proj, rows, rows_dt, _ptr(mask), _ptr(ln_in_w), _ptr(ln_in_b),
            _ptr(w_ap), _ptr(w_ag), _ptr(w_bp), _ptr(w_bg), a, b, n, n, ldn, int(incoming), eps, st)
    _launch("px_trimul_contract", lib.px_trimul_contract, a, b, x, C_Z, n, ldn, st)
    _launch("px_trimul_out", lib.px_trimul_out, x, _ptr(z_in), zn, _ptr(z_out), dt, _ptr(ln_in_w), _ptr(ln_in_b),
            _ptr(ln_out_w), _ptr(ln_out_b), _ptr(w_z), _ptr(w_g), n, n, ldn, int(add_residual), eps, st)
    return z_out


def triangle_attention(z_in: torch.Tensor, z_out: torch.Tensor, mask: Optional[torch.Tensor], ln_w, ln_b, w_bias,
                       w_q, w_k, w_v, w_g, w_o, ending: bool, add_residual: bool, eps: float = 1e-5,
                       inf: float = 1e9, zn: Optional[torch.Tensor] = None) -> torch.Tensor:
    """zn: as for triangle_multiplication."""
    n = _check_pair(z_in, "z_in")
    if _check_pair(z_out, "z_out") != n or z_out.dtype != z_in.dtype:
        raise RuntimeError("z_out must match z_in in shape and dtype")
    mask = _check_mask(mask, n)
    _check_v(ln_w, C_Z, "ln_w")
    _check_v(ln_b, C_Z, "ln_b")
    zf = _zfmt(z_in)
    w_bias = _w(w_bias, zf, (N_HEAD_PAIR, C_Z), "w_bias")
    w_q, w_k, w_v, w_g = (_w(w, zf, (C_Z, C_Z), nm) for w, nm in ((w_q, "w_q"), (w_k, "w_k"), (w_v, "w_v"), (w_g, "w_g")))
    w_o = _w(w_o, F16, (C_Z, C_Z), "w_o")
    lib = _lib.load()
    ws = workspace(z_in.device, lib.px_triatt_workspace_bytes(n))
    ldn = lib.px_ld_mask(n)
    al = lambda nb: (nb + 255) // 256 * 256
    qkv = al(n * N_HEAD_PAIR * lib.px_ld(n) * D_HEAD_PAIR * 2)   # v is [n][4][32][ld(n)], q and k fit as well
    q = ws.data_ptr()
    k, v, o = q + qkv, q + 2 * qkv, q + 3 * qkv
    bias = o + al(n * n * C_Z * 2)
    mbias = bias + al(N_HEAD_PAIR * n * ldn * 4)
    flags = mbias + al(n * ldn * 4)
    dt, st, eps = _pair_dtype(z_in), _stream(z_in), float(eps)
    rows, rows_dt = _ptr(z_in), dt
    zn = _zn_arg(z_in, zn)
    if dt == PX_F32:            # the projection and the output stage normalise the same z: one standardised copy
        if zn is None:
            zn = flags + al(lib.px_triatt_flash_scratch_bytes(n, n))
            _launch("px_standardise_rows", lib.px_standardise_rows, _ptr(z_in), zn, n * n, eps, st)
        rows, rows_dt = zn, PX_F16
    _launch("px_triatt_in_proj", lib.px_triatt_in_proj, rows, rows_dt, _ptr(mask), _ptr(ln_w), _ptr(ln_b),
            _ptr(w_q), _ptr(w_k), _ptr(w_v), _ptr(w_bias), q, k, v, bias, mbias, n, n, ldn, int(ending), eps,
            float(inf), st)
    _launch("px_triatt_flash", lib.px_triatt_flash, q, k, v, bias, mbias, o, flags, n, n, ldn, st)
    _launch("px_triatt_out", lib.px_triatt_out, o, _ptr(z_in), zn, _ptr(z_out), dt, _ptr(ln_w), _ptr(ln_b), _ptr(w_g),
            _ptr(w_o), n, n, int(ending), int(add_residual), eps, st)
    return z_out


def transition(x_in: torch.Tensor, x_out: torch.Tensor, ln_w, ln_b, w_a, w_b, w_o, add_residual: bool,
               eps: float = 1e-5) -> torch.Tensor:
    _need_cuda(x_in, "x_in")
    _need_cuda(x_out, "x_out")
    if x_in.shape[-1] != C_Z or x_out.shape != x_in.shape or x_out.dtype != x_in.dtype:
        raise RuntimeError(f"transition kernel handles [..., {C_Z}] rows with matching output")
    _check_v(ln_w, C_Z, "ln_w")
    _check_v(ln_b, C_Z, "ln_b")
    w_a = _w(w_a, F16, (4 * C_Z, C_Z), "w_a")
    w_b = _w(w_b, F16, (4 * C_Z, C_Z), "w_b")
    w_o = _w(w_o, F16, (C_Z, 4 * C_Z), "w_o")
    rows = x_in.numel() // C_Z
    _launch("px_transition", _lib.load().px_transition, _ptr(x_in), _ptr(x_out), _pair_dtype(x_in), _ptr(ln_w),
            _ptr(ln_b), _ptr(w_a), _ptr(w_b), _ptr(w_o), rows, int(add_residual), float(eps), _stream(x_in))
    return x_out


def pair_bias_proj(z: torch.Tensor, ln_w, ln_b: Optional[torch.Tensor], w: torch.Tensor, eps: float = 1e-5,
                   zn: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bias[h, i, j] = (W LN(z[i, j]))[h] in fp32, for the single-representation attention.  zn: the standardised
    copy of an fp32 z when the caller has it."""
    n = _check_pair(z)
    _check_v(ln_w, C_Z, "ln_w")
    if ln_b is not None:
        _check_v(ln_b, C_Z, "ln_b")
    heads = w.shape[0]
    w = _w(w, _zfmt(z), (heads, C_Z), "w")
    out = torch.empty(heads, n, n, dtype=torch.float32, device=z.device)
    rows, rows_dt = _rows_of(z, zn, eps)
    _launch("px_pair_bias_proj", _lib.load().px_pair_bias_proj, _ptr(rows), rows_dt, _ptr(ln_w), _ptr(ln_b),
            _ptr(w), _ptr(out), n * n, heads, float(eps), _stream(z))
    return out


def recycle_update(z: torch.Tensor, z_init: torch.Tensor, ln_w, ln_b: Optional[torch.Tensor], w: torch.Tensor,
                   eps: float = 1e-5, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = z_init + W LN(z) over rows of 128 channels (any leading shape; `out` may be z or z_init)."""
    _need_cuda(z, "z")
    _need_cuda(z_init, "z_init")
    if z.shape != z_init.shape or z.dtype != z_init.dtype or z.shape[-1] != C_Z:
        raise RuntimeError("z and z_init must have the same shape [..., 128] and dtype")
    if not (z.is_contiguous() and z_init.is_contiguous()):
        raise RuntimeError("z and z_init must be contiguous")
    _check_v(ln_w, C_Z, "ln_w")
    if ln_b is not None:
        _check_v(ln_b, C_Z, "ln_b")
    w = _w(w, _zfmt(z), (C_Z, C_Z), "w")
    if out is None:
        out = torch.empty_like(z)
    elif out.shape != z.shape or out.dtype != z.dtype or not out.is_contiguous():
        raise RuntimeError("out must match z")
    rows = z.numel() // C_Z
    if rows == 0:
        return out
    zdt = _pair_dtype(z)
    z, _ = _rows_of(z, None, eps)          # an fp32 z enters as its standardised fp16 copy
    _launch("px_recycle_update", _lib.load().px_recycle_update, _ptr(z), _ptr(z_init), _ptr(out), zdt,
            _ptr(ln_w), _ptr(ln_b), _ptr(w), rows, float(eps), _stream(z))
    return out


OPM_X_BYTES = 2 << 30      # bound of the outer-product buffer of outer_product_mean


def outer_product_mean(z_in: Optional[torch.Tensor], z_out: torch.Tensor, m: torch.Tensor,
                       msa_mask: Optional[torch.Tensor], ln_w, ln_b, w_1, w_2, w_out, b_out, eps: float = 1e-3,
                       ln_eps: float = 1e-5) -> torch.Tensor:
    """z_out = [z_in +] OuterProductMean(m): m [S, N, c_m] (fp32 or bf16), msa_mask [S, N] or None, w_1 / w_2
    [32, c_m], w_out [128, 1024], b_out [128]; z [N, N, 128] fp32 or bf16.  The S*N-sized preparation (LayerNorm
    kernel, the two small projections on the library GEMM, mask, transposition to [(i, c)][s] in fp16) happens here;
    the outer product and the output projection are the tcgen05 kernels."""
    _need_cuda(m, "m")
    if m.dim() != 3 or not m.is_contiguous():
        raise RuntimeError("m must be a contiguous [N_seq, N_res, c_m] tensor")
    s_rows, n, c_m = m.shape
    if tuple(w_1.shape) != (32, c_m) or tuple(w_2.shape) != (32, c_m) or tuple(w_out.shape) != (C_Z, 1024) or \
            tuple(b_out.shape) != (C_Z,):
        raise RuntimeError("outer_product_mean kernels are built for c_hidden = 32 and c_z = 128")
    if n > 32768 or n < 1 or s_rows < 1:
        raise RuntimeError("outer_product_mean supports 1 <= N <= 32768 tokens")
    if _check_pair(z_out, "z_out") != n or (z_in is not None and (z_in.shape != z_out.shape or z_in.dtype != z_out.dtype)):
        raise RuntimeError("z must be [N, N, 128] with N = m.shape[1]")
    if not z_out.is_contiguous() or (z_in is not None and not z_in.is_contiguous()):
        raise RuntimeError("z must be contiguous")
    dev = m.device
    if msa_mask is None:
        mask = torch.ones(s_rows, n, dtype=torch.float32, device=dev)
    else:
        _need_cuda(msa_mask, "msa_mask")
        if tuple(msa_mask.shape) != (s_rows, n):
            raise RuntimeError("msa_mask must be [N_seq, N_res]")
        mask = msa_mask.to(torch.float32)
    ln = layer_norm(m, ln_w.detach().to(m.dtype), None if ln_b is None else ln_b.detach().to(m.dtype), ln_eps)
    w12 = torch.cat([w_1.detach(), w_2.detach()], 0).float()
    ab = (ln.float().view(s_rows * n, c_m) @ w12.t()).view(s_rows, n, 64) * mask[..., None]
    ld_k = (s_rows + 7) // 8 * 8
    a_t = torch.zeros(n * 32, ld_k, dtype=torch.float16, device=dev)
    b_t = torch.zeros(n * 32, ld_k, dtype=torch.float16, device=dev)
    a_t[:, :s_rows] = ab[..., :32].permute(1, 2, 0).reshape(n * 32, s_rows)
    b_t[:, :s_rows] = ab[..., 32:].permute(1, 2, 0).reshape(n * 32, s_rows)
    inv_norm = torch.reciprocal(mask.t() @ mask + eps).contiguous()
    # blocks of rows i bound the size of x = [32 n_i][32 N] fp16 (OPM_X_BYTES, 2 GiB by default)
    n_blk = max(1, min(n, OPM_X_BYTES // (2048 * n)))
    x = torch.empty(min(n, n_blk) * 32, n * 32, dtype=torch.float16, device=dev)
    lib, st = _lib.load(), _stream(m)
    b32 = b_out.detach().float().contiguous()
    w16 = _w(w_out, F16, (C_Z, 1024), "w_out")
    zb = z_out.element_size() * n * C_Z                # bytes of one row i of z
    for i0 in range(0, n, n_blk):
        ni = min(n_blk, n - i0)
        _launch("px_opm_outer", lib.px_opm_outer, a_t.data_ptr() + i0 * 32 * ld_k * 2, _ptr(b_t), _ptr(x), ni * 32, n * 32,
                ld_k, st)
        _launch("px_opm_out", lib.px_opm_out, _ptr(x), _ptr(w16), _ptr(b32), inv_norm.data_ptr() + i0 * n * 4,
                None if z_in is None else z_in.data_ptr() + i0 * zb, z_out.data_ptr() + i0 * zb, _pair_dtype(z_out), ni, n,
                int(z_in is not None), st)
    return z_out


# ---------------------------------------------------------------------------------------------
# Stage-level calls on rectangular slabs (row-sharded pair tensor).  Outputs are allocated here.
def _slab(z: torch.Tensor, name: str = "z") -> Tuple[int, int]:
    _need_cuda(z, name)
    if z.dim() != 3 or z.shape[2] != C_Z:
        raise RuntimeError(f"{name} must have shape [rows, cols, {C_Z}], got {tuple(z.shape)}")
    return z.shape[0], z.shape[1]


def trimul_in_proj(z: torch.Tensor, mask: Optional[torch.Tensor], ln_w, ln_b, w_ap, w_ag, w_bp, w_bg,
                   incoming: bool, eps: float = 1e-5, zn: Optional[torch.Tensor] = None
                   ) -> Tuple[torch.Tensor, torch.Tensor]:
    """a, b as [128][n_u][ld(n_t)] fp16.  z is [n_u][n_t][128]; with ``incoming`` it is [n_t][n_u][128]."""
    r, c = _slab(z)
    n_u, n_t = (c, r) if incoming else (r, c)
    lib = _lib.load()
    ldt = lib.px_ld(n_t)
    zf = _zfmt(z)
    w_ap, w_ag, w_bp, w_bg = (_w(w, zf, (C_Z, C_Z), "w") for w in (w_ap, w_ag, w_bp, w_bg))
    a = torch.empty(C_Z, n_u, ldt, dtype=torch.float16, device=z.device)
    b = torch.empty_like(a)
    rows, rows_dt = _rows_of(z, zn, eps)
    _launch("px_trimul_in_proj", lib.px_trimul_in_proj, _ptr(rows), rows_dt, _ptr(mask), _ptr(ln_w), _ptr(ln_b),
            _ptr(w_ap), _ptr(w_ag), _ptr(w_bp), _ptr(w_bg), _ptr(a), _ptr(b), n_u, n_t, ldt, int(incoming), float(eps),
            _stream(z))
    return a, b


def trimul_contract(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """x[c][i][j] = X_SCALE * sum_k a[c][i][k] b[c][j][k] for [C][n][ld] fp16 operands (pad columns zero)."""
    _need_cuda(a, "a")
    _need_cuda(b, "b")
    ch, n, ldn = a.shape
    if a.dtype != torch.float16 or b.shape != a.shape or b.dtype != a.dtype or ldn != ld(n):
        raise RuntimeError("contraction operands must be float16 [C][n][ld(n)] of equal shape")
    x = torch.empty_like(a)
    _launch("px_trimul_contract", _lib.load().px_trimul_contract, _ptr(a), _ptr(b), _ptr(x), ch, n, ldn, _stream(a))
    return x


def trimul_out(x: torch.Tensor, z: torch.Tensor, ln_in_w, ln_in_b, ln_out_w, ln_out_b, w_z, w_g,
               eps: float = 1e-5, zn: Optional[torch.Tensor] = None) -> torch.Tensor:
    """z[n_i][n_j] += W_z LN(x) * sigmoid(W_g LN(z)) in place; x is [128][n_i][ld(n_j)]."""
    n_i, n_j = _slab(z)
    _need_cuda(x, "x")
    if x.dtype != torch.float16 or x.dim() != 3 or x.shape[0] != C_Z or x.shape[1] != n_i or x.shape[2] != ld(n_j):
        raise RuntimeError("x must be float16 [128][n_i][ld(n_j)]")
    w_z, w_g = _w(w_z, F16, (C_Z, C_Z), "w_z"), _w(w_g, _zfmt(z), (C_Z, C_Z), "w_g")
    zn = _rows_of(z, zn, eps)[0] if z.dtype == torch.float32 else None
    _launch("px_trimul_out", _lib.load().px_trimul_out, _ptr(x), _ptr(z), _ptr(zn), _ptr(z), _pair_dtype(z), _ptr(ln_in_w),
            _ptr(ln_in_b), _ptr(ln_out_w), _ptr(ln_out_b), _ptr(w_z), _ptr(w_g), n_i, n_j, x.shape[2], 1, float(eps),
            _stream(z))
    return z


def triatt_in_proj(z: torch.Tensor, mask: Optional[torch.Tensor], ln_w, ln_b, w_bias, w_q, w_k, w_v,
                   eps: float = 1e-5, inf: float = 1e9, ending: bool = False, zn: Optional[torch.Tensor] = None):
    """q, k [n_u][4][n_t][32] and v (transposed) [n_u][4][32][ld(n_t)] in fp16, bias [4][n_u][ldm] and
    mask_bias [n_u][ldm] in fp32 for a slab.  z (and the mask) is [n_u][n_t][128]; with ``ending`` it is the
    column slab [n_t][n_u][128] and the attended rows u are its columns."""
    n_u, n_t = _slab(z)
    if ending:
        n_u, n_t = n_t, n_u
    lib = _lib.load()
    ldm = lib.px_ld_mask(n_t)
    zf = _zfmt(z)
    w_bias = _w(w_bias, zf, (N_HEAD_PAIR, C_Z), "w_bias")
    w_q, w_k, w_v = (_w(w, zf, (C_Z, C_Z), "w") for w in (w_q, w_k, w_v))
    q = torch.empty(n_u, N_HEAD_PAIR, n_t, D_HEAD_PAIR, dtype=torch.float16, device=z.device)
    k = torch.empty_like(q)
    v = torch.empty(n_u, N_HEAD_PAIR, D_HEAD_PAIR, lib.px_ld(n_t), dtype=torch.float16, device=z.device)
    bias = torch.empty(N_HEAD_PAIR, n_u, ldm, dtype=torch.float32, device=z.device)
    mb = torch.empty(n_u, ldm, dtype=torch.float32, device=z.device)
    rows, rows_dt = _rows_of(z, zn, eps)
    _launch("px_triatt_in_proj", lib.px_triatt_in_proj, _ptr(rows), rows_dt, _ptr(mask), _ptr(ln_w), _ptr(ln_b),
            _ptr(w_q), _ptr(w_k), _ptr(w_v), _ptr(w_bias), _ptr(q), _ptr(k), _ptr(v), _ptr(bias), _ptr(mb), n_u, n_t,
            ldm, int(ending), float(eps), float(inf), _stream(z))
    return q, k, v, bias, mb


def triatt_flash(q, k, v, bias_full: torch.Tensor, mb) -> torch.Tensor:
    """o [n_u][n][128] fp16 from q,k,v [n_u][4][n][32] (fp16), the full pair bias [4][n][ldm] and mask_bias
    [n_u][ldm] (fp32)."""
    n_u, _, n, _ = q.shape
    for t, nm in ((q, "q"), (k, "k"), (v, "v"), (bias_full, "bias"), (mb, "mask_bias")):
        _need_cuda(t, nm)
    ldm = bias_full.shape[2]
    if tuple(bias_full.shape) != (N_HEAD_PAIR, n, ldm) or tuple(mb.shape) != (n_u, ldm):
        raise RuntimeError("pair bias must be [4][n][ldm] and mask_bias [n_u][ldm]")
    if any(t.dtype != torch.float16 for t in (q, k, v)) or bias_full.dtype != torch.float32 or mb.dtype != torch.float32:
        raise RuntimeError("q, k, v must be float16, the pair bias and mask_bias float32")
    o = torch.empty(n_u, n, C_Z, dtype=torch.float16, device=q.device)
    lib = _lib.load()
    scratch = torch.empty(int(lib.px_triatt_flash_scratch_bytes(n_u, n)), dtype=torch.uint8, device=q.device)
    _launch("px_triatt_flash", lib.px_triatt_flash, _ptr(q), _ptr(k), _ptr(v), _ptr(bias_full), _ptr(mb), _ptr(o),
            _ptr(scratch), n_u, n, ldm, _stream(q))
    return o


def triatt_out(o: torch.Tensor, z: torch.Tensor, ln_w, ln_b, w_g, w_o, eps: float = 1e-5, ending: bool = False,
               zn: Optional[torch.Tensor] = None, update_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """z(u,t) += W_o(o[u][t] * sigmoid(W_g LN(z(u,t)))) in place; z is [n_u][n_t][128], or the column slab
    [n_t][n_u][128] with ``ending``.  With a float16 ``z`` (the standardised copy of rows that live elsewhere) the
    update alone is written, in fp16, to ``update_out`` (same layout as z), which is returned."""
    n_u, n_t = _slab(z)
    if ending:
        n_u, n_t = n_t, n_u
    _need_cuda(o, "o")
    if o.dtype != torch.float16 or tuple(o.shape) != (n_u, n_t, C_Z):
        raise RuntimeError("o must be float16 [n_u][n_t][128]")
    if z.dtype == torch.float16:            # update only, from standardised rows
        w_g, w_o = _w(w_g, F16, (C_Z, C_Z), "w_g"), _w(w_o, F16, (C_Z, C_Z), "w_o")
        if update_out is None:
            update_out = torch.empty_like(z)
        elif update_out.dtype != torch.float16 or update_out.shape != z.shape or not update_out.is_contiguous():
            raise RuntimeError("update_out must be a contiguous float16 tensor of z's shape")
        _launch("px_triatt_out", _lib.load().px_triatt_out, _ptr(o), _ptr(z), None, _ptr(update_out), PX_F16, _ptr(ln_w),
                _ptr(ln_b), _ptr(w_g), _ptr(w_o), n_u, n_t, int(ending), 0, float(eps), _stream(z))
        return update_out
    w_g, w_o = _w(w_g, _zfmt(z), (C_Z, C_Z), "w_g"), _w(w_o, F16, (C_Z, C_Z), "w_o")
    zn = _rows_of(z, zn, eps)[0] if z.dtype == torch.float32 else None
    _launch("px_triatt_out", _lib.load().px_triatt_out, _ptr(o), _ptr(z), _ptr(zn), _ptr(z), _pair_dtype(z), _ptr(ln_w),
            _ptr(ln_b), _ptr(w_g), _ptr(w_o), n_u, n_t, int(ending), 1, float(eps), _stream(z))
    return z


def pair_bias_rows(z: torch.Tensor, ln_w, ln_b: Optional[torch.Tensor], w: torch.Tensor, eps: float = 1e-5,
                   zn: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bias[h, u, t] for a row slab z [n_u][n_t][128].  zn: the standardised copy of an fp32 slab, if at hand."""
    n_u, n_t = _slab(z)
    heads = w.shape[0]
    w = _w(w, _zfmt(z), (heads, C_Z), "w")
    out = torch.empty(heads, n_u, n_t, dtype=torch.float32, device=z.device)
    rows, rows_dt = _rows_of(z, zn, eps)
    _launch("px_pair_bias_proj", _lib.load().px_pair_bias_proj, _ptr(rows), rows_dt, _ptr(ln_w), _ptr(ln_b),
            _ptr(w), _ptr(out), n_u * n_t, heads, float(eps), _stream(z))
    return out


def transition_rows(x: torch.Tensor, ln_w, ln_b, w_a, w_b, w_o, eps: float = 1e-5,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = x + Transition(x) for any [..., 128] slab; in place when ``out`` is None."""
    _need_cuda(x, "x")
    if out is None:
        out = x
    else:
        _need_cuda(out, "out")
        if out.shape != x.shape or out.dtype != x.dtype:
            raise RuntimeError("out must match x")
    w_a, w_b = _w(w_a, F16, (4 * C_Z, C_Z), "w_a"), _w(w_b, F16, (4 * C_Z, C_Z), "w_b")
    w_o = _w(w_o, F16, (C_Z, 4 * C_Z), "w_o")
    _launch("px_transition", _lib.load().px_transition, _ptr(x), _ptr(out), _pair_dtype(x), _ptr(ln_w), _ptr(ln_b),
            _ptr(w_a), _ptr(w_b), _ptr(w_o), x.numel() // C_Z, 1, float(eps), _stream(x))
    return out


# ---------------------------------------------------------------------------------------------
# Buffers other GPUs of the box can write into (row-sharded path) and the strided copy that fills them.
class PeerBuffer:
    """A cudaMalloc allocation of this process together with the handle other processes open it by."""

    def __init__(self, nbytes: int, device: torch.device) -> None:
        import ctypes

        self.nbytes, self.device = int(nbytes), device
        ptr, handle = ctypes.c_void_p(), (ctypes.c_ubyte * 64)()
        with torch.cuda.device(device):
            _lib.check(_lib.load().px_peer_alloc(self.nbytes, ctypes.byref(ptr), handle), "px_peer_alloc")
        self.ptr, self.handle = int(ptr.value), bytes(handle)

    def tensor(self, shape, dtype: torch.dtype, offset_bytes: int = 0) -> torch.Tensor:
        """A tensor over (a part of) the buffer; it does not own the memory."""
        numel = 1
        for d in shape:
            numel *= int(d)
        item = torch.empty(0, dtype=dtype).element_size()
        if offset_bytes + numel * item > self.nbytes:
            raise RuntimeError("peer buffer too small for the requested view")
        typestr = {torch.bfloat16: "<u2", torch.float16: "<f2", torch.float32: "<f4", torch.uint8: "|u1"}[dtype]

        class _View:
            pass

        v = _View()
        v.__cuda_array_interface__ = {"shape": (numel,), "typestr": typestr, "data": (self.ptr + offset_bytes, False),
                                      "version": 3}
        t = torch.as_tensor(v, device=self.device)
        if dtype == torch.bfloat16:
            t = t.view(torch.bfloat16)
        return t.view(*shape)

    def free(self) -> None:
        if self.ptr:
            _lib.load().px_peer_free(self.ptr)
            self.ptr = 0


def peer_open(handle: bytes, device: torch.device) -> int:
    """Opens another process's PeerBuffer; returns its address in this process."""
    import ctypes

    ptr, buf = ctypes.c_void_p(), (ctypes.c_ubyte * 64).from_buffer_copy(handle)
    with torch.cuda.device(device):
        _lib.check(_lib.load().px_peer_open(buf, ctypes.byref(ptr)), "px_peer_open")
    return int(ptr.value)


def peer_close(ptr: int) -> None:
    _lib.load().px_peer_close(ptr)


def peer_barrier(flag_ptrs, rank: int, world: int, epoch: int, device: torch.device) -> None:
    """Stream-ordered barrier between the ranks of a box through flags in peer memory (one small kernel per rank)."""
    import ctypes

    arr = (ctypes.c_void_p * world)(*[int(p) for p in flag_ptrs])
    _launch("px_peer_barrier", _lib.load().px_peer_barrier, arr, int(rank), int(world), int(epoch) & 0xFFFFFFFF,
            torch.cuda.current_stream(device).cuda_stream)


def copy_2d(dst_ptr: int, dpitch: int, src: torch.Tensor, src_offset_bytes: int, spitch: int, width_bytes: int,
            height: int) -> None:
    """height rows of width_bytes from src (+offset) to the raw address dst_ptr, on src's current stream."""
    _launch("px_copy_2d", _lib.load().px_copy_2d, dst_ptr, int(dpitch), src.data_ptr() + int(src_offset_bytes),
            int(spitch), int(width_bytes), int(height), _stream(src))


DMA_MIN_WIDTH = 16384     # rows at least this wide go to the copy engines, narrower ones to the copy kernel


def copy_2d_batch(dst_ptrs, src: torch.Tensor, src_offsets, dpitch: int, spitch: int, width_bytes: int, height: int) -> None:
    """For every i, height rows of width_bytes from src (+src_offsets[i]) to the raw address dst_ptrs[i], on src's
    current stream, in one launch of the copy kernel (measured at about 590 GB/s per direction between two B200s).
    ``PX_PEER_DMA=1`` sends wide rows through the copy engines instead (one pitched transfer per destination, no SM
    involved; measured at about 280 GB/s, which is why it is not the default)."""
    import ctypes

    n = len(dst_ptrs)
    if width_bytes >= DMA_MIN_WIDTH and os.environ.get("PX_PEER_DMA", "0") == "1":
        lib, st = _lib.load(), _stream(src)
        for d, o in zip(dst_ptrs, src_offsets):
            _launch("px_copy_2d_dma", lib.px_copy_2d_dma, int(d), int(dpitch), src.data_ptr() + int(o), int(spitch),
                    int(width_bytes), int(height), st)
        return
    d = (ctypes.c_void_p * n)(*[int(p) for p in dst_ptrs])
    s_ = (ctypes.c_void_p * n)(*[src.data_ptr() + int(o) for o in src_offsets])
    _launch("px_copy_2d_batch", _lib.load().px_copy_2d_batch, d, s_, n, int(dpitch), int(spitch), int(width_bytes),
            int(height), _stream(src))
