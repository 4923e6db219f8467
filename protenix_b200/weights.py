"""16-bit copies of fp32 parameters, cached until the parameter changes.

The kernels consume 16-bit weight matrices: bf16 where the weight multiplies rows of a bf16 pair tensor, fp16
where it multiplies fp16 operands (rows of an fp32 pair tensor, which the kernels standardise and round to fp16,
and every intermediate tensor).  The modules keep fp32 parameters with the reference's names so that its
checkpoints load with ``strict=True``.  A cached copy is keyed on the parameter's storage pointer, device, in-place
version counter and the wanted format, so ``load_state_dict``, ``.to()`` and optimiser steps all invalidate it.
"""
from __future__ import annotations

import weakref
from typing import Dict, Tuple

import torch

_cache: Dict[Tuple[int, torch.dtype], Tuple[Tuple, torch.Tensor, "weakref.ref"]] = {}


def w16_of(p: torch.Tensor, fmt: torch.dtype) -> torch.Tensor:
    """``p`` as a contiguous tensor of the 16-bit format ``fmt`` (``torch.bfloat16`` or ``torch.float16``)."""
    if p.dtype == fmt and p.is_contiguous() and not p.requires_grad:
        return p
    key = (p.data_ptr(), p._version, p.device, tuple(p.shape), p.dtype)
    ent = _cache.get((id(p), fmt))
    if ent is not None and ent[0] == key and ent[2]() is p:
        return ent[1]
    w = p.detach().to(fmt).contiguous()
    ck = (id(p), fmt)
    _cache[ck] = (key, w, weakref.ref(p, lambda _r, ck=ck: _cache.pop(ck, None)))
    return w


def bf16_of(p: torch.Tensor) -> torch.Tensor:
    return w16_of(p, torch.bfloat16)


def f16_of(p: torch.Tensor) -> torch.Tensor:
    return w16_of(p, torch.float16)


def clear() -> None:
    _cache.clear()
