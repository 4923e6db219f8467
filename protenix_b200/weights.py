"""bf16 copies of fp32 parameters, cached until the parameter changes.

The kernels consume bf16 weight matrices; the modules keep fp32 parameters with the
reference's names so that its checkpoints load with ``strict=True``.  A cached copy is keyed on
the parameter's storage pointer, device and in-place version counter, so ``load_state_dict``,
``.to()`` and optimiser steps all invalidate it.
"""
from __future__ import annotations

import weakref
from typing import Dict, Tuple

import torch

_cache: Dict[int, Tuple[Tuple, torch.Tensor, "weakref.ref"]] = {}


def bf16_of(p: torch.Tensor) -> torch.Tensor:
    key = (p.data_ptr(), p._version, p.device, tuple(p.shape), p.dtype)
    ent = _cache.get(id(p))
    if ent is not None and ent[0] == key and ent[2]() is p:
        return ent[1]
    w = p.detach().to(torch.bfloat16).contiguous()
    pid = id(p)
    _cache[pid] = (key, w, weakref.ref(p, lambda _r, pid=pid: _cache.pop(pid, None)))
    return w


def clear() -> None:
    _cache.clear()
