"""Deterministic parameter randomisation for tests and benchmarks.

With the reference's own initialisers every residual branch of a Pairformer block ends in a
zero-initialised projection (protenix/model/triangular/layers.py:90-97 "final"/"gating";
protenix/model/modules/primitives.py:72-73 "zeros"), so a freshly constructed block is the
identity.  Parity and throughput are therefore evaluated on re-drawn parameters.  The draw
depends only on (seed, parameter name, shape), so the same call applied to the reference's
modules and to this package's modules (identical ``state_dict`` keys) yields identical bits.
"""
from __future__ import annotations

import zlib

import torch


def _gen_for(seed: int, name: str) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed((seed * 1000003 + zlib.crc32(name.encode())) % (2 ** 63))
    return g


@torch.no_grad()
def randomize_parameters_(module: torch.nn.Module, seed: int = 1, out_scale: float = 1.0) -> torch.nn.Module:
    """Re-draw every parameter of ``module`` in place.

    * 2-D weights: N(0, 1/fan_in); projections that close a residual branch
      (``linear_z``, ``linear_o``, ``linear_no_bias``) are further scaled by ``out_scale``.
    * 1-D ``*.weight`` (LayerNorm scale): 1 + 0.1 N(0,1).
    * 1-D ``*.bias``: 0.1 N(0,1).
    Values are drawn on the CPU in fp32 and copied to the parameter's device / dtype.
    """
    closing = ("linear_z.weight", "linear_o.weight", "linear_no_bias.weight")
    for name, p in sorted(module.named_parameters(), key=lambda kv: kv[0]):
        g = _gen_for(seed, name)
        r = torch.randn(p.shape, generator=g, dtype=torch.float32)
        if p.dim() == 2:
            r = r * (1.0 / p.shape[1]) ** 0.5
            if name.endswith(closing):
                r = r * out_scale
        elif name.endswith("weight"):
            r = 1.0 + 0.1 * r
        else:
            r = 0.1 * r
        p.copy_(r.to(device=p.device, dtype=p.dtype))
    return module
