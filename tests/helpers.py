"""Shared helpers: build modules with seeded weights and hand the same weights to the oracle."""
from __future__ import annotations

import os

import numpy as np
import torch

import protenix_b200 as px
from protenix_b200.init_utils import randomize_parameters_

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "pairformer_golden.npz")


def golden():
    return np.load(GOLDEN)


def build_module(kind: str, case: dict) -> torch.nn.Module:
    """The package's module for a golden-case kind, parameters drawn from the case's weight seed."""
    if kind == "block":
        m = px.PairformerBlock(c_s=case["c_s"])
    elif kind == "stack":
        m = px.PairformerStack(n_blocks=case["n_blocks"], c_s=case["c_s"])
    elif kind == "tri_mul_out":
        m = px.TriangleMultiplicationOutgoing(c_z=128, c_hidden=128)
    elif kind == "tri_mul_in":
        m = px.TriangleMultiplicationIncoming(c_z=128, c_hidden=128)
    elif kind == "tri_att_start":
        m = px.TriangleAttention(c_in=128, c_hidden=32, no_heads=4, starting=True)
    elif kind == "tri_att_end":
        m = px.TriangleAttention(c_in=128, c_hidden=32, no_heads=4, starting=False)
    elif kind == "transition":
        m = px.Transition(c_in=case["c"], n=case["n"])
    elif kind == "layer_norm":
        m = px.LayerNorm(case["c"], create_scale=case["scale"], create_offset=case["offset"])
    elif kind == "opm":
        m = px.OuterProductMean(c_m=case.get("c_m", 64), c_z=128, c_hidden=case.get("c_hidden", 32))
    elif kind == "msa_block":
        from protenix_b200.msa import MSABlock
        m = MSABlock(c_m=case.get("c_m", 64), c_z=128, c_hidden=32, is_last_block=case.get("last", False))
    elif kind == "msa_module":
        from golden_cases import MSA_CONFIGS
        from protenix_b200.msa import MSAModule
        m = MSAModule(n_blocks=case["n_blocks"], c_s_inputs=case["c_s_inputs"], msa_configs=MSA_CONFIGS)
    elif kind == "trunk_msa":
        from golden_cases import MSA_CONFIGS
        m = px.RecyclingTrunk(n_blocks=case["n_blocks"], c_s=case["c_s"], N_cycle=case["n_cycle"],
                              msa_n_blocks=case["msa_n_blocks"], c_s_inputs=case["c_s_inputs"], msa_configs=MSA_CONFIGS)
    elif kind == "recycle":
        m = px.RecyclingTrunk(n_blocks=case["n_blocks"], c_s=case["c_s"], N_cycle=case["n_cycle"])
    else:
        raise ValueError(kind)
    randomize_parameters_(m, case["wseed"])
    return m.eval()


def params_of(module: torch.nn.Module, dtype=torch.float32) -> dict:
    return {k: v.detach().to("cpu", dtype) for k, v in module.state_dict().items()}


def relf(a, b) -> float:
    a = torch.as_tensor(np.asarray(a) if not torch.is_tensor(a) else a).double().cpu()
    b = torch.as_tensor(np.asarray(b) if not torch.is_tensor(b) else b).double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))
