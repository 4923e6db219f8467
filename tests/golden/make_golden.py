"""Generate the golden vectors in this folder by running the reference itself on the CPU.

Usage (only where a checkout of bytedance/Protenix v2.0.0 is available):

    python tests/golden/make_golden.py --reference /path/to/Protenix

The reference's torch back-end is imported with two in-memory stand-ins for packages that
its hot path never really uses (``optree`` -> torch pytree, ``rdkit.Chem.GetPeriodicTable``)
and with ``LAYERNORM_TYPE=torch``.  Modules are built with the reference's constructors,
their parameters re-drawn by ``protenix_b200.init_utils.randomize_parameters_`` (a function of
seed, parameter name and shape only), and run in fp32 and eval mode.  Inputs are re-created
from the recorded seeds by ``golden_cases.py`` beside this script; only outputs are stored.
"""
from __future__ import annotations

import argparse
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))


def import_reference(path: str):
    os.environ["LAYERNORM_TYPE"] = "torch"
    sys.path.insert(0, path)
    import torch.utils._pytree as pt

    opt = types.ModuleType("optree")
    opt.tree_map = lambda f, tree: pt.tree_map(f, tree)
    opt.tree_flatten = lambda tree: pt.tree_flatten(tree)
    sys.modules["optree"] = opt
    rd = types.ModuleType("rdkit")
    ch = types.ModuleType("rdkit.Chem")

    class _Table:
        def GetElementSymbol(self, i):
            return f"E{i}"

    ch.GetPeriodicTable = lambda: _Table()
    rd.Chem = ch
    sys.modules["rdkit"] = rd
    sys.modules["rdkit.Chem"] = ch
    from protenix.model.modules import pairformer as ref_pf
    from protenix.model.modules import primitives as ref_prim
    from protenix.model.triangular import layers as ref_layers
    from protenix.model.triangular import triangular as ref_tri

    return ref_pf, ref_prim, ref_layers, ref_tri


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a bytedance/Protenix checkout")
    args = ap.parse_args()
    ref_pf, ref_prim, ref_layers, ref_tri = import_reference(args.reference)

    from protenix_b200.init_utils import randomize_parameters_
    sys.path.insert(0, HERE)
    from golden_cases import CASES, make_inputs

    torch.set_grad_enabled(False)
    out = {}
    for name, case in CASES.items():
        kind = case["kind"]
        inp = make_inputs(case)
        torch.manual_seed(0)
        np.random.seed(0)
        if kind == "block":
            mod = ref_pf.PairformerBlock(c_s=case["c_s"]).eval()
            randomize_parameters_(mod, case["wseed"])
            for inplace in (False, True):
                s, z = mod(inp["s"].clone() if inp["s"] is not None else None, inp["z"].clone(),
                           inp["mask"], inplace_safe=inplace)
                if not inplace:
                    out[name + ".z"] = z.numpy()
                    if s is not None:
                        out[name + ".s"] = s.numpy()
                else:  # the reference's in-place branch must agree with its functional one
                    assert np.abs(z.numpy() - out[name + ".z"]).max() <= 1e-4 * np.abs(out[name + ".z"]).max()
        elif kind == "stack":
            mod = ref_pf.PairformerStack(n_blocks=case["n_blocks"], c_s=case["c_s"]).eval()
            randomize_parameters_(mod, case["wseed"])
            s, z = mod(inp["s"], inp["z"], inp["mask"])
            out[name + ".z"] = z.numpy()
            out[name + ".s"] = s.numpy()
        elif kind in ("tri_mul_out", "tri_mul_in"):
            cls = ref_tri.TriangleMultiplicationOutgoing if kind == "tri_mul_out" else ref_tri.TriangleMultiplicationIncoming
            mod = cls(c_z=128, c_hidden=128).eval()
            randomize_parameters_(mod, case["wseed"])
            out[name + ".y"] = mod(inp["z"], mask=inp["mask"]).numpy()
        elif kind in ("tri_att_start", "tri_att_end"):
            mod = ref_tri.TriangleAttention(c_in=128, c_hidden=32, no_heads=4, starting=(kind == "tri_att_start")).eval()
            randomize_parameters_(mod, case["wseed"])
            out[name + ".y"] = mod(inp["z"], mask=inp["mask"]).numpy()
        elif kind == "transition":
            mod = ref_prim.Transition(c_in=case["c"], n=case["n"]).eval()
            randomize_parameters_(mod, case["wseed"])
            out[name + ".y"] = mod(inp["x"]).numpy()
        elif kind == "layer_norm":
            mod = ref_layers.LayerNorm(case["c"], create_scale=case["scale"], create_offset=case["offset"]).eval()
            randomize_parameters_(mod, case["wseed"])
            out[name + ".y"] = mod(inp["x"]).numpy()
        elif kind == "recycle":
            # the recycling loop of Protenix.get_pairformer_output (protenix/model/protenix.py:230-296) with the
            # reference's own layers, template embedder and MSA module left out
            class Trunk(torch.nn.Module):
                def __init__(self):
                    super().__init__()
                    self.linear_no_bias_z_cycle = ref_prim.LinearNoBias(in_features=128, out_features=128)
                    self.linear_no_bias_s = ref_prim.LinearNoBias(in_features=case["c_s"], out_features=case["c_s"])
                    self.layernorm_z_cycle = ref_layers.LayerNorm(128)
                    self.layernorm_s = ref_layers.LayerNorm(case["c_s"])
                    self.pairformer_stack = ref_pf.PairformerStack(n_blocks=case["n_blocks"], c_s=case["c_s"])

            mod = Trunk().eval()
            randomize_parameters_(mod, case["wseed"])
            z, s = torch.zeros_like(inp["z"]), torch.zeros_like(inp["s"])
            for _ in range(case["n_cycle"]):
                z = inp["z"] + mod.linear_no_bias_z_cycle(mod.layernorm_z_cycle(z))
                s = inp["s"] + mod.linear_no_bias_s(mod.layernorm_s(s))
                s, z = mod.pairformer_stack(s, z, pair_mask=inp["mask"])
            out[name + ".z"] = z.numpy()
            out[name + ".s"] = s.numpy()
        elif kind == "opm":
            mod = ref_layers.OuterProductMean(c_m=case["c_m"], c_z=128, c_hidden=case["c_hidden"]).eval()
            randomize_parameters_(mod, case["wseed"])
            out[name + ".y"] = mod(inp["m"], mask=inp["msa_mask"]).numpy()
        elif kind == "msa_block":
            mod = ref_pf.MSABlock(c_m=case["c_m"], c_z=128, c_hidden=32, is_last_block=case["last"]).eval()
            randomize_parameters_(mod, case["wseed"])
            m, z = mod(inp["m"].clone(), inp["z"].clone(), inp["mask"])
            out[name + ".z"] = z.numpy()
            if m is not None:
                out[name + ".m"] = m.numpy()
        elif kind == "msa_module":
            from golden_cases import MSA_CONFIGS

            mod = ref_pf.MSAModule(n_blocks=case["n_blocks"], c_s_inputs=case["c_s_inputs"], msa_configs=MSA_CONFIGS).eval()
            randomize_parameters_(mod, case["wseed"])
            feat = {k: inp[k] for k in ("msa", "has_deletion", "deletion_value")}
            out[name + ".z"] = mod(feat, inp["z"].clone(), inp["s_inputs"], inp["mask"]).numpy()
        elif kind == "trunk_msa":
            from golden_cases import MSA_CONFIGS

            class TrunkMsa(torch.nn.Module):        # protenix/model/protenix.py:230-296 without the template embedder
                def __init__(self):
                    super().__init__()
                    self.linear_no_bias_z_cycle = ref_prim.LinearNoBias(in_features=128, out_features=128)
                    self.linear_no_bias_s = ref_prim.LinearNoBias(in_features=case["c_s"], out_features=case["c_s"])
                    self.layernorm_z_cycle = ref_layers.LayerNorm(128)
                    self.layernorm_s = ref_layers.LayerNorm(case["c_s"])
                    self.pairformer_stack = ref_pf.PairformerStack(n_blocks=case["n_blocks"], c_s=case["c_s"])
                    self.msa_module = ref_pf.MSAModule(n_blocks=case["msa_n_blocks"], c_s_inputs=case["c_s_inputs"],
                                                       msa_configs=MSA_CONFIGS)

            mod = TrunkMsa().eval()
            randomize_parameters_(mod, case["wseed"])
            feat = {k: inp[k] for k in ("msa", "has_deletion", "deletion_value")}
            z, s = torch.zeros_like(inp["z"]), torch.zeros_like(inp["s"])
            for _ in range(case["n_cycle"]):
                z = inp["z"] + mod.linear_no_bias_z_cycle(mod.layernorm_z_cycle(z))
                z = mod.msa_module(feat, z, inp["s_inputs"], pair_mask=inp["mask"])
                s = inp["s"] + mod.linear_no_bias_s(mod.layernorm_s(s))
                s, z = mod.pairformer_stack(s, z, pair_mask=inp["mask"])
            out[name + ".z"] = z.numpy()
            out[name + ".s"] = s.numpy()
        else:
            raise ValueError(kind)
        print(name, {k: v.shape for k, v in out.items() if k.startswith(name + ".")})
    # state_dict layout of one reference block: the drop-in must load it with strict=True
    import json

    torch.manual_seed(0)
    np.random.seed(0)
    blk = ref_pf.PairformerBlock().eval()
    keys = {k: list(v.shape) for k, v in blk.state_dict().items()}
    with open(os.path.join(HERE, "block_state_dict_keys.json"), "w") as f:
        json.dump(keys, f, indent=0, sort_keys=True)
    torch.manual_seed(0)
    np.random.seed(0)
    msa = ref_pf.MSABlock().eval()
    with open(os.path.join(HERE, "msa_block_state_dict_keys.json"), "w") as f:
        json.dump({k: list(v.shape) for k, v in msa.state_dict().items()}, f, indent=0, sort_keys=True)
    from golden_cases import MSA_CONFIGS

    mm = ref_pf.MSAModule(n_blocks=2, msa_configs=MSA_CONFIGS).eval()
    with open(os.path.join(HERE, "msa_module_state_dict_keys.json"), "w") as f:
        json.dump({k: list(v.shape) for k, v in mm.state_dict().items()}, f, indent=0, sort_keys=True)
    path = os.path.join(HERE, "pairformer_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
