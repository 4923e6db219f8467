"""Seeded inputs shared by the golden-vector generator and the tests that consume them."""
from __future__ import annotations

import torch


def padding_mask(n: int, n_pad: int) -> torch.Tensor:
    """pair_mask = t t^T with the last ``n_pad`` tokens masked."""
    t = torch.ones(n)
    if n_pad:
        t[n - n_pad:] = 0
    return t[:, None] * t[None, :]


def random_mask(n: int, seed: int, p_drop: float = 0.2) -> torch.Tensor:
    """A general (non-separable) 0/1 pair mask; column 0 is kept so no row is fully masked."""
    g = torch.Generator().manual_seed(seed)
    m = (torch.rand(n, n, generator=g) > p_drop).float()
    m[:, 0] = 1
    m[0, :] = 1
    return m


CASES = {
    # whole block with the single-representation branch, padding mask
    "block_n24": dict(kind="block", n=24, c_s=384, seed=11, wseed=1, pad=3),
    # pair-only block (as embedded in the MSA module), no mask
    "block_pair_n20": dict(kind="block", n=20, c_s=0, seed=12, wseed=2, pad=0, no_mask=True),
    "stack2_n16": dict(kind="stack", n=16, c_s=384, n_blocks=2, seed=13, wseed=3, pad=2),
    "tri_mul_out_n20": dict(kind="tri_mul_out", n=20, seed=21, wseed=4, rand_mask=True),
    "tri_mul_in_n20": dict(kind="tri_mul_in", n=20, seed=22, wseed=5, rand_mask=True),
    "tri_att_start_n20": dict(kind="tri_att_start", n=20, seed=23, wseed=6, rand_mask=True),
    "tri_att_end_n20": dict(kind="tri_att_end", n=20, seed=24, wseed=7, rand_mask=True),
    "transition_pair": dict(kind="transition", rows=300, c=128, n=4, seed=31, wseed=8),
    "transition_single": dict(kind="transition", rows=50, c=384, n=4, seed=32, wseed=9),
    "ln_128_both": dict(kind="layer_norm", rows=200, c=128, scale=True, offset=True, seed=41, wseed=10),
    "ln_384_both": dict(kind="layer_norm", rows=64, c=384, scale=True, offset=True, seed=42, wseed=11),
    "ln_833_scale": dict(kind="layer_norm", rows=33, c=833, scale=True, offset=False, seed=43, wseed=12),
    "ln_64_none": dict(kind="layer_norm", rows=77, c=64, scale=False, offset=False, seed=44, wseed=13),
    # recycling loop around a 2-block stack: z, s are z_init, s_init
    "recycle_n16": dict(kind="recycle", n=16, c_s=384, n_blocks=2, n_cycle=3, seed=51, wseed=14, pad=2),
    # the MSA module's OuterProductMean: MSA embedding [n_msa, n, 64] -> pair update [n, n, 128]; random MSA mask
    "opm_n24": dict(kind="opm", n=24, n_msa=20, c_m=64, c_hidden=32, seed=61, wseed=15, p_drop=0.25),
    "opm_n40_nomask": dict(kind="opm", n=40, n_msa=9, c_m=64, c_hidden=32, seed=62, wseed=16, p_drop=0.0),
    # one block of the MSA module (outer product mean, MSA stack, pair-only Pairformer block), padding mask
    "msa_block_n20": dict(kind="msa_block", n=20, n_msa=12, c_m=64, seed=71, wseed=17, pad=3, last=False),
    "msa_block_last_n16": dict(kind="msa_block", n=16, n_msa=7, c_m=64, seed=72, wseed=18, pad=0, last=True),
    # the whole MSA module: feature embedding, 3 blocks (the last without an MSA stack); all MSA rows are used, in order
    "msa_module_n18": dict(kind="msa_module", n=18, n_msa=11, n_blocks=3, c_s_inputs=449, seed=81, wseed=19, pad=2),
    # the trunk's recycling loop with the MSA module inside: 2 cycles x (2 MSA blocks + 2 Pairformer blocks)
    "trunk_msa_n16": dict(kind="trunk_msa", n=16, n_msa=6, c_s=384, n_blocks=2, msa_n_blocks=2, n_cycle=2, c_s_inputs=449,
                          seed=91, wseed=20, pad=2),
}

# sampling made deterministic: the lower bound exceeds the number of rows, so all of them are taken, first to last
MSA_CONFIGS = {"enable": True, "strategy": "topk", "sample_cutoff": {"train": 512, "test": 16384},
               "min_size": {"train": 1, "test": 1 << 30}}


def make_inputs(case: dict) -> dict:
    g = torch.Generator().manual_seed(case["seed"])
    kind = case["kind"]
    if kind in ("transition", "layer_norm"):
        return {"x": torch.randn(case["rows"], case["c"], generator=g)}
    if kind == "opm":
        m = torch.randn(case["n_msa"], case["n"], case["c_m"], generator=g)
        mask = None
        if case["p_drop"] > 0:
            mask = (torch.rand(case["n_msa"], case["n"], generator=g) > case["p_drop"]).float()
            mask[0] = 1                                  # the query sequence is never masked
        return {"m": m, "msa_mask": mask}
    if kind in ("msa_module", "trunk_msa"):
        n, sr = case["n"], case["n_msa"]
        extra = {"s": torch.randn(n, case["c_s"], generator=g)} if kind == "trunk_msa" else {}
        return {**extra, "msa": torch.randint(0, 32, (sr, n), generator=g), "has_deletion": (torch.rand(sr, n, generator=g) > 0.8).float(),
                "deletion_value": torch.rand(sr, n, generator=g), "z": torch.randn(n, n, 128, generator=g),
                "s_inputs": torch.randn(n, case["c_s_inputs"], generator=g), "mask": padding_mask(n, case.get("pad", 0))}
    if kind == "msa_block":
        n = case["n"]
        return {"m": torch.randn(case["n_msa"], n, case["c_m"], generator=g), "z": torch.randn(n, n, 128, generator=g),
                "mask": padding_mask(n, case.get("pad", 0))}
    n = case["n"]
    z = torch.randn(n, n, 128, generator=g)
    s = torch.randn(n, case["c_s"], generator=g) if case.get("c_s", 0) > 0 else None
    if case.get("no_mask"):
        mask = None
    elif case.get("rand_mask"):
        mask = random_mask(n, case["seed"] + 1000)
    else:
        mask = padding_mask(n, case.get("pad", 0))
    return {"z": z, "s": s, "mask": mask}
