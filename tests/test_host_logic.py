"""Host-side behaviour that needs no GPU: state_dict layout, weight cache, error paths."""
import json
import os

import pytest
import torch

import protenix_b200 as px
from protenix_b200 import weights
from protenix_b200.init_utils import randomize_parameters_

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_block_state_dict_matches_reference_layout():
    ref = json.load(open(os.path.join(ROOT, "tests", "golden", "block_state_dict_keys.json")))
    mine = {k: list(v.shape) for k, v in px.PairformerBlock().state_dict().items()}
    assert mine == ref
    assert sum(p.numel() for p in px.PairformerBlock().parameters()) == 3070848


def test_msa_block_state_dict_matches_reference_layout():
    from protenix_b200.msa import MSABlock

    ref = json.load(open(os.path.join(ROOT, "tests", "golden", "msa_block_state_dict_keys.json")))
    assert {k: list(v.shape) for k, v in MSABlock().state_dict().items()} == ref
    last = MSABlock(is_last_block=True).state_dict()
    assert not any(k.startswith("msa_stack") for k in last) and "outer_product_mean_msa.linear_out.bias" in last


def test_msa_module_state_dict_matches_reference_layout():
    import sys
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    from golden_cases import MSA_CONFIGS
    from protenix_b200.msa import MSAModule

    ref = json.load(open(os.path.join(ROOT, "tests", "golden", "msa_module_state_dict_keys.json")))
    mod = MSAModule(n_blocks=2, msa_configs=MSA_CONFIGS)
    assert {k: list(v.shape) for k, v in mod.state_dict().items()} == ref
    assert mod.msa_configs["test_lowerb"] == 1 << 30 and mod.msa_max_size == 512
    with pytest.raises(RuntimeError):          # no CPU path
        mod.eval()({"msa": torch.zeros(3, 4, dtype=torch.long), "has_deletion": torch.zeros(3, 4),
                    "deletion_value": torch.zeros(3, 4)}, torch.zeros(4, 4, 128), torch.zeros(4, 449), torch.ones(4, 4))


def test_stack_keys_and_pair_only_block():
    st = px.PairformerStack(n_blocks=2)
    keys = list(st.state_dict())
    assert keys[0].startswith("blocks.0.") and any(k.startswith("blocks.1.pair_transition") for k in keys)
    blk = px.PairformerBlock(c_s=0)
    assert not any(k.startswith("attention_pair_bias") for k in blk.state_dict())


def test_reference_initialisers_zero_the_residual_branches():
    torch.manual_seed(0)
    blk = px.PairformerBlock()
    for name in ("tri_mul_out.linear_z", "tri_mul_in.linear_g", "tri_att_start.mha.linear_o",
                 "tri_att_end.mha.linear_g", "pair_transition.linear_no_bias",
                 "attention_pair_bias.attention.linear_o", "single_transition.linear_no_bias"):
        assert float(blk.get_submodule(name).weight.abs().sum()) == 0.0
    w = blk.tri_mul_out.linear_a_p.weight
    assert abs(float(w.std()) - (1 / 128) ** 0.5) < 0.01 and float(w.abs().max()) <= 2 * (1 / 128) ** 0.5 / 0.8796 + 1e-6


def test_randomize_is_a_function_of_name_seed_shape():
    a, b = px.PairformerBlock(), px.PairformerBlock()
    randomize_parameters_(a, 5)
    randomize_parameters_(b, 5)
    for (ka, va), (kb, vb) in zip(a.state_dict().items(), b.state_dict().items()):
        assert ka == kb and torch.equal(va, vb)
    randomize_parameters_(b, 6)
    assert not torch.equal(a.tri_mul_out.linear_z.weight, b.tri_mul_out.linear_z.weight)


def test_weight_cache_tracks_parameter_updates():
    lin = px.OpenfoldLinear(8, 4, bias=False)
    w1 = weights.bf16_of(lin.weight)
    assert weights.bf16_of(lin.weight) is w1
    with torch.no_grad():
        lin.weight.add_(1.0)
    w2 = weights.bf16_of(lin.weight)
    assert w2 is not w1 and torch.equal(w2, lin.weight.detach().to(torch.bfloat16))
    lin.load_state_dict({"weight": torch.zeros(4, 8)})
    assert float(weights.bf16_of(lin.weight).abs().sum()) == 0.0


def test_cpu_tensors_are_rejected_not_silently_computed():
    blk = px.PairformerBlock(c_s=0).eval()
    z = torch.randn(8, 8, 128)
    with pytest.raises(RuntimeError, match="CUDA"):
        blk(None, z, None)
    with pytest.raises(RuntimeError, match="CUDA"):
        px.LayerNorm(128)(z)
    with pytest.raises(RuntimeError, match="CUDA"):
        px.Transition(128, 4).eval()(z)


def test_unsupported_shapes_raise_clear_errors():
    # the reference's regression test builds 16 pair heads; that is outside the compiled kernels
    att = px.TriangleAttention(c_in=128, c_hidden=32, no_heads=16)
    with pytest.raises(RuntimeError, match="specialised"):
        att._kernel_args()
    mul = px.TriangleMultiplicationOutgoing(c_z=64, c_hidden=128)
    with pytest.raises(RuntimeError, match="specialised"):
        mul._kernel_args()


def test_dropout_add_rowwise_eval_is_plain_add():
    r, x = torch.randn(3, 4, 5), torch.randn(3, 4, 5)
    assert torch.equal(px.dropout_add_rowwise(r, x, 0.25, False), r + x)
    assert torch.equal(px.dropout_add_rowwise(r, x, 0.0, True), r + x)
    with pytest.raises(RuntimeError):
        px.dropout_add_rowwise(r, x, 0.25, True)


def test_msa_row_sampling_follows_the_reference_rules():
    """protenix/model/utils.py:290-311: a size drawn from [min(lower_bound, n), n], then the first rows ('topk') or a
    random subset without replacement ('random')."""
    from protenix_b200.msa import sample_msa_indices

    torch.manual_seed(0)
    idx = sample_msa_indices(10, "cpu", lower_bound=1 << 30, strategy="topk")
    assert idx.tolist() == list(range(10))                       # lower bound beyond n: every row, in order
    torch.manual_seed(0)
    sizes = {len(sample_msa_indices(10, "cpu", lower_bound=4, strategy="random")) for _ in range(200)}
    assert min(sizes) >= 4 and max(sizes) == 10
    torch.manual_seed(1)
    idx = sample_msa_indices(50, "cpu", lower_bound=50, strategy="random")
    assert sorted(idx.tolist()) == list(range(50)) and idx.tolist() != list(range(50))
    torch.manual_seed(5)
    a = sample_msa_indices(20, "cpu", 1, "random")
    torch.manual_seed(5)                                          # the same generator calls as the reference's function
    size = int(torch.randint(low=1, high=21, size=(1,)).item())
    assert torch.equal(a, torch.randperm(20)[:size])
    with pytest.raises(ValueError):
        sample_msa_indices(5, "cpu", 1, "sequential")
