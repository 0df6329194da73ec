"""Policy validation, divide-factor table, buffer assignment rules (single process)."""

import pytest
import torch

from yafsdp_b200 import MixedPrecisionPolicy
from yafsdp_b200.comm.backends import gradient_divide_factors


def test_policy_validation():
    MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.bfloat16, bit32_acc_for_bit16_reduce_scatter=True)
    with pytest.raises(ValueError):
        MixedPrecisionPolicy(reduce_dtype=torch.float32, bit32_acc_for_bit16_reduce_scatter=True)
    assert MixedPrecisionPolicy().cast_forward_inputs is False


@pytest.mark.parametrize(
    "n,dtype,factor,force,want",
    [
        (8, torch.float32, None, False, (None, None, "avg", None)),
        (1, torch.float32, None, False, (None, None, "sum", None)),
        (8, torch.bfloat16, 8, False, (None, None, "avg", None)),
        (8, torch.float32, 32.0, False, (None, None, "premul_sum", 1 / 32.0)),
        (8, torch.float32, None, True, (None, 8.0, "sum", None)),
        (8, torch.float16, None, False, (4.0, 2.0, "sum", None)),
        (64, torch.float16, None, True, (8.0, 8.0, "sum", None)),
    ],
)
def test_divide_factor_table(n, dtype, factor, force, want):
    assert gradient_divide_factors(n, dtype, factor, force) == want


def test_llama_family_configs_match_published_sizes_and_build_on_meta():
    """Every named configuration has the published parameter count, and the module tree built on the meta device holds
    exactly that many parameters under Hugging Face names."""
    import torch

    from yafsdp_b200.models.llama import CONFIGS, LlamaForCausalLM

    want = {"llama2-7b": 6.738e9, "llama2-13b": 13.016e9, "llama3-8b": 8.030e9, "llama2-34b": 33.744e9,
            "llama2-70b": 68.977e9, "llama3-70b": 70.554e9}
    for name, n in want.items():
        cfg = CONFIGS[name]
        assert abs(cfg.num_params() - n) < 2e6, (name, cfg.num_params())
        with torch.device("meta"):
            model = LlamaForCausalLM(cfg)
        assert sum(p.numel() for p in model.parameters()) == cfg.num_params()
        names = dict(model.named_parameters())
        assert "model.embed_tokens.weight" in names and "lm_head.weight" in names
        assert f"model.layers.{cfg.num_hidden_layers - 1}.mlp.down_proj.weight" in names
