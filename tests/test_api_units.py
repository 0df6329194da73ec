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


def test_symm_transport_selection_rules():
    """Transport names are checked when they are set: the push all-gather exists only for the all-gather and only when the
    gather outputs were placed in the shared arena; multicast falls back to the default when the box has none."""
    import types

    import pytest

    from yafsdp_b200.comm.symm import SymmBackend

    def stub(**kw):
        base = dict(world=8, rank=1, has_multicast=False, symmetric_gather_output=False, ag_transport="ce", rs_transport="sm",
                    ag_ctas=0, rs_ctas=0, DEFAULT_TRANSPORTS=SymmBackend.DEFAULT_TRANSPORTS, arena=types.SimpleNamespace())
        base.update(kw)
        return types.SimpleNamespace(**base)

    be = stub()
    SymmBackend.set_transports(be, "sm", "ce", ag_ctas=32)
    assert (be.ag_transport, be.rs_transport, be.ag_ctas, be.rs_ctas) == ("sm", "ce", 32, 0)
    with pytest.raises(ValueError):
        SymmBackend.set_transports(be, "nvl", None)
    with pytest.raises(ValueError):
        SymmBackend.set_transports(be, None, "cp")  # the push form exists for the all-gather only
    with pytest.raises(ValueError):
        SymmBackend.set_transports(be, "cp", None)  # gather outputs are private to this rank
    SymmBackend.set_transports(be, "mc", "mc")  # no multicast on this box: the defaults are used
    assert (be.ag_transport, be.rs_transport) == ("ce", "sm")
    be = stub(symmetric_gather_output=True, has_multicast=True)
    SymmBackend.set_transports(be, "cp", "mc")
    assert (be.ag_transport, be.rs_transport) == ("cp", "mc")


def test_keep_gathered_rule():
    """Gathered bf16 weights are kept from forward to backward only when the whole bf16 model fits beside the sharded plan in
    60 % of a GPU: Llama-2-7B and Llama-3-8B on 8 ranks do, the 34B and 70B shapes do not, a single rank gathers nothing."""
    from yafsdp_b200.models.llama import CONFIGS
    from yafsdp_b200.utils.memory import keep_gathered_fits

    assert keep_gathered_fits(CONFIGS["llama2-7b"], 8, 2048)
    assert keep_gathered_fits(CONFIGS["llama2-7b"], 2, 2048)
    assert keep_gathered_fits(CONFIGS["llama3-8b"], 8, 4096)
    assert not keep_gathered_fits(CONFIGS["llama2-34b"], 8, 2048, checkpoint_layers=5)
    assert not keep_gathered_fits(CONFIGS["llama2-70b"], 8, 2048, checkpoint_layers=80)
    assert not keep_gathered_fits(CONFIGS["llama2-7b"], 1, 2048)
