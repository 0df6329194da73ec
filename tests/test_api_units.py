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
