"""Public policy dataclasses.

Parity: ``ya_fsdp/_api.py:6-22``.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class MixedPrecisionPolicy:
    """Mixed-precision configuration of one ``fully_shard`` group.

    ``param_dtype``: dtype of the all-gathered (compute) parameters; ``None`` keeps the original dtype.
    ``reduce_dtype``: dtype of the gradient reduce-scatter; ``None`` means ``param_dtype``.
    ``output_dtype``: cast floating-point forward outputs to this dtype.
    ``cast_forward_inputs``: cast floating-point forward inputs to ``param_dtype`` (default off).
    ``bit32_acc_for_bit16_reduce_scatter``: bf16 on the wire, fp32 accumulation (needs ``reduce_dtype=bf16``).
    ``all_gather_dtype_to_param_cls``: all-gather dtype -> parameter tensor class (or tuple of classes) gathered in
    that dtype through the ``fsdp_pre_all_gather`` / ``fsdp_post_all_gather`` tensor-extension hooks (fp8-style
    parameters).  A group gathers in one dtype: such parameters go into ``fully_shard`` groups of their own.
    """

    param_dtype: torch.dtype | None = None
    reduce_dtype: torch.dtype | None = None
    output_dtype: torch.dtype | None = None
    cast_forward_inputs: bool = False
    bit32_acc_for_bit16_reduce_scatter: bool = False
    all_gather_dtype_to_param_cls: dict[torch.dtype, tuple[type, ...]] | None = None

    def __post_init__(self) -> None:
        if self.bit32_acc_for_bit16_reduce_scatter and self.reduce_dtype != torch.bfloat16:
            raise ValueError("bit32_acc_for_bit16_reduce_scatter requires reduce_dtype=torch.bfloat16")
