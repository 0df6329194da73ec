"""Activation checkpointing that composes with ``fully_shard``.

The reference relies on ``torch.distributed.algorithms`` checkpoint wrappers applied by the training
stack (``patches/accelerate.diff:71-89``); here a module's ``forward`` is simply routed through
non-reentrant ``torch.utils.checkpoint`` in place, so parameter names do not change.  The recompute
runs inside backward, where the group is already gathered and the forward hooks are no-ops.
"""

from __future__ import annotations

from typing import Any

import torch.nn as nn
from torch.utils.checkpoint import checkpoint


def checkpoint_module(module: nn.Module) -> nn.Module:
    """Recompute ``module``'s forward during backward instead of keeping its activations."""
    if getattr(module, "_yf_checkpointed", False):
        return module
    inner = module.forward

    def forward(*args: Any, **kwargs: Any) -> Any:
        return checkpoint(inner, *args, use_reentrant=False, **kwargs)

    module.__dict__["forward"] = forward
    module.__dict__["_yf_checkpointed"] = True
    return module
