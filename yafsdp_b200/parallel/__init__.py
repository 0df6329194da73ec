"""Parallelism helpers: the shard mesh and the ZeRO-stage presets.

What is supported (and what is not) mirrors the reference:

* fully sharded data parallel over a 1-D mesh (ZeRO-3: parameters, gradients and optimizer state sharded;
  parameters gathered per layer and freed after use) — the default of ``fully_shard``;
* ZeRO-2 style (parameters stay gathered after their first use in a step, gradients and optimizer state sharded):
  ``reshard_after_forward=False`` on every group, which gives every group its own gather buffer;
* ZeRO-1 style (additionally one gradient buffer per group, so unreduced gradients can be kept across micro-batches):
  ``allow_no_grad_reduce=True`` at lazy init together with ``set_requires_gradient_sync``;
* gradient accumulation, mixed precision, activation checkpointing, hooks for external pipeline schedules.

* hierarchical partitioning (secondary shards inside a smaller group for the backward gather):
  ``module.set_secondary_shard_group(group)``;
* parameters that already are ``DTensor``s of an external tensor- or expert-parallel mesh: their local tensors are
  sharded over the data-parallel mesh and gathered back as ``DTensor``s of the outer mesh.

Not implemented, as in the reference: tensor / pipeline / sequence / context parallelism themselves, hybrid (2-D) sharding.
"""

from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.distributed.device_mesh import DeviceMesh, init_device_mesh

from ..common import ShardMeshInfo

__all__ = ["init_shard_mesh", "zero_stage_kwargs", "enable_unreduced_accumulation", "ShardMeshInfo"]


def init_shard_mesh(device_type: str | None = None, group: dist.ProcessGroup | None = None) -> DeviceMesh:
    """1-D mesh over ``group`` (default: the world).  ``device_type`` defaults to CUDA when the backend is not gloo."""
    if not dist.is_initialized():
        raise RuntimeError("initialise torch.distributed first (see yafsdp_b200.train.init_distributed)")
    if device_type is None:
        device_type = "cuda" if torch.cuda.is_available() and dist.get_backend(group) != "gloo" else "cpu"
    if group is None:
        return init_device_mesh(device_type, (dist.get_world_size(),))
    return DeviceMesh.from_group(group, device_type)


def zero_stage_kwargs(stage: int) -> dict[str, Any]:
    """``fully_shard`` keyword arguments for a ZeRO stage (apply the same stage to every group of a model)."""
    if stage >= 3:
        return {"reshard_after_forward": True}
    if stage in (1, 2):
        return {"reshard_after_forward": False}
    raise ValueError("stage must be 1, 2 or 3 (plain replicated data parallel is not part of this framework)")


def enable_unreduced_accumulation(root: nn.Module) -> None:
    """Give every group its own gradient buffer so that ``set_requires_gradient_sync(False)`` can be used on the whole
    model (micro-batch gradients accumulate unreduced; the reduction runs once, on the last micro-batch).  Call before
    the first forward."""
    root._get_fsdp_state()._lazy_init(allow_no_grad_reduce=True)  # type: ignore[attr-defined]
