"""Small shared definitions: mesh info, training states, the library logger.

Parity: ``ya_fsdp/_common.py:13-74``.
"""

from __future__ import annotations

import enum
import logging
import traceback
from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist
from torch.distributed.device_mesh import DeviceMesh

logger = logging.getLogger("yafsdp_b200")


class TrainingState(enum.Enum):
    """State of one ``fully_shard`` group inside a training step."""

    FORWARD = enum.auto()
    PRE_BACKWARD = enum.auto()
    POST_BACKWARD = enum.auto()
    IDLE = enum.auto()


@dataclass
class ShardMeshInfo:
    """The 1-D mesh a group is sharded over."""

    mesh: DeviceMesh
    shard_mesh_dim: int = 0

    def __post_init__(self) -> None:
        self.shard_process_group: dist.ProcessGroup = self.mesh.get_group(self.shard_mesh_dim)
        self.shard_mesh_size: int = self.mesh.size(self.shard_mesh_dim)
        self.shard_mesh_rank: int = self.shard_process_group.rank()


def raise_assert_with_print(*args: Any, **kwargs: Any) -> None:
    rank = dist.get_rank() if dist.is_initialized() else 0
    print(f"[Rank {rank}] ", end="")
    print(*args, **kwargs)
    traceback.print_stack()
    raise AssertionError(*args, **kwargs)


def cast_fp_tensor(dtype: torch.dtype, x: Any) -> Any:
    if not isinstance(x, torch.Tensor) or not torch.is_floating_point(x) or x.dtype == dtype:
        return x
    return x.to(dtype)


def is_backward_running() -> bool:
    """True while the autograd engine is executing a backward pass on this thread."""
    return torch._C._current_graph_task_id() != -1
