"""B200-native sharded data parallel training (ZeRO-3 style) with flat ragged per-layer shards.

Public API (same names as the reference package, ``ya_fsdp/__init__.py:1-12``):
``fully_shard``, ``YaFSDPModule``, ``MixedPrecisionPolicy``, ``RaggedShard``, ``RaggedShardDTensor``,
``UnshardHandle``; plus the class-style ``YaFSDP`` wrapper of the reference's first generation.
"""

from .api import MixedPrecisionPolicy
from .fully_shard import UnshardHandle, YaFSDPModule, fully_shard
from .tensor import RaggedShard, RaggedShardDTensor

__version__ = "0.1.0"

__all__ = [
    "MixedPrecisionPolicy",
    "RaggedShard",
    "RaggedShardDTensor",
    "UnshardHandle",
    "YaFSDPModule",
    "fully_shard",
]
