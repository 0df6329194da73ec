"""B200-native sharded data parallel training (ZeRO-3 style) with flat ragged per-layer shards."""

__version__ = "0.1.0"
