"""Utilities: activation checkpointing, profiling / logging helpers, failure detection."""

from .checkpointing import checkpoint_module
from .failure import Heartbeat, RankFailure, check_device_status
from .profiling import StepLogger, StepTimer, dump_memory_snapshot, profile_steps

__all__ = ["checkpoint_module", "Heartbeat", "RankFailure", "check_device_status", "StepLogger", "StepTimer",
           "dump_memory_snapshot", "profile_steps"]
