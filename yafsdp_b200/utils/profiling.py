"""Tracing and per-step metrics.

The library labels its phases with ``torch.profiler.record_function`` ranges (``YaFSDP::all_gather``,
``YaFSDP::pre_forward``, ``YaFSDP::post_backward_reduce`` ..., the names the reference uses,
``ya_fsdp/_param_group.py:563-820``) and logs state transitions on the ``yafsdp_b200`` logger at DEBUG level.
This module adds what the reference's example scripts patch into the trainer
(``patches/transformers.diff:146-180``): a profiler context that writes a Chrome trace for a window of
steps, an iteration timer (host wall clock and CUDA events) and a memory-snapshot helper.
"""

from __future__ import annotations

import contextlib
import json
import time
from typing import Any, Iterator

import torch

__all__ = ["StepTimer", "profile_steps", "dump_memory_snapshot", "StepLogger"]


class StepTimer:
    """Host and device time of each step: ``with timer.step(): train_step()``; ``timer.summary()``."""

    def __init__(self, device: torch.device | None = None):
        self.cuda = device is not None and device.type == "cuda"
        self.host_ms: list[float] = []
        self._events: list[tuple[Any, Any]] = []

    @contextlib.contextmanager
    def step(self) -> Iterator[None]:
        t0 = time.perf_counter()
        if self.cuda:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
        yield
        if self.cuda:
            e.record()
            self._events.append((s, e))
        self.host_ms.append((time.perf_counter() - t0) * 1e3)

    def device_ms(self) -> list[float]:
        if not self.cuda:
            return []
        torch.cuda.synchronize()
        return [s.elapsed_time(e) for s, e in self._events]

    def summary(self) -> dict[str, float]:
        dev = self.device_ms()
        out = {"steps": float(len(self.host_ms)), "host_ms_mean": sum(self.host_ms) / max(1, len(self.host_ms))}
        if dev:
            out["device_ms_mean"] = sum(dev) / len(dev)
        return out


@contextlib.contextmanager
def profile_steps(path: str, wait: int = 10, warmup: int = 10, active: int = 1) -> Iterator[Any]:
    """``torch.profiler`` with the example scripts' schedule; call ``prof.step()`` after every training step.  The Chrome
    trace of the active window is written to ``path``."""
    from torch.profiler import ProfilerActivity, profile, schedule

    acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])

    def on_ready(prof: Any) -> None:
        prof.export_chrome_trace(path)

    with profile(activities=acts, schedule=schedule(wait=wait, warmup=warmup, active=active), on_trace_ready=on_ready) as prof:
        yield prof


def dump_memory_snapshot(path: str) -> None:
    """Write the CUDA caching-allocator history recorded so far (start it with ``torch.cuda.memory._record_memory_history()``)."""
    torch.cuda.memory._dump_snapshot(path)


class StepLogger:
    """One JSON line per step: loss, iteration time, tokens/s/GPU, peak memory."""

    def __init__(self, tokens_per_step_per_gpu: int, stream: Any = None):
        self.tokens = tokens_per_step_per_gpu
        self.stream = stream
        self.step = 0

    def log(self, loss: float, iter_time_s: float, **extra: Any) -> dict[str, Any]:
        rec = {"step": self.step, "loss": round(float(loss), 5), "iter_time_s": round(iter_time_s, 5),
               "tokens_per_s_per_gpu": round(self.tokens / iter_time_s, 1)}
        if torch.cuda.is_available():
            rec["peak_mem_gb"] = round(torch.cuda.max_memory_allocated() / 2**30, 2)
        rec.update(extra)
        print(json.dumps(rec), file=self.stream, flush=True)
        self.step += 1
        return rec
