"""Failure detection: host-side heartbeats through the rendezvous store, and the device status word.

The reference has no failure detection of its own (it relies on the process-group watchdog).  Because the
peer-memory backend replaces NCCL's collectives with kernels that wait on flags written by other GPUs,
this framework adds two small mechanisms:

* every device-side wait is bounded; a wait that runs out records a code in the library status word and the
  kernel returns (the CUDA context stays usable).  ``check_device_status()`` reads and clears it;
* ``Heartbeat``: each rank bumps a counter in the ``torch.distributed`` store from a background thread; ``check()``
  (called between steps, never while kernels of a collective are in flight) raises ``RankFailure`` when a peer's
  counter has not moved within the timeout, so the surviving ranks learn about a dead peer on the host before
  their next launch instead of timing out on the device.
"""

from __future__ import annotations

import threading
import time

import torch.distributed as dist

__all__ = ["Heartbeat", "RankFailure", "check_device_status"]


class RankFailure(RuntimeError):
    def __init__(self, ranks: list[int], message: str):
        super().__init__(message)
        self.ranks = ranks


class Heartbeat:
    """Store-based liveness: ``start()`` begins beating, ``check()`` raises ``RankFailure`` for silent peers."""

    def __init__(self, store: dist.Store, rank: int, world_size: int, interval_s: float = 0.5, timeout_s: float = 10.0,
                 prefix: str = "yafsdp_hb"):
        self.store = store
        self.rank = rank
        self.world_size = world_size
        self.interval_s = interval_s
        self.timeout_s = timeout_s
        self.prefix = prefix
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._last_seen: dict[int, tuple[int, float]] = {}

    def _key(self, rank: int) -> str:
        return f"{self.prefix}/{rank}"

    def start(self) -> None:
        self.store.add(self._key(self.rank), 1)
        self._thread = threading.Thread(target=self._beat, name="yafsdp-heartbeat", daemon=True)
        self._thread.start()

    def _beat(self) -> None:
        while not self._stop.wait(self.interval_s):
            try:
                self.store.add(self._key(self.rank), 1)
            except Exception:
                return  # the store went away with its host: the job is ending

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval_s + 1.0)

    def check(self) -> None:
        now = time.monotonic()
        dead: list[int] = []
        for r in range(self.world_size):
            if r == self.rank:
                continue
            try:
                count = int(self.store.add(self._key(r), 0))
            except Exception as e:  # store unreachable: treat like a failure of the store's host
                raise RankFailure([0], f"heartbeat store unreachable: {e}") from e
            seen = self._last_seen.get(r)
            if seen is None or seen[0] != count:
                self._last_seen[r] = (count, now)
            elif now - seen[1] > self.timeout_s:
                dead.append(r)
        if dead:
            raise RankFailure(dead, f"rank(s) {dead} stopped sending heartbeats for more than {self.timeout_s:.1f} s")


def check_device_status() -> None:
    """Raise if a kernel of the native library recorded a failed bounded wait since the last check (synchronises)."""
    from ..ops import kernels

    kernels.check_status()
