"""Collective backends used by the parameter groups.

``TorchBackend`` goes through ``torch.distributed`` (NCCL on GPUs, gloo on CPU) and is the measured
baseline / CPU plumbing path.  ``SymmBackend`` (:mod:`yafsdp_b200.comm.symm`) runs the hand-written
peer-memory kernels over NVLink and is the product path on a multi-GPU box.

Both expose the same five operations; all of them enqueue on the *current* stream and none blocks
the host:

* ``alloc(numel, dtype, device, kind)``: memory for a gather input / gather output / reduce input (the
  symmetric backend returns peer-mapped memory here, which is why allocation belongs to the backend,
  like the registered buffers of the closed-source library the reference can attach,
  ``ya_fsdp/_param_group.py:46-69``);
* ``all_gather(out, inp, group)``;
* ``reduce_scatter(dst, inp, group, scale=, accumulate=, ...)``: ``dst (+)= scale * sum_ranks inp[chunk]``
  with fp32 accumulation, fusing the divide and the accumulation into the sharded gradient
  (``ya_fsdp/_collectives.py:93-218``).

Gradient divide factors follow ``ya_fsdp/_collectives.py:221-267``.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

__all__ = ["CommBackend", "TorchBackend", "gradient_divide_factors", "make_backend"]


def gradient_divide_factors(
    group_size: int,
    reduce_dtype: torch.dtype,
    gradient_divide_factor: float | None,
    force_sum_reduction: bool,
) -> tuple[float | None, float | None, str, float | None]:
    """``(pre_divide, post_divide, op, premul)`` with ``op`` one of ``"avg"``, ``"sum"``, ``"premul_sum"``.

    fp32/bf16 without a forced sum: a single AVG (or a pre-multiplied sum for a custom factor); with a
    forced sum: SUM then one division of the shard; other dtypes (fp16): overflow-safe split of the
    factor into a pre- and a post-division around a SUM.
    """
    overflow_risk = reduce_dtype not in (torch.float32, torch.bfloat16)
    factor = gradient_divide_factor
    if not overflow_risk and not force_sum_reduction:
        if factor is None or factor == group_size:
            return None, None, ("avg" if group_size > 1 else "sum"), None
        return None, None, "premul_sum", 1.0 / factor
    if factor is None:
        factor = float(group_size)
    if overflow_risk:
        pre = 1.0
        while factor % pre == 0 and factor / pre > pre:
            pre *= 2
        return pre, factor / pre, "sum", None
    return None, factor, "sum", None


class CommBackend:
    """Interface of a collective backend (see the module docstring)."""

    name = "abstract"
    #: True when gather inputs / reduce inputs must come from ``alloc`` (peer-mapped memory)
    needs_registered_buffers = False
    #: True when all-gathers and reduce-scatters should share one communication stream
    prefers_single_comm_stream = False

    def alloc(self, numel: int, dtype: torch.dtype, device: torch.device, kind: str) -> torch.Tensor:
        return torch.empty(numel, dtype=dtype, device=device)

    def all_gather(self, out: torch.Tensor, inp: torch.Tensor, group: dist.ProcessGroup | None) -> None:
        raise NotImplementedError

    def reduce_scatter(
        self,
        dst: torch.Tensor,
        inp: torch.Tensor,
        group: dist.ProcessGroup | None,
        *,
        scale: float,
        accumulate: bool,
        acc_fp32: bool = True,
        sumsq: torch.Tensor | None = None,
    ) -> bool:
        """Returns True when ``sumsq`` was given and the squared norm of the final ``dst`` values was added to it."""
        raise NotImplementedError

    def step_barrier(self) -> None:
        """Called once per iteration after the optimizer refreshed the gather inputs (symmetric backends
        need every peer's shard to be final before anyone pulls it)."""

    def before_write(self, buf: torch.Tensor) -> None:
        """``buf`` was the input of an earlier ``reduce_scatter`` and is about to be overwritten on the current stream.
        Backends whose peers read the buffer remotely wait here until all of them are done with it."""

    def check(self) -> None:
        """Raise if a device-side bounded wait ran out since the last call."""


class TorchBackend(CommBackend):
    """``torch.distributed`` collectives (NCCL / gloo)."""

    name = "torch"

    def all_gather(self, out: torch.Tensor, inp: torch.Tensor, group: dist.ProcessGroup | None) -> None:
        world = 1 if group is None else group.size()
        # gloo bumps the output's autograd version counter (NCCL does not); the gather outputs are shared
        # rotating buffers that autograd has saved views of, so the counter must not move.
        with torch.autograd._unsafe_preserve_version_counter(out):
            if world == 1:
                out[: inp.numel()].copy_(inp)
            else:
                dist.all_gather_into_tensor(out, inp, group=group)

    def reduce_scatter(
        self,
        dst: torch.Tensor,
        inp: torch.Tensor,
        group: dist.ProcessGroup | None,
        *,
        scale: float,
        accumulate: bool,
        acc_fp32: bool = True,
        sumsq: torch.Tensor | None = None,
    ) -> bool:
        world = 1 if group is None else group.size()
        shard = inp.numel() // world
        rank = 0 if group is None else group.rank()
        own = inp[rank * shard : (rank + 1) * shard]
        if world > 1:
            if scale == 1.0 / world:
                dist.reduce_scatter_tensor(own, inp, op=dist.ReduceOp.AVG, group=group)
            else:
                dist.reduce_scatter_tensor(own, inp, op=dist.ReduceOp.SUM, group=group)
                if scale != 1.0:
                    own.mul_(scale)
        elif scale != 1.0:
            own.mul_(scale)
        if accumulate:
            dst.add_(own)
        elif dst.data_ptr() != own.data_ptr():
            dst.copy_(own)
        return False


def make_backend(name: str | None, device: torch.device, group: dist.ProcessGroup | None, **options: object) -> CommBackend:
    """``"torch"`` (default), ``"symm"`` (peer-memory kernels; CUDA, one node) or ``"auto"``.  ``options`` are the
    peer-memory backend's constructor arguments (transports, multicast, CTA counts); the NCCL backend has none."""
    name = (name or "torch").lower()
    if name == "auto":
        name = "symm" if device.type == "cuda" and group is not None and 1 < group.size() <= 16 else "torch"
    if name == "torch":
        return TorchBackend()
    if name == "symm":
        from .symm import SymmBackend

        return SymmBackend(device, group, **options)  # type: ignore[arg-type]
    raise ValueError(f"unknown comm backend {name!r}")
