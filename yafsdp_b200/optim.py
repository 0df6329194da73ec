"""Sharded AdamW on the flat master shards, fused with the compute-dtype refresh and the clip scale.

The reference leaves the optimizer to ``torch.optim`` running foreach / fused kernels over the
``RaggedShardDTensor`` parameters (``ya_fsdp/_tensor.py:212-312``) and re-casts fp32 -> bf16 in the next
step's first all-gather (``ya_fsdp/_collectives.py:47-55``).  That path works here too (any
``torch.optim`` optimizer accepts the sharded parameters).  ``ShardedAdamW`` is the fast path: one
kernel launch per parameter group that reads gradient / master / moments once, writes master /
moments and *also* the bf16 all-gather input, and multiplies the gradient by a device-side clip
coefficient, so clipping costs no extra pass over the gradients and there is no host sync.
"""

from __future__ import annotations

import math
from typing import Any, Iterable

import torch
import torch.distributed as dist
import torch.nn as nn

from .group import ParamGroup
from .state import get_module_state
from .tensor import RaggedShardDTensor

__all__ = ["ShardedAdamW", "param_groups_of", "clip_grad_norm_"]


def param_groups_of(module: nn.Module) -> list[ParamGroup]:
    """Every ``fully_shard`` parameter group under ``module`` in ``named_modules()`` order."""
    out: list[ParamGroup] = []
    for m in module.modules():
        s = get_module_state(m)
        if s is not None and s._param_group is not None:
            for g in getattr(s._param_group, "groups", [s._param_group]):  # a GroupSet contributes its member groups
                if not any(g is o for o in out):
                    out.append(g)
    return out


class ShardedAdamW:
    """AdamW over all ``fully_shard`` groups of ``module`` (decoupled weight decay, bias correction).

    ``step()`` is a handful of kernel launches and never synchronises with the host.  ``max_grad_norm``
    enables global-norm clipping: the squared norms of all shards are summed on the device, all-reduced
    over the shard group, and the resulting coefficient is consumed by the update kernels directly.

    ``overlap_with_forward`` (single-rank groups on CUDA): the update kernels run on a side stream in forward order and
    every group's next forward waits only for its own update, so the memory-bound optimizer pass runs underneath the
    compute-bound GEMMs of the next step's forward instead of in front of them.  Code that reads parameters outside the
    module's forward / ``state_dict`` must call ``join()`` first.  Off by default: on a B200 at its 1000 W cap the
    Llama-2-7B step did not get shorter (125.8 / 127.4 ms with, 126.2 ms without): the GEMMs already run power-limited
    at ~1650 MHz and slow down by what the concurrent memory traffic draws.
    """

    def __init__(self, module: nn.Module, lr: float = 1e-3, betas: tuple[float, float] = (0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, max_grad_norm: float | None = None, overlap_with_forward: bool = False):
        self.module = module
        self.groups = param_groups_of(module)
        if not self.groups:
            raise ValueError("ShardedAdamW needs a module that fully_shard was applied to")
        self.lr = lr
        self.betas = betas
        self.eps = eps
        self.weight_decay = weight_decay
        self.max_grad_norm = max_grad_norm
        self.step_count = 0
        self.overlap_with_forward = overlap_with_forward
        self._side_stream: Any = None
        self._n_sms = torch.cuda.get_device_properties(self.groups[0].device).multi_processor_count if self.groups[0].device.type == "cuda" else 1
        self.exp_avg = [torch.zeros_like(g.master_flat, dtype=torch.float32) for g in self.groups]
        self.exp_avg_sq = [torch.zeros_like(g.master_flat, dtype=torch.float32) for g in self.groups]
        dev = self.groups[0].device
        self._norm_sq = torch.zeros(1, device=dev, dtype=torch.float32)
        # one slot per group: weight-gradient kernels add the squared norm of what they write (single-rank fusion)
        self._group_norm_sq = torch.zeros(len(self.groups), device=dev, dtype=torch.float32)
        if max_grad_norm is not None and dev.type == "cuda":
            for i, g in enumerate(self.groups):
                g._norm_sq = self._group_norm_sq[i : i + 1]
        self._coef = torch.ones(1, device=dev, dtype=torch.float32)
        self.last_grad_norm = torch.zeros(1, device=dev, dtype=torch.float32)

    # ------------------------------------------------------------------ helpers
    def zero_grad(self, set_to_none: bool = True) -> None:
        for g in self.groups:
            for sp in g.params:
                if sp.sharded_param is not None:
                    if set_to_none:
                        sp.sharded_param.grad = None
                    elif sp.sharded_param.grad is not None:
                        sp.sharded_param.grad._local_tensor.zero_()  # type: ignore[union-attr]

    def _active(self) -> list[int]:
        return [i for i, g in enumerate(self.groups) if g._has_sharded_grads()]

    def _compute_clip_coef(self, active: list[int]) -> torch.Tensor | None:
        if self.max_grad_norm is None:
            return None
        from .ops import kernels

        dev = self._norm_sq.device
        self._norm_sq.zero_()
        # groups may be sharded over different process groups: sum each group's shards over its own ranks
        by_pg: dict[Any, list[int]] = {}
        for i in active:
            by_pg.setdefault(self.groups[i].process_group, []).append(i)
        for n_pg, (pg, members) in enumerate(by_pg.items()):
            part = self._norm_sq if len(by_pg) == 1 else torch.zeros_like(self._norm_sq)
            fused = []
            for i in members:
                grp = self.groups[i]
                if grp._norm_sq is not None and grp._norm_fused_ok:
                    fused.append(i)  # the kernels that wrote the gradients already summed their squares
                    continue
                g = grp.sharded_grad_flat
                if dev.type == "cuda":
                    kernels.sumsq_(g, part)
                else:
                    part += g.float().pow(2).sum()
            if fused:
                part += self._group_norm_sq[fused].sum() if len(fused) < len(self.groups) else self._group_norm_sq.sum()
            if pg is not None and pg.size() > 1:
                dist.all_reduce(part, group=pg)
            if part is not self._norm_sq:
                self._norm_sq += part
        if dev.type == "cuda":
            kernels.clip_coef_(self._norm_sq, self.max_grad_norm, self._coef, self.last_grad_norm)
        else:
            self.last_grad_norm.copy_(self._norm_sq.sqrt())
            self._coef.copy_(torch.clamp(self.max_grad_norm / (self.last_grad_norm + 1e-6), max=1.0))
        return self._coef

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self) -> None:
        active = self._active()
        if not active:
            return
        if self._norm_sq.is_cuda:
            from .ops import kernels

            kernels.poll_status()
        self.step_count += 1
        coef = self._compute_clip_coef(active)
        b1, b2 = self.betas
        side = None
        if self.overlap_with_forward and self._norm_sq.is_cuda and all(self.groups[i].world_size == 1 for i in active):
            if self._side_stream is None:
                self._side_stream = torch.cuda.Stream(device=self._norm_sq.device)
            side = self._side_stream
            side.wait_stream(torch.cuda.current_stream(self._norm_sq.device))  # gradients and the clip coefficient are ready
        for i in active:
            g = self.groups[i]
            if side is not None:
                with torch.cuda.stream(side):
                    self._update_group(i, coef, b1, b2, max_ctas=3 * self._n_sms)
                    ev = torch.cuda.Event()
                    ev.record(side)
                g._optim_event = ev
                continue
            self._update_group(i, coef, b1, b2)

    def join(self) -> None:
        """Make the current stream wait for updates still running on the side stream (``overlap_with_forward``)."""
        if self._side_stream is not None:
            torch.cuda.current_stream(self._norm_sq.device).wait_stream(self._side_stream)
            for g in self.groups:
                g._optim_event = None

    @staticmethod
    def _segments(g: ParamGroup) -> list[tuple[int, int]] | None:
        """``None`` when every parameter of which this rank holds a piece has a gradient (the whole flat shard is updated in
        one launch); otherwise the local ranges of those that have one.  Parameters without a gradient (frozen, or unused
        in this step) are left alone entirely - no weight decay, no moment decay - as ``torch.optim.AdamW`` does."""
        segs: list[tuple[int, int]] = []
        full = True
        for sp in g.params:
            pl = sp.placement
            assert pl is not None
            if not pl.local_numel:
                continue
            if sp.sharded_param is None or sp.sharded_param.grad is None:
                full = False
                continue
            lo, hi = pl.shard_offset, pl.shard_offset + pl.local_numel
            if segs and segs[-1][1] == lo:
                segs[-1] = (segs[-1][0], hi)
            else:
                segs.append((lo, hi))
        return None if full else segs

    def _update_group(self, i: int, coef: torch.Tensor | None, b1: float, b2: float, max_ctas: int = 0) -> None:
        g = self.groups[i]
        p, grad, m, v = g.master_flat, g.sharded_grad_flat, self.exp_avg[i], self.exp_avg_sq[i]
        ag = g.gather_input
        bf16_out = ag if (ag is not None and ag is not p and ag.dtype == torch.bfloat16) else None
        segs = self._segments(g)
        if segs is not None:
            # some parameters have no gradient: update the others range by range with tensor ops
            bc1 = 1 - b1 ** self.step_count
            bc2 = 1 - b2 ** self.step_count
            for lo, hi in segs:
                gr = grad[lo:hi].float() * (coef if coef is not None else 1.0)
                pf = p[lo:hi].float()
                pf.mul_(1 - self.lr * self.weight_decay)
                m[lo:hi].mul_(b1).add_(gr, alpha=1 - b1)
                v[lo:hi].mul_(b2).addcmul_(gr, gr, value=1 - b2)
                denom = (v[lo:hi].sqrt() / math.sqrt(bc2)).add_(self.eps)
                pf.addcdiv_(m[lo:hi], denom, value=-self.lr / bc1)
                p[lo:hi].copy_(pf)
            g._ag_input_fresh = False
            return
        if p.is_cuda and p.dtype == torch.float32:
            from .ops import kernels

            kernels.adamw_(p, grad, m, v, bf16_out, coef, lr=self.lr, beta1=b1, beta2=b2, eps=self.eps,
                           weight_decay=self.weight_decay, step=self.step_count, max_ctas=max_ctas)
            if bf16_out is not None:
                g.mark_gather_input_fresh()
            else:
                g._ag_input_fresh = False  # the kernel updated the master behind autograd's version counter
        else:
            gr = grad.float() * (coef if coef is not None else 1.0)
            pf = p.float()
            pf.mul_(1 - self.lr * self.weight_decay)
            m.mul_(b1).add_(gr, alpha=1 - b1)
            v.mul_(b2).addcmul_(gr, gr, value=1 - b2)
            bc1 = 1 - b1 ** self.step_count
            bc2 = 1 - b2 ** self.step_count
            denom = (v.sqrt() / math.sqrt(bc2)).add_(self.eps)
            pf.addcdiv_(m, denom, value=-self.lr / bc1)
            p.copy_(pf)

    # ------------------------------------------------------------------ checkpointing
    def state_dict(self) -> dict[str, Any]:
        """``{"state": {param_fqn: {"exp_avg", "exp_avg_sq"}}, "step": n}`` with ``RaggedShardDTensor`` moments
        (saved by ``torch.distributed.checkpoint`` in the same flat per-parameter format as the parameters)."""
        state: dict[str, Any] = {}
        self.join()
        for g in self.groups:
            g._to_sharded_for_state_dict()
        names = {p: n for n, p in self.module.named_parameters(remove_duplicate=False)}
        for g, m, v in zip(self.groups, self.exp_avg, self.exp_avg_sq):
            for sp in g.params:
                pl = sp.placement
                assert pl is not None and sp.sharded_param is not None
                spec = sp.sharded_param._spec.with_dtype(torch.float32)
                sl = slice(pl.shard_offset, pl.shard_offset + pl.local_numel)
                key = names.get(sp.sharded_param) or sp.fqn or f"{g._module_fqn}.{sp.info.param_name}"
                state[key] = {"exp_avg": RaggedShardDTensor(m[sl], spec), "exp_avg_sq": RaggedShardDTensor(v[sl], spec)}
        return {"state": state, "step": self.step_count, "lr": self.lr, "betas": self.betas, "eps": self.eps,
                "weight_decay": self.weight_decay}

    def load_state_dict(self, sd: dict[str, Any]) -> None:
        cur = self.state_dict()["state"]
        for key, entry in sd["state"].items():
            for name in ("exp_avg", "exp_avg_sq"):
                src = entry[name]
                dst = cur[key][name]
                dst._local_tensor.copy_(src._local_tensor if isinstance(src, RaggedShardDTensor) else
                                        src.reshape(-1)[dst._spec.placement.global_offset:
                                                        dst._spec.placement.global_offset + dst._spec.placement.local_numel])
        self.step_count = int(sd.get("step", self.step_count))


def clip_grad_norm_(parameters: Iterable[torch.Tensor] | nn.Module, max_norm: float, norm_type: float = 2.0) -> torch.Tensor:
    """Global gradient-norm clipping for sharded (and plain) parameters; returns the total norm as a plain tensor.

    ``torch.nn.utils.clip_grad_norm_`` also works on ``RaggedShardDTensor`` parameters (through the norm-partial
    dispatch); this helper avoids DTensor overhead and accepts a module."""
    params = list(parameters.parameters()) if isinstance(parameters, nn.Module) else list(parameters)
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return torch.zeros(())
    dev = grads[0].device
    inf = norm_type == math.inf

    def fold(acc: torch.Tensor, local: torch.Tensor) -> torch.Tensor:
        if inf:
            return torch.maximum(acc, local.abs().max().float()) if local.numel() else acc
        return acc + local.float().abs().pow(norm_type).sum()

    # sharded gradients: every rank holds a piece, summed (or maximised) over the ranks of their shard group; plain
    # gradients (replicated or ignored parameters) are whole on every rank and enter once
    plain = torch.zeros((), device=dev, dtype=torch.float32)
    sharded: dict[Any, torch.Tensor] = {}
    for g in grads:
        if isinstance(g, RaggedShardDTensor):
            pg = g._spec.group()
            sharded[pg] = fold(sharded.get(pg, torch.zeros((), device=dev, dtype=torch.float32)), g._local_tensor)
        else:
            plain = fold(plain, g)
    total = plain
    for pg, part in sharded.items():
        if pg is not None and pg.size() > 1:
            dist.all_reduce(part, op=dist.ReduceOp.MAX if inf else dist.ReduceOp.SUM, group=pg)
        total = torch.maximum(total, part) if inf else total + part
    if not inf:
        total = total.pow(1.0 / norm_type)
    coef = torch.clamp(max_norm / (total + 1e-6), max=1.0)
    for g in grads:
        (g._local_tensor if isinstance(g, RaggedShardDTensor) else g).mul_(coef)
    return total
