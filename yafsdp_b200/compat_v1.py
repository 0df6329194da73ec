"""Class-style ``YaFSDP`` wrapper with the reference's first-generation constructor.

Parity: ``ya_fsdp/ya_fsdp.py:70-602`` (``YaFSDP``), the argument mapping of ``docs/migration_guide.md``.
The class maps the old arguments onto the same core that ``fully_shard`` uses:

* every ``(module, name)`` of ``modules_to_wrap_with_names`` becomes one parameter group (the reference's
  ``SuperTensorModule``); all modules of ``layer_norm_module_cls`` plus those of
  ``rogue_layer_norm_modules_with_names`` form ONE further group with buffers of its own, gathered once per forward
  and kept until the end of backward (the reference's norm super-tensor); the wrapped model is the root;
* ``is_trainable=False``: the model is kept in ``param_dtype`` with no master copy and no gradient buffers;
* ``zero_stage=3``: gathered weights are freed after use (two rotating weight buffers); ``zero_stage<=2``:
  weights stay gathered after the first use (one buffer per group);
* ``bit16_reduce_scatter`` / ``bit32_acc_for_bit16_reduce_scatter`` select the reduce dtype; gradients are
  divided by ``dp_size * gradient_accumulation_steps`` as they are reduced, so after the last micro-batch the flat
  fp32 gradients hold the mean (the reference divides once at the end, ``ya_fsdp.py:499-501``);
* ``parameters()`` yields ONE flat fp32 ``nn.Parameter`` per group whose ``.grad`` is the group's flat fp32
  gradient shard (the reference exposes two flat parameters, ``ya_fsdp.py:364-410``); any ``torch.optim`` optimizer
  then runs a few large foreach kernels;
* ``clip_grad_norm_``, ``local_state_dict`` / ``load_state_dict`` (local format with ``"meta"``), ``state_dict`` (full,
  gathered to CPU on rank 0) and ``zero_grad`` (``set_to_none=True`` refused: the gradients are persistent flat
  buffers) behave as in the reference.

``model_parallel_process_group``: the wrapper shards over the data-parallel group only; with
``all_reduce_grads_across_model_parallel_group`` the norm group's reduced gradients are summed over the model-parallel
group, and ``clip_grad_norm_`` adds the squared norms over it.

Not carried over: the closed-source communication library switches (``use_yccl*``: accepted and ignored with
a warning; the peer-memory backend plays that role, ``comm_backend="symm"``), ``yccl_intra_inter_expr`` (an
``eval`` of a user string).  ``hpz_first_layers_num`` keeps a secondary shard of the first layers' weights inside
``intra_node_data_parallel_process_group`` (default: one group per node) and gathers them for backward from there.
"""

from __future__ import annotations

import warnings
from typing import Any, Callable, Iterator

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.distributed.device_mesh import DeviceMesh, init_device_mesh

from . import checkpoint as _ckpt
from .api import MixedPrecisionPolicy
from .fully_shard import fully_shard
from .optim import param_groups_of

__all__ = ["YaFSDP"]


class YaFSDP(nn.Module):
    def __init__(
        self,
        module: nn.Module,
        zero_stage: int = 3,
        param_dtype: torch.dtype = torch.bfloat16,
        modules_to_wrap_with_names: list[tuple[nn.Module, str]] | None = None,
        layer_norm_module_cls: type | tuple[type, ...] | None = None,
        gradient_accumulation_steps: int = 1,
        data_parallel_process_group: dist.ProcessGroup | None = None,
        intra_node_data_parallel_process_group: dist.ProcessGroup | None = None,
        model_parallel_process_group: dist.ProcessGroup | None = None,
        all_reduce_grads_across_model_parallel_group: bool = False,
        bit16_reduce_scatter: bool = False,
        bit32_acc_for_bit16_reduce_scatter: bool = False,
        hpz_first_layers_num: int = 0,
        rogue_layer_norm_modules_with_names: dict[nn.Module, str] | list[tuple[nn.Module, str]] | None = None,
        sync_module_states: bool = False,
        param_init_fn: Callable[[nn.Module], None] | None = None,
        device_id: int | torch.device | None = None,
        is_trainable: bool = True,
        use_yccl: bool = False,
        use_yccl_padding: bool = False,
        yccl_intra_inter_expr: str | None = None,
        yccl_all_gather_stages: int | None = None,
        profile: bool = False,
        comm_backend: str = "auto",
    ):
        super().__init__()
        if hpz_first_layers_num and zero_stage < 3:
            raise ValueError("hpz_first_layers_num needs zero_stage=3: with weights kept gathered there is no backward all-gather")
        if use_yccl or yccl_intra_inter_expr is not None or yccl_all_gather_stages is not None:
            warnings.warn("the closed-source communication library options are ignored; use comm_backend='symm'", stacklevel=2)
        if all_reduce_grads_across_model_parallel_group and model_parallel_process_group is None:
            raise ValueError("all_reduce_grads_across_model_parallel_group needs model_parallel_process_group")
        self._mp_group = model_parallel_process_group
        if not modules_to_wrap_with_names:
            raise ValueError("modules_to_wrap_with_names must list the (module, name) pairs to shard as units")
        self.module = module
        self.zero_stage = zero_stage
        self.gradient_accumulation_steps = gradient_accumulation_steps
        self.is_trainable = is_trainable
        self._profile = profile

        pg = data_parallel_process_group or dist.group.WORLD
        device_type = "cpu"
        if device_id is not None or (torch.cuda.is_available() and dist.get_backend(pg) != "gloo"):
            device_type = "cuda"
            if device_id is not None:
                torch.cuda.set_device(device_id)
        if data_parallel_process_group is None:
            mesh = init_device_mesh(device_type, (dist.get_world_size(),))
        else:
            mesh = DeviceMesh.from_group(pg, device_type)
        self._mesh = mesh
        self._dp_size = pg.size()

        reduce_dtype = torch.bfloat16 if bit16_reduce_scatter else torch.float32
        dev = torch.device(device_type, torch.cuda.current_device()) if device_type == "cuda" else torch.device("cpu")
        rogue = rogue_layer_norm_modules_with_names or []
        rogue_items = list(rogue.items()) if isinstance(rogue, dict) else list(rogue)
        # materialise / synchronise first: the norm modules inside the wrapped modules are sharded before their parents
        for sub in [m for m, _ in modules_to_wrap_with_names] + [m for m, _ in rogue_items]:
            if param_init_fn is not None and any(p.device.type == "meta" for p in sub.parameters()):
                sub.to_empty(device=dev)
                param_init_fn(sub)
            if sync_module_states:
                _broadcast_module(sub, pg)
        if not is_trainable:
            # inference: no fp32 master and no gradient buffers; the flat parameters are kept in param_dtype and are the
            # all-gather input themselves (ya_fsdp/ya_fsdp.py:355-360)
            module.to(param_dtype)
            module.requires_grad_(False)
        policy = MixedPrecisionPolicy(
            param_dtype=param_dtype if is_trainable else None,
            reduce_dtype=reduce_dtype if is_trainable else None,
            bit32_acc_for_bit16_reduce_scatter=bool(is_trainable and bit16_reduce_scatter and bit32_acc_for_bit16_reduce_scatter),
        )
        reshard = zero_stage >= 3
        # with zero_stage <= 2 nobody reshards after forward, so every group gets its own weight buffer
        kw: dict[str, Any] = dict(mesh=mesh, mp_policy=policy, reshard_after_forward=reshard if reshard else False)

        # ---- all norm weights of the model form ONE group that is gathered once per forward and stays gathered until the end
        # of backward (the reference's "layernorm super-tensor", ya_fsdp/ya_fsdp.py:313-323,469-471), in its own buffers
        wrapped_set = {m for m, _ in modules_to_wrap_with_names}
        norm_modules: list[nn.Module] = []
        if layer_norm_module_cls is not None:
            norm_modules = [m for m in module.modules() if isinstance(m, layer_norm_module_cls) and m not in wrapped_set]
        for m, _ in rogue_items:
            if m not in norm_modules and m not in wrapped_set:
                norm_modules.append(m)
        norm_modules = [m for m in norm_modules if next(m.parameters(), None) is not None]
        self._norm_group: Any = None
        if norm_modules:
            fully_shard(norm_modules if len(norm_modules) > 1 else norm_modules[0], **{**kw, "reshard_after_forward": False})
            self._norm_group = norm_modules[0]._get_fsdp_state()._param_group  # type: ignore[attr-defined]
            self._norm_group.dedicated_buffers = True
            self._norm_group.is_norm_group = True
            if all_reduce_grads_across_model_parallel_group and self._mp_group is not None and self._mp_group.size() > 1:
                # norm weights are replicated over the model-parallel group and see different activations there:
                # their reduced gradients are summed over it (ya_fsdp/ya_fsdp.py:989-990)
                mp = self._mp_group
                self._norm_group.post_reduce_hook = lambda shard: dist.all_reduce(shard, group=mp)
        wrapped: list[nn.Module] = []
        for sub, _name in modules_to_wrap_with_names:
            fully_shard(sub, **kw)
            wrapped.append(sub)
        leftover = [p for p in module.parameters() if not hasattr(p, "_spec")]
        if leftover:
            warnings.warn(f"{len(leftover)} parameters are outside the wrapped modules; they are sharded with the root group", stacklevel=2)
        fully_shard(module, **kw)
        if hpz_first_layers_num:
            intra = intra_node_data_parallel_process_group or _intra_node_group(pg, device_type)
            for sub in wrapped[:hpz_first_layers_num]:
                sub.set_secondary_shard_group(intra)  # type: ignore[attr-defined]
        module.set_comm_backend(comm_backend, num_grad_buffers=2 if zero_stage >= 2 else None)  # type: ignore[attr-defined]
        if zero_stage <= 1:
            module._get_fsdp_state()._lazy_init(allow_no_grad_reduce=True)  # type: ignore[attr-defined]
        # reduced gradients are divided by dp_size * accumulation steps, so the flat gradients hold the mean after the last micro-batch
        module.set_gradient_divide_factor(float(self._dp_size * gradient_accumulation_steps))  # type: ignore[attr-defined]
        self._flat_params: list[nn.Parameter] | None = None

    # ------------------------------------------------------------------ module protocol
    def forward(self, *args: Any, **kwargs: Any) -> Any:
        return self.module(*args, **kwargs)

    def __getattr__(self, name: str) -> Any:
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.module, name)

    # ------------------------------------------------------------------ optimizer contract
    def _groups(self) -> list[Any]:
        return param_groups_of(self.module)

    def parameters(self, recurse: bool = True) -> Iterator[nn.Parameter]:  # type: ignore[override]
        """One flat parameter (original dtype) per group; ``.grad`` is bound to the group's flat gradient shard."""
        if self._flat_params is None:
            self._flat_params = []
            for g in self._groups():
                p = nn.Parameter(g.master_flat, requires_grad=self.is_trainable)
                if self.is_trainable:
                    p.grad = g.sharded_grad_flat
                self._flat_params.append(p)
        return iter(self._flat_params)

    def zero_grad(self, set_to_none: bool = False) -> None:
        if set_to_none:
            raise ValueError("YaFSDP keeps persistent flat gradient buffers: zero_grad(set_to_none=True) is not supported")
        for g in self._groups():
            g.sharded_grad_flat.zero_()
            for sp in g.params:
                if sp.sharded_param is not None and sp.sharded_param.grad is None and sp.requires_grad:
                    _ = g.sharded_grad_flat
                    sp.sharded_param.grad = sp.sharded_grad

    @torch.no_grad()
    def clip_grad_norm_(self, max_norm: float, norm_type: float = 2.0) -> torch.Tensor:
        """L2 only: local squared norms of the flat gradients, one all-reduce, in-place scale."""
        if norm_type != 2.0:
            raise NotImplementedError("only the L2 norm is supported")
        groups = self._groups()
        total = torch.zeros((), device=groups[0].device, dtype=torch.float32)
        for g in groups:
            total = total + g.sharded_grad_flat.float().pow(2).sum()
        if self._dp_size > 1:
            dist.all_reduce(total, group=groups[0].process_group)
        if self._mp_group is not None and self._mp_group.size() > 1:
            dist.all_reduce(total, group=self._mp_group)
        total = total.sqrt()
        coef = torch.clamp(max_norm / (total + 1e-6), max=1.0)
        for g in groups:
            g.sharded_grad_flat.mul_(coef)
        return total

    # ------------------------------------------------------------------ checkpoints
    def local_state_dict(self) -> dict[str, Any]:
        return _ckpt.local_state_dict_v1(self.module)

    def state_dict(self, *args: Any, **kwargs: Any) -> dict[str, torch.Tensor]:  # type: ignore[override]
        return _ckpt.full_state_dict(self.module, rank0_only=True)

    def load_state_dict(self, state_dict: dict[str, Any], *args: Any, **kwargs: Any) -> None:  # type: ignore[override]
        _ckpt.load_local_state_dict_v1(self.module, state_dict)


def _intra_node_group(pg: dist.ProcessGroup, device_type: str) -> dist.ProcessGroup | None:
    """Groups of consecutive ranks, one per node (``ya_fsdp/ya_fsdp.py:180-184``); every rank creates every group."""
    per_node = torch.cuda.device_count() if device_type == "cuda" else 1
    world = pg.size()
    if per_node <= 1 or per_node >= world or world % per_node:
        return None
    ranks = dist.get_process_group_ranks(pg)
    mine = None
    for lo in range(0, world, per_node):
        g = dist.new_group(ranks[lo : lo + per_node])
        if pg.rank() // per_node == lo // per_node:
            mine = g
    return mine


def _broadcast_module(module: nn.Module, group: dist.ProcessGroup) -> None:
    src = dist.get_global_rank(group, 0)
    with torch.no_grad():
        for t in list(module.parameters()) + list(module.buffers()):
            if t.device.type != "meta":
                dist.broadcast(t.data, src=src, group=group)
