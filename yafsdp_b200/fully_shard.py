"""``fully_shard`` and the module mixin it installs.

Parity: ``ya_fsdp/fully_shard.py:67-275`` (entry point, ``YaFSDPModule`` method set, ``UnshardHandle``) and
``ya_fsdp/_init.py:22-220`` (mesh default, managed modules / parameters / buffers, device placement).
"""

from __future__ import annotations

import itertools
from typing import Any, Iterable, NoReturn, cast

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.distributed.device_mesh import DeviceMesh, init_device_mesh

from .api import MixedPrecisionPolicy
from .common import ShardMeshInfo
from .group import GroupSet, ParamGroup
from .state import FSDPState, get_module_state

__all__ = ["fully_shard", "YaFSDPModule", "UnshardHandle"]

_cls_to_fsdp_cls: dict[type, type] = {}


# --------------------------------------------------------------------------------------- init helpers
def _default_mesh() -> DeviceMesh:
    if not dist.is_initialized():
        dist.init_process_group()
    device_type = "cuda" if torch.cuda.is_available() and dist.get_backend() != "gloo" else "cpu"
    return init_device_mesh(device_type, (dist.get_world_size(),))


def _device_from_mesh(mesh: DeviceMesh) -> torch.device:
    if mesh.device_type == "cpu":
        return torch.device("cpu")
    return torch.device(mesh.device_type, torch.cuda.current_device())


def _root_modules(modules: Iterable[nn.Module]) -> tuple[nn.Module, ...]:
    mods = list(modules)
    descendants: set[nn.Module] = set()
    for m in mods:
        for sub in itertools.islice(m.modules(), 1, None):
            descendants.add(sub)
    return tuple(m for m in mods if m not in descendants)


def _managed_modules(roots: tuple[nn.Module, ...], ignored_params: set[nn.Parameter] | None) -> list[nn.Module]:
    """Post-order DFS below the roots, skipping subtrees that already have their own ``fully_shard``."""
    out: list[nn.Module] = []
    visited: set[nn.Module] = set()

    def dfs(m: nn.Module) -> None:
        if m in visited:
            return
        if m not in roots and get_module_state(m) is not None:
            return  # nested fully_shard: managed by its own state
        visited.add(m)
        for child in m.children():
            dfs(child)
        out.append(m)

    for r in roots:
        dfs(r)
    return out


def _managed_states(modules: list[nn.Module], ignored_params: set[nn.Parameter] | None) -> tuple[list[nn.Parameter], list[torch.Tensor]]:
    params: list[nn.Parameter] = []
    buffers: list[torch.Tensor] = []
    seen_p: set[nn.Parameter] = set()
    seen_b: set[torch.Tensor] = set()
    for m in modules:
        for p in m.parameters(recurse=False):
            if p in seen_p or (ignored_params is not None and p in ignored_params):
                continue
            if p.dim() == 0:
                raise ValueError("fully_shard does not support 0-dim parameters; view them as 1-D first")
            seen_p.add(p)
            params.append(p)
        for b in m.buffers(recurse=False):
            if b not in seen_b:
                seen_b.add(b)
                buffers.append(b)
    return params, buffers


def _move_states_to_device(params: list[nn.Parameter], buffers: list[torch.Tensor], device: torch.device) -> None:
    """Buffers (and parameters that are neither on the target device nor on meta) move to the device;
    meta tensors become uninitialised device tensors (parameters are initialised later through the
    sharded parameters, so the full meta parameter is never materialised)."""
    for t in itertools.chain(params, buffers):
        if t.device == device:
            continue
        if t.device.type == "meta":
            if isinstance(t, nn.Parameter):
                continue
            t.data = torch.empty_like(t, device=device)
        elif hasattr(t.data, "__tensor_flatten__"):
            # wrapper tensor subclass (inner tensors): `.data =` would only move the outer shell, so swap the whole object
            # (``ya_fsdp/_init.py:209-216``)
            with torch.no_grad():
                moved = nn.Parameter(t.to(device), requires_grad=t.requires_grad) if isinstance(t, nn.Parameter) else t.to(device)
            torch.utils.swap_tensors(t, moved)
        else:
            t.data = t.data.to(device)


# --------------------------------------------------------------------------------------- entry point
def _split_by_all_gather_dtype(params: list[nn.Parameter], mp_policy: MixedPrecisionPolicy) -> list[list[nn.Parameter]]:
    """Parameters whose class is listed in ``all_gather_dtype_to_param_cls`` travel in that dtype: one list per dtype,
    ordinary parameters first (``ya_fsdp/_param_group.py:194-228``)."""
    mapping = mp_policy.all_gather_dtype_to_param_cls
    if not mapping:
        return [params]
    buckets: dict[Any, list[nn.Parameter]] = {None: []}
    for p in params:
        key = None
        for dtype, classes in mapping.items():
            if isinstance(p.data, classes if isinstance(classes, tuple) else (classes,)):
                key = dtype
                break
        buckets.setdefault(key, []).append(p)
    return [ps for ps in buckets.values() if ps]


def fully_shard(
    module: nn.Module | list[nn.Module],
    *,
    mesh: DeviceMesh | None = None,
    reshard_after_forward: bool | None = True,
    mp_policy: MixedPrecisionPolicy = MixedPrecisionPolicy(),
    ignored_params: set[nn.Parameter] | None = None,
    shard_alignment: int = 8,
) -> Any:
    """Shard the parameters of ``module`` (or of a list of modules that run forward together) over a 1-D mesh.

    Parameters become ``RaggedShardDTensor`` views of one flat shard per group; they are all-gathered
    before the group's forward / backward and freed afterwards; gradients are reduce-scattered after the
    group's backward.  Apply bottom-up (each transformer layer, then a parameter-less root).

    ``reshard_after_forward``: ``True`` / ``False`` free / keep the gathered parameters after forward and
    leave *auto mode* on (the last group of each rotating buffer keeps its parameters, since backward needs
    them right away); ``None`` always frees and turns auto mode off.
    """
    if isinstance(module, (nn.ModuleList, nn.ModuleDict)):
        raise ValueError(f"fully_shard does not support containers that do not implement forward: {module}")
    mesh = mesh or _default_mesh()
    if mesh.ndim != 1:
        raise ValueError(f"fully_shard expects a 1D DeviceMesh but got {mesh}")
    if reshard_after_forward is not None and not isinstance(reshard_after_forward, bool):
        raise ValueError(f"reshard_after_forward must be a bool or None, got {reshard_after_forward!r}")
    mesh_info = ShardMeshInfo(mesh, 0)
    device = _device_from_mesh(mesh)
    auto = reshard_after_forward is not None
    reshard = True if reshard_after_forward is None else reshard_after_forward

    arg_module = module
    modules = (module,) if isinstance(module, nn.Module) else _root_modules(module)
    state = FSDPState()
    state.init(modules, device, mp_policy, auto)

    for root_m in modules:  # remember the enclosing state so that a nested module can find its root before any forward
        for sub in root_m.modules():
            sub_state = get_module_state(sub)
            if sub_state is not None and sub_state is not state:
                sub_state._outer = state

    managed = _managed_modules(modules, ignored_params)
    params, buffers = _managed_states(managed, ignored_params)
    _move_states_to_device(params, buffers, device)
    if params:
        by_class = _split_by_all_gather_dtype(params, mp_policy)
        groups = [ParamGroup(ps, modules, mesh_info, reshard, device, mp_policy, shard_alignment) for ps in by_class]
        state._param_group = groups[0] if len(groups) == 1 else GroupSet(groups)  # type: ignore[assignment]

    for m in modules:
        cls = m.__class__
        new_cls = _cls_to_fsdp_cls.get(cls)
        if new_cls is None:
            new_cls = type(f"YaFSDP{cls.__name__}", (YaFSDPModule, cls), {"__deepcopy__": _unimplemented_deepcopy})
            _cls_to_fsdp_cls[cls] = new_cls
        m.__class__ = new_cls
    return arg_module


def _unimplemented_deepcopy(*args: Any, **kwargs: Any) -> NoReturn:
    raise AssertionError("fully_shard modules do not support deepcopy; copy the model before sharding it")


# --------------------------------------------------------------------------------------- module mixin
class UnshardHandle:
    """Returned by ``unshard(async_op=True)``; ``wait()`` makes the gathered parameters usable."""

    def __init__(self, group: ParamGroup | None):
        self._group = group

    def wait(self) -> None:
        if self._group is not None:
            self._group.wait_for_unshard()
            self._group = None


class YaFSDPModule:
    """Methods added to every module that ``fully_shard`` was applied to."""

    def __new__(cls, *args: Any, **kwargs: Any) -> Any:
        # constructing YaFSDP<Cls>(...) builds the original class (index 2 of the MRO: [YaFSDPCls, YaFSDPModule, Cls, ...])
        orig_cls = cls.__mro__[2]
        return orig_cls.__new__(orig_cls, *args, **kwargs)

    def _get_fsdp_state(self) -> FSDPState:
        state = get_module_state(cast(nn.Module, self))
        if state is None:
            raise AssertionError(f"no fully_shard state on {self.__class__.__name__}")
        return state

    def _states(self, recurse: bool) -> list[FSDPState]:
        me = cast(nn.Module, self)
        mods = list(me.modules()) if recurse else [me]
        out: list[FSDPState] = []
        for m in mods:
            s = get_module_state(m)
            if s is not None and s not in out:
                out.append(s)
        return out

    def reshard(self) -> None:
        """Free the gathered parameters (the sharded ones are registered again)."""
        if (g := self._get_fsdp_state()._param_group) is not None:
            g.reshard()

    def unshard(self, async_op: bool = False) -> UnshardHandle | None:
        """Gather this module's parameters now.  With ``async_op`` the gather is only enqueued and the
        returned handle's ``wait()`` (or the module's next pre-forward) finishes it."""
        state = self._get_fsdp_state()
        root = state
        while root._outer is not None:
            root = root._outer
        root._lazy_init()
        g = state._param_group
        if g is not None:
            g.unshard(async_op=async_op)
        handle = UnshardHandle(g)
        if async_op:
            return handle
        handle.wait()
        return None

    def set_is_last_backward(self, is_last_backward: bool) -> None:
        """``False`` postpones the end-of-backward bookkeeping (waiting for the last reduction) to a later
        backward: for pipeline schedules that run several backward passes per step."""
        self._get_fsdp_state()._state_ctx.is_last_backward = is_last_backward

    def set_requires_gradient_sync(self, requires_gradient_sync: bool, *, recurse: bool = True) -> None:
        """Turn the gradient reduce-scatter off (gradients accumulate unreduced in the reduce buffer) or on."""
        states = self._states(recurse)
        for s in states:
            if s._param_group is not None:
                s._param_group.reduce_grads = requires_gradient_sync
        root = self._get_fsdp_state()
        if root._is_root:
            root._validate_shared_state()

    def set_reshard_after_forward(self, reshard_after_forward: bool, recurse: bool = True) -> None:
        if not isinstance(reshard_after_forward, bool):
            raise ValueError(f"reshard_after_forward should be a bool, got {type(reshard_after_forward)}")
        for s in self._states(recurse):
            s._auto_reshard_after_forward = False
            if s._param_group is not None:
                s._param_group.reshard_after_forward = reshard_after_forward

    def set_reshard_after_backward(self, reshard_after_backward: bool, *, recurse: bool = True) -> None:
        for s in self._states(recurse):
            if s._param_group is not None:
                s._param_group.reshard_after_backward = reshard_after_backward

    def set_modules_to_forward_prefetch(self, modules: list["YaFSDPModule"]) -> None:
        """Gather these modules' parameters right after this module's own gather in forward."""
        _assert_all_fsdp_modules(modules)
        self._get_fsdp_state()._states_to_forward_prefetch = [m._get_fsdp_state() for m in modules]

    def set_modules_to_backward_prefetch(self, modules: list["YaFSDPModule"]) -> None:
        """Replace the default backward prefetch (the previous module in forward order) by this list."""
        _assert_all_fsdp_modules(modules)
        self._get_fsdp_state()._states_to_backward_prefetch = [m._get_fsdp_state() for m in modules]

    def set_post_optim_event(self, event: Any) -> None:
        """The next root pre-forward waits only for this event (recorded after the optimizer step) instead
        of the whole compute stream."""
        self._get_fsdp_state()._state_ctx.post_optim_event = event

    def set_unshard_in_backward(self, unshard_in_backward: bool) -> None:
        """``False`` skips the backward gather for modules whose parameters are not needed in backward."""
        if (g := self._get_fsdp_state()._param_group) is not None:
            g.unshard_in_backward = unshard_in_backward

    def set_gradient_divide_factor(self, factor: float) -> None:
        """Divide reduced gradients by ``factor`` instead of the shard world size."""
        for s in self._states(True):
            if s._param_group is not None:
                s._param_group.gradient_divide_factor = factor

    def set_force_sum_reduction_for_comms(self, enable: bool) -> None:
        """Reduce with SUM and divide the shard afterwards (instead of AVG / pre-multiplied SUM)."""
        for s in self._states(True):
            if s._param_group is not None:
                s._param_group.force_sum_reduction_for_comms = enable

    def set_post_reduce_hook(self, hook: Any) -> None:
        """``hook(flat_shard)`` runs on the reduce-scatter stream on this rank's reduced flat gradient shard of every
        micro-batch, before accumulation (the place where the reference all-reduces norm gradients over the
        model-parallel group, ``ya_fsdp/ya_fsdp.py:989-990``; upstream FSDP2 calls it ``set_all_reduce_hook``)."""
        if (g := self._get_fsdp_state()._param_group) is not None:
            g.post_reduce_hook = hook

    def set_fused_gradient_reduce(self, enable: bool = True, *, recurse: bool = True) -> None:
        """Fuse the gradient reduce-scatter into the weight-gradient GEMMs (peer-memory backend, fp32 reduction): the GEMM
        epilogue pushes each fp32 row of dW over NVLink into the slot that the owning rank keeps for this rank, and the
        owner sums its slots locally.  Replaces copy-into-buffer + reduce-scatter + divide + accumulate
        (``ya_fsdp/_param_group.py:655-771``, ``ya_fsdp/_collectives.py:93-218``).  For groups whose every parameter gets
        exactly one gradient per backward pass (no weight used twice); other backends ignore the flag."""
        for state in self._states(recurse):
            if state._param_group is not None:
                state._param_group.fused_reduce = enable

    def set_fused_gather(self, enable: bool = True, prefix_params: Iterable[nn.Parameter] = ()) -> None:
        """Fuse this module's all-gather into its first GEMM (peer-memory backend, bf16 gather): a forward pass whose gather
        has not been started yet (nothing could prefetch it: the first layer of a step) skips the all-gather; the module's
        forward redeems ``ParamGroup.take_in_kernel_gather`` and runs ``kernels.gemm_gathered``, which pulls the whole layer
        from the peers while it computes (replaces ``ya_fsdp/_collectives.py:47-72`` + the GEMM).  ``prefix_params``: the
        parameters read before that GEMM (copied ahead of it).  Only for modules whose forward does so (the Llama decoder
        layer of this package)."""
        g = self._get_fsdp_state()._param_group
        if g is None:
            return
        wanted = {id(p) for p in prefix_params}
        for grp in getattr(g, "groups", [g]):
            grp.fused_gather = enable
            grp.fused_gather_prefix = [sp.index for sp in grp.params if id(sp.sharded_param) in wanted or id(sp.unsharded_param) in wanted]

    def set_secondary_shard_group(self, group: Any, *, recurse: bool = False) -> None:
        """Hierarchical partitioning for this module's parameter group: gather the weights for backward inside ``group``
        (e.g. the ranks of one node) from a secondary shard saved after the forward all-gather."""
        for state in self._states(recurse):
            if state._param_group is not None:
                state._param_group.set_secondary_shard_group(group)

    def set_comm_backend(self, name: Any, *, num_grad_buffers: int | None = None, **backend_options: Any) -> None:
        """Root only, before the first forward: ``"torch"`` (NCCL / gloo), ``"symm"`` (peer-memory kernels),
        ``"auto"``, or a ready :class:`~yafsdp_b200.comm.backends.CommBackend` instance; optionally the number of rotating
        gradient buffers.  ``backend_options`` go to the backend's constructor, e.g. ``ag_transport="ce"``,
        ``rs_transport="sm"``, ``multicast=True`` for the peer-memory backend."""
        state = self._get_fsdp_state()
        if state._is_root is not None:
            raise RuntimeError("set_comm_backend must be called before the first forward")
        state._backend_name = name
        state._backend_options = dict(backend_options)
        state._num_grad_buffers = num_grad_buffers

    def _apply(self, *args: Any, **kwargs: Any) -> Any:
        # .to() / .float() / .cuda(): run on the sharded parameters, then rebuild the flat master from them
        self.reshard()
        ret = super()._apply(*args, **kwargs)  # type: ignore[misc]
        for s in self._states(True):
            if s._param_group is not None:
                s._param_group.reset_sharded_params()
        return ret


def _assert_all_fsdp_modules(modules: Iterable[Any]) -> None:
    for m in modules:
        if not isinstance(m, YaFSDPModule):
            raise ValueError(f"Expects YaFSDPModule but got {type(m)}: {m}")
