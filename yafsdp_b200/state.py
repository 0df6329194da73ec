"""Runtime scheduler: per-module state, forward / backward hooks, root lazy init, buffer sharing.

Flow of one step (``ya_fsdp/_state.py:39-678`` is the reference for the behaviour):

* the root's pre-forward runs the lazy init once (collects every state under the root in
  ``named_modules()`` order, assigns the rotating buffers, validates the sharing, builds the views);
* a group's pre-forward gathers its parameters on the side stream and swaps them into the module; its
  post-forward swaps the sharded parameters back and releases the buffer;
* tensor hooks on the forward outputs give the pre-backward (re-gather + prefetch of the previous
  group), an identity autograd node over the inputs gives the post-backward (gradient reduction);
* a callback queued on the autograd engine finishes the step (groups autograd never reached, waits
  for the last reduction, clears per-step state).
"""

from __future__ import annotations

import functools
from typing import Any

import torch
import torch.nn as nn
from torch.autograd import Variable
from torch.autograd.graph import register_multi_grad_hook
from torch.profiler import record_function
from torch.utils._pytree import tree_flatten, tree_map, tree_unflatten

from .api import MixedPrecisionPolicy
from .comm.backends import CommBackend, make_backend
from .common import TrainingState, cast_fp_tensor, logger
from .group import BufferContext, CommContext, ParamGroup, RegisterPostBackwardFunction

__all__ = ["FSDPState", "StateContext", "get_module_state"]

_STATE_ATTR = "_yafsdp_state"


def get_module_state(module: nn.Module) -> "FSDPState | None":
    return module.__dict__.get(_STATE_ATTR)


class StateContext:
    """Shared by every state under one root."""

    def __init__(self) -> None:
        self.all_states: list[FSDPState] = []
        self.iter_forward_root: FSDPState | None = None
        self.post_backward_final_callback_queued = False
        self.is_last_backward = True
        self.post_optim_event: Any = None


class FSDPState:
    def __init__(self) -> None:
        self._param_group: ParamGroup | None = None
        self._is_root: bool | None = None
        self._state_ctx = StateContext()
        self._comm_ctx = CommContext()
        self._training_state = TrainingState.IDLE
        self._modules: tuple[nn.Module, ...] = ()
        self._pre_backward_hook_handles: list[Any] = []
        self._hook_handles: list[Any] = []
        self._modules_to_run_forward: set[nn.Module] = set()
        self._states_to_forward_prefetch: list[FSDPState] = []
        self._states_to_backward_prefetch: list[FSDPState] = []
        self._module_fqn: str | None = None
        self._backend_name: Any = None
        self._backend_options: dict[str, Any] = {}
        self._num_grad_buffers: int | None = None
        self._outer: FSDPState | None = None  # state of the enclosing fully_shard module, if any

    # ------------------------------------------------------------------ construction
    def init(self, modules: tuple[nn.Module, ...], device: torch.device, mp_policy: MixedPrecisionPolicy,
             auto_reshard_after_forward: bool) -> None:
        for m in modules:
            if get_module_state(m) is not None:
                raise AssertionError("fully_shard was already applied to this module")
            m.__dict__[_STATE_ATTR] = self
        self._modules = modules
        self._device = device
        self._mp_policy = mp_policy
        self._auto_reshard_after_forward = auto_reshard_after_forward
        if len(modules) == 1:
            self._hook_handles.append(modules[0].register_forward_pre_hook(self._pre_forward, prepend=True, with_kwargs=True))
            self._hook_handles.append(modules[0].register_forward_hook(self._post_forward, prepend=False))
        else:
            self._register_group_forward_hooks(modules)

    def _register_group_forward_hooks(self, modules: tuple[nn.Module, ...]) -> None:
        """Several modules in one group: pre-forward fires on the first that runs, post-forward on the last."""
        modules_set = set(modules)

        def pre(module: nn.Module, args: Any, kwargs: Any) -> Any:
            if self._training_state == TrainingState.PRE_BACKWARD:
                return None  # activation-checkpoint recompute of some of the modules: not a forward pass of the group
            if not self._modules_to_run_forward:
                self._modules_to_run_forward = set(modules_set)
                return self._pre_forward(module, args, kwargs)
            return None

        def post(module: nn.Module, args: Any, output: Any) -> Any:
            if self._training_state == TrainingState.PRE_BACKWARD:
                return None
            self._modules_to_run_forward.discard(module)
            if not self._modules_to_run_forward:
                return self._post_forward(module, args, output)
            return None

        for m in modules:
            self._hook_handles.append(m.register_forward_pre_hook(pre, prepend=True, with_kwargs=True))
            self._hook_handles.append(m.register_forward_hook(post, prepend=False, always_call=True))

    # ------------------------------------------------------------------ root
    def _root_pre_forward(self, module: nn.Module, args: Any, kwargs: Any) -> tuple[Any, Any]:
        self._lazy_init()
        if self._state_ctx.iter_forward_root is not None:
            return args, kwargs
        logger.debug("root pre-forward")
        self._state_ctx.iter_forward_root = self
        if self._device.type == "cuda":
            from .ops import kernels

            kernels.poll_status()  # a bounded device-side wait that ran out during the previous step surfaces here
        with record_function("YaFSDP::root_pre_forward"):
            st = self._comm_ctx.streams
            assert st is not None
            # a previous forward that was never followed by a backward left its last groups gathered: release them
            if self._comm_ctx.post_forward_order and not self._state_ctx.post_backward_final_callback_queued:
                for s in self._state_ctx.all_states:
                    g = s._param_group
                    if g is not None and g._kept_after_forward and g.reshard_after_backward and g._training_state == TrainingState.IDLE:
                        g.reshard()
                        g._kept_after_forward = False
                        g._post_forward_indices.clear()
                self._comm_ctx.post_forward_order.clear()
            # the gathers of this step read what the optimizer step wrote on the compute stream
            if (ev := self._state_ctx.post_optim_event) is not None:
                st.wait_event(self._comm_ctx.all_gather_stream, ev)
                self._state_ctx.post_optim_event = None
            else:
                st.wait_stream(self._comm_ctx.all_gather_stream, st.current())
            self._comm_ctx.sync_gather_inputs(self._comm_ctx.all_gather_stream)
            if self._device.type == "cuda":
                with record_function("YaFSDP::inputs_to_device"):
                    args, kwargs = tree_map(lambda x: x.to(self._device, non_blocking=True) if isinstance(x, torch.Tensor) and x.device.type == "cpu" else x, (args, kwargs))
        return args, kwargs

    def _lazy_init(
        self,
        allow_no_grad_reduce: bool = False,
        param_group_to_data_buffer_ctx_idx: dict[ParamGroup, int] | None = None,
        param_group_to_grad_buffer_ctx_idx: dict[ParamGroup, int] | None = None,
        *,
        num_grad_buffers: int | None = None,
        comm_backend: str | CommBackend | None = None,
    ) -> None:
        """Root-only, once.  ``allow_no_grad_reduce`` gives every group its own grad buffer (needed for
        ``set_requires_gradient_sync(False)`` on more than one group); the two maps override the default
        round-robin buffer assignment; ``num_grad_buffers`` rotates that many grad buffers (default 1, the
        Llama trainer uses 2 so that a layer's weight-gradient kernels never wait for the previous layer's
        reduction); ``comm_backend`` selects ``"torch"`` / ``"symm"`` / ``"auto"``."""
        if self._is_root is not None:
            return
        self._is_root = True
        if len(self._modules) != 1:
            raise RuntimeError(f"fully_shard requires a single root module but got {self._modules}")
        root = self._modules[0]
        visited: set[FSDPState] = set()
        for name, m in root.named_modules():
            state = get_module_state(m)
            if state is None or state in visited:
                continue
            visited.add(state)
            if state is not self:
                if state._is_root is not None:
                    raise RuntimeError(f"fully_shard module {name!r} ran forward before its root; call the root first")
                state._is_root = False
            state._module_fqn = name
            self._state_ctx.all_states.append(state)
        self._init_fqns()
        self._init_shared_state(
            allow_no_grad_reduce, param_group_to_data_buffer_ctx_idx, param_group_to_grad_buffer_ctx_idx,
            num_grad_buffers if num_grad_buffers is not None else self._num_grad_buffers,
            comm_backend if comm_backend is not None else self._backend_name,
        )
        self._validate_shared_state()
        for state in self._state_ctx.all_states:
            g = state._param_group
            if g is not None:
                g.lazy_init(self._comm_ctx, g.data_ctx, g.grad_ctx)  # type: ignore[arg-type]
                self._comm_ctx.groups.extend(getattr(g, "groups", [g]))

    def _init_fqns(self) -> None:
        root = self._modules[0]
        module_to_name = {m: n for n, m in root.named_modules()}
        param_to_name = {p: n for n, p in root.named_parameters(remove_duplicate=False)}
        for state in self._state_ctx.all_states:
            g = state._param_group
            if g is None:
                continue
            names = [module_to_name.get(m, "?") for m in g.modules]
            g._module_fqn = names[0] if len(names) == 1 else "[" + ", ".join(names) + "]"
            for sp in g.params:
                sp.fqn = param_to_name.get(sp.sharded_param)  # type: ignore[arg-type]

    def _init_shared_state(self, allow_no_grad_reduce: bool, data_map: Any, grad_map: Any, num_grad_buffers: int | None,
                           comm_backend: Any) -> None:
        groups = [s._param_group for s in self._state_ctx.all_states if s._param_group is not None]
        pg = groups[0].process_group if groups else None
        if isinstance(comm_backend, CommBackend):
            backend = comm_backend
        else:
            backend = make_backend(comm_backend, self._device, pg, **self._backend_options)
        self._comm_ctx.lazy_init(self._device, backend)
        for s in self._state_ctx.all_states:
            s._state_ctx = self._state_ctx
            s._comm_ctx = self._comm_ctx
        if not groups:
            return
        # ---- data buffers: two per process group, or one per group when nobody reshards after forward
        nobody_reshards = all(not g.reshard_after_forward for g in groups if not g.dedicated_buffers)
        by_pg: dict[Any, list[ParamGroup]] = {}
        for g in groups:
            by_pg.setdefault(g.process_group, []).append(g)
        self._data_ctxs: list[BufferContext] = []
        self._grad_ctxs: list[BufferContext] = []
        for all_pg_groups in by_pg.values():
            # a group that stays gathered while others come and go (e.g. all norm weights of a model) owns its buffers
            for g in all_pg_groups:
                if g.dedicated_buffers:
                    g.data_ctx = BufferContext("data", len(self._data_ctxs))
                    g.grad_ctx = BufferContext("grad", len(self._grad_ctxs))
                    g.data_ctx.users.append(g)
                    g.grad_ctx.users.append(g)
                    self._data_ctxs.append(g.data_ctx)
                    self._grad_ctxs.append(g.grad_ctx)
            pg_groups = [g for g in all_pg_groups if not g.dedicated_buffers]
            if not pg_groups:
                continue
            n_data = len(pg_groups) if nobody_reshards else min(2, len(pg_groups))
            n_grad = len(pg_groups) if allow_no_grad_reduce else min(max(1, num_grad_buffers or 1), len(pg_groups))
            data = [BufferContext("data", len(self._data_ctxs) + i) for i in range(n_data)]
            grad = [BufferContext("grad", len(self._grad_ctxs) + i) for i in range(n_grad)]
            self._data_ctxs += data
            self._grad_ctxs += grad
            for i, g in enumerate(pg_groups):
                di = data_map[g] if data_map is not None and g in data_map else i % n_data
                gi = grad_map[g] if grad_map is not None and g in grad_map else i % n_grad
                g.data_ctx = data[di]
                g.grad_ctx = grad[gi]
                data[di].users.append(g)
                grad[gi].users.append(g)
        for ctx in self._data_ctxs:
            users = [g for g in ctx.users if g.world_size > 1]
            if users:
                ctx.lazy_init(max(g.data_buffer_nbytes() for g in users), self._device, backend)
        for ctx in self._grad_ctxs:
            users = [g for g in ctx.users if not (g.world_size == 1 and g.reduce_scatter_dtype == g.orig_dtype)
                     and any(sp.requires_grad for sp in g.params)]
            if users:
                ctx.lazy_init(max(g.grad_buffer_nbytes() for g in users), self._device, backend)
        # ---- auto mode: the last user of every data buffer keeps its parameters after forward, because
        # backward would gather it again immediately
        if self._auto_reshard_after_forward:
            for ctx in self._data_ctxs:
                if ctx.users:
                    ctx.users[-1].reshard_after_forward = False

    def _validate_shared_state(self) -> None:
        groups = [s._param_group for s in self._state_ctx.all_states if s._param_group is not None]
        if not groups:
            return
        if len(self._data_ctxs) < min(2, len(groups)):
            raise AssertionError(f"Expected at least min(2, {len(groups)}) data buffers, got {len(self._data_ctxs)}")
        if len(self._grad_ctxs) < min(1, len(groups)):
            raise AssertionError(f"Expected at least min(1, {len(groups)}) grad buffers, got {len(self._grad_ctxs)}")
        for ctx in self._data_ctxs:
            keep_fwd = [g for g in ctx.users if not g.reshard_after_forward]
            if len(keep_fwd) > 1 and len(ctx.users) > 1:
                raise AssertionError(
                    "Only one parameter group across groups which share a data buffer can have reshard_after_forward=False, "
                    f"but {[g._module_fqn for g in keep_fwd]} share data buffer {ctx.index}"
                )
            keep_bwd = [g for g in ctx.users if not g.reshard_after_backward]
            if len(keep_bwd) > 1 and len(ctx.users) > 1:
                raise AssertionError(
                    "Only one parameter group across groups which share a data buffer can have reshard_after_backward=False, "
                    f"but {[g._module_fqn for g in keep_bwd]} share data buffer {ctx.index}"
                )
        for ctx in self._grad_ctxs:
            no_reduce = [g for g in ctx.users if not g.reduce_grads]
            if len(no_reduce) > 1 or (no_reduce and len(ctx.users) > 1):
                raise AssertionError(
                    "Only one parameter group across groups which share a grad buffer can have reduce_grads=False "
                    "(its unreduced gradients live in the buffer), "
                    f"but {[g._module_fqn for g in ctx.users]} share grad buffer {ctx.index}; "
                    "call root._get_fsdp_state()._lazy_init(allow_no_grad_reduce=True) before the first forward"
                )
        # two groups that share a buffer must never be active at the same time: none may be an ancestor of the other
        module_to_group: dict[nn.Module, ParamGroup] = {}
        for g in groups:
            for m in g.modules:
                module_to_group[m] = g
        root = self._modules[0]

        def walk(module: nn.Module, active: list[ParamGroup]) -> None:
            g = module_to_group.get(module)
            pushed = False
            if g is not None and g not in active:
                for a in active:
                    if a.data_ctx is g.data_ctx and not (a._shares_nothing_data() or g._shares_nothing_data()):
                        raise AssertionError(f"Param groups of {g._module_fqn} and {a._module_fqn} share a data buffer but one contains the other")
                    if a.grad_ctx is g.grad_ctx and not (a._shares_nothing_grad() or g._shares_nothing_grad()):
                        raise AssertionError(f"Param groups of {g._module_fqn} and {a._module_fqn} share a grad buffer but one contains the other")
                active.append(g)
                pushed = True
            for child in module.children():
                walk(child, active)
            if pushed:
                active.pop()

        walk(root, [])

    # ------------------------------------------------------------------ forward hooks
    @torch.compiler.disable
    def _pre_forward(self, module: nn.Module, args: Any, kwargs: Any) -> tuple[Any, Any]:
        if self._training_state == TrainingState.PRE_BACKWARD:  # activation-checkpoint recompute inside backward
            return args, kwargs
        self._training_state = TrainingState.FORWARD
        if self._is_root is None or self._is_root:
            args, kwargs = self._root_pre_forward(module, args, kwargs)
        if self._mp_policy.cast_forward_inputs and self._mp_policy.param_dtype:
            with record_function("YaFSDP::cast_forward_inputs"):
                cast = functools.partial(cast_fp_tensor, self._mp_policy.param_dtype)
                args, kwargs = tree_map(cast, args), tree_map(cast, kwargs)
        g = self._param_group
        if g is not None:
            g.pre_forward()
            args, kwargs = self._register_post_backward_hook(args, kwargs)
        for s in self._states_to_forward_prefetch:
            if (t := s._param_group) is not None:
                ParamGroup._prefetch_unshard(t, "forward")
        return args, kwargs

    @torch.compiler.disable
    def _post_forward(self, module: nn.Module, input: Any, output: Any) -> Any:
        if self._training_state == TrainingState.PRE_BACKWARD:
            return output
        if self._param_group is not None:
            self._param_group.post_forward()
        output = self._register_pre_backward_hooks(output)
        self._training_state = TrainingState.IDLE
        if self._state_ctx.iter_forward_root is self:
            self._state_ctx.iter_forward_root = None
            if not torch.is_grad_enabled():
                # no backward will follow: release what auto mode kept unsharded
                for s in self._state_ctx.all_states:
                    if s._param_group is not None:
                        s._param_group.reshard()
                self._comm_ctx.post_forward_order.clear()
        if self._mp_policy.output_dtype is not None:
            with record_function("YaFSDP::cast_forward_outputs"):
                output = tree_map(functools.partial(cast_fp_tensor, self._mp_policy.output_dtype), output)
        return output

    def _register_post_backward_hook(self, args: Any, kwargs: Any) -> tuple[Any, Any]:
        if not torch.is_grad_enabled():
            return args, kwargs
        flat, spec = tree_flatten((args, kwargs))
        idx = [i for i, t in enumerate(flat) if isinstance(t, torch.Tensor) and t.requires_grad]
        if not idx:
            return args, kwargs
        outs = RegisterPostBackwardFunction.apply(self._post_backward, *[flat[i] for i in idx])
        for i, o in zip(idx, outs):
            flat[i] = o
        return tree_unflatten(flat, spec)

    def _register_pre_backward_hooks(self, output: Any) -> Any:
        if not torch.is_grad_enabled():
            return output
        flat, _ = tree_flatten(output)
        tensors = [t for t in flat if isinstance(t, torch.Tensor) and t.requires_grad]
        if tensors:
            handle = register_multi_grad_hook(tensors, self._pre_backward, mode="any")
            self._pre_backward_hook_handles.append(handle)
        return output

    # ------------------------------------------------------------------ backward hooks
    def _pre_backward(self, grad: torch.Tensor) -> None:
        self._training_state = TrainingState.PRE_BACKWARD
        self._register_root_post_backward_final_callback()
        if self._param_group is not None:
            default_prefetch = len(self._states_to_backward_prefetch) == 0
            self._param_group.pre_backward(default_prefetch)
        for s in self._states_to_backward_prefetch:
            if (t := s._param_group) is not None:
                ParamGroup._prefetch_unshard(t, "backward")

    def _post_backward(self) -> None:
        if self._param_group is not None:
            self._param_group.post_backward()
        self._training_state = TrainingState.POST_BACKWARD

    def _register_root_post_backward_final_callback(self) -> None:
        if self._state_ctx.post_backward_final_callback_queued:
            return
        self._state_ctx.post_backward_final_callback_queued = True
        Variable._execution_engine.queue_callback(self._root_post_backward_final_callback)

    def _root_post_backward_final_callback(self) -> None:
        logger.debug("root post-backward final callback")
        with record_function("YaFSDP::root_post_backward_callback"):
            ctx = self._state_ctx
            for state in ctx.all_states:
                g = state._param_group
                if g is not None and state._training_state == TrainingState.PRE_BACKWARD:
                    # autograd never ran this group's post-backward node (its inputs need no gradient, e.g. embeddings)
                    g.post_backward()
                state._training_state = TrainingState.IDLE
                if g is not None:
                    g._training_state = TrainingState.IDLE
                for h in state._pre_backward_hook_handles:
                    h.remove()
                state._pre_backward_hook_handles.clear()
            if ctx.is_last_backward:
                for state in ctx.all_states:
                    if state._param_group is not None:
                        state._param_group.finalize_backward()
                self._comm_ctx.post_forward_order.clear()
            ctx.post_backward_final_callback_queued = False
