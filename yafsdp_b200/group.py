"""Parameter groups: flat ragged shards, rotating gather / reduce buffers, unshard / reshard.

One ``ParamGroup`` holds every parameter that one ``fully_shard`` call manages:

* a persistent flat master shard (original dtype, e.g. fp32) and a flat sharded gradient, both of
  ``layout.shard_numel`` elements; every ``RaggedShardDTensor`` parameter / gradient is a view of them;
* a flat all-gather input in the compute dtype (bf16 under mixed precision), refreshed from the master
  once per optimizer step (or written directly by the fused AdamW kernel);
* views into a *shared, rotating* gather buffer (the unsharded parameters) and a shared reduce buffer
  (the unsharded fp32 gradients).  Buffers have an owner and a release event instead of going through
  the caching allocator, so a layer's gather can be enqueued on the communication stream as soon as the
  previous owner released the buffer.

Blackwell-specific design on top of the reference's scheme (``ya_fsdp/_param_group.py:32-992``,
``ya_fsdp/_param.py:44-372``):

* *gradient sinks*: every unsharded parameter exposes ``_yf_grad_sink``; weight-gradient kernels (the
  tcgen05 GEMM with an fp32 accumulating epilogue, RMSNorm / embedding backward) write straight into
  the fp32 reduce buffer, so the bf16 gradient tensor, its cast and the copy into the flat buffer
  disappear.  Plain ``autograd`` gradients (``param.grad``) still work and are copied in post-backward.
* *single-rank aliasing*: with one rank the gather input IS the unsharded parameter storage and the
  sharded gradient IS the reduce buffer, so there is no gather copy and no reduce copy at all.
* the reduce-scatter fuses the averaging and the accumulation into the sharded gradient.
"""

from __future__ import annotations

import contextlib
from typing import Any, Callable, Iterator, NamedTuple

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.profiler import record_function

from .api import MixedPrecisionPolicy
from .comm.backends import CommBackend, TorchBackend, gradient_divide_factors
from .common import ShardMeshInfo, TrainingState, is_backward_running, logger
from .layout import FlatLayout, ParamPlacement
from .tensor import RaggedShard, RaggedShardDTensor, RaggedSpec, _contiguous_stride

__all__ = ["ParamGroup", "BufferContext", "CommContext", "GradSink", "ShardedParam"]


# ----------------------------------------------------------------------------------------- streams
class _DeviceStreams:
    """Stream / event helper that degrades to no-ops on CPU."""

    def __init__(self, device: torch.device):
        self.device = device
        self.is_cuda = device.type == "cuda"

    def current(self) -> Any:
        return torch.cuda.current_stream(self.device) if self.is_cuda else None

    def new_stream(self, priority: int = 0) -> Any:
        return torch.cuda.Stream(self.device, priority=priority) if self.is_cuda else None

    def record(self, stream: Any = None) -> Any:
        if not self.is_cuda:
            return None
        ev = torch.cuda.Event()
        ev.record(stream if stream is not None else self.current())
        return ev

    def wait_event(self, stream: Any, event: Any) -> None:
        if self.is_cuda and event is not None:
            (stream if stream is not None else self.current()).wait_event(event)

    def wait_stream(self, stream: Any, other: Any) -> None:
        if self.is_cuda and stream is not None and other is not None:
            stream.wait_stream(other)

    @contextlib.contextmanager
    def use(self, stream: Any) -> Iterator[None]:
        if self.is_cuda and stream is not None:
            with torch.cuda.stream(stream):
                yield
        else:
            yield


class BufferContext:
    """One shared rotating buffer (bytes) with an owner and a release event."""

    def __init__(self, kind: str, index: int):
        self.kind = kind  # "data" | "grad"
        self.index = index
        self.nbytes = 0
        self.tensor: torch.Tensor | None = None
        self.owner: "ParamGroup | None" = None
        self.release_event: Any = None
        self.users: list["ParamGroup"] = []

    def lazy_init(self, nbytes: int, device: torch.device, backend: CommBackend) -> None:
        if self.tensor is not None and self.nbytes >= nbytes:
            return
        self.nbytes = nbytes
        self.tensor = backend.alloc(nbytes, torch.uint8, device, "gather_output" if self.kind == "data" else "reduce_input")

    def view(self, dtype: torch.dtype, numel: int, byte_offset: int = 0) -> torch.Tensor:
        assert self.tensor is not None
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        return self.tensor[byte_offset : byte_offset + nbytes].view(dtype)

    def __repr__(self) -> str:
        return f"BufferContext({self.kind}#{self.index}, {self.nbytes} B)"


class CommContext:
    """Streams shared by all groups of one root.  The reference runs all-gathers and reduce-scatters on ONE
    high-priority side stream (``ya_fsdp/_param_group.py:74-101``); here they get a stream each, so a backward
    prefetch is never queued behind the previous layer's reduction and its cross-GPU barriers."""

    def __init__(self) -> None:
        self.streams: _DeviceStreams | None = None
        self.all_gather_stream: Any = None
        self.reduce_scatter_stream: Any = None
        self.post_forward_order: list["ParamGroup"] = []
        self.backend: CommBackend = TorchBackend()
        self.groups: list["ParamGroup"] = []  # every group under the root, in module order (set at the root's lazy init)
        self.secondary_synced = False  # hierarchical partitioning: the ranks have met since the secondary shards were written

    def lazy_init(self, device: torch.device, backend: CommBackend | None = None) -> None:
        self.streams = _DeviceStreams(device)
        if backend is not None:
            self.backend = backend
        self.all_gather_stream = self.streams.new_stream(priority=-1)
        if self.backend.prefers_single_comm_stream:
            self.reduce_scatter_stream = self.all_gather_stream
        else:
            self.reduce_scatter_stream = self.streams.new_stream(priority=-1)

    def sync_gather_inputs(self, stream: Any) -> None:
        """Peer-memory backends: peers pull this rank's shards straight out of its gather inputs, so all of them are
        brought up to date together (not lazily per group) and nobody pulls before every rank has finished writing its
        own.  Runs on ``stream``; a no-op for backends that exchange data through ``torch.distributed``."""
        if not self.backend.needs_registered_buffers:
            return
        assert self.streams is not None
        with self.streams.use(stream):
            for g in self.groups:
                if g._lazy_inited and not g._alias_data:
                    g.wait_optimizer()
                    g._refresh_gather_input()
            self.backend.step_barrier()

    def get_all_gather_stream(self, async_op: bool, training_state: TrainingState) -> Any:
        assert self.streams is not None
        if not async_op and training_state in (TrainingState.FORWARD, TrainingState.PRE_BACKWARD):
            return self.all_gather_stream
        return self.streams.current()


class GradSink:
    """Destination of one parameter's weight gradient inside the flat fp32 reduce buffer.

    ``begin()`` returns ``(fp32 view with the parameter's shape, accumulate)``: the first write of a
    backward pass overwrites (the buffer holds another layer's stale data), later writes accumulate.
    Kernels that can only add (atomics) call ``begin(zero=True)``.
    """

    __slots__ = ("group", "index", "view")

    def __init__(self, group: "ParamGroup", index: int, view: torch.Tensor):
        self.group = group
        self.index = index
        self.view = view

    def norm_target(self, accumulate: bool) -> torch.Tensor | None:
        """Where a kernel that writes this gradient once, completely and finally may add the sum of its squares (the
        gradient norm then needs no pass of its own).  ``None`` when the value written is not final: another write will
        accumulate into it, or a reduction over ranks follows."""
        g = self.group
        if g._norm_sq is None or not g._alias_grad:
            return None
        if accumulate:
            g._norm_fused_ok = False
            return None
        return g._norm_sq

    def would_accumulate(self) -> bool:
        """True when the next write adds to a value that is already there: an earlier write of this backward pass, or
        (single rank, where the sink is the persistent sharded gradient itself) the sum of earlier micro-batches."""
        g = self.group
        if g._sink_written[self.index]:
            return True
        if g._alias_grad:
            sp = g.params[self.index].sharded_param
            return sp is not None and sp.grad is not None
        return False

    # ---- fused gradient reduction: the producing kernel pushes the gradient to the ranks that own it
    def pushes(self) -> bool:
        """True when this backward pass sends the group's gradients straight to their owners' reduce-scatter slots
        (``ParamGroup.fused_reduce``) instead of writing them into the local flat buffer."""
        return self.group._push_mode()

    @property
    def local_ok(self) -> bool:
        """Kernels may write this sink locally (fp32 view of the flat reduce buffer).  With a bf16 reduce dtype the sink
        only exists for pushing: the pushed pieces are rounded to bf16 on the way and summed in fp32 by the owner."""
        return self.view.dtype == torch.float32

    def begin_push(self) -> tuple[Any, int, int, int, int, bool]:
        """Claim the reduce buffers for a pushed write of the whole parameter; returns what the pushing kernel needs:
        ``(peer buffer pointers, flat offset of the parameter, shard size, rank, world, bf16 wire format)``."""
        g = self.group
        g._acquire_grad_buffer()
        if g._sink_written[self.index]:
            raise RuntimeError(
                f"parameter {g.params[self.index].fqn!r} receives a second gradient in one backward pass: pushed gradients "
                "cannot accumulate at the owner; disable fused_reduce for this group")
        g._sink_counts[self.index] += 1
        g._sink_written[self.index] = True
        g._pushed = True
        return (g._push_ptrs, g.layout.flat_offsets[self.index], g.layout.shard_numel, g.rank, g.world_size,
                g.reduce_scatter_dtype == torch.bfloat16)

    def push_from(self, grad: torch.Tensor | None) -> None:
        """Push a complete fp32 gradient of this parameter (``None``: zeros) that some other kernel produced."""
        from .ops import kernels

        ptrs, off, shard, rank, world, bf16 = self.begin_push()
        kernels.push_flat(None if grad is None else grad.reshape(-1), self.group.params[self.index].numel, off, ptrs, shard, rank, world,
                          wire_bf16=bf16)

    def begin(self, zero: bool = False) -> tuple[torch.Tensor, bool]:
        g = self.group
        g._acquire_grad_buffer()
        g._sink_counts[self.index] += 1
        accumulate = self.would_accumulate()
        g._sink_written[self.index] = True
        if zero and not accumulate:
            self.view.zero_()
            accumulate = True
        return self.view, accumulate


class ParamModuleInfo(NamedTuple):
    module: nn.Module
    param_name: str
    shared_modules: list[nn.Module]
    shared_param_names: list[str]


class ShardedParam:
    """Sharded and unsharded incarnations of one parameter."""

    def __init__(self, info: ParamModuleInfo, param: nn.Parameter, index: int):
        self.info = info
        self.index = index
        # A parameter that already is a DTensor of an outer 1-D mesh (expert / tensor parallel, Shard(0)) is sharded
        # further: this group flat-shards the piece that this rank holds on the outer mesh.
        self.outer_mesh: Any = None
        self.outer_placements: Any = None
        self.outer_shape: torch.Size | None = None
        inner = _outer_local(param, self)
        self.orig_shape = inner.shape
        self.orig_dtype = param.dtype
        self.numel = inner.numel()
        self.requires_grad = param.requires_grad
        # all-gather extension (``fsdp_pre_all_gather`` / ``fsdp_post_all_gather`` defined by the parameter's tensor class):
        # the local shard is presented to the hooks as an instance of that class
        data = param.data
        has_pre, has_post = hasattr(data, "fsdp_pre_all_gather"), hasattr(data, "fsdp_post_all_gather")
        if has_pre != has_post:
            raise AssertionError(f"Both fsdp_pre_all_gather and fsdp_post_all_gather should be defined if using all-gather extensions: {type(data)}")
        self.ext_cls: type | None = type(data) if has_pre else None
        self.ext_local: torch.Tensor | None = None
        self.ext_metadata: Any = None
        self.placement: ParamPlacement | None = None
        self.sharded_param: nn.Parameter | None = None
        self.sharded_grad: RaggedShardDTensor | None = None
        self.unsharded_param: nn.Parameter | None = None
        self.rs_view: torch.Tensor | None = None
        self.gathered_view: torch.Tensor | None = None
        self.sink: GradSink | None = None
        self.is_unsharded = False
        self.fqn: str | None = None

    def _set(self, p: nn.Parameter) -> None:
        # write module._parameters directly: nn.Module.__setattr__ is slow and these swaps are on the hot path
        self.info.module._parameters[self.info.param_name] = p
        for m, n in zip(self.info.shared_modules, self.info.shared_param_names):
            m._parameters[n] = p

    def to_sharded(self) -> None:
        assert self.sharded_param is not None
        self._set(self.sharded_param)
        self.is_unsharded = False

    def to_unsharded(self) -> None:
        assert self.unsharded_param is not None
        self._set(self.unsharded_param)
        self.is_unsharded = True


def _outer_local(param: torch.Tensor, sp: "ShardedParam | None" = None) -> torch.Tensor:
    """The tensor to flat-shard: the parameter itself, or its local piece when it is a DTensor of an outer mesh."""
    from torch.distributed.tensor import DTensor, Shard

    if not isinstance(param, DTensor):
        return param
    mesh, placements = param.device_mesh, param.placements
    if mesh.ndim != 1 or len(placements) != 1 or not (isinstance(placements[0], Shard) and placements[0].dim == 0):
        raise NotImplementedError(f"fully_shard composes with parameters sharded as Shard(0) on a 1-D mesh, got {placements} on {mesh}")
    if param.shape[0] % mesh.size() != 0:
        raise NotImplementedError("the outer Shard(0) dimension must divide evenly over the outer mesh")
    if sp is not None:
        sp.outer_mesh, sp.outer_placements, sp.outer_shape = mesh, placements, param.shape
    return param._local_tensor


def _get_param_module_infos(params: list[nn.Parameter], modules: tuple[nn.Module, ...]) -> list[ParamModuleInfo]:
    """Find the owning (module, name) of every parameter, plus other attributes sharing it (tied weights)."""
    params_set = set(params)
    found: dict[nn.Parameter, ParamModuleInfo] = {}
    visited: set[nn.Module] = set()
    for root in modules:
        for _, sub in root.named_modules(remove_duplicate=False):
            if sub in visited:
                continue
            visited.add(sub)
            for name, p in sub.named_parameters(recurse=False):
                if p in params_set:
                    if p not in found:
                        found[p] = ParamModuleInfo(sub, name, [], [])
                    else:
                        found[p].shared_modules.append(sub)
                        found[p].shared_param_names.append(name)
    if len(found) != len(params):
        raise AssertionError(f"some parameters are not reachable from the wrapped modules ({len(found)} of {len(params)})")
    return [found[p] for p in params]


class ParamGroup:
    """All parameters of one ``fully_shard`` call, communicated as one flat tensor."""

    def __init__(
        self,
        params: list[nn.Parameter],
        modules: tuple[nn.Module, ...],
        mesh_info: ShardMeshInfo,
        reshard_after_forward: bool,
        device: torch.device,
        mp_policy: MixedPrecisionPolicy,
        shard_alignment: int = 8,
    ):
        self.modules = modules
        self.mesh_info = mesh_info
        self.device = device
        self.mp_policy = mp_policy
        self.world_size = mesh_info.shard_mesh_size
        self.rank = mesh_info.shard_mesh_rank
        self.process_group = mesh_info.shard_process_group
        self._training_state = TrainingState.IDLE
        self._module_fqn: str | None = None

        infos = _get_param_module_infos(params, modules)
        self.params = [ShardedParam(info, p, i) for i, (info, p) in enumerate(zip(infos, params))]
        self._init_mp_dtypes(params)

        # ---- flat layout and persistent shards
        self.layout = FlatLayout([sp.numel for sp in self.params], self.world_size, shard_alignment)
        self._master = torch.zeros(self.layout.shard_numel, dtype=self.orig_dtype, device=device)
        self._sharded_grad_flat: torch.Tensor | None = None
        mesh = mesh_info.mesh
        with torch.no_grad():
            for sp, p in zip(self.params, params):
                pl = self.layout.placement(sp.index, self.rank)
                sp.placement = pl
                local = self._master[pl.shard_offset : pl.shard_offset + pl.local_numel]
                wrapper = sp.ext_cls is not None and hasattr(p.data, "__tensor_flatten__")
                if pl.local_numel and p.device.type != "meta":
                    # a wrapper subclass keeps its values in its first inner tensor: that is what the master shards
                    full = getattr(p.data, p.data.__tensor_flatten__()[0][0]) if wrapper else _outer_local(p.detach())
                    local.copy_(full.reshape(-1)[pl.global_offset : pl.global_offset + pl.local_numel])
                spec = RaggedSpec(
                    mesh, (RaggedShard(pl.local_numel, pl.global_offset, pl.shard_numels),), torch.Size(sp.orig_shape),
                    _contiguous_stride(sp.orig_shape), self.orig_dtype, sp.outer_mesh, sp.outer_placements, sp.outer_shape,
                )
                sp.sharded_param = nn.Parameter(RaggedShardDTensor(local, spec), requires_grad=sp.requires_grad)
                if wrapper:
                    # the hooks are called on a wrapper of the local size whose first inner tensor IS the master slice
                    # (``ya_fsdp/_param.py:146-155``); its other inner tensors (scales, ...) are whatever new_zeros gives them
                    shell = p.data.new_zeros(pl.local_numel)
                    inner0 = getattr(shell, shell.__tensor_flatten__()[0][0])
                    if inner0.dtype != local.dtype or inner0.numel() != pl.local_numel:
                        raise AssertionError(
                            f"all-gather extension {type(p.data).__name__}: the first inner tensor of new_zeros(n) must have n "
                            f"elements of the parameter's dtype, got {inner0.numel()} x {inner0.dtype}")
                    torch.utils.swap_tensors(inner0, self._master[pl.shard_offset : pl.shard_offset + pl.local_numel])
                    sp.ext_local = shell
                elif sp.ext_cls is not None:
                    sp.ext_local = local.as_subclass(sp.ext_cls)
                for attr in ("_yf_init_fn",):
                    if hasattr(p, attr):
                        setattr(sp.sharded_param, attr, getattr(p, attr))
                sp.to_sharded()
        del params

        # ---- runtime configuration
        self.reshard_after_forward = reshard_after_forward
        self.reshard_after_backward = True
        self.reduce_grads = True
        self.unshard_in_backward = True
        self.unshard_async_op = False
        self.gradient_divide_factor: float | None = None
        self.force_sum_reduction_for_comms = False

        # ---- set at lazy init
        self.comm_ctx: CommContext | None = None
        self.data_ctx: BufferContext | None = None
        self.grad_ctx: BufferContext | None = None
        self._lazy_inited = False
        self._ag_input: torch.Tensor | None = None
        self._ag_input_version = -1
        self._ag_input_fresh = False
        self._alias_data = False
        self._alias_grad = False
        self._ag_event: Any = None
        self._unshard_pending = False
        self._is_unsharded = False
        self._post_reduce_event: Any = None
        self._sink_written: list[bool] = [False] * len(self.params)
        self._sink_counts: list[int] = [0] * len(self.params)
        self._holds_grad_buffer = False
        self._post_forward_indices: list[int] = []
        self._partial_reduce_pending = False
        self._kept_after_forward = False
        self._has_extensions = False
        self._optim_event: Any = None
        # gradient-norm fusion (single rank): kernels that write a final gradient add its squared norm here
        self._norm_sq: torch.Tensor | None = None
        self._norm_fused_ok = False
        self.modules_to_backward_prefetch: list[Any] = []
        self.modules_to_forward_prefetch: list[Any] = []
        # who owns a shared buffer while this group uses it: the group itself, or the GroupSet it is part of; and where
        # this group's bytes start inside the shared buffers (groups of one set lie side by side)
        self._owner: Any = self
        self._data_byte_offset = 0
        self._grad_byte_offset = 0
        # called on the reduce-scatter stream with this rank's freshly reduced flat gradient shard (before it is
        # accumulated into the sharded gradient)
        self.post_reduce_hook: Callable[[torch.Tensor], None] | None = None
        # True: this group never shares its gather / reduce buffers with the rotating ones
        self.dedicated_buffers = False
        # fused gradient reduction (peer-memory backend, fp32 reduce): weight-gradient GEMMs push their rows from the epilogue
        # into the owners' reduce-scatter slots, the owners sum their slots locally; every parameter of the group must get
        # exactly one gradient per backward pass
        self.fused_reduce = False
        self._push_ptrs: Any = None
        self._pushed = False
        # fused all-gather -> GEMM (peer-memory backend): a forward pass whose gather has not been started yet does not
        # gather at all; the module's first GEMM (``kernels.gemm_gathered``) pulls the layer while it computes.  Only for
        # modules whose forward asks for it (``take_in_kernel_gather``); ``fused_gather_prefix`` lists the parameters that
        # are read before that GEMM and are therefore copied ahead of it (a norm weight).
        self.fused_gather = False
        self.fused_gather_prefix: list[int] = []
        self._in_kernel_gather: dict[str, Any] | None = None
        self._gather_counters: torch.Tensor | None = None
        self._gather_epoch = 0
        # hierarchical partitioning: a secondary shard of the gathered weights kept inside a smaller (intra-node) group
        self.secondary_group: dist.ProcessGroup | None = None
        self._secondary_shard: torch.Tensor | None = None
        self._secondary_valid = False
        self._secondary_backend: CommBackend | None = None
        self._gathered_from_secondary = False

    # ------------------------------------------------------------------ hierarchical partitioning
    def set_secondary_shard_group(self, group: dist.ProcessGroup | None) -> None:
        """Keep, after each forward all-gather, this rank's ``1 / group.size()`` piece of the gathered weights, and gather
        the weights for backward inside ``group`` only (ZeRO++-style hierarchical partitioning; the reference's
        ``hpz_first_layers_num``, ``ya_fsdp/ya_fsdp.py:832-838,925-935,1015-1021``).  ``group`` must hold consecutive
        ranks of the shard group, the same number on every rank."""
        if group is not None:
            n = group.size()
            if self.world_size % n != 0:
                raise ValueError(f"the secondary group's size {n} must divide the shard group's size {self.world_size}")
            if n == self.world_size or self.world_size == 1:
                group = None  # the primary shards already are what a group of that size would keep
        self.secondary_group = group
        self._secondary_shard = None
        self._secondary_valid = False

    def _secondary_chunk(self) -> torch.Tensor:
        assert self.secondary_group is not None
        n = self.secondary_group.size()
        chunk = self.layout.padded_numel // n
        r = self.secondary_group.rank()
        return self._data_flat[r * chunk : (r + 1) * chunk]

    def _save_secondary_shard(self) -> None:
        assert self.comm_ctx is not None
        self.comm_ctx.secondary_synced = False
        chunk = self._secondary_chunk()
        if self._secondary_shard is None:
            assert self.comm_ctx is not None
            backend = self.comm_ctx.backend
            if backend.needs_registered_buffers and hasattr(backend, "subgroup_barrier"):
                # peer-memory backend: the secondary shards live in peer-mapped memory and are pulled over NVLink
                self._secondary_shard = backend.alloc(chunk.numel(), chunk.dtype, self.device, "gather_input")
                self._secondary_backend = backend
            else:
                self._secondary_shard = torch.empty_like(chunk)
                self._secondary_backend = TorchBackend()
        self._secondary_shard.copy_(chunk)
        self._secondary_valid = True

    # ------------------------------------------------------------------ dtypes
    def _init_mp_dtypes(self, params: list[nn.Parameter]) -> None:
        orig = {p.dtype for p in params}
        if len(orig) != 1:
            raise AssertionError(f"fully_shard expects uniform original parameter dtype per group, got {orig}")
        self.orig_dtype = next(iter(orig))
        pd, rd = self.mp_policy.param_dtype, self.mp_policy.reduce_dtype
        if rd == pd:
            rd = None
        if pd == self.orig_dtype:
            pd = None
        self.param_dtype = pd
        self.reduce_dtype = rd
        self.all_gather_dtype = pd or self.orig_dtype
        self.reduce_scatter_dtype = rd or pd or self.orig_dtype
        # parameter classes that are gathered in their own dtype through the tensor-extension hooks; one all-gather dtype
        # per group, so a group holds either only such parameters (of one dtype) or none
        mapping = self.mp_policy.all_gather_dtype_to_param_cls
        if mapping:
            for dtype, classes in mapping.items():
                classes = classes if isinstance(classes, tuple) else (classes,)
                hits = [isinstance(p.data, classes) for p in params]
                if all(hits):
                    self.all_gather_dtype = dtype
                elif any(hits):
                    raise AssertionError(
                        f"a fully_shard group gathers in one dtype: put the {classes} parameters (gathered as {dtype}) in a group of their own")

    # ------------------------------------------------------------------ sizes
    @property
    def padded_unsharded_numel(self) -> int:
        return self.layout.padded_numel

    def data_buffer_nbytes(self) -> int:
        return self.layout.padded_numel * torch.empty((), dtype=self.all_gather_dtype).element_size()

    def grad_buffer_nbytes(self) -> int:
        return self.layout.padded_numel * torch.empty((), dtype=self.reduce_scatter_dtype).element_size()

    @property
    def sharded_grad_flat(self) -> torch.Tensor:
        if self._sharded_grad_flat is None:
            self._sharded_grad_flat = torch.zeros(self.layout.shard_numel, dtype=self.orig_dtype, device=self.device)
            self._bind_sharded_grads()
        return self._sharded_grad_flat

    def _bind_sharded_grads(self) -> None:
        assert self._sharded_grad_flat is not None
        for sp in self.params:
            pl = sp.placement
            assert pl is not None and sp.sharded_param is not None
            local = self._sharded_grad_flat[pl.shard_offset : pl.shard_offset + pl.local_numel]
            sp.sharded_grad = RaggedShardDTensor(local, sp.sharded_param._spec.with_dtype(local.dtype))

    @property
    def master_flat(self) -> torch.Tensor:
        return self._master

    @property
    def gather_input(self) -> torch.Tensor | None:
        return self._ag_input

    # ------------------------------------------------------------------ lazy init (root calls it once)
    def lazy_init(self, comm_ctx: CommContext, data_ctx: BufferContext, grad_ctx: BufferContext) -> None:
        self.comm_ctx = comm_ctx
        self.data_ctx = data_ctx
        self.grad_ctx = grad_ctx
        backend = comm_ctx.backend
        single = self.world_size == 1
        self._has_extensions = any(sp.ext_cls is not None for sp in self.params)
        need_cast = self.all_gather_dtype != self.orig_dtype or self._has_extensions
        # all-gather input
        if need_cast or backend.needs_registered_buffers:
            self._ag_input = backend.alloc(self.layout.shard_numel, self.all_gather_dtype, self.device, "gather_input")
        else:
            self._ag_input = self._master
        self._ag_input_version = -1
        self._ag_input_fresh = False
        # unsharded parameter storage
        self._alias_data = single
        data_flat = self._ag_input if self._alias_data else data_ctx.view(self.all_gather_dtype, self.layout.padded_numel,
                                                                          self._data_byte_offset)
        # unsharded gradient storage
        self._alias_grad = single and self.reduce_scatter_dtype == self.orig_dtype
        trainable = any(sp.requires_grad for sp in self.params)
        grad_flat = None
        if trainable:
            grad_flat = self.sharded_grad_flat if self._alias_grad else grad_ctx.view(self.reduce_scatter_dtype, self.layout.padded_numel,
                                                                                      self._grad_byte_offset)
        self._data_flat = data_flat
        self._grad_flat = grad_flat
        for sp in self.params:
            o = self.layout.flat_offsets[sp.index]
            view = data_flat[o : o + sp.numel].view(sp.orig_shape)
            if sp.outer_mesh is not None:
                from torch.distributed.tensor import DTensor

                view = DTensor.from_local(view, sp.outer_mesh, sp.outer_placements, run_check=False, shape=sp.outer_shape,
                                          stride=_contiguous_stride(sp.outer_shape))
            sp.gathered_view = view
            # extension parameters get their unsharded tensor from fsdp_post_all_gather at the first unshard
            sp.unsharded_param = nn.Parameter(view, requires_grad=sp.requires_grad) if sp.ext_cls is None else None
            sp.rs_view = grad_flat[o : o + sp.numel].view(sp.orig_shape) if grad_flat is not None else None
            # kernels write fp32 gradients into the sink; with a bf16 reduce dtype the sink only serves pushed gradients
            # (GradSink.local_ok) and the autograd .grad path is used otherwise
            sp.sink = (GradSink(self, sp.index, sp.rs_view)
                       if sp.requires_grad and self.reduce_scatter_dtype in (torch.float32, torch.bfloat16) and sp.outer_mesh is None
                       and sp.ext_cls is None and sp.rs_view is not None else None)
            if sp.unsharded_param is not None:
                sp.unsharded_param._yf_grad_sink = sp.sink  # type: ignore[attr-defined]
                sp.unsharded_param._yf_group_index = (self, sp.index)  # type: ignore[attr-defined]
        self._push_ptrs = None
        al = 8 if self.reduce_scatter_dtype == torch.bfloat16 else 4  # elements per 16 bytes on the wire
        if (grad_flat is not None and not self._alias_grad and hasattr(backend, "reduce_pushed")
                and self.reduce_scatter_dtype in (torch.float32, torch.bfloat16) and self.layout.shard_numel % al == 0
                and all(sp.numel % al == 0 and sp.sink is not None for sp in self.params if sp.requires_grad)
                and all(sp.requires_grad for sp in self.params)):
            self._push_ptrs = backend.peer_pointers(grad_flat)  # type: ignore[attr-defined]
        self._register_state_dict_hooks()
        self._lazy_inited = True

    # ------------------------------------------------------------------ gather input refresh
    def _refresh_gather_input(self) -> None:
        """master (orig dtype) -> gather input (compute dtype), once per optimizer step."""
        assert self._ag_input is not None
        if self._ag_input is self._master:
            return
        if self._ag_input_fresh and self._ag_input_version == self._master._version:
            return
        with torch.no_grad(), torch.autograd._unsafe_preserve_version_counter(self._ag_input):
            if self._has_extensions:
                for sp in self.params:
                    pl = sp.placement
                    assert pl is not None
                    dst = self._ag_input[pl.shard_offset : pl.shard_offset + pl.local_numel]
                    if sp.ext_cls is not None:
                        assert sp.ext_local is not None
                        (src,), sp.ext_metadata = sp.ext_local.fsdp_pre_all_gather(self.mesh_info.mesh)
                        if src.dtype != self.all_gather_dtype or src.numel() != pl.local_numel:
                            raise AssertionError(
                                f"fsdp_pre_all_gather must return one tensor of dtype {self.all_gather_dtype} with the local shard's "
                                f"{pl.local_numel} elements, got {src.dtype} with {src.numel()}")
                        dst.copy_(src.reshape(-1))
                    else:
                        dst.copy_(self._master[pl.shard_offset : pl.shard_offset + pl.local_numel])
            elif self._master.is_cuda and self.orig_dtype == torch.float32 and self.all_gather_dtype == torch.bfloat16:
                from .ops import kernels

                kernels.cast_f32_to_bf16_(self._master, self._ag_input)
            else:
                self._ag_input.copy_(self._master)
        self._ag_input_version = self._master._version
        self._ag_input_fresh = True

    def wait_optimizer(self) -> None:
        """An optimizer that updates this group on a side stream (overlapped with the next forward) leaves an event here;
        whoever reads the parameters next on the current stream waits for it first."""
        ev = self._optim_event
        if ev is not None:
            self._optim_event = None
            if self.comm_ctx is not None and self.comm_ctx.streams is not None:
                self.comm_ctx.streams.wait_event(None, ev)
            elif self.device.type == "cuda":
                torch.cuda.current_stream(self.device).wait_event(ev)

    def mark_gather_input_fresh(self) -> None:
        """The fused optimizer kernel wrote the compute-dtype copy itself."""
        self._ag_input_version = self._master._version
        self._ag_input_fresh = True
        self._secondary_valid = False

    # ------------------------------------------------------------------ unshard / reshard
    def unshard(self, async_op: bool = False) -> None:
        assert self._lazy_inited and self.comm_ctx is not None and self.data_ctx is not None
        if self._is_unsharded or self._unshard_pending:
            return
        cc = self.comm_ctx
        st = cc.streams
        assert st is not None
        logger.debug("unshard %s", self._module_fqn)
        with record_function(self._with_fqn("YaFSDP::all_gather")):
            if self._alias_data:
                self.wait_optimizer()
                self._refresh_gather_input()
                self._ag_event = None
                self._unshard_pending = True
                return
            ctx = self.data_ctx
            if ctx.owner is not None and ctx.owner is not self._owner:
                raise RuntimeError(
                    f"Data buffer {ctx.index} is still owned by {ctx.owner._module_fqn!r} while {self._module_fqn!r} "
                    "needs it: two groups that share a buffer are unsharded at the same time"
                )
            ctx.owner = self._owner
            stream = cc.get_all_gather_stream(async_op, self._training_state)
            stale = not (self._ag_input_fresh and self._ag_input_version == self._master._version)
            if stream is not st.current() and stale:
                # the gather input may have just been produced on the compute stream (first gather after the step)
                st.wait_stream(stream, st.current())
            if stale and cc.backend.needs_registered_buffers:
                # a gather outside a root forward (explicit unshard() after an optimizer step): every rank refreshes all of
                # its gather inputs and the ranks meet before anyone pulls
                cc.sync_gather_inputs(stream)
            st.wait_event(stream, ctx.release_event)
            with st.use(stream):
                if (self.secondary_group is not None and self._secondary_valid
                        and (self._training_state != TrainingState.FORWARD or is_backward_running())):
                    # backward of a hierarchically partitioned group: the weights come from the secondary shards
                    assert self._secondary_shard is not None and self._secondary_backend is not None
                    if self._secondary_backend.needs_registered_buffers and not cc.secondary_synced:
                        # the peers wrote their secondary shards during their forward pass: meet once before the first pull
                        st.wait_stream(stream, st.current())
                        self._secondary_backend.subgroup_barrier()  # type: ignore[attr-defined]
                        cc.secondary_synced = True
                    self._secondary_backend.all_gather(self._data_flat, self._secondary_shard, self.secondary_group)
                    self._gathered_from_secondary = True
                else:
                    self._refresh_gather_input()
                    assert self._ag_input is not None
                    cc.backend.all_gather(self._data_flat, self._ag_input, self.process_group)
                    self._gathered_from_secondary = False
                self._ag_event = st.record(stream)
            self._unshard_pending = True

    def wait_for_unshard(self) -> None:
        if not self._unshard_pending:
            return
        assert self.comm_ctx is not None and self.comm_ctx.streams is not None
        self.comm_ctx.streams.wait_event(None, self._ag_event)
        self._ag_event = None
        if (self.secondary_group is not None and not self._alias_data and not self._gathered_from_secondary
                and self._training_state == TrainingState.FORWARD and self.reshard_after_forward and torch.is_grad_enabled()
                and not is_backward_running()):
            self._save_secondary_shard()
        if self._has_extensions:
            self._run_post_all_gather_hooks()
        for sp in self.params:
            sp.to_unsharded()
        self._unshard_pending = False
        self._is_unsharded = True

    def _run_post_all_gather_hooks(self) -> None:
        """Extension parameters: the hook turns the gathered data into the tensor the module computes with; the first call
        creates it, later calls refresh it in place (``out=``)."""
        compute_dtype = self.param_dtype or self.orig_dtype
        with torch.no_grad():
            for sp in self.params:
                if sp.ext_cls is None:
                    continue
                assert sp.ext_local is not None
                if sp.unsharded_param is None:
                    unsharded, _ = sp.ext_local.fsdp_post_all_gather((sp.gathered_view,), sp.ext_metadata, compute_dtype)
                    sp.unsharded_param = nn.Parameter(unsharded, requires_grad=sp.requires_grad)
                    sp.unsharded_param._yf_grad_sink = None  # type: ignore[attr-defined]
                else:
                    sp.ext_local.fsdp_post_all_gather((sp.gathered_view,), sp.ext_metadata, compute_dtype, out=sp.unsharded_param.data)

    def reshard(self) -> None:
        if self._unshard_pending:
            self.wait_for_unshard()
        if not self._is_unsharded:
            return
        logger.debug("reshard %s", self._module_fqn)
        for sp in self.params:
            sp.to_sharded()
        self._is_unsharded = False
        if not self._alias_data:
            assert self.data_ctx is not None and self.comm_ctx is not None and self.comm_ctx.streams is not None
            self.data_ctx.release_event = self.comm_ctx.streams.record()
            self.data_ctx.owner = None

    # ------------------------------------------------------------------ forward
    def pre_forward(self) -> None:
        logger.debug("pre_forward %s", self._module_fqn)
        with record_function(self._with_fqn("YaFSDP::pre_forward")):
            self._training_state = TrainingState.FORWARD
            if self._can_gather_in_kernel():
                self._begin_in_kernel_gather()
                return
            self.unshard(self.unshard_async_op)
            self.wait_for_unshard()

    # ------------------------------------------------------------------ fused all-gather -> GEMM
    def _can_gather_in_kernel(self) -> bool:
        if not self.fused_gather or self._is_unsharded or self._unshard_pending or self._alias_data or is_backward_running():
            return False
        cc = self.comm_ctx
        return (cc is not None and hasattr(cc.backend, "gather_ranges") and not getattr(cc.backend, "dry_run", False)
                and self.all_gather_dtype == torch.bfloat16 and not self._has_extensions and self.secondary_group is None
                and self._ag_input_fresh and self._ag_input_version == self._master._version)

    def _begin_in_kernel_gather(self) -> None:
        """Forward pass without a gather: take the layer buffer, copy the few parameters that are read before the fusing
        GEMM, register the (still empty) unsharded parameters and leave a ticket that the module's forward redeems with
        :meth:`take_in_kernel_gather`."""
        assert self.comm_ctx is not None and self.data_ctx is not None and self.comm_ctx.streams is not None
        cc, st, ctx = self.comm_ctx, self.comm_ctx.streams, self.data_ctx
        if ctx.owner is not None and ctx.owner is not self._owner:
            raise RuntimeError(f"Data buffer {ctx.index} is still owned by {ctx.owner._module_fqn!r} while {self._module_fqn!r} needs it")
        ctx.owner = self._owner
        st.wait_event(None, ctx.release_event)
        st.wait_stream(st.current(), cc.all_gather_stream)  # the step barrier (every rank's shards are final) sits there
        backend = cc.backend
        ranges = [(self.layout.flat_offsets[i], self.layout.flat_offsets[i] + self.params[i].numel) for i in self.fused_gather_prefix]
        backend.gather_ranges(self._data_flat, self._ag_input, ranges)  # type: ignore[attr-defined]
        if self._gather_counters is None:
            self._gather_counters = torch.zeros(4096, dtype=torch.int64, device=self.device)
        self._in_kernel_gather = {"peer_in": backend.peer_pointers(self._ag_input), "layer_buf": self._data_flat,  # type: ignore[attr-defined]
                                  "shard_bytes": self.layout.shard_numel * 2, "rank": self.rank, "world": self.world_size,
                                  "counters": self._gather_counters}
        self._gathered_from_secondary = False
        for sp in self.params:
            sp.to_unsharded()
        self._is_unsharded = True

    def take_in_kernel_gather(self, first_param_index: int, rows: int) -> dict[str, Any] | None:
        """Called by a module's forward right before its first GEMM over ``rows`` weight rows that start at parameter
        ``first_param_index``: the arguments for ``kernels.gemm_gathered`` when this forward pass gathers in that kernel,
        else ``None`` (the parameters are already there)."""
        t = self._in_kernel_gather
        if t is None:
            return None
        self._in_kernel_gather = None
        if rows > 128 * t["counters"].numel():
            raise RuntimeError("fused all-gather -> GEMM: more weight rows than column-block counters")
        self._gather_epoch += 1
        t["epoch"] = self._gather_epoch
        t["b_byte_off"] = self.layout.flat_offsets[first_param_index] * 2
        return t

    def post_forward(self) -> None:
        logger.debug("post_forward %s", self._module_fqn)
        if self._in_kernel_gather is not None:
            self._in_kernel_gather = None
            raise RuntimeError(f"{self._module_fqn}: fused_gather is set but the module's forward never gathered its parameters "
                               "(only modules that call take_in_kernel_gather may use it)")
        with record_function(self._with_fqn("YaFSDP::post_forward")):
            if not is_backward_running():  # inside backward (checkpoint recompute) the backward owns the buffer
                if self.reshard_after_forward:
                    self.reshard()
                else:
                    self._kept_after_forward = True
                self._record_post_forward()
            self._training_state = TrainingState.IDLE

    def _record_post_forward(self) -> None:
        assert self.comm_ctx is not None
        if self._owner is not self:
            return  # the set this group belongs to takes the place in the order
        idx = len(self.comm_ctx.post_forward_order)
        self.comm_ctx.post_forward_order.append(self)
        self._post_forward_indices.append(idx)

    # ------------------------------------------------------------------ backward
    def pre_backward(self, default_prefetch: bool = True) -> None:
        if self._training_state == TrainingState.PRE_BACKWARD:
            return
        logger.debug("pre_backward %s", self._module_fqn)
        with record_function(self._with_fqn("YaFSDP::pre_backward")):
            self._training_state = TrainingState.PRE_BACKWARD
            self._kept_after_forward = False
            if self._norm_sq is not None and self._alias_grad and not self._has_sharded_grads():
                self._norm_sq.zero_()
                self._norm_fused_ok = True
            if not self._holds_grad_buffer:
                self._sink_written = [False] * len(self.params)
                self._sink_counts = [0] * len(self.params)
            if self.unshard_in_backward:
                self.unshard(self.unshard_async_op)
                self.wait_for_unshard()
            if default_prefetch:
                self._backward_prefetch()

    def _backward_prefetch(self) -> None:
        """Start the gather of the group that ran just before this one in forward, if it uses the other buffer."""
        if self._training_state != TrainingState.PRE_BACKWARD or not self._post_forward_indices:
            return
        assert self.comm_ctx is not None
        curr = self._post_forward_indices.pop()
        target_idx = curr - 1
        if target_idx < 0:
            return
        target = self.comm_ctx.post_forward_order[target_idx]
        if target._alias_data or (target.data_ctx is not self.data_ctx):
            if target.unshard_in_backward:
                self._prefetch_unshard(target, "backward")

    @staticmethod
    def _prefetch_unshard(target: "ParamGroup", pass_type: str) -> None:
        state = TrainingState.PRE_BACKWARD if pass_type == "backward" else TrainingState.FORWARD
        if target._is_unsharded or target._unshard_pending:
            return
        ctx = target.data_ctx
        if not target._alias_data and ctx is not None and ctx.owner is not None and ctx.owner is not target._owner:
            return  # the buffer is not free yet: the target gathers itself when its turn comes
        with record_function(target._with_fqn(f"YaFSDP::{pass_type}_prefetch")):
            old = target._training_state
            target._training_state = state
            target.unshard(target.unshard_async_op)
            target._training_state = old

    def _push_mode(self) -> bool:
        """Gradients of this backward pass go to their owners from the producing kernels.  Decided by the first gradient
        of the pass: not while unreduced gradients of earlier micro-batches sit in the local flat buffer."""
        if self._pushed:
            return True
        if not (self.fused_reduce and self.reduce_grads and self._push_ptrs is not None) or self.post_reduce_hook is not None:
            return False
        return not (self._holds_grad_buffer and any(self._sink_written))

    def _acquire_grad_buffer(self) -> None:
        if self._holds_grad_buffer or self._alias_grad:
            self._holds_grad_buffer = True
            return
        assert self.grad_ctx is not None and self.comm_ctx is not None and self.comm_ctx.streams is not None
        ctx = self.grad_ctx
        if ctx.owner is not None and ctx.owner is not self._owner:
            raise RuntimeError(
                f"Grad buffer {ctx.index} is still owned by {ctx.owner._module_fqn!r} (gradients kept for accumulation "
                f"without reduction) while {self._module_fqn!r} needs it; give such groups their own grad buffers"
            )
        self.comm_ctx.streams.wait_event(None, ctx.release_event)
        if self._grad_flat is not None:
            self.comm_ctx.backend.before_write(self._grad_flat)
        ctx.owner = self._owner
        self._holds_grad_buffer = True

    def post_backward(self) -> None:
        logger.debug("post_backward %s", self._module_fqn)
        self._training_state = TrainingState.POST_BACKWARD
        assert self.comm_ctx is not None and self.comm_ctx.streams is not None
        st = self.comm_ctx.streams
        with record_function(self._with_fqn("YaFSDP::post_backward_accumulate")):
            with_grad: list[ShardedParam] = []
            for sp in self.params:
                up = sp.unsharded_param
                has_autograd_grad = up is not None and up.grad is not None
                if has_autograd_grad or self._sink_written[sp.index]:
                    with_grad.append(sp)
            if not with_grad:
                if self.reshard_after_backward:
                    self.reshard()
                return
            if self._pushed:
                self._finish_pushes()
                with record_function(self._with_fqn("YaFSDP::post_backward_reshard")):
                    if self.reshard_after_backward:
                        self.reshard()
                with record_function(self._with_fqn("YaFSDP::post_backward_reduce")):
                    self._reduce([sp for sp in self.params if sp.requires_grad], st)
                return
            self._acquire_grad_buffer()
            fresh = self._alias_grad and not self._has_sharded_grads()
            dsts_copy, dsts_add = [], []
            with torch.no_grad():
                for sp in self.params:
                    up = sp.unsharded_param
                    assert up is not None and sp.rs_view is not None
                    g = up.grad
                    if g is not None and sp.outer_mesh is not None:
                        # gradient of a DTensor parameter: bring it to the parameter's own placement, take the local piece
                        if tuple(g.placements) != tuple(sp.outer_placements):
                            g = g.redistribute(placements=sp.outer_placements)
                        g = g._local_tensor
                    if g is not None:
                        self._norm_fused_ok = False
                        accumulate = self._sink_written[sp.index] or (self._alias_grad and not fresh and sp.sharded_param.grad is not None)  # type: ignore[union-attr]
                        (dsts_add if accumulate else dsts_copy).append((sp.rs_view, g))
                        up.grad = None
                        self._sink_written[sp.index] = True
                    elif not self._sink_written[sp.index] and not self._alias_grad:
                        # unused this step, or frozen: do not reduce another layer's stale bytes into the flat gradient
                        # (flat consumers - fused optimizer, norm over the whole shard - read these positions too)
                        sp.rs_view.zero_()
                if not self._alias_grad and self.layout.padded_numel > self.layout.total_numel:
                    # padding tail: never written by any gradient, must not carry another layer's bytes into the reduction
                    self._grad_flat[self.layout.total_numel :].zero_()
                if dsts_copy:
                    torch._foreach_copy_([d for d, _ in dsts_copy], [s for _, s in dsts_copy])
                if dsts_add:
                    torch._foreach_add_([d for d, _ in dsts_add], [s.to(d.dtype) if s.dtype != d.dtype else s for d, s in dsts_add])
        if not self.reduce_grads:
            with record_function(self._with_fqn("YaFSDP::post_backward_reshard")):
                if self.reshard_after_backward:
                    self.reshard()
            return  # keeps the grad buffer: the unsharded accumulated gradients live there
        with record_function(self._with_fqn("YaFSDP::post_backward_reshard")):
            if self.reshard_after_backward:
                self.reshard()
        with record_function(self._with_fqn("YaFSDP::post_backward_reduce")):
            self._reduce(with_grad, st)

    def _finish_pushes(self) -> None:
        """End of a backward pass in push mode: gradients that autograd produced (``.grad``) are pushed now, parameters
        that got no gradient push zeros, so every position of every owner's slot for this rank has been written."""
        with torch.no_grad():
            for sp in self.params:
                if not sp.requires_grad:
                    continue
                up = sp.unsharded_param
                g = up.grad if up is not None else None
                assert sp.sink is not None
                if g is not None:
                    up.grad = None  # type: ignore[union-attr]
                    sp.sink.push_from(g.to(torch.float32).contiguous())
                elif not self._sink_written[sp.index]:
                    sp.sink.push_from(None)

    def _has_sharded_grads(self) -> bool:
        return any(sp.sharded_param is not None and sp.sharded_param.grad is not None for sp in self.params)

    def _reduce(self, with_grad: list[ShardedParam], st: _DeviceStreams) -> None:
        assert self.comm_ctx is not None
        pre, post, op, premul = gradient_divide_factors(
            self.world_size, self.reduce_scatter_dtype, self.gradient_divide_factor, self.force_sum_reduction_for_comms
        )
        if op == "avg":
            scale = 1.0 / self.world_size
        elif op == "premul_sum":
            scale = float(premul)  # type: ignore[arg-type]
        else:
            scale = 1.0
        if post is not None and post != 1.0:
            scale = scale / post
        if self.world_size == 1 and self.gradient_divide_factor is not None and pre is None and post is None:
            scale = 1.0 / self.gradient_divide_factor
        if self._alias_grad:
            # single rank, gradients already sit in the sharded gradient: at most a scale
            if scale != 1.0 or (pre or 1.0) != 1.0:
                self._norm_fused_ok = False
                with torch.no_grad():
                    self.sharded_grad_flat.mul_(scale / (pre or 1.0))
            self._finish_reduce(with_grad, None)
            return
        had = [sp.sharded_param.grad is not None for sp in self.params]  # type: ignore[union-attr]
        producing = [sp.index for sp in with_grad]
        all_fresh = not any(had)
        all_have = all(had[i] for i in producing) and len(producing) == len([sp for sp in self.params if sp.requires_grad])
        stream = self.comm_ctx.reduce_scatter_stream
        st.wait_stream(stream, st.current())
        with st.use(stream), torch.no_grad():
            if pre is not None and pre != 1.0:
                self._grad_flat.div_(pre)
            dst = self.sharded_grad_flat
            if self._pushed:
                # every rank's contribution already sits in this rank's slots: wait for all of them, sum locally
                self._pushed = False
                whole = all_fresh or all_have
                target = self._norm_sq if (self._norm_sq is not None and all_fresh and dst.dtype == torch.float32) else None
                if target is not None:
                    target.zero_()
                out = dst if whole else torch.empty_like(dst)
                fused = self.comm_ctx.backend.reduce_pushed(  # type: ignore[attr-defined]
                    out, self._grad_flat, scale=scale, accumulate=whole and not all_fresh, sumsq=target if whole else None,
                    valid_numel=self.layout.total_numel)
                self._norm_fused_ok = bool(fused)
                if not whole:
                    for sp in with_grad:
                        pl = sp.placement
                        assert pl is not None
                        src = out[pl.shard_offset : pl.shard_offset + pl.local_numel]
                        tgt = dst[pl.shard_offset : pl.shard_offset + pl.local_numel]
                        if had[sp.index]:
                            tgt.add_(src)
                        else:
                            tgt.copy_(src)
            elif (all_fresh or all_have) and self.post_reduce_hook is None:
                # the reduction kernel can also sum the squares of the final shard (gradient-norm fusion) when this is the
                # only contribution of the step to the sharded gradient
                target = self._norm_sq if (self._norm_sq is not None and all_fresh and dst.dtype == torch.float32) else None
                if target is not None:
                    target.zero_()
                fused = self.comm_ctx.backend.reduce_scatter(
                    dst, self._grad_flat, self.process_group, scale=scale, accumulate=all_have and not all_fresh,
                    acc_fp32=True, sumsq=target,
                )
                self._norm_fused_ok = bool(fused)
            else:
                # mixed: some parameters accumulate, some start fresh -> reduce into the own chunk, then per parameter
                self._norm_fused_ok = False
                own = self._grad_flat[self.rank * self.layout.shard_numel : (self.rank + 1) * self.layout.shard_numel]
                self.comm_ctx.backend.reduce_scatter(own, self._grad_flat, self.process_group, scale=scale, accumulate=False)
                if self.post_reduce_hook is not None:
                    self.post_reduce_hook(own)  # e.g. an all-reduce of this micro-batch's reduced shard over another group
                for sp in with_grad:
                    pl = sp.placement
                    assert pl is not None
                    src = own[pl.shard_offset : pl.shard_offset + pl.local_numel]
                    tgt = dst[pl.shard_offset : pl.shard_offset + pl.local_numel]
                    if had[sp.index]:
                        tgt.add_(src)
                    else:
                        tgt.copy_(src)
            event = st.record(stream)
        self._finish_reduce(with_grad, event)

    def _finish_reduce(self, with_grad: list[ShardedParam], event: Any) -> None:
        self._post_reduce_event = event
        if not self._alias_grad:
            assert self.grad_ctx is not None
            self.grad_ctx.release_event = event
            self.grad_ctx.owner = None
        self._holds_grad_buffer = False
        self._sink_written = [False] * len(self.params)
        for sp in with_grad:
            assert sp.sharded_param is not None
            _ = self.sharded_grad_flat
            sp.sharded_param.grad = sp.sharded_grad

    def finalize_backward(self) -> None:
        assert self.comm_ctx is not None and self.comm_ctx.streams is not None
        if self._post_reduce_event is not None:
            self.comm_ctx.streams.wait_event(None, self._post_reduce_event)
            self._post_reduce_event = None
        if self._unshard_pending:
            # a prefetch that nothing consumed (e.g. unused module): finish and release it
            self.wait_for_unshard()
            if self.reshard_after_backward:
                self.reshard()
        self._post_forward_indices.clear()
        self._secondary_valid = False
        # an optimizer step normally follows: the compute-dtype copy is re-derived at the next gather unless the fused
        # optimizer writes it itself (it then marks it fresh again)
        self._ag_input_fresh = False

    # ------------------------------------------------------------------ state dict
    def _register_state_dict_hooks(self) -> None:
        if getattr(self, "_sd_hooks", None):
            return
        handles = []
        for m in self.modules:
            handles.append(m.register_state_dict_pre_hook(lambda *a, **k: self._to_sharded_for_state_dict()))
            handles.append(m._register_load_state_dict_pre_hook(lambda *a, **k: self._to_sharded_for_state_dict()))
        self._sd_hooks = handles

    def _to_sharded_for_state_dict(self) -> None:
        self.wait_optimizer()
        if self._is_unsharded or self._unshard_pending:
            self.reshard()

    def reset_sharded_params(self) -> None:
        """``module._apply`` (``.to()``, ``.float()``, ``.cuda()``) replaced the sharded parameters by transformed copies.

        Before the first forward the flat master is re-derived from them, so the group really changes dtype / device.
        After it, buffers, streams and views are bound to the master's storage: like the reference
        (``ya_fsdp/_param.py:349-357``) the group then keeps its storage, takes over the transformed *values* (cast back to
        the master's dtype) and registers its own sharded parameters again."""
        def local_of(t: torch.Tensor) -> torch.Tensor:
            return t._local_tensor if isinstance(t, RaggedShardDTensor) else t.data._local_tensor  # type: ignore[union-attr]

        changed = False
        for sp in self.params:
            cur = sp.info.module._parameters[sp.info.param_name]
            pl = sp.placement
            assert pl is not None
            if not isinstance(cur, torch.Tensor):
                continue
            # either a new Parameter object, or the same object whose data was swapped for the transformed tensor
            if cur is not sp.sharded_param or (pl.local_numel and local_of(cur).data_ptr() != self._master[pl.shard_offset:].data_ptr()) \
                    or cur.dtype != self._master.dtype:
                changed = True
        if not changed:
            return
        locals_ = []
        for sp in self.params:
            cur = sp.info.module._parameters[sp.info.param_name]
            locals_.append(local_of(cur))
        if self._lazy_inited:
            with torch.no_grad():
                for sp, local in zip(self.params, locals_):
                    pl = sp.placement
                    assert pl is not None and sp.sharded_param is not None
                    mine = self._master[pl.shard_offset : pl.shard_offset + pl.local_numel]
                    if pl.local_numel and (local.data_ptr() != mine.data_ptr() or local.dtype != mine.dtype):
                        mine.copy_(local.reshape(-1))
                    if local_of(sp.sharded_param) is not mine and (local_of(sp.sharded_param).dtype != mine.dtype
                                                                   or local_of(sp.sharded_param).data_ptr() != mine.data_ptr()):
                        # the registered Parameter object (the one optimizers hold) had its contents swapped for the transformed
                        # tensor: swap the master-backed contents back in, so the object keeps its identity
                        fresh = nn.Parameter(RaggedShardDTensor(mine, sp.sharded_param._spec.with_dtype(mine.dtype)),
                                             requires_grad=sp.requires_grad)
                        torch.utils.swap_tensors(sp.sharded_param, fresh)
                    # gradients were transformed along with the parameters: drop them (the reference's re-created parameters
                    # have none either) and bind fresh views of the flat sharded gradient
                    sp.sharded_param.grad = None
                    sp.to_sharded()
                if self._sharded_grad_flat is not None:
                    self._bind_sharded_grads()
            self._ag_input_fresh = False  # the next gather re-derives the compute-dtype copy from the new values
            self._secondary_valid = False
            return
        new_dtype = locals_[0].dtype
        device = locals_[0].device
        master = torch.zeros(self.layout.shard_numel, dtype=new_dtype, device=device)
        for sp, local in zip(self.params, locals_):
            pl = sp.placement
            assert pl is not None
            master[pl.shard_offset : pl.shard_offset + pl.local_numel].copy_(local)
        self._master = master
        self.device = device
        self.orig_dtype = new_dtype
        self._init_dtypes_after_apply()
        self._sharded_grad_flat = None
        for sp in self.params:
            pl = sp.placement
            assert pl is not None and sp.sharded_param is not None
            spec = sp.sharded_param._spec.with_dtype(new_dtype)
            sp.orig_dtype = new_dtype
            local = master[pl.shard_offset : pl.shard_offset + pl.local_numel]
            sp.sharded_param = nn.Parameter(RaggedShardDTensor(local, spec), requires_grad=sp.requires_grad)
            sp.sharded_grad = None
            sp.to_sharded()

    def _init_dtypes_after_apply(self) -> None:
        pd, rd = self.mp_policy.param_dtype, self.mp_policy.reduce_dtype
        if rd == pd:
            rd = None
        if pd == self.orig_dtype:
            pd = None
        self.param_dtype, self.reduce_dtype = pd, rd
        self.all_gather_dtype = pd or self.orig_dtype
        self.reduce_scatter_dtype = rd or pd or self.orig_dtype

    def _sink_written_twice(self, index: int) -> bool:
        """True when the parameter's gradient already held a contribution before the latest sink write (so a kernel that
        added into it did not produce the final value alone)."""
        return self._sink_counts[index] > 1

    def _shares_nothing_data(self) -> bool:
        return self.world_size == 1

    def _shares_nothing_grad(self) -> bool:
        return self.world_size == 1 and self.reduce_scatter_dtype == self.orig_dtype

    # ------------------------------------------------------------------ misc
    def _with_fqn(self, label: str) -> str:
        return f"{label} ({self._module_fqn})" if self._module_fqn else label

    def __repr__(self) -> str:
        return f"ParamGroup(fqn={self._module_fqn!r}, {self.layout})"


class RegisterPostBackwardFunction(torch.autograd.Function):
    """Identity over the forward inputs that require grad; its backward runs once the gradients with
    respect to the group's inputs exist, i.e. after the group's own backward: that is where the gradient
    reduction is issued (``ya_fsdp/_param_group.py:979-992``)."""

    @staticmethod
    def forward(ctx: Any, hook: Callable[[], None], *inputs: torch.Tensor) -> Any:  # type: ignore[override]
        ctx.hook = hook
        ctx.set_materialize_grads(False)
        return inputs

    @staticmethod
    def backward(ctx: Any, *grads: torch.Tensor) -> Any:  # type: ignore[override]
        ctx.hook()
        return (None,) + grads


class GroupSet:
    """Several :class:`ParamGroup` s of ONE ``fully_shard`` call, driven by the scheduler as one group.

    A module whose parameters are gathered in different dtypes (ordinary parameters in the compute dtype, extension
    parameters in their own wire dtype, ``MixedPrecisionPolicy.all_gather_dtype_to_param_cls``) gets one flat layout,
    one shard and one all-gather / reduce-scatter per dtype class (the reference splits a group the same way,
    ``ya_fsdp/_param_group.py:194-228,577-594``).  The groups of a set lie side by side in the shared rotating buffers,
    own them together and take one place in the forward order.

    Attribute reads go to the first group (the scheduler's flags are kept equal in all of them), attribute writes and
    method calls go to every group, in order.
    """

    _OWN = ("groups", "_post_forward_indices")

    def __init__(self, groups: list[ParamGroup]):
        object.__setattr__(self, "groups", list(groups))
        object.__setattr__(self, "_post_forward_indices", [])
        for g in groups:
            g._owner = self

    # ---- generic forwarding
    def __getattr__(self, name: str) -> Any:
        groups = object.__getattribute__(self, "groups")
        attr = getattr(groups[0], name)
        if callable(attr) and getattr(attr, "__self__", None) is groups[0]:
            def broadcast(*args: Any, **kwargs: Any) -> Any:
                results = [getattr(g, name)(*args, **kwargs) for g in groups]
                return results[0]

            return broadcast
        return attr

    def __setattr__(self, name: str, value: Any) -> None:
        if name in GroupSet._OWN:
            object.__setattr__(self, name, value)
            return
        for g in self.groups:
            setattr(g, name, value)

    # ---- what differs from a single group
    @property
    def _owner(self) -> "GroupSet":
        return self

    @property
    def params(self) -> list[ShardedParam]:
        return [sp for g in self.groups for sp in g.params]

    @property
    def _is_unsharded(self) -> bool:
        return all(g._is_unsharded for g in self.groups)

    @property
    def _unshard_pending(self) -> bool:
        return any(g._unshard_pending for g in self.groups)

    def _finish_pushes(self) -> None:
        """End of a backward pass in push mode: gradients that autograd produced (``.grad``) are pushed now, parameters
        that got no gradient push zeros, so every position of every owner's slot for this rank has been written."""
        with torch.no_grad():
            for sp in self.params:
                if not sp.requires_grad:
                    continue
                up = sp.unsharded_param
                g = up.grad if up is not None else None
                assert sp.sink is not None
                if g is not None:
                    up.grad = None  # type: ignore[union-attr]
                    sp.sink.push_from(g.to(torch.float32).contiguous())
                elif not self._sink_written[sp.index]:
                    sp.sink.push_from(None)

    def _has_sharded_grads(self) -> bool:
        return any(g._has_sharded_grads() for g in self.groups)

    @staticmethod
    def _aligned(nbytes: int) -> int:
        return (nbytes + 1023) // 1024 * 1024

    def data_buffer_nbytes(self) -> int:
        return sum(self._aligned(g.data_buffer_nbytes()) for g in self.groups)

    def grad_buffer_nbytes(self) -> int:
        return sum(self._aligned(g.grad_buffer_nbytes()) for g in self.groups)

    def lazy_init(self, comm_ctx: CommContext, data_ctx: BufferContext, grad_ctx: BufferContext) -> None:
        d = r = 0
        for g in self.groups:
            g._data_byte_offset, g._grad_byte_offset = d, r
            d += self._aligned(g.data_buffer_nbytes())
            r += self._aligned(g.grad_buffer_nbytes())
            g.lazy_init(comm_ctx, data_ctx, grad_ctx)

    # ---- one place in the forward order, one backward prefetch
    def post_forward(self) -> None:
        for g in self.groups:
            g.post_forward()
        if not is_backward_running():
            cc = self.groups[0].comm_ctx
            assert cc is not None
            self._post_forward_indices.append(len(cc.post_forward_order))
            cc.post_forward_order.append(self)  # type: ignore[arg-type]

    def pre_backward(self, default_prefetch: bool = True) -> None:
        for g in self.groups:
            g.pre_backward(default_prefetch=False)
        if default_prefetch and self._post_forward_indices:
            cc = self.groups[0].comm_ctx
            assert cc is not None
            target_idx = self._post_forward_indices.pop() - 1
            if target_idx >= 0:
                target = cc.post_forward_order[target_idx]
                if (target._alias_data or target.data_ctx is not self.groups[0].data_ctx) and target.unshard_in_backward:
                    ParamGroup._prefetch_unshard(target, "backward")

    def finalize_backward(self) -> None:
        for g in self.groups:
            g.finalize_backward()
        self._post_forward_indices.clear()

    def __repr__(self) -> str:
        return f"GroupSet({', '.join(repr(g) for g in self.groups)})"
