"""Hugging Face ``transformers`` integration: shard any decoder-only causal LM, checkpoint its first N layers, and
``Trainer`` callbacks for iteration time, memory snapshots and profiler traces.

The reference ships this as patches against ``accelerate`` / ``transformers`` / ``trl``
(``patches/accelerate.diff:41-54,71-89,98-159``: the plugin that wraps ``embed_tokens``, every decoder layer and
``lm_head``, treats the final norm as a "rogue" norm module and checkpoints the first ``num_layers_to_checkpoint``
layers; ``patches/transformers.diff:69-90``: weights only on local rank 0, meta elsewhere; ``:146-205``: profiler,
``IterTimeCallback``, ``MemorySnapshotCallback``; ``patches/trl.diff``: the same for supervised fine-tuning).
Here it is a module that works with stock libraries:

* :func:`find_decoder_parts` locates embedding, decoder layers, final norm and head of a ``PreTrainedModel``;
* :func:`shard_causal_lm` materialises (from rank 0, part by part, so no rank ever holds more than one unsharded part
  besides rank 0), shards with :func:`~yafsdp_b200.fully_shard` (default) or the class-style wrapper, and applies
  activation checkpointing;
* :func:`trainer_callbacks` returns the three callbacks for ``transformers.Trainer`` / ``trl.SFTTrainer``.

Hugging Face modules run their own (PyTorch) forward; the hand-written sm_100a kernels of this package are used by
``yafsdp_b200.models.llama`` (same parameter names, so checkpoints are interchangeable).
"""

from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist
import torch.nn as nn

from ..api import MixedPrecisionPolicy
from ..fully_shard import fully_shard
from ..utils.checkpointing import checkpoint_module

__all__ = ["DecoderParts", "find_decoder_parts", "shard_causal_lm", "materialize_from_rank0", "trainer_callbacks"]

_LAYER_LIST_NAMES = ("layers", "h", "blocks", "block")
_FINAL_NORM_NAMES = ("norm", "ln_f", "final_layer_norm", "final_layernorm", "norm_f")


@dataclass
class DecoderParts:
    embed: nn.Module
    layers: list[nn.Module]
    norm: nn.Module | None
    head: nn.Module | None
    tied: bool
    names: dict[int, str]  # id(module) -> qualified name inside the model

    def name(self, module: nn.Module) -> str:
        return self.names[id(module)]


def find_decoder_parts(model: nn.Module) -> DecoderParts:
    """Embedding, decoder layers, final norm and LM head of a decoder-only ``transformers`` model (Llama, Mistral, Qwen,
    GPT-2/NeoX style layouts)."""
    names = {id(m): n for n, m in model.named_modules()}
    embed = model.get_input_embeddings() if hasattr(model, "get_input_embeddings") else None
    head = model.get_output_embeddings() if hasattr(model, "get_output_embeddings") else None
    base = getattr(model, getattr(model, "base_model_prefix", "model"), None) or model
    layers: list[nn.Module] | None = None
    for holder in (base, getattr(base, "decoder", None), model):
        if holder is None:
            continue
        for n in _LAYER_LIST_NAMES:
            cand = getattr(holder, n, None)
            if isinstance(cand, nn.ModuleList) and len(cand) > 0:
                layers = list(cand)
                base = holder
                break
        if layers is not None:
            break
    if embed is None or layers is None:
        raise ValueError("could not find the input embedding and the decoder layer list of this model")
    norm = None
    for n in _FINAL_NORM_NAMES:
        cand = getattr(base, n, None)
        if isinstance(cand, nn.Module):
            norm = cand
            break
    tied = head is not None and getattr(head, "weight", None) is getattr(embed, "weight", object())
    return DecoderParts(embed=embed, layers=layers, norm=norm, head=head, tied=tied, names=names)


def materialize_from_rank0(module: nn.Module, device: torch.device, group: dist.ProcessGroup | None = None) -> None:
    """Give ``module`` real storage on ``device`` and the values of rank 0 (which holds the loaded weights; the other ranks
    may have built the model on the meta device)."""
    if any(t.device.type == "meta" for t in list(module.parameters()) + list(module.buffers())):
        module.to_empty(device=device)
    else:
        module.to(device)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        src = dist.get_global_rank(group, 0) if group is not None else 0
        with torch.no_grad():
            for t in list(module.parameters()) + list(module.buffers()):
                dist.broadcast(t.data, src=src, group=group)


def shard_causal_lm(
    model: nn.Module,
    *,
    mesh: Any = None,
    mp_policy: MixedPrecisionPolicy | None = None,
    num_layers_to_checkpoint: int = 0,
    sync_from_rank0: bool = False,
    device: torch.device | None = None,
    api: str = "fully_shard",
    comm_backend: str = "auto",
    **v1_kwargs: Any,
) -> nn.Module:
    """Shard a decoder-only causal LM: one group per decoder layer, one for the embedding, one for final norm + head (with
    tied embeddings: embedding, final norm and head share one group that stays gathered, in buffers of its own).

    ``api="fully_shard"`` returns the model itself (now a ``YaFSDPModule``); ``api="v1"`` returns the class-style
    ``YaFSDP`` wrapper (``zero_stage``, ``gradient_accumulation_steps`` ... go through ``v1_kwargs``).
    ``num_layers_to_checkpoint`` recomputes the first N decoder layers in backward.  ``sync_from_rank0`` materialises
    every part from rank 0 before it is sharded."""
    parts = find_decoder_parts(model)
    if mp_policy is None:
        mp_policy = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() and (
            not dist.is_initialized() or dist.get_backend() != "gloo") else torch.device("cpu")
    for layer in parts.layers[: max(0, num_layers_to_checkpoint)]:
        checkpoint_module(layer)
    if hasattr(model, "config") and num_layers_to_checkpoint > 0:
        model.config.use_cache = False  # a key/value cache cannot be recomputed
    if sync_from_rank0:
        for m in [parts.embed, *parts.layers, parts.norm, parts.head]:
            if m is not None:
                materialize_from_rank0(m, device)
        if parts.tied:
            # giving a meta parameter storage creates a new Parameter per module: restore the sharing
            parts.head.weight = parts.embed.weight  # type: ignore[union-attr]
        materialize_from_rank0(model, device)  # whatever is left (rotary tables, ...)

    if api == "v1":
        from ..compat_v1 import YaFSDP

        wrap = [(parts.embed, parts.name(parts.embed))] + [(l, parts.name(l)) for l in parts.layers]
        if parts.head is not None and not parts.tied:
            wrap.append((parts.head, parts.name(parts.head)))
        elif parts.tied:
            raise NotImplementedError("tied embeddings with the class-style wrapper: use api='fully_shard'")
        norm_cls = type(parts.norm) if parts.norm is not None else None
        rogue = {parts.norm: parts.name(parts.norm)} if parts.norm is not None else None
        v1_kwargs.setdefault("zero_stage", 3)
        v1_kwargs.setdefault("gradient_accumulation_steps", 1)
        return YaFSDP(model, param_dtype=mp_policy.param_dtype or torch.float32, modules_to_wrap_with_names=wrap,
                      layer_norm_module_cls=norm_cls, rogue_layer_norm_modules_with_names=rogue,
                      bit16_reduce_scatter=mp_policy.reduce_dtype == torch.bfloat16, comm_backend=comm_backend, **v1_kwargs)
    if api != "fully_shard":
        raise ValueError(f"api must be 'fully_shard' or 'v1', got {api!r}")

    kw: dict[str, Any] = dict(mesh=mesh, mp_policy=mp_policy)
    tail = [m for m in (parts.norm, parts.head) if m is not None]
    # modules outside the known parts that own parameters themselves (e.g. learned position embeddings): they join the
    # embedding's group, which then keeps buffers of its own because such modules may run anywhere in the forward
    covered = {id(p) for m in (parts.embed, *parts.layers, *tail) for p in m.parameters()}
    inside = {id(sub) for m in (parts.embed, *parts.layers, *tail) for sub in m.modules()}
    extra = [m for m in model.modules()
             if id(m) not in inside and any(id(p) not in covered for p in m.parameters(recurse=False))]
    if parts.tied or extra:
        fully_shard([parts.embed, *extra, *(tail if parts.tied else [])], reshard_after_forward=False, **kw)
        parts.embed._get_fsdp_state()._param_group.dedicated_buffers = True  # type: ignore[attr-defined]
    else:
        fully_shard(parts.embed, **kw)
    for layer in parts.layers:
        fully_shard(layer, **kw)
    if tail and not parts.tied:
        fully_shard(tail if len(tail) > 1 else tail[0], **kw)
    fully_shard(model, **kw)
    if comm_backend != "auto":
        model.set_comm_backend(comm_backend)  # type: ignore[attr-defined]
    return model


def trainer_callbacks(*, trace_path: str | None = None, memory_snapshot_path: str | None = None, snapshot_step: int = 10,
                      profiler_schedule: tuple[int, int, int] = (10, 10, 1)) -> list[Any]:
    """``transformers.TrainerCallback`` objects: iteration time logged as ``iter_time`` every step; optionally a
    CUDA memory snapshot dumped at ``snapshot_step`` and a ``torch.profiler`` Chrome trace from rank 0 with the
    (wait, warmup, active) schedule of the reference's example scripts."""
    from transformers import TrainerCallback

    class IterTimeCallback(TrainerCallback):  # type: ignore[misc]
        def __init__(self) -> None:
            self._t0: float | None = None
            self.times: list[float] = []

        def on_step_begin(self, args: Any, state: Any, control: Any, **kw: Any) -> None:
            self._t0 = time.perf_counter()

        def on_step_end(self, args: Any, state: Any, control: Any, **kw: Any) -> None:
            if self._t0 is not None:
                self.times.append(time.perf_counter() - self._t0)
                state.log_history.append({"iter_time": self.times[-1], "step": state.global_step})

    class MemorySnapshotCallback(TrainerCallback):  # type: ignore[misc]
        def on_train_begin(self, args: Any, state: Any, control: Any, **kw: Any) -> None:
            if torch.cuda.is_available():
                torch.cuda.memory._record_memory_history()

        def on_step_end(self, args: Any, state: Any, control: Any, **kw: Any) -> None:
            if state.global_step == snapshot_step and torch.cuda.is_available() and memory_snapshot_path:
                rank = dist.get_rank() if dist.is_initialized() else 0
                if rank < 8:
                    torch.cuda.memory._dump_snapshot(f"{memory_snapshot_path}.rank{rank}.pickle")
                torch.cuda.memory._record_memory_history(enabled=None)

    class ProfilerCallback(TrainerCallback):  # type: ignore[misc]
        def __init__(self) -> None:
            self._prof: Any = None

        def on_train_begin(self, args: Any, state: Any, control: Any, **kw: Any) -> None:
            from torch.profiler import ProfilerActivity, profile, schedule

            if dist.is_initialized() and dist.get_rank() != 0:
                return
            acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
            w, wu, a = profiler_schedule
            self._prof = profile(activities=acts, schedule=schedule(wait=w, warmup=wu, active=a),
                                 on_trace_ready=lambda p: p.export_chrome_trace(trace_path))
            self._prof.__enter__()

        def on_step_end(self, args: Any, state: Any, control: Any, **kw: Any) -> None:
            if self._prof is not None:
                self._prof.step()

        def on_train_end(self, args: Any, state: Any, control: Any, **kw: Any) -> None:
            if self._prof is not None:
                self._prof.__exit__(None, None, None)
                self._prof = None

    cbs: list[Any] = [IterTimeCallback()]
    if memory_snapshot_path:
        cbs.append(MemorySnapshotCallback())
    if trace_path:
        cbs.append(ProfilerCallback())
    return cbs
