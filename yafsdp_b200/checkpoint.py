"""Checkpoint save / load / reshard for ragged-sharded models.

On-disk format (identical to what the reference produces through ``torch.distributed.checkpoint``,
``ya_fsdp/_tensor.py:365-432``): every parameter (and every optimizer moment) is a 1-D tensor of
``numel`` elements; each rank writes one chunk at offset ``(global_offset,)`` of size
``(local_numel,)``; keys are the original module FQNs.

What the reference does not ship and this module adds:

* ``RaggedLoadPlanner``: the default DCP load planner rejects the flat format ("Size mismatch between
  saved torch.Size([numel]) and current torch.Size([rows, cols])"); this planner reads exactly the
  slices a rank needs, from however many saved chunks cover them, so a checkpoint written by W ranks
  loads into any other world size (resharding) or into an unsharded model;
* ``full_state_dict``: gather every parameter to rank 0 on CPU under its original name and shape;
* ``local_state_dict_v1``: the per-rank "local" checkpoint layout of the reference's first-generation
  wrapper (``ya_fsdp/ya_fsdp.py:236-311,566-573``) including its ``"meta"`` dictionary.
"""

from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp
import torch.nn as nn
from torch.distributed.checkpoint.default_planner import DefaultLoadPlanner
from torch.distributed.checkpoint.metadata import BytesStorageMetadata, MetadataIndex, TensorStorageMetadata
from torch.distributed.checkpoint.planner import LoadItemType, LoadPlan, ReadItem
from torch.distributed.checkpoint.planner_helpers import _create_read_items

from .optim import param_groups_of
from .tensor import RaggedShardDTensor

__all__ = ["save", "load", "RaggedLoadPlanner", "full_state_dict", "local_state_dict_v1", "load_local_state_dict_v1"]


def _flat_read_items(fqn: str, md: TensorStorageMetadata, lo: int, n: int, dest_offset_index: tuple[int, ...]) -> list[ReadItem]:
    """Read items that fill the flat range ``[lo, lo + n)`` of a saved 1-D tensor from its saved chunks."""
    items: list[ReadItem] = []
    hi = lo + n
    for idx, chunk in enumerate(md.chunks):
        c_lo = int(chunk.offsets[0])
        c_hi = c_lo + int(chunk.sizes[0])
        a, b = max(lo, c_lo), min(hi, c_hi)
        if b <= a:
            continue
        items.append(
            ReadItem(
                type=LoadItemType.TENSOR,
                dest_index=MetadataIndex(fqn, torch.Size(dest_offset_index)),
                dest_offsets=torch.Size([a - lo]),
                storage_index=MetadataIndex(fqn, chunk.offsets, idx),
                storage_offsets=torch.Size([a - c_lo]),
                lengths=torch.Size([b - a]),
            )
        )
    return items


class RaggedLoadPlanner(DefaultLoadPlanner):
    """Load planner that understands the flat per-parameter format for ``RaggedShardDTensor`` destinations and for
    plain tensors whose saved form is flat (an unsharded model loading a sharded checkpoint)."""

    def create_local_plan(self) -> LoadPlan:
        assert self.metadata is not None
        requests: list[ReadItem] = []
        self._flat_views: dict[str, torch.Tensor] = {}
        for fqn, obj in self.state_dict.items():
            if fqn not in self.metadata.state_dict_metadata:
                if self.allow_partial_load:
                    continue
                raise RuntimeError(f"Missing key in checkpoint state_dict: {fqn}.")
            md = self.metadata.state_dict_metadata[fqn]
            if isinstance(obj, RaggedShardDTensor):
                if not isinstance(md, TensorStorageMetadata) or len(md.size) != 1 or int(md.size[0]) != obj._spec.global_numel:
                    raise ValueError(f"{fqn}: saved entry {getattr(md, 'size', None)} is not the flat form of a tensor with {obj._spec.global_numel} elements")
                pl = obj._spec.placement
                lo = obj._spec.outer_offset + pl.global_offset
                requests += _flat_read_items(fqn, md, lo, pl.local_numel, (lo,))
            elif (isinstance(obj, torch.Tensor) and isinstance(md, TensorStorageMetadata) and len(md.size) == 1
                  and obj.dim() != 1 and int(md.size[0]) == obj.numel()):
                if not obj.is_contiguous():
                    raise ValueError(f"{fqn}: loading a flat checkpoint entry into a non-contiguous tensor")
                self._flat_views[fqn] = obj.detach().view(-1)
                requests += _flat_read_items(fqn, md, 0, obj.numel(), (0,))
            elif isinstance(md, BytesStorageMetadata) or isinstance(obj, torch.Tensor):
                requests += _create_read_items(fqn, md, obj)
            else:
                requests += _create_read_items(fqn, md, obj)
        return LoadPlan(requests)

    def lookup_tensor(self, index: MetadataIndex) -> torch.Tensor:
        flat = getattr(self, "_flat_views", {}).get(index.fqn)
        if flat is not None:
            return flat
        return super().lookup_tensor(index)


def _state(model: nn.Module, optimizer: Any | None) -> dict[str, Any]:
    sd: dict[str, Any] = {"model": model.state_dict()}
    if optimizer is not None:
        sd["optim"] = optimizer.state_dict()
    return sd


def save(path: str, model: nn.Module, optimizer: Any | None = None, extra: dict[str, Any] | None = None) -> None:
    """Write a sharded checkpoint directory (every rank calls this)."""
    sd = _state(model, optimizer)
    if extra:
        sd["extra"] = dict(extra)
    dcp.save(sd, checkpoint_id=path)


def load(path: str, model: nn.Module, optimizer: Any | None = None, extra: dict[str, Any] | None = None) -> dict[str, Any]:
    """Load a checkpoint written by :func:`save` (by any world size) into ``model`` / ``optimizer`` in place."""
    sd = _state(model, optimizer)
    if extra is not None:
        sd["extra"] = dict(extra)
    dcp.load(sd, checkpoint_id=path, planner=RaggedLoadPlanner())
    if optimizer is not None and hasattr(optimizer, "load_state_dict"):
        optimizer.load_state_dict(sd["optim"])
    for g in param_groups_of(model):
        g._ag_input_fresh = False  # the compute-dtype copies are stale now
    return sd.get("extra", {})


def full_state_dict(model: nn.Module, rank0_only: bool = True) -> dict[str, torch.Tensor]:
    """Unsharded CPU tensors under the original names (a collective: every rank must call it).  With
    ``rank0_only`` other ranks return an empty dict (the reference's first-generation ``state_dict()``,
    ``ya_fsdp/ya_fsdp.py:575-584``)."""
    out: dict[str, torch.Tensor] = {}
    keep = (not rank0_only) or (not dist.is_initialized()) or dist.get_rank() == 0
    for name, t in model.state_dict().items():
        if isinstance(t, RaggedShardDTensor):
            full = t.full_tensor()
            if keep:
                out[name] = full.cpu()
        elif keep:
            out[name] = t.detach().cpu()
    return out


def _split_norm_group(model: nn.Module) -> tuple[list[Any], list[Any]]:
    groups = param_groups_of(model)
    return [g for g in groups if not getattr(g, "is_norm_group", False)], [g for g in groups if getattr(g, "is_norm_group", False)]


def local_state_dict_v1(model: nn.Module) -> dict[str, Any]:
    """Per-rank local checkpoint in the first-generation layout: ``"main_parameter"`` is the concatenation of this rank's flat
    shard of every wrapped group (in wrap order), ``"layernorm_parameter"`` this rank's flat shard of the norm group (empty
    when the model was wrapped without one), and rank 0 adds ``"meta"`` with the shard sizes, padded sizes and per-group
    parameter names, sizes and shapes (key spellings as in the reference, including ``main_parameter_shard_bounaries``)."""
    groups, norm = _split_norm_group(model)
    dev = groups[0].device if groups else torch.device("cpu")
    sd: dict[str, Any] = {
        "main_parameter": torch.cat([g.master_flat.detach().reshape(-1) for g in groups]) if groups else torch.empty(0),
        "layernorm_parameter": torch.cat([g.master_flat.detach().reshape(-1) for g in norm]) if norm else torch.empty(0, device=dev),
    }
    for name, buf in model.named_buffers():
        if name.rpartition(".")[2] not in getattr(model.get_submodule(name.rpartition(".")[0]), "_non_persistent_buffers_set", ()):
            sd["module." + name] = buf
    rank = dist.get_rank() if dist.is_initialized() else 0
    if rank == 0:
        sd["meta"] = {
            "main_parameter_shard_bounaries": [g.layout.shard_numel for g in groups],
            "main_parameter_padded_numels": [g.layout.padded_numel for g in groups],
            "main_shards_fqns": [[sp.fqn or sp.info.param_name for sp in g.params] for g in groups],
            "main_shards_numels": [[sp.numel for sp in g.params] for g in groups],
            "main_parameter_orig_shapes": [[tuple(sp.orig_shape) for sp in g.params] for g in groups],
            "layernorm_fqns": [[sp.fqn or sp.info.param_name for sp in g.params] for g in norm],
            "layernorm_numels": [[sp.numel for sp in g.params] for g in norm],
            "layernorm_orig_shapes": [[tuple(sp.orig_shape) for sp in g.params] for g in norm],
        }
    return sd


def load_local_state_dict_v1(model: nn.Module, sd: dict[str, Any]) -> None:
    """Inverse of :func:`local_state_dict_v1` (same world size and padding only, like the reference)."""
    sd = dict(sd)
    sd.pop("meta", None)
    groups, norm = _split_norm_group(model)
    with torch.no_grad():
        for key, gs in (("main_parameter", groups), ("layernorm_parameter", norm)):
            flat = sd[key]
            o = 0
            for g in gs:
                n = g.layout.shard_numel
                g.master_flat.copy_(flat[o : o + n])
                g._ag_input_fresh = False
                o += n
            if o != flat.numel():
                raise ValueError(f"local state dict entry {key!r} has {flat.numel()} elements, the model's shards hold {o}")
        buffers = dict(model.named_buffers())
        for k, v in sd.items():
            if k.startswith("module.") and k[len("module."):] in buffers:
                buffers[k[len("module."):]].copy_(v)
