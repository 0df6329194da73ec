"""Training entry points: model construction, the step function, a small trainer loop.

``build_llama`` creates the model on the meta device, shards it, then initialises the sharded
parameters (every rank draws the same full tensors and keeps its slices), so no rank ever holds an
unsharded copy of the model (the reference's examples do the same through ``init_empty_weights``,
``patches/transformers.diff:69-90``).

Run ``python -m yafsdp_b200.train --model llama2-7b --steps 10`` (under ``torchrun`` for several GPUs).
"""

from __future__ import annotations

import argparse
import json
import os
import time
from typing import Any

import torch
import torch.distributed as dist

from .api import MixedPrecisionPolicy
from .models.llama import CONFIGS, LlamaConfig, LlamaForCausalLM, shard_llama
from .optim import ShardedAdamW

__all__ = ["build_llama", "TrainStep", "smoke_step", "init_distributed"]


def init_distributed(device_type: str | None = None) -> tuple[int, int, torch.device]:
    """Initialise the default process group from the torchrun environment (or a single-process group)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available() if device_type is None else device_type == "cuda"
    if use_cuda:
        torch.cuda.set_device(local_rank)
        device = torch.device("cuda", local_rank)
    else:
        device = torch.device("cpu")
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29577")
        kw: dict[str, Any] = {}
        if use_cuda:
            kw["device_id"] = device
        dist.init_process_group("nccl" if use_cuda else "gloo", rank=rank, world_size=world, **kw)
    return rank, world, device


def build_llama(cfg: LlamaConfig, device: torch.device, *, seed: int = 0, comm_backend: Any = "auto", checkpoint_layers: int = 0,
                mp_policy: MixedPrecisionPolicy | None = None, num_grad_buffers: int = 2, mesh: Any = None,
                fused_reduce: bool | None = None, fused_gather: bool | None = None, reshard_after_forward: bool | None = True,
                **backend_options: Any) -> LlamaForCausalLM:
    from torch.distributed.device_mesh import init_device_mesh

    if mesh is None:
        mesh = init_device_mesh(device.type, (dist.get_world_size(),))
    with torch.device("meta"):
        model = LlamaForCausalLM(cfg)
    shard_llama(model, mesh=mesh, mp_policy=mp_policy, reshard_after_forward=reshard_after_forward, comm_backend=comm_backend,
                num_grad_buffers=num_grad_buffers,
                checkpoint_layers=checkpoint_layers, fused_reduce=fused_reduce, fused_gather=fused_gather, **backend_options)
    model.init_weights(seed)
    return model


class TrainStep:
    """``loss = step(input_ids_host)``: host-to-device copy of the batch from pinned memory, forward, backward, clipped AdamW."""

    def __init__(self, model: LlamaForCausalLM, optimizer: ShardedAdamW, device: torch.device):
        self.model = model
        self.optimizer = optimizer
        self.device = device
        self._ids_dev: torch.Tensor | None = None

    def __call__(self, input_ids: torch.Tensor) -> torch.Tensor:
        if input_ids.device != self.device:
            if self._ids_dev is None or self._ids_dev.shape != input_ids.shape:
                self._ids_dev = torch.empty(input_ids.shape, dtype=input_ids.dtype, device=self.device)
            self._ids_dev.copy_(input_ids, non_blocking=True)
            input_ids = self._ids_dev
        self.optimizer.zero_grad()
        loss = self.model(input_ids, labels=input_ids)
        loss.backward()
        self.optimizer.step()
        return loss


def smoke_step(device: torch.device) -> float:
    """One tiny forward + backward + optimizer step on ``device`` through the public API."""
    created = False
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29578")
        if device.type == "cuda":
            torch.cuda.set_device(device)
        dist.init_process_group("nccl" if device.type == "cuda" else "gloo", rank=0, world_size=1)
        created = True
    try:
        model = build_llama(CONFIGS["tiny-gpu"], device)
        opt = ShardedAdamW(model, lr=1e-3, max_grad_norm=1.0)
        step = TrainStep(model, opt, device)
        ids = torch.randint(0, 1024, (2, 256), generator=torch.Generator().manual_seed(0))
        if device.type == "cuda":
            ids = ids.pin_memory()
        first = float(step(ids).item())
        for _ in range(3):
            last = float(step(ids).item())
        if device.type == "cuda":
            from .ops import kernels

            kernels.check_status()
        assert last < first, f"loss did not decrease: {first} -> {last}"
        return last
    finally:
        if created:
            dist.destroy_process_group()


def parse_with_config(ap: argparse.ArgumentParser, argv: list[str] | None = None) -> argparse.Namespace:
    """``--config file.yaml`` provides defaults (keys = option names, dashes or underscores); explicit flags override them."""
    pre, _ = ap.parse_known_args(argv)
    if getattr(pre, "config", None):
        import yaml

        with open(pre.config) as f:
            values = yaml.safe_load(f) or {}
        known = {a.dest for a in ap._actions}
        defaults = {}
        for k, v in values.items():
            dest = str(k).replace("-", "_")
            if dest not in known:
                raise SystemExit(f"{pre.config}: unknown option {k!r}")
            defaults[dest] = v
        ap.set_defaults(**defaults)
    return ap.parse_args(argv)


def main() -> None:
    ap = argparse.ArgumentParser(description="Train a Llama-family model on synthetic tokens with sharded data parallelism")
    ap.add_argument("--model", default="llama2-7b", choices=sorted(CONFIGS))
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=1, help="sequences per GPU")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--max-grad-norm", type=float, default=1.0)
    ap.add_argument("--checkpoint-layers", type=int, default=0)
    ap.add_argument("--comm-backend", default="auto", choices=["auto", "torch", "symm"])
    ap.add_argument("--config", default=None, help="YAML file with defaults for the options above (command line wins)")
    args = parse_with_config(ap)
    rank, world, device = init_distributed()
    cfg = CONFIGS[args.model]
    if rank == 0:
        from .utils.memory import estimate_memory

        plan = estimate_memory(cfg, world, args.seq_len, args.batch, args.checkpoint_layers)
        print(json.dumps({"memory_plan_gib": {k: round(v / 2**30, 1) for k, v in plan.items() if k != "fits"},
                          "fits_b200": bool(plan["fits"])}), flush=True)
    model = build_llama(cfg, device, comm_backend=args.comm_backend, checkpoint_layers=args.checkpoint_layers)
    opt = ShardedAdamW(model, lr=args.lr, betas=(0.9, 0.95), weight_decay=0.1, max_grad_norm=args.max_grad_norm)
    step = TrainStep(model, opt, device)
    gen = torch.Generator().manual_seed(1 + rank)
    for i in range(args.steps):
        ids = torch.randint(0, cfg.vocab_size, (args.batch, args.seq_len), generator=gen)
        if device.type == "cuda":
            ids = ids.pin_memory()
        t0 = time.perf_counter()
        loss = step(ids).item()
        dt = time.perf_counter() - t0
        if device.type == "cuda":
            from .ops import kernels

            kernels.check_status()  # a device-side wait that ran out (a peer that stopped answering) raises here
        if rank == 0:
            print(json.dumps({"step": i, "loss": round(loss, 4), "iter_time_s": round(dt, 4),
                              "tokens_per_s_per_gpu": round(args.batch * args.seq_len / dt, 1),
                              "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2**30, 2) if device.type == "cuda" else None}))
    opt.join()
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
