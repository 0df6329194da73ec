"""Headline benchmark: Llama-2-7B pre-training step, sequence length 2048, one sequence per GPU.

``python bench.py --gpus N --steps K --warmup W`` (under ``torch.distributed.run`` for N > 1) trains on
synthetic uniform-random tokens with random-init weights: bf16 compute, fp32 sharded master weights,
fp32 gradient reduction, AdamW with global-norm clipping, no activation checkpointing.  Rank 0 prints
one JSON line.  ``value`` is total tokens/s over all GPUs from CUDA-event timing of exactly K steps
(max over ranks); ``e2e`` repeats K steps through the public API with the per-step host-to-device copy
of the batch from pinned memory and a device-to-host read of the loss inside the timed region.

``--impl reference`` runs the unmodified reference package from ``baseline/_ref`` (its ``fully_shard``
around the Hugging Face Llama model and ``torch.optim.AdamW``) on the same config and prints the
same line with ``"impl": "reference"``.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch
import torch.distributed as dist

REPO = os.path.dirname(os.path.abspath(__file__))

# The reference's published iteration times (its README, A100-80G clusters, one sequence per GPU): seconds per iteration by
# (model, sequence length); tokens/s/GPU = sequence length / iteration time.  The headline row is Llama-2-7B at 2048 tokens.
PUBLISHED_ITER_S = {
    ("llama2-7b", 2048): 0.81, ("llama2-7b", 4096): 1.16, ("llama2-7b", 8192): 2.23,
    ("llama2-13b", 2048): 1.55, ("llama2-13b", 4096): 2.06,
    ("llama2-34b", 2048): 3.39, ("llama2-34b", 4096): 5.33,
    ("llama2-70b", 2048): 6.97, ("llama2-70b", 4096): 11.07,
    ("llama3-8b", 2048): 0.97, ("llama3-8b", 4096): 1.36,
    ("llama3-70b", 2048): 7.17,
}


# ----------------------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks / throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc: subprocess.Popen | None = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, power = [], [], []
        reasons: set[str] = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for n, v in zip(names, parts[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(mx) if mx else None,
            "power_w_max": max(power) if power else None,
            "samples": len(sm),
            "reasons": sorted(reasons),
        }


# ----------------------------------------------------------------------------------------- common
def setup_dist(n_gpus: int) -> tuple[int, int, torch.device]:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}: launch with python -m torch.distributed.run --nproc-per-node {n_gpus}")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29591")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    return rank, world, device


def max_over_ranks(x: float, device: torch.device) -> float:
    t = torch.tensor([x], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def timed_steps(step_fn, batches, k: int, device: torch.device, finish=None) -> float:
    """Milliseconds for exactly k calls of step_fn, CUDA events on the launching stream, barrier + sync on both sides.
    ``finish`` joins work that the steps left on side streams (an optimizer overlapped with the next forward) into the
    launching stream before the closing event, so the timed region contains all of the k steps' work."""
    dist.barrier()
    torch.cuda.synchronize()
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(k):
        step_fn(batches[i % len(batches)])
    if finish is not None:
        finish()
    end.record()
    torch.cuda.synchronize()
    dist.barrier()
    return max_over_ranks(start.elapsed_time(end), device)


def run(args, make_step) -> dict:
    rank, world, device = setup_dist(args.gpus)
    cfg_name, seq, batch = args.model, args.seq_len, args.batch
    step_dev, step_e2e, vocab, launch_counter, extra = make_step(args, rank, world, device)
    finish = extra.pop("_finish", None)
    gen = torch.Generator().manual_seed(1 + rank)
    n_batches = 4
    host_batches = [torch.randint(0, vocab, (batch, seq), generator=gen).pin_memory() for _ in range(n_batches)]
    dev_batches = [b.to(device) for b in host_batches]
    for i in range(args.warmup):
        step_dev(dev_batches[i % n_batches])
    torch.cuda.synchronize()
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    if rank == 0:
        sampler.start()
    l0 = launch_counter()
    ms = timed_steps(step_dev, dev_batches, args.steps, device, finish)
    launches = launch_counter() - l0
    step_e2e(host_batches[0])  # one untimed pass through the end-to-end path
    ms_e2e = timed_steps(step_e2e, host_batches, args.steps, device, finish)
    clocks = sampler.stop() if rank == 0 else {}
    # exposed communication, measured: the same steps once more with the collectives moving nothing between the GPUs
    # (compute-only step at this world size; the values it computes are meaningless, it runs last)
    ms_dry = None
    dry = extra.pop("_dry_run", None)
    if dry is not None and world > 1:
        dry(True)
        for i in range(2):
            step_dev(dev_batches[i % n_batches])
        ms_dry = timed_steps(step_dev, dev_batches, args.steps, device, finish)
        dry(False)
    # host time to issue one step into an empty queue (no device wait inside): when it approaches ms_per_step the step is
    # bound by the launching CPU thread, not by the GPU
    torch.cuda.synchronize()
    dist.barrier()
    t0 = time.perf_counter()
    step_dev(dev_batches[0])
    host_issue_ms = max_over_ranks((time.perf_counter() - t0) * 1e3, device)
    torch.cuda.synchronize()
    tokens = batch * seq * world * args.steps
    value = tokens / (ms / 1e3)
    e2e_value = tokens / (ms_e2e / 1e3)
    peak_gb = torch.cuda.max_memory_allocated() / 2**30
    result = {
        "metric": "tokens_per_second",
        "value": round(value, 1),
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(ms / args.steps, 3),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": (round(value / world / (seq / PUBLISHED_ITER_S[(cfg_name, seq)]), 3) if (cfg_name, seq) in PUBLISHED_ITER_S else None),
        "dtype": "bf16",
        "data": "synthetic uniform-random tokens, random-init N(0,0.02) weights",
        "impl": args.impl,
        "config": {
            "model": cfg_name,
            "global_batch": batch * world,
            "seq_len": seq,
            "parallelism": f"dp{world} fully sharded (ZeRO-3)",
            "optimizer": "AdamW fp32 master/grad/moments, global-norm clip 1.0",
            "activation_checkpointing": args.checkpoint_layers,
            "params": extra.pop("params"),
            "l2": "no explicit flush: every step streams far more than the 126 MB L2 (weights, gradients, optimizer state)",
            "vs_baseline_is": "tokens/s/GPU over the reference's published figure for this model and sequence length (A100-80G clusters; 2528 tokens/s/GPU for Llama-2-7B at 2048)",
            "impl_detail": extra,
        },
        "clocks": clocks,
        "e2e": {
            "value": round(e2e_value, 1),
            "unit": "tokens/s",
            "ms_per_step": round(ms_e2e / args.steps, 3),
            "h2d_bytes_per_step": batch * seq * 8,
            "d2h_bytes_per_step": 4,
        },
        "gpu_launches": int(launches),
        "tokens_per_s_per_gpu": round(value / world, 1),
        "peak_mem_gb": round(peak_gb, 2),
        "host_issue_ms_per_step": round(host_issue_ms, 2),
    }
    if ms_dry is not None:
        result["compute_only_ms_per_step"] = round(ms_dry / args.steps, 3)
        result["exposed_comm_ms"] = round((ms - ms_dry) / args.steps, 3)
        result["exposed_comm_fraction"] = round((ms - ms_dry) / ms, 4)
    if rank == 0:
        print(json.dumps(result), flush=True)
    dist.destroy_process_group()
    return result


def resolve_reshard(args, world: int) -> bool:
    """``--reshard-after-forward auto`` (both arms alike): layers keep their gathered bf16 parameters between forward and
    backward (one all-gather per layer and step instead of two) when the whole bf16 model fits beside the sharded plan in
    60 % of a B200's memory, else they are freed after forward and gathered again for backward."""
    if args.reshard_after_forward != "auto":
        return args.reshard_after_forward == "true"
    from yafsdp_b200.models.llama import CONFIGS
    from yafsdp_b200.utils.memory import keep_gathered_fits

    return not keep_gathered_fits(CONFIGS[args.model], world, args.seq_len, args.batch, args.checkpoint_layers)


# ----------------------------------------------------------------------------------------- ours
def make_step_ours(args, rank: int, world: int, device: torch.device):
    from yafsdp_b200.models.llama import CONFIGS
    from yafsdp_b200.ops import kernels
    from yafsdp_b200.optim import ShardedAdamW
    from yafsdp_b200.train import TrainStep, build_llama

    cfg = CONFIGS[args.model]
    reshard = resolve_reshard(args, world)
    model = build_llama(cfg, device, comm_backend=args.comm_backend, checkpoint_layers=args.checkpoint_layers,
                        reshard_after_forward=reshard)
    opt = ShardedAdamW(model, lr=1e-5, betas=(0.9, 0.95), weight_decay=0.1, max_grad_norm=1.0)
    step = TrainStep(model, opt, device)

    def step_dev(ids_dev: torch.Tensor) -> None:
        step(ids_dev)

    def step_e2e(ids_host: torch.Tensor) -> float:
        return step(ids_host).item()

    backend = args.comm_backend if args.comm_backend != "auto" else ("symm" if world > 1 else "none (single rank: buffers aliased)")

    pushed_groups: list = []

    def dry_run(on: bool) -> None:
        be = model._get_fsdp_state()._comm_ctx.backend
        if hasattr(be, "dry_run"):
            torch.cuda.synchronize()
            dist.barrier()
            be.dry_run = on
            # gradients pushed from the GEMM epilogues would still cross NVLink: the compute-only step reduces locally
            from yafsdp_b200.optim import param_groups_of

            if on:
                pushed_groups[:] = [g for g in param_groups_of(model) if g.fused_reduce]
            for g in pushed_groups:
                g.fused_reduce = not on

    detail = {"comm_backend": backend, "params": cfg.num_params(), "_finish": opt.join, "reshard_after_forward": reshard}
    if backend == "symm":
        detail["_dry_run"] = dry_run
    return step_dev, step_e2e, cfg.vocab_size, kernels.launch_count, detail


# ----------------------------------------------------------------------------------------- reference
def make_step_reference(args, rank: int, world: int, device: torch.device):
    ref_root = os.path.join(REPO, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "ya_fsdp")):
        raise RuntimeError("baseline/_ref/ya_fsdp is missing (reference not installed)")
    sys.path.insert(0, ref_root)
    import ya_fsdp  # the unmodified reference
    from torch.distributed.device_mesh import init_device_mesh
    from transformers import LlamaConfig as HFLlamaConfig
    from transformers import LlamaForCausalLM as HFLlama

    from yafsdp_b200.models.llama import CONFIGS  # shapes only

    c = CONFIGS[args.model]
    attn_impl = args.ref_attn
    hf_cfg = HFLlamaConfig(
        vocab_size=c.vocab_size, hidden_size=c.hidden_size, intermediate_size=c.intermediate_size,
        num_hidden_layers=c.num_hidden_layers, num_attention_heads=c.num_attention_heads,
        num_key_value_heads=c.num_key_value_heads, rms_norm_eps=c.rms_norm_eps, rope_theta=c.rope_theta,
        max_position_embeddings=max(c.max_position_embeddings, args.seq_len), tie_word_embeddings=False,
        use_cache=False, attn_implementation=attn_impl,
    )
    torch.manual_seed(0)
    with torch.device(device):
        model = HFLlama(hf_cfg)
    model.train()
    mesh = init_device_mesh("cuda", (world,))
    mp = ya_fsdp.MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    # With one rank the reference's all-gather is `output.copy_(input)`, which bumps the autograd version
    # counter of its shared rotating buffers, so its default configuration fails in backward ("modified by
    # an inplace operation").  Its public `reshard_after_forward=False` gives every group its own buffer and
    # skips the backward re-gather, which runs; with one rank there is no communication either way.
    kw = dict(mesh=mesh, mp_policy=mp)
    reshard = resolve_reshard(args, world)  # the same rule as in the other arm
    if world == 1 or not reshard:
        kw["reshard_after_forward"] = False
    if args.checkpoint_layers:
        # the reference's recipe: non-reentrant activation checkpointing on the first N decoder layers, applied before sharding
        from torch.distributed.algorithms._checkpoint.checkpoint_wrapper import CheckpointImpl, checkpoint_wrapper

        for i in range(min(args.checkpoint_layers, len(model.model.layers))):
            model.model.layers[i] = checkpoint_wrapper(model.model.layers[i], checkpoint_impl=CheckpointImpl.NO_REENTRANT)
    ya_fsdp.fully_shard(model.model.embed_tokens, **kw)
    for layer in model.model.layers:
        ya_fsdp.fully_shard(layer, **kw)
    ya_fsdp.fully_shard([model.model.norm, model.lm_head], **kw)
    ya_fsdp.fully_shard(model, **kw)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-5, betas=(0.9, 0.95), weight_decay=0.1, fused=True)
    ids_dev = torch.empty((args.batch, args.seq_len), dtype=torch.int64, device=device)

    def one(ids: torch.Tensor) -> torch.Tensor:
        opt.zero_grad(set_to_none=True)
        loss = model(input_ids=ids, labels=ids).loss
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0, foreach=True)
        opt.step()
        return loss

    def step_dev(ids: torch.Tensor) -> None:
        one(ids)

    def step_e2e(ids_host: torch.Tensor) -> float:
        ids_dev.copy_(ids_host, non_blocking=True)
        return one(ids_dev).item()

    return step_dev, step_e2e, c.vocab_size, (lambda: 0), {
        "attn_implementation": attn_impl, "params": c.num_params(), "model_code": "transformers.LlamaForCausalLM",
        "reshard_after_forward": world != 1 and reshard}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama2-7b")
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=1, help="sequences per GPU")
    ap.add_argument("--comm-backend", default="auto", choices=["auto", "torch", "symm"])
    ap.add_argument("--ref-attn", default="sdpa", choices=["sdpa", "flash_attention_2", "eager"])
    ap.add_argument("--checkpoint-layers", type=int, default=0, help="activation checkpointing on the first N decoder layers")
    ap.add_argument("--reshard-after-forward", default="auto", choices=["auto", "true", "false"],
                    help="free the gathered parameters after forward (true), keep them until backward (false), or keep them when they fit (auto)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        try:
            run(args, make_step_reference)
        except Exception as e:  # the reference arm must never fail the driver: report why instead
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:300]}"}), flush=True)
            if dist.is_initialized():
                dist.destroy_process_group()
        return
    run(args, make_step_ours)


if __name__ == "__main__":
    main()
