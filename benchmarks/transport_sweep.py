"""Step time of the Llama trainer for every transport combination of the peer-memory backend, in ONE process launch.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 benchmarks/transport_sweep.py \
        [--model llama2-7b] [--seq-len 2048] [--steps 5] [--warmup 3] [--configs ce/sm,ce/ce,...]

The model is built once (multicast arena when the box has NVSwitch multicast), then the transports are switched between
measurements with ``SymmBackend.set_transports``: a configuration costs a few steps, not a start-up.  A configuration is
``<all-gather>[:CTAs]/<reduce-scatter>[:CTAs][+1s]`` with transports ``ce`` (copy engines), ``sm`` (pull kernels),
``mc`` (NVSwitch multicast), ``cp`` (all-gather only: copy engines writing to the peers); ``+1s`` puts both collectives on one communication stream, ``+fr`` fuses the gradient
reduce-scatter into the weight-gradient GEMMs (rows pushed to their owners from the epilogue), ``+fg`` lets the first
layer gather inside its QKV GEMM, ``+rs`` (with ``--keep-gathered``) frees the parameters after forward as usual.  The configuration ``dry``
times the step with collectives that move nothing (compute-only step at this world size); put it last.  Rank 0 prints one JSON line per
configuration: CUDA-event time of ``--steps`` steps, max over ranks.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

try:
    import yafsdp_b200  # noqa: F401  (installed: pip install -e . --no-build-isolation)
except ImportError:  # run from a checkout that was not installed
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from yafsdp_b200.models.llama import CONFIGS  # noqa: E402
from yafsdp_b200.ops import kernels  # noqa: E402
from yafsdp_b200.optim import ShardedAdamW  # noqa: E402
from yafsdp_b200.train import TrainStep, build_llama, init_distributed  # noqa: E402

DEFAULT = "ce/sm,ce/sm:64,ce/sm:32,ce/ce,ce/mc,sm/sm,sm/sm+1s,mc/mc,sm:32/sm:32"


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama2-7b")
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--configs", default=DEFAULT)
    ap.add_argument("--checkpoint-layers", type=int, default=0)
    ap.add_argument("--num-grad-buffers", type=int, default=2, help="rotating fp32 gradient buffers (reduce-scatter inputs)")
    ap.add_argument("--keep-gathered", action="store_true",
                    help="give every layer its own gather buffer (reshard_after_forward=False); the flag '+rs' of a configuration then "
                         "frees and re-gathers as usual, configurations without it keep the parameters from forward to backward")
    a = ap.parse_args()
    rank, world, dev = init_distributed("cuda")
    if world < 2:
        raise SystemExit("transport_sweep needs at least 2 ranks")
    cfg = CONFIGS[a.model]
    wants_mc = "mc" in a.configs
    model = build_llama(cfg, dev, comm_backend="symm", checkpoint_layers=a.checkpoint_layers, multicast=wants_mc,
                        symmetric_gather_output="cp" in a.configs, reshard_after_forward=not a.keep_gathered, num_grad_buffers=a.num_grad_buffers)
    opt = ShardedAdamW(model, lr=1e-5, betas=(0.9, 0.95), weight_decay=0.1, max_grad_norm=1.0)
    step = TrainStep(model, opt, dev)
    ids = torch.randint(0, cfg.vocab_size, (1, a.seq_len), generator=torch.Generator().manual_seed(1 + rank)).to(dev)
    step(ids)  # lazy init
    cc = model._get_fsdp_state()._comm_ctx
    be = cc.backend
    own_rs_stream = cc.reduce_scatter_stream if cc.reduce_scatter_stream is not cc.all_gather_stream else torch.cuda.Stream(dev, priority=-1)
    for spec in a.configs.split(","):
        be.dry_run = spec == "dry"  # "dry": collectives move nothing, i.e. the compute-only step at this world size
        if spec == "dry":
            spec_run = "ce/sm"
        else:
            spec_run = spec
        flags = spec_run.split("+")[1:]
        single, fused = "1s" in flags, "fr" in flags
        first = model.model.layers[0]
        first.set_fused_gather("fg" in flags, prefix_params=[first.input_layernorm.weight])  # '+fg': layer 0 gathers inside its QKV GEMM
        if a.keep_gathered:
            from yafsdp_b200.optim import param_groups_of

            for g in param_groups_of(model):
                g.reshard_after_forward = "rs" in flags
        body = spec_run.split("+")[0]
        ag_s, rs_s = body.split("/")
        ag_p, rs_p = ag_s.split(":"), rs_s.split(":")
        ag, rs = ag_p[0], rs_p[0]
        ag_ctas = int(ag_p[1]) if len(ag_p) > 1 else 0
        rs_ctas = int(rs_p[1]) if len(rs_p) > 1 else 0
        if "mc" in (ag, rs) and not be.has_multicast:
            if rank == 0:
                print(json.dumps({"config": spec, "skipped": "no NVSwitch multicast"}), flush=True)
            continue
        torch.cuda.synchronize()
        dist.barrier()
        be.set_transports(ag, rs, ag_ctas=ag_ctas, rs_ctas=rs_ctas)
        cc.reduce_scatter_stream = cc.all_gather_stream if single else own_rs_stream
        for layer in model.model.layers:
            layer.set_fused_gradient_reduce(fused)
        model.lm_head.set_fused_gradient_reduce(fused)
        for _ in range(a.warmup):
            step(ids)
        torch.cuda.synchronize()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(a.steps):
            loss = step(ids)
        e.record()
        torch.cuda.synchronize()
        kernels.check_status()
        t = torch.tensor([s.elapsed_time(e) / a.steps], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            print(json.dumps({"config": spec, "keep_gathered": a.keep_gathered, "grad_buffers": a.num_grad_buffers, "world": world, "ms_per_step": round(float(t.item()), 2), "loss": round(float(loss.item()), 4),
                              "tokens_per_s": round(world * a.seq_len / float(t.item()) * 1e3, 1)}), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
