"""How much each communication transport slows a co-running tcgen05 GEMM, and what the GEMM costs the transfer.

Run under torchrun on N >= 2 GPUs of one box::

    YAFSDP_SYMM_TRANSPORT=mc python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        benchmarks/comm_interference.py

(the environment variable only makes the arena multicast-capable, so that the ``mc`` variants can run too).  For every
variant the GEMM loop (main stream) and the collective loop (side stream) are timed alone and side by side with CUDA
events, max over ranks; one JSON line per variant: GEMM ms alone / beside, slowdown, collective ms alone / beside and
its bytes-per-GPU rate.  Sizes: the GEMM is a Llama-2-7B gate/up projection of 2048 tokens; the collectives move what
one GPU receives per 7B layer at 8 ranks (354 MB of bf16 parameters, 709 MB of fp32 gradients).
"""

from __future__ import annotations

import json
import math
import os
import sys

import torch
import torch.distributed as dist

try:
    import yafsdp_b200  # noqa: F401  (installed: pip install -e . --no-build-isolation)
except ImportError:  # run from a checkout that was not installed
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from yafsdp_b200.comm.symm import SymmBackend  # noqa: E402
from yafsdp_b200.ops import kernels  # noqa: E402


def max_over_ranks(x: float, dev: torch.device) -> float:
    t = torch.tensor([x], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29657")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    if world < 2:
        raise SystemExit("needs at least 2 GPUs")
    be = SymmBackend(dev, dist.group.WORLD)
    side = torch.cuda.Stream(device=dev, priority=-1)

    # ---- operands
    a = torch.randn(2048, 4096, device=dev).bfloat16()
    w = torch.randn(22016, 4096, device=dev).bfloat16()
    c = torch.empty(2048, 22016, device=dev, dtype=torch.bfloat16)
    ag_in_bytes = 354 * 2**20  # received per GPU per all-gather
    ag_shard = ag_in_bytes // 2 // (world - 1) // 8 * 8  # bf16 elements per rank
    rs_in_bytes = 709 * 2**20
    rs_shard = rs_in_bytes // 4 // (world - 1) // 8 * 8  # fp32 elements per rank
    want_mc = be.has_multicast
    saved = be.ag_transport
    be.ag_transport = "mc" if want_mc else saved  # so that the gather output comes from the arena
    ag_out = be.alloc(ag_shard * world, torch.bfloat16, dev, "gather_output")
    be.ag_transport = saved
    ag_inp = be.alloc(ag_shard, torch.bfloat16, dev, "gather_input")
    ag_inp.normal_()
    rs_inp = be.alloc(rs_shard * world, torch.float32, dev, "reduce_input")
    rs_inp.normal_()
    rs_dst = torch.zeros(rs_shard, device=dev, dtype=torch.float32)
    torch.cuda.synchronize()
    dist.barrier()
    be.step_barrier()

    def gemm() -> None:
        kernels.gemm(a, w, out=c)

    def all_gather() -> None:
        be.all_gather(ag_out, ag_inp, dist.group.WORLD)

    def reduce_scatter() -> None:
        be.reduce_scatter(rs_dst, rs_inp, dist.group.WORLD, scale=1.0 / world, accumulate=False)

    def timed(fn, iters: int, stream: torch.cuda.Stream | None = None) -> float:
        st = stream or torch.cuda.current_stream()
        torch.cuda.synchronize()
        dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(st):
            s.record()
            for _ in range(iters):
                fn()
            e.record()
        torch.cuda.synchronize()
        return max_over_ranks(s.elapsed_time(e) / iters, dev)

    def together(comm, gemm_iters: int, comm_iters: int) -> tuple[float, float]:
        torch.cuda.synchronize()
        dist.barrier()
        gs, ge = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        cs, ce = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(side):
            cs.record()
            for _ in range(comm_iters):
                comm()
            ce.record()
        gs.record()
        for _ in range(gemm_iters):
            gemm()
        ge.record()
        torch.cuda.synchronize()
        return max_over_ranks(gs.elapsed_time(ge) / gemm_iters, dev), max_over_ranks(cs.elapsed_time(ce) / comm_iters, dev)

    gemm_iters = 40
    for _ in range(3):
        gemm()
    gemm_alone = timed(gemm, gemm_iters)
    flops = 2.0 * 2048 * 22016 * 4096
    if rank == 0:
        print(json.dumps({"variant": "gemm_alone", "gemm_ms": round(gemm_alone, 4), "tflops": round(flops / gemm_alone / 1e9, 1)}), flush=True)

    variants = [
        ("ag_sm", "ag", "sm", 0), ("ag_sm_32cta", "ag", "sm", 32), ("ag_sm_8cta", "ag", "sm", 8), ("ag_ce", "ag", "ce", 0),
        ("rs_sm", "rs", "sm", 0), ("rs_sm_32cta", "rs", "sm", 32), ("rs_ce", "rs", "ce", 0),
    ]
    if want_mc:
        variants += [("ag_mc", "ag", "mc", 0), ("rs_mc", "rs", "mc", 0)]
    for name, kind, transport, ctas in variants:
        if kind == "ag":
            be.ag_transport, be.ag_ctas, comm, nbytes = transport, ctas, all_gather, ag_in_bytes
        else:
            be.rs_transport, be.rs_ctas, comm, nbytes = transport, ctas, reduce_scatter, rs_in_bytes
        for _ in range(2):
            comm()
        comm_alone = timed(comm, 6, side)
        comm_iters = max(4, min(200, math.ceil(1.5 * gemm_alone * gemm_iters / comm_alone)))
        gemm_with, comm_with = together(comm, gemm_iters, comm_iters)
        if rank == 0:
            print(json.dumps({
                "variant": name, "gemm_ms_alone": round(gemm_alone, 4), "gemm_ms_beside": round(gemm_with, 4),
                "gemm_slowdown": round(gemm_with / gemm_alone, 3), "comm_ms_alone": round(comm_alone, 4),
                "comm_ms_beside": round(comm_with, 4), "comm_gbs_alone": round(nbytes / comm_alone / 1e6, 1),
                "comm_gbs_beside": round(nbytes / comm_with / 1e6, 1), "comm_iters": comm_iters}), flush=True)
    be.ag_ctas = be.rs_ctas = 0
    kernels.check_status()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
