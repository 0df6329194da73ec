"""Fused compute + collective kernels against their rooflines, on Llama-2-7B layer shapes.

Run under torchrun on N GPUs of one box::

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/fused_paths.py

Reports (device-timed with CUDA events, max over ranks, inputs far larger than L2):

* all-gather -> GEMM: the layer's bf16 all-gather (pull) followed by the QKV GEMM, unfused vs the single fused
  kernel; roofline = max(GEMM FLOPs / measured bf16 peak, bytes that must cross NVLink / 770 GB/s);
* GEMM -> reduce-scatter: the layer's weight-gradient GEMMs (fp32) + pull reduce-scatter, unfused vs epilogue
  push + local slot reduction; same roofline rule.
"""

from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from yafsdp_b200.comm.symm import SymmBackend, _ptr_array  # noqa: E402
from yafsdp_b200.ops import kernels  # noqa: E402

NVLINK_GBS = 770.0


def peaks() -> float:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["bf16_tflops"])
    except Exception:
        return 1590.0


def timed(fn, dev, iters=8, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main() -> None:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    be = SymmBackend(dev, dist.group.WORLD)
    peak = peaks()
    d, f, t = 4096, 11008, 2048
    # flat layer: [norm1 | wq wk wv | wo | norm2 | gate up | down]
    numels = [d, 3 * d * d, d * d, d, 2 * f * d, f * d]
    total = sum(numels)
    total = (total + world * 8 - 1) // (world * 8) * (world * 8)
    shard = total // world
    qkv_off = d
    x = torch.randn(t, d, device=dev).bfloat16()
    inp = be.alloc(shard, torch.bfloat16, dev, "gather_input")
    inp.copy_(torch.randn(shard, device=dev).bfloat16() * 0.02)
    layer = torch.empty(total, device=dev, dtype=torch.bfloat16)
    flags = torch.zeros(world * 1024 + 64, device=dev, dtype=torch.int32)
    out = torch.empty(t, 3 * d, device=dev, dtype=torch.bfloat16)
    torch.cuda.synchronize()
    be.step_barrier()
    wqkv = layer[qkv_off : qkv_off + 3 * d * d].view(3 * d, d)
    epoch = [0]

    def unfused_ag_gemm():
        be.all_gather(layer, inp, None)
        kernels.gemm(x, wqkv, out=out)

    def fused_ag_gemm():
        epoch[0] += 1
        kernels.gemm_gathered(x, 3 * d, d, peer_in=be._peers(inp), layer_buf=layer, shard_bytes=shard * 2, b_byte_off=qkv_off * 2,
                              rank=rank, world=world, flags=flags, epoch=epoch[0], chunk_bytes=1 << 20, n_comm=int(os.environ.get("YF_NCOMM", "32")),
                              out=out)

    t_ag = timed(lambda: be.all_gather(layer, inp, None), dev)
    t_gemm = timed(lambda: kernels.gemm(x, wqkv, out=out), dev)
    t_unf = timed(unfused_ag_gemm, dev)
    t_fus = timed(fused_ag_gemm, dev)
    flops = 2.0 * t * 3 * d * d
    roof_ag = max(flops / (peak * 1e9), (world - 1) * shard * 2 / (NVLINK_GBS * 1e6))  # ms
    # ---- gradient side: dW of the four fused weights, fp32
    gbuf = be.alloc(total, torch.float32, dev, "reduce_input")
    dst = torch.zeros(shard, device=dev, dtype=torch.float32)
    acts = {
        "qkv": (torch.randn(t, 3 * d, device=dev).bfloat16(), x, d),
        "o": (torch.randn(t, d, device=dev).bfloat16(), x, d + 3 * d * d),
        "gateup": (torch.randn(t, 2 * f, device=dev).bfloat16(), x, d + 4 * d * d + d),
        "down": (torch.randn(t, d, device=dev).bfloat16(), torch.randn(t, f, device=dev).bfloat16(), d + 4 * d * d + d + 2 * f * d),
    }
    local_slots = _ptr_array([gbuf.data_ptr() + (r - rank) * shard * 4 for r in range(world)])

    def unfused_dw_rs():
        for dy, xx, off in acts.values():
            view = gbuf[off : off + dy.shape[1] * xx.shape[1]].view(dy.shape[1], xx.shape[1])
            kernels.gemm(dy, xx, a_mn_major=True, b_mn_major=True, out=view)
        be.reduce_scatter(dst, gbuf, None, scale=1.0 / world, accumulate=False)

    def fused_dw_rs():
        for dy, xx, off in acts.values():
            kernels.gemm_scatter(dy, xx, a_mn_major=True, b_mn_major=True, peer_grad=be._peers(gbuf), c_flat_off=off, shard_numel=shard,
                                 rank=rank, world=world)
        be.barrier(1)
        rc = kernels._native.lib().yf_reduce_scatter_pull(local_slots, dst.data_ptr(), shard, rank, world, 1.0 / world, 0, 0, 0,
                                                          torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        be.barrier(2)

    def dw_only():
        for dy, xx, off in acts.values():
            view = gbuf[off : off + dy.shape[1] * xx.shape[1]].view(dy.shape[1], xx.shape[1])
            kernels.gemm(dy, xx, a_mn_major=True, b_mn_major=True, out=view)

    def scatter_only():
        for dy, xx, off in acts.values():
            kernels.gemm_scatter(dy, xx, a_mn_major=True, b_mn_major=True, peer_grad=be._peers(gbuf), c_flat_off=off, shard_numel=shard,
                                 rank=rank, world=world)

    # steady state of a backward pass: the reduction of layer l runs on a side stream under the GEMMs of layer l+1
    side = torch.cuda.Stream()
    n_layers = 4

    def pipelined(fused: bool):
        def run():
            for _ in range(n_layers):
                scatter_only() if fused else dw_only()
                ev = torch.cuda.Event()
                ev.record()
                with torch.cuda.stream(side):
                    side.wait_event(ev)
                    if fused:
                        be.barrier(1)
                        kernels._native.lib().yf_reduce_scatter_pull(local_slots, dst.data_ptr(), shard, rank, world, 1.0 / world, 0, 0, 0,
                                                                     side.cuda_stream)
                        be.barrier(2)
                    else:
                        be.reduce_scatter(dst, gbuf, None, scale=1.0 / world, accumulate=False)
                    done = torch.cuda.Event()
                    done.record()
                torch.cuda.current_stream().wait_event(done) if False else None
            torch.cuda.current_stream().wait_stream(side)
        return run

    t_dw = timed(dw_only, dev)
    t_scatter = timed(scatter_only, dev)
    t_pipe_unf = timed(pipelined(False), dev) / n_layers
    t_pipe_fus = timed(pipelined(True), dev) / n_layers
    t_rs = timed(lambda: be.reduce_scatter(dst, gbuf, None, scale=1.0 / world, accumulate=False), dev)
    t_unf2 = timed(unfused_dw_rs, dev)
    t_fus2 = timed(fused_dw_rs, dev)
    flops2 = 2.0 * t * (4 * d * d + 3 * f * d)
    roof_rs = max(flops2 / (peak * 1e9), (world - 1) * shard * 4 / (NVLINK_GBS * 1e6))
    code, site = kernels.status()
    if rank == 0:
        print(json.dumps({
            "n_gpus": world, "layer_params": sum(numels), "bf16_peak_tflops_measured": peak, "nvlink_gbs": NVLINK_GBS, "status": [code, site],
            "ag_gemm": {"all_gather_ms": round(t_ag, 4), "gemm_ms": round(t_gemm, 4), "unfused_ms": round(t_unf, 4), "fused_ms": round(t_fus, 4),
                        "roofline_ms": round(roof_ag, 4), "fused_fraction_of_roofline": round(roof_ag / t_fus, 3),
                        "unfused_fraction_of_roofline": round(roof_ag / t_unf, 3)},
            "gemm_rs": {"dw_gemms_ms": round(t_dw, 4), "scatter_gemms_ms": round(t_scatter, 4),
                        "scatter_gemms_fraction_of_roofline": round(roof_rs / t_scatter, 3),
                        "pipelined_per_layer_unfused_ms": round(t_pipe_unf, 4), "pipelined_per_layer_fused_ms": round(t_pipe_fus, 4),
                        "pipelined_fused_fraction_of_roofline": round(roof_rs / t_pipe_fus, 3), "reduce_scatter_ms": round(t_rs, 4), "unfused_ms": round(t_unf2, 4), "fused_ms": round(t_fus2, 4),
                        "roofline_ms": round(roof_rs, 4), "fused_fraction_of_roofline": round(roof_rs / t_fus2, 3),
                        "unfused_fraction_of_roofline": round(roof_rs / t_unf2, 3)},
        }))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
