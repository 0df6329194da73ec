"""Fused compute + collective kernels against their rooflines, on Llama-2-7B layer shapes.

Run under torchrun on N GPUs of one box::

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/fused_paths.py

Reports (device-timed with CUDA events, max over ranks, inputs far larger than L2):

* all-gather -> GEMM: the layer's bf16 all-gather (copy engines or pull kernel) followed by the QKV GEMM, unfused vs the
  single fused kernel; roofline = max(GEMM FLOPs / measured bf16 peak, bytes that must cross NVLink / 770 GB/s);
* GEMM -> reduce-scatter: the layer's weight-gradient GEMMs (fp32) + reduce-scatter, unfused vs epilogue push + local
  slot reduction, one layer at a time and pipelined as in a backward pass (two rotating buffers, the reduction on a side
  stream under the next layer's GEMMs); same roofline rule.
"""

from __future__ import annotations

import json
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
    counters = torch.zeros(3 * d // 128, device=dev, dtype=torch.int64)
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
                              rank=rank, world=world, counters=counters, epoch=epoch[0], out=out)

    t_gemm = timed(lambda: kernels.gemm(x, wqkv, out=out), dev)
    t_ag, t_unf = {}, {}
    for tr in ("ce", "sm"):
        be.set_transports(ag=tr)
        t_ag[tr] = timed(lambda: be.all_gather(layer, inp, None), dev)
        t_unf[tr] = timed(unfused_ag_gemm, dev)
    t_fus = timed(fused_ag_gemm, dev)
    # the fused kernel must leave the same bytes behind as the plain all-gather
    be.set_transports(ag="ce")
    be.all_gather(layer, inp, None)
    want = layer.clone()
    layer.zero_()
    fused_ag_gemm()
    torch.cuda.synchronize()
    same = bool(torch.equal(layer, want))
    flops = 2.0 * t * 3 * d * d
    roof_ag = max(flops / (peak * 1e9), (world - 1) * shard * 2 / (NVLINK_GBS * 1e6))  # ms
    # ---- gradient side: dW of the four fused weights, fp32, two reduce buffers in rotation as in a backward pass
    gbufs = [be.alloc(total, torch.float32, dev, "reduce_input") for _ in range(2)]
    dst = torch.zeros(shard, device=dev, dtype=torch.float32)
    acts = {
        "qkv": (torch.randn(t, 3 * d, device=dev).bfloat16(), x, d),
        "o": (torch.randn(t, d, device=dev).bfloat16(), x, d + 3 * d * d),
        "gateup": (torch.randn(t, 2 * f, device=dev).bfloat16(), x, d + 4 * d * d + d),
        "down": (torch.randn(t, d, device=dev).bfloat16(), torch.randn(t, f, device=dev).bfloat16(), d + 4 * d * d + d + 2 * f * d),
    }

    def dw_local(gbuf):
        for dy, xx, off in acts.values():
            view = gbuf[off : off + dy.shape[1] * xx.shape[1]].view(dy.shape[1], xx.shape[1])
            kernels.gemm(dy, xx, a_mn_major=True, b_mn_major=True, out=view)

    def dw_pushed(gbuf):
        ptrs = be._peers(gbuf)
        for dy, xx, off in acts.values():
            kernels.gemm_scatter(dy, xx, a_mn_major=True, b_mn_major=True, peer_grad=ptrs, c_flat_off=off, shard_numel=shard,
                                 rank=rank, world=world)

    def dw_pushed_grouped(gbuf):
        kernels.gemm_scatter_grouped([(dy, xx, off) for dy, xx, off in acts.values()], peer_grad=be._peers(gbuf), shard_numel=shard,
                                     rank=rank, world=world)

    grouped = os.environ.get("YF_GROUPED", "1") == "1"  # one grouped launch for the layer (0: one launch per weight)
    if grouped:
        dw_pushed = dw_pushed_grouped  # noqa: F811

    def serial(fused: bool):
        def run():
            be.before_write(gbufs[0])
            if fused:
                dw_pushed(gbufs[0])
                be.reduce_pushed(dst, gbufs[0], scale=1.0 / world, accumulate=False)
            else:
                dw_local(gbufs[0])
                be.reduce_scatter(dst, gbufs[0], None, scale=1.0 / world, accumulate=False)
        return run

    # steady state of a backward pass: the reduction of layer l runs on a side stream under the GEMMs of layer l+1
    side = torch.cuda.Stream()
    n_layers = 4

    def pipelined(fused: bool):
        def run():
            cur = torch.cuda.current_stream()
            released = [None, None]
            for l in range(n_layers):
                g = gbufs[l % 2]
                if released[l % 2] is not None:
                    cur.wait_event(released[l % 2])
                be.before_write(g)
                dw_pushed(g) if fused else dw_local(g)
                ev = torch.cuda.Event()
                ev.record()
                with torch.cuda.stream(side):
                    side.wait_event(ev)
                    if fused:
                        be.reduce_pushed(dst, g, scale=1.0 / world, accumulate=False)
                    else:
                        be.reduce_scatter(dst, g, None, scale=1.0 / world, accumulate=False)
                    done = torch.cuda.Event()
                    done.record()
                released[l % 2] = done
            cur.wait_stream(side)
        return run

    be.set_transports(rs="sm")
    t_dw = timed(lambda: dw_local(gbufs[0]), dev)
    t_rs = {}
    t_unf2, t_pipe_unf = {}, {}
    for tr in ("sm", "ce"):
        be.set_transports(rs=tr)
        t_rs[tr] = timed(lambda: (be.before_write(gbufs[0]), be.reduce_scatter(dst, gbufs[0], None, scale=1.0 / world, accumulate=False)), dev)
        t_unf2[tr] = timed(serial(False), dev)
        t_pipe_unf[tr] = timed(pipelined(False), dev) / n_layers
    t_fus2 = timed(serial(True), dev)
    t_pipe_fus = timed(pipelined(True), dev) / n_layers
    # pushed GEMMs alone (nobody sums the slots): the epilogue's store rate over NVLink
    torch.cuda.synchronize()
    dist.barrier()
    be.before_write(gbufs[0])
    be.before_write(gbufs[1])
    t_scatter = timed(lambda: dw_pushed(gbufs[0]), dev)
    flops2 = 2.0 * t * (4 * d * d + 3 * f * d)
    roof_rs = max(flops2 / (peak * 1e9), (world - 1) * shard * 4 / (NVLINK_GBS * 1e6))
    # the same fused path with the gradients on the wire as bf16 (reduce_dtype=bfloat16; the owner sums in fp32)
    hbufs = [be.alloc(total, torch.bfloat16, dev, "reduce_input") for _ in range(2)]

    def fused_bf16(gbuf):
        be.before_write(gbuf)
        kernels.gemm_scatter_grouped([(dy, xx, off) for dy, xx, off in acts.values()], peer_grad=be._peers(gbuf), shard_numel=shard,
                                     rank=rank, world=world, wire_bf16=True)
        be.reduce_pushed(dst, gbuf, scale=1.0 / world, accumulate=False)

    t_fus_bf16 = timed(lambda: fused_bf16(hbufs[0]), dev)
    roof_rs_bf16 = max(flops2 / (peak * 1e9), (world - 1) * shard * 2 / (NVLINK_GBS * 1e6))
    code, site = kernels.status()
    if rank == 0:
        best_unf = min(t_unf.values())
        best_unf2 = min(t_unf2.values())
        print(json.dumps({
            "n_gpus": world, "layer_params": sum(numels), "bf16_peak_tflops_measured": peak, "nvlink_gbs": NVLINK_GBS, "status": [code, site],
            "ag_gemm": {"all_gather_ms": {k: round(v, 4) for k, v in t_ag.items()}, "gemm_ms": round(t_gemm, 4),
                        "unfused_ms": {k: round(v, 4) for k, v in t_unf.items()}, "fused_ms": round(t_fus, 4),
                        "fused_layer_buffer_equals_all_gather": same,
                        "roofline_ms": round(roof_ag, 4), "fused_fraction_of_roofline": round(roof_ag / t_fus, 3),
                        "best_unfused_fraction_of_roofline": round(roof_ag / best_unf, 3)},
            "gemm_rs": {"grouped_launch": grouped, "dw_gemms_ms": round(t_dw, 4), "pushed_gemms_ms": round(t_scatter, 4),
                        "pushed_gemms_fraction_of_roofline": round(roof_rs / t_scatter, 3),
                        "reduce_scatter_ms": {k: round(v, 4) for k, v in t_rs.items()},
                        "unfused_ms": {k: round(v, 4) for k, v in t_unf2.items()}, "fused_ms": round(t_fus2, 4),
                        "pipelined_per_layer_unfused_ms": {k: round(v, 4) for k, v in t_pipe_unf.items()},
                        "pipelined_per_layer_fused_ms": round(t_pipe_fus, 4),
                        "roofline_ms": round(roof_rs, 4), "fused_fraction_of_roofline": round(roof_rs / t_fus2, 3),
                        "pipelined_fused_fraction_of_roofline": round(roof_rs / t_pipe_fus, 3),
                        "best_unfused_fraction_of_roofline": round(roof_rs / best_unf2, 3),
                        "bf16_wire": {"fused_ms": round(t_fus_bf16, 4), "roofline_ms": round(roof_rs_bf16, 4),
                                      "fused_fraction_of_roofline": round(roof_rs_bf16 / t_fus_bf16, 3)}},
        }))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
