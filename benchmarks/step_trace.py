"""Where a training step's device time goes: per-stream kernel totals and the idle gaps of the compute stream.

Run under torchrun on N GPUs of one box (or plain ``python`` for one GPU)::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 benchmarks/step_trace.py \
        [--model llama2-7b] [--seq-len 2048] [--steps 2] [--out DIR]

Rank 0 records ``--steps`` steps with ``torch.profiler`` (CUDA activities only) after 4 warm-up steps, prints

* per stream: number of kernels, busy time, and the top kernels with count / median / max duration;
* the compute stream's idle gaps longer than 20 us, grouped by the pair of kernels around them,

* the GEMM time of the last step by what ran beside each GEMM (all-gather kernel, reduce-scatter kernel, nothing),

and writes the same text plus the gzipped Chrome trace into ``--out``.  ``--analyze TRACE [--baseline TRACE]`` repeats the
last report on a stored trace without a GPU and compares launch by launch with a baseline trace (e.g. one GPU).  Kernels run slower under the profiler than in
``bench.py``; compare shares and per-kernel medians between world sizes, not the span.
"""

from __future__ import annotations

import argparse
import collections
import gzip
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist
from torch.profiler import ProfilerActivity, profile

try:
    import yafsdp_b200  # noqa: F401  (installed: pip install -e . --no-build-isolation)
except ImportError:  # run from a checkout that was not installed
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from yafsdp_b200.models.llama import CONFIGS  # noqa: E402
from yafsdp_b200.optim import ShardedAdamW  # noqa: E402
from yafsdp_b200.train import TrainStep, build_llama  # noqa: E402


def summarize(trace_path: str, world: int, steps: int) -> str:
    d = json.load(open(trace_path))
    ev = [e for e in d["traceEvents"] if e.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset") and "dur" in e]
    ev.sort(key=lambda e: e["ts"])
    t0 = ev[0]["ts"]
    t1 = max(e["ts"] + e["dur"] for e in ev)
    out = [f"world {world} span ms {(t1 - t0) / 1e3:.2f} events {len(ev)} ({steps} steps)"]
    streams: dict = collections.defaultdict(list)
    for e in ev:
        streams[e["args"].get("stream")].append(e)
    main = max(streams, key=lambda s: len(streams[s]))
    for s, es in streams.items():
        out.append(f"stream {s}{' (main)' if s == main else ''} n {len(es)} busy ms {sum(e['dur'] for e in es) / 1e3:.2f}")
        agg: dict = collections.defaultdict(list)
        for e in es:
            agg[e["name"][:48]].append(e["dur"] / 1e3)
        for k, v in sorted(agg.items(), key=lambda x: -sum(x[1]))[: 28 if s == main else 8]:
            out.append(f"    {sum(v):8.2f} ms n={len(v):4d} med {statistics.median(v):.3f} max {max(v):.3f}  {k}")
    es = streams[main]
    gaps = []
    for a, b in zip(es, es[1:]):
        g = b["ts"] - (a["ts"] + a["dur"])
        if g > 20:
            gaps.append((g, a["name"][:40], b["name"][:40]))
    out.append(f"main stream gaps >20us: total {sum(g for g, *_ in gaps) / 1e3:.2f} ms n {len(gaps)}")
    hist: dict = collections.defaultdict(lambda: [0, 0.0])
    for g, a, b in gaps:
        hist[f"{a} -> {b}"][0] += 1
        hist[f"{a} -> {b}"][1] += g / 1e3
    for k, (n, t) in sorted(hist.items(), key=lambda x: -x[1][1])[:20]:
        out.append(f"    {t:7.2f} ms n={n:3d} {k}")
    return "\n".join(out)


def _load_kernels(path: str) -> list:
    with (gzip.open(path) if path.endswith(".gz") else open(path, "rb")) as f:
        d = json.load(f)
    ev = [e for e in d["traceEvents"] if e.get("cat") in ("kernel", "gpu_memcpy") and "dur" in e]
    ev.sort(key=lambda e: e["ts"])
    return ev


def overlap_report(trace_path: str, baseline_path: str | None, steps: int) -> str:
    """GEMM time of the last recorded step by what ran beside each GEMM (all-gather kernel, reduce-scatter kernel, nothing),
    and, with a baseline trace of the same model (e.g. one GPU), the same launches' time there."""
    ev = _load_kernels(trace_path)
    is_gemm = lambda e: "gemm_bf16" in e["name"]  # noqa: E731
    gemms = [e for e in ev if is_gemm(e)]
    # the all-gather is a kernel (pull / multicast transports) or peer copies on the copy engines
    ag = [e for e in ev if "allgather" in e["name"] or (e.get("cat") == "gpu_memcpy" and ("PtoP" in e["name"] or "DtoD" in e["name"]) and e["dur"] > 50)]
    rs = [e for e in ev if "reduce_scatter" in e["name"]]
    per = len(gemms) // steps
    last = gemms[-per:]
    base = None
    if baseline_path:
        bg = [e for e in _load_kernels(baseline_path) if is_gemm(e)]
        if len(bg) >= per and len(bg) % per == 0:
            base = bg[-per:]

    def frac(e: dict, others: list) -> float:
        s, t = e["ts"], e["ts"] + e["dur"]
        return sum(max(0.0, min(t, c["ts"] + c["dur"]) - max(s, c["ts"])) for c in others) / e["dur"]

    cls: dict = collections.defaultdict(lambda: [0, 0.0, 0.0])
    for i, e in enumerate(last):
        a, r = frac(e, ag), frac(e, rs)
        key = (("all-gather " if a > 0.5 else "") + ("reduce-scatter" if r > 0.5 else "")).strip() or ("partial" if a + r > 0.05 else "alone")
        cls[key][0] += 1
        cls[key][1] += e["dur"] / 1e3
        if base is not None:
            cls[key][2] += base[i]["dur"] / 1e3
    out = [f"GEMM launches of the last step: {per}, total {sum(e['dur'] for e in last) / 1e3:.2f} ms"
           + (f" (baseline trace: {sum(e['dur'] for e in base) / 1e3:.2f} ms)" if base is not None else "")]
    for k, (n, t, tb) in sorted(cls.items(), key=lambda x: -x[1][1]):
        out.append(f"    beside {k:28s} n={n:4d} {t:7.2f} ms" + (f"   same launches in the baseline {tb:7.2f} ms  x{t / tb:.2f}" if tb else ""))
    return "\n".join(out)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--analyze", default=None, help="only analyse this trace (.json or .json.gz); needs no GPU")
    ap.add_argument("--baseline", default=None, help="with --analyze: a trace of the same model to compare GEMM launches with")
    ap.add_argument("--model", default="llama2-7b", choices=sorted(CONFIGS))
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--out", default="trace_out")
    args = ap.parse_args()
    if args.analyze:
        print(overlap_report(args.analyze, args.baseline, args.steps))
        return
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29655")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    cfg = CONFIGS[args.model]
    from yafsdp_b200.utils.memory import keep_gathered_fits

    keep = keep_gathered_fits(cfg, world, args.seq_len)  # the rule bench.py applies: keep the gathered weights when they fit
    model = build_llama(cfg, dev, comm_backend="symm" if world > 1 else "auto", reshard_after_forward=not keep)
    opt = ShardedAdamW(model, lr=1e-5, betas=(0.9, 0.95), weight_decay=0.1, max_grad_norm=1.0)
    step = TrainStep(model, opt, dev)
    ids = torch.randint(0, cfg.vocab_size, (1, args.seq_len), device=dev)
    for _ in range(4):
        step(ids)
    torch.cuda.synchronize()
    dist.barrier()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(args.steps):
            step(ids)
        torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        os.makedirs(args.out, exist_ok=True)
        path = os.path.join(args.out, f"step_trace_{args.model}_{world}gpu.json")
        prof.export_chrome_trace(path)
        txt = summarize(path, world, args.steps) + "\n" + overlap_report(path, None, args.steps)
        print(txt)
        with open(path.replace(".json", "_summary.txt"), "w") as f:
            f.write(txt)
        with open(path, "rb") as f, gzip.open(path + ".gz", "wb") as g:
            g.write(f.read())
        os.remove(path)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
