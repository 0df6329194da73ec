"""One small, self-contained case per native kernel, for profiling with ncu and for timing.

    python benchmarks/kernel_cases.py <case> [--iters N]

Cases hold a few hundred MB on the device (inputs larger than the 126 MB L2, far below the few-GB limit that keeps an
ncu capture short) and launch the kernel a handful of times.  Each prints the CUDA-event time of one launch and the
achieved fraction of the measured peak (``MEASURED_PEAKS.json``: copy bandwidth / cuBLAS bf16 throughput).

Cases: gemm_fwd, gemm_dx, gemm_dw, attn_fwd, attn_bwd, adamw, rmsnorm, swiglu, cross_entropy, and the memory-bound kernels at
the size they have inside a Llama-2-7B step (2048 tokens), cycling through enough copies of their operands that no launch
finds them in the L2: step_rmsnorm_fwd, step_rmsnorm_bwd, step_swiglu_fwd, step_swiglu_bwd, step_rope.  ``all_step`` runs those five.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

try:
    import yafsdp_b200  # noqa: F401  (installed: pip install -e . --no-build-isolation)
except ImportError:  # run from a checkout that was not installed
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from yafsdp_b200.ops import kernels  # noqa: E402


def peaks() -> tuple[float, float]:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        d = json.load(open(path))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"])
    except Exception:
        return 6650.0, 1590.0


def run(fn, iters: int) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def step_case(name: str, iters: int, hbm: float) -> dict:
    """One memory-bound kernel at its in-step size; operands rotate through ``copies`` buffers (> 2 x L2 in total)."""
    dev, bf = "cuda", torch.bfloat16
    t, d, f, hq = 2048, 4096, 11008, 32
    from yafsdp_b200.ops.functional import rope_table

    if name == "step_rmsnorm_fwd":
        nbytes = 2 * 2.0 * t * d
        mk = lambda: (torch.randn(t, d, device=dev, dtype=bf),)
        w = torch.ones(d, device=dev, dtype=bf)
        call = lambda x: kernels.rmsnorm_fwd(x, w, 1e-5)
    elif name == "step_rmsnorm_bwd":
        nbytes = 4 * 2.0 * t * d
        w = torch.ones(d, device=dev, dtype=bf)
        dw = torch.zeros(d, device=dev, dtype=torch.float32)
        rstd = torch.ones(t, device=dev, dtype=torch.float32)
        mk = lambda: tuple(torch.randn(t, d, device=dev, dtype=bf) for _ in range(3))
        call = lambda x, dy, dres: kernels.rmsnorm_bwd(x, w, dy, rstd, dw, dres=dres, zero_dw=True)
    elif name == "step_swiglu_fwd":
        nbytes = 3 * 2.0 * t * f
        mk = lambda: (torch.randn(t, 2 * f, device=dev, dtype=bf),)
        call = lambda gu: kernels.swiglu_fwd(gu)
    elif name == "step_swiglu_bwd":
        nbytes = 5 * 2.0 * t * f
        mk = lambda: (torch.randn(t, 2 * f, device=dev, dtype=bf), torch.randn(t, f, device=dev, dtype=bf))
        call = lambda gu, da: kernels.swiglu_bwd(gu, da)
    elif name == "step_rope":
        nbytes = 2 * 2.0 * t * 2 * hq * 128
        cs = rope_table(t, 128, 10000.0, torch.device(dev))
        mk = lambda: (torch.randn(t, 3 * hq * 128, device=dev, dtype=bf),)
        call = lambda qkv: kernels.rope_(qkv, cs, t, 0, 2 * hq, 128)
    else:
        raise SystemExit(f"unknown case {name}")
    copies = max(2, int(300e6 // nbytes) + 1)
    bufs = [mk() for _ in range(copies)]
    for b in bufs:  # warm-up (also outside the graph: first-use initialisation must not be captured)
        call(*b)
    torch.cuda.synchronize()
    # one CUDA graph of a launch per copy: the kernels run back to back, without the host's launch cost between them
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for b in bufs:
            call(*b)
    ms = run(graph.replay, max(iters, 5)) / copies
    return {"case": name, "us": round(ms * 1e3, 2), "gbs": round(nbytes / ms / 1e6, 1), "fraction_of_measured_hbm_peak": round(nbytes / ms / 1e6 / hbm, 3)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    hbm, tf = peaks()
    dev = "cuda"
    t, d, f = 2048, 4096, 11008
    bf = torch.bfloat16
    flops = bytes_ = 0.0
    if a.case == "all_step" or a.case.startswith("step_"):
        names = ["step_rmsnorm_fwd", "step_rmsnorm_bwd", "step_swiglu_fwd", "step_swiglu_bwd", "step_rope"] if a.case == "all_step" else [a.case]
        for n in names:
            rec = step_case(n, a.iters, hbm)
            rec["status"] = list(kernels.status())
            print(json.dumps(rec))
        return
    if a.case == "gemm_fwd":  # gate/up projection: [T,d] x [2f,d]^T
        x, w = torch.randn(t, d, device=dev, dtype=bf), torch.randn(2 * f, d, device=dev, dtype=bf)
        out = torch.empty(t, 2 * f, device=dev, dtype=bf)
        fn = lambda: kernels.gemm(x, w, out=out)
        flops = 2.0 * t * d * 2 * f
    elif a.case == "gemm_dx":  # dX = dY W, W stored [out, in]: MN-major B
        dy, w = torch.randn(t, 2 * f, device=dev, dtype=bf), torch.randn(2 * f, d, device=dev, dtype=bf)
        out = torch.empty(t, d, device=dev, dtype=bf)
        fn = lambda: kernels.gemm(dy, w, b_mn_major=True, out=out)
        flops = 2.0 * t * d * 2 * f
    elif a.case == "gemm_dw":  # dW = dY^T X in fp32 into a flat gradient buffer
        dy, x = torch.randn(t, 2 * f, device=dev, dtype=bf), torch.randn(t, d, device=dev, dtype=bf)
        out = torch.empty(2 * f, d, device=dev, dtype=torch.float32)
        fn = lambda: kernels.gemm(dy, x, a_mn_major=True, b_mn_major=True, out=out)
        flops = 2.0 * t * d * 2 * f
    elif a.case in ("attn_fwd", "attn_bwd"):
        b, s, hq, hkv = 2, 4096, 32, 8
        qkv = torch.randn(b * s, (hq + 2 * hkv) * 128, device=dev, dtype=bf)
        q, k, v = qkv[:, : hq * 128], qkv[:, hq * 128 : (hq + hkv) * 128], qkv[:, (hq + hkv) * 128 :]
        sc = 1 / math.sqrt(128)
        out, lse = kernels.attn_fwd(q, k, v, b, s, hq, hkv, sc, True)
        fl = 4.0 * b * hq * s * s * 128 / 2
        if a.case == "attn_fwd":
            fn = lambda: kernels.attn_fwd(q, k, v, b, s, hq, hkv, sc, True)
            flops = fl
        else:
            dout = torch.randn_like(out)
            dqkv = torch.empty_like(qkv)
            fn = lambda: kernels.attn_bwd(q, k, v, out, dout, lse, dqkv[:, : hq * 128], dqkv[:, hq * 128 : (hq + hkv) * 128],
                                          dqkv[:, (hq + hkv) * 128 :], b, s, hq, hkv, sc, True)
            flops = 2.5 * fl
    elif a.case == "adamw":
        n = 100 * 1000 * 1000
        p, g, m, v = (torch.randn(n, device=dev) for _ in range(4))
        v.abs_()
        pb = torch.empty(n, device=dev, dtype=bf)
        fn = lambda: kernels.adamw_(p, g, m, v, pb, None, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=3)
        bytes_ = 30.0 * n
    elif a.case == "rmsnorm":
        rows = 32768
        x, w = torch.randn(rows, d, device=dev, dtype=bf), torch.ones(d, device=dev, dtype=bf)
        fn = lambda: kernels.rmsnorm_fwd(x, w, 1e-5)
        bytes_ = 4.0 * rows * d
    elif a.case == "swiglu":
        rows = 16384
        gu = torch.randn(rows, 2 * f, device=dev, dtype=bf)
        fn = lambda: kernels.swiglu_fwd(gu)
        bytes_ = 6.0 * rows * f
    elif a.case == "cross_entropy":
        rows, vocab = 4096, 32000
        logits = torch.randn(rows, vocab, device=dev, dtype=bf)
        labels = torch.randint(0, vocab, (rows,), device=dev)
        fn = lambda: kernels.cross_entropy_(logits, labels, 1.0)
        bytes_ = 3 * 2.0 * rows * vocab
    else:
        raise SystemExit(f"unknown case {a.case}")
    ms = run(fn, a.iters)
    rec = {"case": a.case, "ms": round(ms, 4)}
    if flops:
        rec["tflops"] = round(flops / ms / 1e9, 1)
        rec["fraction_of_measured_bf16_peak"] = round(flops / ms / 1e9 / tf, 3)
    if bytes_:
        rec["gbs"] = round(bytes_ / ms / 1e6, 1)
        rec["fraction_of_measured_hbm_peak"] = round(bytes_ / ms / 1e6 / hbm, 3)
    code, site = kernels.status()
    rec["status"] = [code, site]
    print(json.dumps(rec))


if __name__ == "__main__":
    main()
