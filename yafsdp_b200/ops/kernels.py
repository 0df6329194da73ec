"""Thin tensor-level wrappers over the native sm_100a kernels (``csrc/*.cu``).

Each function checks its arguments on the host, launches on the current CUDA stream and raises on a
non-zero return code.  ``launch_count()`` counts every launch made through this module (the
benchmark reports it).  Nothing here falls back to PyTorch: a missing library on a GPU machine is an
error, and the autograd-level ops in :mod:`yafsdp_b200.ops.functional` choose between this module
(CUDA tensors) and plain PyTorch math (CPU tensors).
"""

from __future__ import annotations

import ctypes
from typing import Any

import torch

from .. import _native

_launches = 0


def launch_count() -> int:
    return _launches


def reset_launch_count() -> None:
    global _launches
    _launches = 0


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check(rc: int, name: str) -> None:
    global _launches
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc}")
    _launches += 1


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def status(clear: bool = True) -> tuple[int, int]:
    """(code, site) of the first error any kernel recorded since the last clearing read.  The status word sits in host
    memory: this is a plain read that neither synchronises nor touches the GPU; synchronise first to cover kernels that
    are still running."""
    code = ctypes.c_int(0)
    site = ctypes.c_int(0)
    rc = _native.lib().yf_status_read(ctypes.byref(code), ctypes.byref(site), int(clear))
    if rc != 0:
        raise RuntimeError(f"yf_status_read failed with code {rc}")
    return code.value, site.value


def check_status() -> None:
    code, site = status()
    if code != 0:
        raise RuntimeError(f"a native kernel reported error {code} at site {site} (a bounded wait ran out: a peer rank is late or "
                           "gone); the results of the kernels that ran since are undefined")


def poll_status() -> None:
    """:func:`check_status` when the native library is loaded in this process, nothing otherwise (CPU runs).  Cheap enough
    for once per step: the framework calls it at every root pre-forward and in the fused optimizer step."""
    if _native.loaded():
        check_status()


# --------------------------------------------------------------------------------------- GEMM
def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn_major: bool = False,
    b_mn_major: bool = False,
    out: torch.Tensor | None = None,
    out_dtype: torch.dtype = torch.bfloat16,
    accumulate: bool = False,
    alpha: float = 1.0,
    sm_limit: int = 0,
    sumsq: torch.Tensor | None = None,
    residual: torch.Tensor | None = None,
) -> torch.Tensor:
    """``out[M,N] = alpha * A @ B^T (+ out)`` with bf16 inputs and fp32 accumulation (tcgen05).

    ``a`` is ``[M,K]`` (K-major) or, with ``a_mn_major``, the stored tensor is ``[K,M]``; ``b`` is
    ``[N,K]`` or, with ``b_mn_major``, stored ``[K,N]``.  Rows must be contiguous (stride 1 in the last
    dimension); the row pitch may exceed the row length.  ``sumsq`` (fp32 output without accumulation only): a
    one-element fp32 tensor that receives ``+= sum(out**2)`` from the same kernel.  ``residual`` (bf16 output without
    accumulation only): a bf16 ``[M,N]`` tensor added in fp32 inside the epilogue, before the output is rounded.
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.is_cuda and b.is_cuda
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    if a_mn_major:
        k, m = a.shape
    else:
        m, k = a.shape
    if b_mn_major:
        kb, n = b.shape
    else:
        n, kb = b.shape
    assert k == kb, f"inner dimensions differ: {k} vs {kb}"
    if out is None:
        assert not accumulate
        out = torch.empty((m, n), device=a.device, dtype=out_dtype)
    assert out.shape == (m, n) and out.stride(1) == 1 and out.dtype in (torch.bfloat16, torch.float32)
    if residual is not None:
        assert out.dtype == torch.bfloat16 and not accumulate and sumsq is None
        assert residual.dtype == torch.bfloat16 and residual.shape == (m, n) and residual.stride(1) == 1
        rc = _native.lib().yf_gemm_bf16_residual(
            a.data_ptr(), b.data_ptr(), out.data_ptr(), residual.data_ptr(), m, n, k, a.stride(0), b.stride(0), out.stride(0),
            residual.stride(0), int(a_mn_major), int(b_mn_major), float(alpha), int(sm_limit), _stream(),
        )
        _check(rc, "yf_gemm_bf16_residual")
        return out
    rc = _native.lib().yf_gemm_bf16_sumsq(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), m, n, k, a.stride(0), b.stride(0), out.stride(0),
        int(a_mn_major), int(b_mn_major), int(out.dtype == torch.float32), int(accumulate), float(alpha),
        int(sm_limit), _ptr(sumsq), _stream(),
    )
    _check(rc, "yf_gemm_bf16")
    return out


def gemm_gathered(a: torch.Tensor, n: int, k: int, *, peer_in: Any, layer_buf: torch.Tensor, shard_bytes: int, b_byte_off: int,
                  rank: int, world: int, counters: torch.Tensor, epoch: int, out: torch.Tensor | None = None,
                  out_dtype: torch.dtype = torch.bfloat16, a_mn_major: bool = False) -> torch.Tensor:
    """All-gather -> GEMM in one kernel: ``out = A @ B^T`` where ``B [n, k]`` (bf16, contiguous) starts ``b_byte_off`` bytes
    into ``layer_buf``, which the same kernel fills from every rank's shard (``peer_in``: ctypes array of ``world`` peer
    pointers).  ``counters``: int64 tensor with one word per 256-row block of ``B``, zero before the first call;
    ``epoch`` = 1, 2, ... counts the calls made with these counters."""
    m = a.shape[1] if a_mn_major else a.shape[0]
    if out is None:
        out = torch.empty((m, n), device=a.device, dtype=out_dtype)
    assert counters.dtype == torch.int64 and counters.numel() >= (n + 127) // 128 and epoch >= 1
    rc = _native.lib().yf_gemm_bf16_gathered(
        a.data_ptr(), out.data_ptr(), m, n, k, a.stride(0), out.stride(0), int(a_mn_major), int(out.dtype == torch.float32),
        peer_in, layer_buf.data_ptr(), shard_bytes, b_byte_off, rank, world, counters.data_ptr(), epoch, _stream())
    _check(rc, "yf_gemm_bf16_gathered")
    return out


def gemm_scatter(a: torch.Tensor, b: torch.Tensor, *, a_mn_major: bool, b_mn_major: bool, peer_grad: Any, c_flat_off: int,
                 shard_numel: int, rank: int, world: int, alpha: float = 1.0, sm_limit: int = 0, wire_bf16: bool = False) -> None:
    """GEMM -> reduce-scatter push: the fp32 product goes piece by piece to the owners' staging slots for this rank
    (``peer_grad``: ctypes array of every rank's reduce-buffer base); nothing is stored locally."""
    m = a.shape[1] if a_mn_major else a.shape[0]
    n = b.shape[1] if b_mn_major else b.shape[0]
    k = a.shape[0] if a_mn_major else a.shape[1]
    rc = _native.lib().yf_gemm_bf16_scatter(a.data_ptr(), b.data_ptr(), m, n, k, a.stride(0), b.stride(0), int(a_mn_major),
                                            int(b_mn_major), float(alpha), peer_grad, c_flat_off, shard_numel, rank, world,
                                            int(wire_bf16), int(sm_limit), _stream())
    _check(rc, "yf_gemm_bf16_scatter")


def gemm_scatter_grouped(problems: list[tuple[torch.Tensor, torch.Tensor, int]], *, peer_grad: Any, shard_numel: int, rank: int,
                         world: int, alpha: float = 1.0, sm_limit: int = 0, wire_bf16: bool = False) -> None:
    """The weight-gradient GEMMs of a layer as one launch pushed to their owners.  ``problems``: up to four
    ``(dy [T, out], x [T, in], flat offset of the [out, in] gradient)`` in ascending flat order; every ``dW = dy^T x``
    goes to the owners' slots for this rank.  The owners' tiles are dealt round-robin, so every rank pushes to all owners
    all the time and no owner's NVLink ingress becomes a hot spot."""
    n = len(problems)
    assert 1 <= n <= 4
    k = problems[0][0].shape[0]
    a_ptrs = (ctypes.c_void_p * n)(*[dy.data_ptr() for dy, _, _ in problems])
    b_ptrs = (ctypes.c_void_p * n)(*[x.data_ptr() for _, x, _ in problems])
    ms = (ctypes.c_int * n)(*[dy.shape[1] for dy, _, _ in problems])
    ns = (ctypes.c_int * n)(*[x.shape[1] for _, x, _ in problems])
    ldas = (ctypes.c_longlong * n)(*[dy.stride(0) for dy, _, _ in problems])
    ldbs = (ctypes.c_longlong * n)(*[x.stride(0) for _, x, _ in problems])
    offs = (ctypes.c_longlong * n)(*[off for _, _, off in problems])
    for dy, x, _ in problems:
        assert dy.dtype == x.dtype == torch.bfloat16 and dy.shape[0] == x.shape[0] == k and dy.stride(1) == 1 and x.stride(1) == 1
    rc = _native.lib().yf_gemm_bf16_scatter_grouped(n, a_ptrs, b_ptrs, ms, ns, k, ldas, ldbs, 1, 1, float(alpha), peer_grad, offs,
                                                    shard_numel, rank, world, int(wire_bf16), int(sm_limit), _stream())
    _check(rc, "yf_gemm_bf16_scatter_grouped")


def push_flat(src: torch.Tensor | None, numel: int, flat_off: int, peer_grad: Any, shard_numel: int, rank: int, world: int,
              wire_bf16: bool = False) -> None:
    """Push ``numel`` fp32 values (``src``, or zeros when ``None``) that start at position ``flat_off`` of the flat layer
    gradient into the owners' reduce-scatter slots for this rank."""
    if src is not None:
        assert src.dtype == torch.float32 and src.is_contiguous() and src.numel() == numel
    rc = _native.lib().yf_push_flat(_ptr(src), numel, flat_off, peer_grad, shard_numel, rank, world, int(wire_bf16), _stream())
    _check(rc, "yf_push_flat")


# --------------------------------------------------------------------------------------- norms etc.
def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float) -> tuple[torch.Tensor, torch.Tensor]:
    t, d = x.shape
    y = torch.empty_like(x)
    rstd = torch.empty(t, device=x.device, dtype=torch.float32)
    _check(_native.lib().yf_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), t, d, float(eps), _stream()),
           "yf_rmsnorm_fwd")
    return y, rstd


def rmsnorm_bwd(x: torch.Tensor, w: torch.Tensor, dy: torch.Tensor, rstd: torch.Tensor, dw_f32: torch.Tensor,
                dres: torch.Tensor | None = None, zero_dw: bool = False) -> torch.Tensor:
    """Returns dx (+ dres when given); accumulates the weight gradient into the fp32 tensor ``dw_f32`` (``zero_dw``: the
    kernel clears it first, which saves the caller a fill launch)."""
    t, d = x.shape
    dx = torch.empty_like(x)
    assert dw_f32.dtype == torch.float32 and dw_f32.numel() == d
    _check(_native.lib().yf_rmsnorm_bwd(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(), _ptr(dres), dx.data_ptr(),
                                        dw_f32.data_ptr(), int(zero_dw), t, d, _stream()), "yf_rmsnorm_bwd")
    return dx


def rope_(qkv: torch.Tensor, cos_sin: torch.Tensor, seq_len: int, col0: int, n_heads: int, head_dim: int,
          backward: bool = False) -> torch.Tensor:
    """Rotate ``n_heads`` heads of ``qkv[T, :]`` starting at column ``col0`` in place."""
    t = qkv.shape[0]
    assert qkv.dim() == 2 and qkv.stride(1) == 1 and cos_sin.dtype == torch.float32
    _check(_native.lib().yf_rope(qkv.data_ptr(), cos_sin.data_ptr(), t, seq_len, qkv.stride(0), col0, n_heads, head_dim,
                                 int(backward), _stream()), "yf_rope")
    return qkv


def swiglu_fwd(gu: torch.Tensor) -> torch.Tensor:
    t, f2 = gu.shape
    h = torch.empty((t, f2 // 2), device=gu.device, dtype=gu.dtype)
    _check(_native.lib().yf_swiglu_fwd(gu.data_ptr(), h.data_ptr(), t, f2 // 2, _stream()), "yf_swiglu_fwd")
    return h


def swiglu_bwd(gu: torch.Tensor, dh: torch.Tensor) -> torch.Tensor:
    t, f2 = gu.shape
    dgu = torch.empty_like(gu)
    _check(_native.lib().yf_swiglu_bwd(gu.data_ptr(), dh.data_ptr(), dgu.data_ptr(), t, f2 // 2, _stream()), "yf_swiglu_bwd")
    return dgu


def cross_entropy_(logits: torch.Tensor, labels: torch.Tensor, grad_scale: float, write_grad: bool = True,
                   scale: torch.Tensor | None = None) -> torch.Tensor:
    """Per-row losses; ``logits`` is overwritten by ``(softmax - onehot) * grad_scale`` when ``write_grad``.  ``scale``: a
    one-element fp32 device tensor whose value multiplies ``grad_scale`` (read by the kernel: no host synchronisation)."""
    t, v = logits.shape
    assert labels.dtype == torch.int64 and logits.stride(1) == 1
    loss_rows = torch.empty(t, device=logits.device, dtype=torch.float32)
    _check(_native.lib().yf_cross_entropy(logits.data_ptr(), labels.data_ptr(), loss_rows.data_ptr(), t, v, logits.stride(0),
                                          float(grad_scale), _ptr(scale), int(write_grad), _stream()), "yf_cross_entropy")
    return loss_rows


def embedding_fwd(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    v, d = table.shape
    t = ids.numel()
    out = torch.empty((t, d), device=table.device, dtype=table.dtype)
    _check(_native.lib().yf_embedding_fwd(table.data_ptr(), ids.data_ptr(), out.data_ptr(), t, d, v, _stream()), "yf_embedding_fwd")
    return out


def embedding_bwd_(dout: torch.Tensor, ids: torch.Tensor, dtable_f32: torch.Tensor) -> None:
    v, d = dtable_f32.shape
    _check(_native.lib().yf_embedding_bwd(dout.data_ptr(), ids.data_ptr(), dtable_f32.data_ptr(), ids.numel(), d, v, _stream()),
           "yf_embedding_bwd")


def adamw_(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, p_bf16: torch.Tensor | None,
           grad_scale: torch.Tensor | None, *, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float,
           step: int, max_ctas: int = 0) -> None:
    n = p.numel()
    assert p.dtype == g.dtype == m.dtype == v.dtype == torch.float32
    _check(_native.lib().yf_adamw(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), _ptr(p_bf16), _ptr(grad_scale), n,
                                  float(lr), float(beta1), float(beta2), float(eps), float(weight_decay), int(step), int(max_ctas),
                                  _stream()),
           "yf_adamw")


def sumsq_(g: torch.Tensor, out: torch.Tensor) -> None:
    """``out[0] += sum(g*g)`` (fp32)."""
    _check(_native.lib().yf_sumsq(g.data_ptr(), g.numel(), out.data_ptr(), _stream()), "yf_sumsq")


def clip_coef_(total_sq: torch.Tensor, max_norm: float, coef: torch.Tensor, norm_out: torch.Tensor | None) -> None:
    _check(_native.lib().yf_clip_coef(total_sq.data_ptr(), float(max_norm), coef.data_ptr(), _ptr(norm_out), _stream()), "yf_clip_coef")


def cast_f32_to_bf16_(src: torch.Tensor, dst: torch.Tensor) -> None:
    assert src.numel() == dst.numel()
    _check(_native.lib().yf_cast_f32_to_bf16(src.data_ptr(), dst.data_ptr(), src.numel(), _stream()), "yf_cast_f32_to_bf16")


def accum_bf16_to_f32_(src: torch.Tensor, dst: torch.Tensor, scale: float = 1.0, accumulate: bool = False) -> None:
    assert src.numel() == dst.numel()
    _check(_native.lib().yf_accum_bf16_to_f32(src.data_ptr(), dst.data_ptr(), src.numel(), float(scale), int(accumulate), _stream()),
           "yf_accum_bf16_to_f32")


def add_bf16(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    out = torch.empty_like(a) if out is None else out
    _check(_native.lib().yf_add_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), _stream()), "yf_add_bf16")
    return out


# --------------------------------------------------------------------------------------- attention
def attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, batch: int, seq: int, n_heads: int, n_kv_heads: int,
             scale: float, causal: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    """Flash attention forward, head_dim 128.  ``q``: ``[B*S, Hq*128]`` view, ``k``/``v``: ``[B*S, Hkv*128]``
    views (column blocks of the fused QKV projection output are fine).  Returns ``out [B*S, Hq*128]`` and
    ``lse [B, Hq, S]``."""
    t = batch * seq
    assert q.shape == (t, n_heads * 128) and k.shape == (t, n_kv_heads * 128) and v.shape == k.shape
    assert q.stride(1) == 1 and k.stride(1) == 1 and v.stride(1) == 1 and k.stride(0) == v.stride(0)
    out = torch.empty((t, n_heads * 128), device=q.device, dtype=torch.bfloat16)
    lse = torch.empty((batch, n_heads, seq), device=q.device, dtype=torch.float32)
    _check(_native.lib().yf_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), batch, seq,
                                     n_heads, n_kv_heads, q.stride(0), k.stride(0), out.stride(0), float(scale), int(causal),
                                     _stream()), "yf_attn_fwd")
    return out, lse


def attn_bwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, dout: torch.Tensor, lse: torch.Tensor,
             dq: torch.Tensor, dk: torch.Tensor, dv: torch.Tensor, batch: int, seq: int, n_heads: int, n_kv_heads: int,
             scale: float, causal: bool = True) -> None:
    """Flash attention backward into the given ``dq``/``dk``/``dv`` views (bf16, unit column stride)."""
    t = batch * seq
    assert dout.stride(1) == 1 and out.stride(1) == 1 and dq.stride(1) == 1 and dk.stride(1) == 1 and dv.stride(1) == 1
    assert dk.stride(0) == dv.stride(0)
    delta = torch.empty((batch, n_heads, seq), device=q.device, dtype=torch.float32)
    dq_acc = torch.empty((t, n_heads * 128), device=q.device, dtype=torch.float32)
    global _launches
    _check(_native.lib().yf_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
                                     delta.data_ptr(), dq_acc.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), batch, seq,
                                     n_heads, n_kv_heads, q.stride(0), k.stride(0), out.stride(0), dout.stride(0), dq.stride(0),
                                     dk.stride(0), float(scale), int(causal), _stream()), "yf_attn_bwd")
    _launches += 2  # delta pre-pass and dq conversion post-pass
