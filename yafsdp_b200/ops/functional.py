"""Autograd-level ops of the Llama training step.

CUDA tensors run the hand-written sm_100a kernels (:mod:`yafsdp_b200.ops.kernels`) through three
coarse autograd Functions with hand-derived backward passes: the embedding, a whole decoder layer,
and final-norm + LM head + cross-entropy.  Coarse Functions keep the gradient adds of the residual
stream fused into the RMSNorm backward kernel and let every weight gradient go straight from the
tcgen05 GEMM epilogue (fp32, accumulating) into the parameter's *gradient sink* (see
``yafsdp_b200.group.GradSink``) when the parameter is managed by ``fully_shard``.

CPU tensors (gloo plumbing tests) run the same math in plain PyTorch and rely on autograd.  On a CUDA
device the native path is the only one: there is no fallback to library kernels.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

import torch
import torch.nn.functional as F

from . import kernels


def rope_table(seq_len: int, head_dim: int, theta: float, device: torch.device | str) -> torch.Tensor:
    """``[seq_len, head_dim/2, 2]`` fp32 table of (cos, sin) for the rotate-half RoPE convention."""
    half = head_dim // 2
    inv_freq = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float64) * 2.0 / head_dim))
    ang = torch.arange(seq_len, dtype=torch.float64)[:, None] * inv_freq[None, :]
    return torch.stack([ang.cos(), ang.sin()], dim=-1).to(torch.float32).to(device).contiguous()


@dataclass(frozen=True)
class LayerDims:
    batch: int
    seq: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    eps: float


# ------------------------------------------------------------------------------------- helpers
def _sink(p: torch.Tensor) -> Any:
    return getattr(p, "_yf_grad_sink", None)


def fuse_adjacent(ts: list[torch.Tensor]) -> torch.Tensor:
    """One ``[sum(rows), cols]`` view over 2-D tensors that sit back to back in memory (consecutive
    parameters of a flat group buffer); a concatenated copy otherwise."""
    first = ts[0]
    cols = first.shape[1]
    adjacent = all(t.is_contiguous() and t.shape[1] == cols and t.dtype == first.dtype for t in ts)
    if adjacent:
        base = first.untyped_storage().data_ptr()
        end = first.data_ptr() + first.numel() * first.element_size()
        for t in ts[1:]:
            # back to back AND inside one allocation (two allocator blocks can touch by accident)
            if t.data_ptr() != end or t.untyped_storage().data_ptr() != base:
                adjacent = False
                break
            end += t.numel() * t.element_size()
    if not adjacent:
        return torch.cat([t.detach() for t in ts], dim=0)
    rows = sum(t.shape[0] for t in ts)
    return torch.as_strided(first.detach(), (rows, cols), (cols, 1))


class _WeightGrad:
    """Where the gradient of one (possibly fused) weight goes: the fp32 sinks of the parameters when all
    of them have one and they are adjacent, else a fresh bf16 tensor split per parameter."""

    def __init__(self, params: list[torch.Tensor]):
        self.params = params
        self.sinks = [_sink(p) for p in params]
        self.use_sinks = all(s is not None for s in self.sinks)

    def run(self, dy: torch.Tensor, x: torch.Tensor, deferred: "list[tuple[Any, ...]] | None" = None) -> list[torch.Tensor | None]:
        """dW = dy^T x for the fused weight; returns per-parameter gradients (None when sunk).  ``deferred``: in push mode
        the GEMM is not launched but recorded there, for one grouped launch at the end of the layer's backward
        (:func:`flush_pushed`)."""
        if self.use_sinks and all(s.pushes() for s in self.sinks):
            # fused GEMM -> reduce-scatter: parameters that follow each other in the flat gradient are one GEMM
            i, r0 = 0, 0
            while i < len(self.sinks):
                ptrs, off, shard, rank, world, bf16 = self.sinks[i].begin_push()
                rows, nxt, j = self.params[i].shape[0], off + self.params[i].numel(), i + 1
                while j < len(self.sinks) and self.sinks[j].group is self.sinks[i].group:
                    _, off_j, *_ = self.sinks[j].begin_push()
                    assert off_j == nxt, "fused weights must be adjacent in the flat layout"
                    rows, nxt, j = rows + self.params[j].shape[0], nxt + self.params[j].numel(), j + 1
                if deferred is not None:
                    deferred.append((dy[:, r0 : r0 + rows], x, off, ptrs, shard, rank, world, bf16))
                else:
                    kernels.gemm_scatter(dy[:, r0 : r0 + rows], x, a_mn_major=True, b_mn_major=True, peer_grad=ptrs, c_flat_off=off,
                                         shard_numel=shard, rank=rank, world=world, wire_bf16=bf16)
                i, r0 = j, r0 + rows
            return [None] * len(self.params)
        if self.use_sinks and all(s.local_ok for s in self.sinks):
            views, accs = zip(*[s.begin() for s in self.sinks])
            fused = fuse_adjacent(list(views)) if len(views) > 1 else views[0]
            targets = [s.norm_target(acc) for s, acc in zip(self.sinks, accs)]
            if len(views) == 1 or (fused.data_ptr() == views[0].data_ptr() and len(set(accs)) == 1):
                kernels.gemm(dy, x, a_mn_major=True, b_mn_major=True, out=fused, accumulate=accs[0], sumsq=targets[0])
            else:
                r0 = 0
                for v, acc, tgt in zip(views, accs, targets):
                    kernels.gemm(dy[:, r0 : r0 + v.shape[0]], x, a_mn_major=True, b_mn_major=True, out=v, accumulate=acc, sumsq=tgt)
                    r0 += v.shape[0]
            return [None] * len(self.params)
        dw = kernels.gemm(dy, x, a_mn_major=True, b_mn_major=True)
        out: list[torch.Tensor | None] = []
        r0 = 0
        for p in self.params:
            out.append(dw[r0 : r0 + p.shape[0]])
            r0 += p.shape[0]
        return out


def flush_pushed(deferred: "list[tuple[Any, ...]]") -> None:
    """Launch the recorded weight-gradient GEMMs of a layer: one grouped launch (owners' tiles dealt round-robin) when they share the token
    dimension and the destination (the usual case), one launch each otherwise."""
    if not deferred:
        return
    deferred.sort(key=lambda d: d[2])
    _, _, _, ptrs, shard, rank, world, bf16 = deferred[0]
    same = all(d[3] is ptrs and d[0].shape[0] == deferred[0][0].shape[0] for d in deferred)
    if same and len(deferred) <= 4:
        kernels.gemm_scatter_grouped([(dy, x, off) for dy, x, off, *_ in deferred], peer_grad=ptrs, shard_numel=shard, rank=rank, world=world,
                                     wire_bf16=bf16)
    else:
        for dy, x, off, p, sh, r, w, b16 in deferred:
            kernels.gemm_scatter(dy, x, a_mn_major=True, b_mn_major=True, peer_grad=p, c_flat_off=off, shard_numel=sh, rank=r, world=w,
                                 wire_bf16=b16)
    deferred.clear()


def _norm_weight_grad(w: torch.Tensor, fn: Any, self_zeroing: bool = False) -> torch.Tensor | None:
    """Run ``fn(dw_fp32)`` (a kernel that atomically accumulates into dw); returns the gradient unless sunk.
    ``self_zeroing``: the kernel can clear its target itself and is called as ``fn(dw, zero)``."""
    s = _sink(w)
    if s is not None and s.pushes():
        dw = torch.empty(w.shape, device=w.device, dtype=torch.float32) if self_zeroing else torch.zeros(w.shape, device=w.device, dtype=torch.float32)
        fn(dw, True) if self_zeroing else fn(dw)
        s.push_from(dw)
        return None
    if s is not None and s.local_ok:
        zeroed_now = not s.would_accumulate()
        if self_zeroing:
            view, _ = s.begin(zero=False)
            fn(view, zeroed_now)
        else:
            view, _ = s.begin(zero=True)
            fn(view)
        # the value is final (and its squares may be summed here) only if this call started from zeros: an earlier write
        # of this backward pass or an earlier micro-batch's gradient makes it a partial sum
        tgt = s.norm_target(not zeroed_now)
        if tgt is not None:
            kernels.sumsq_(view.reshape(-1), tgt)
        return None
    if self_zeroing:
        dw = torch.empty(w.shape, device=w.device, dtype=torch.float32)
        fn(dw, True)
    else:
        dw = torch.zeros(w.shape, device=w.device, dtype=torch.float32)
        fn(dw)
    return dw.to(w.dtype)


def _c(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_contiguous() else t.contiguous()


# ------------------------------------------------------------------------------------- embedding
class EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:  # type: ignore[override]
        ctx.save_for_backward(ids)
        ctx.table = table
        return kernels.embedding_fwd(table.detach(), ids.reshape(-1)).view(*ids.shape, table.shape[1])

    @staticmethod
    def backward(ctx: Any, dout: torch.Tensor) -> Any:  # type: ignore[override]
        (ids,) = ctx.saved_tensors
        table = ctx.table
        dout2 = _c(dout).view(-1, table.shape[1])
        grad = _norm_weight_grad(table, lambda dw: kernels.embedding_bwd_(dout2, ids.reshape(-1), dw))
        return None, grad


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    if table.is_cuda:
        return EmbeddingFn.apply(ids, table)
    return F.embedding(ids, table)


# ------------------------------------------------------------------------------------- decoder layer
class DecoderLayerFn(torch.autograd.Function):
    """x -> x + Attn(RMSNorm(x)) -> h + MLP(RMSNorm(h)); tokens flattened to ``[B*S, d]``."""

    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, w_n1: torch.Tensor, wq: torch.Tensor, wk: torch.Tensor, wv: torch.Tensor,  # type: ignore[override]
                wo: torch.Tensor, w_n2: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor,
                cos_sin: torch.Tensor, dims: LayerDims) -> torch.Tensor:
        x = _c(x)
        hd, hq, hkv = dims.head_dim, dims.n_heads, dims.n_kv_heads
        w_qkv = fuse_adjacent([wq, wk, wv])
        w_gu = fuse_adjacent([wg, wu])
        n1, rstd1 = kernels.rmsnorm_fwd(x, w_n1.detach(), dims.eps)
        owner = getattr(wq, "_yf_group_index", None)
        ticket = owner[0].take_in_kernel_gather(owner[1], w_qkv.shape[0]) if owner is not None else None
        if ticket is not None:
            # this forward pass has not gathered the layer: the QKV GEMM pulls it from the peers while it computes
            qkv = kernels.gemm_gathered(n1, w_qkv.shape[0], w_qkv.shape[1], peer_in=ticket["peer_in"], layer_buf=ticket["layer_buf"],
                                        shard_bytes=ticket["shard_bytes"], b_byte_off=ticket["b_byte_off"], rank=ticket["rank"],
                                        world=ticket["world"], counters=ticket["counters"], epoch=ticket["epoch"])
        else:
            qkv = kernels.gemm(n1, w_qkv)
        kernels.rope_(qkv, cos_sin, dims.seq, 0, hq + hkv, hd)
        q, k, v = qkv[:, : hq * hd], qkv[:, hq * hd : (hq + hkv) * hd], qkv[:, (hq + hkv) * hd :]
        att, lse = kernels.attn_fwd(q, k, v, dims.batch, dims.seq, hq, hkv, 1.0 / math.sqrt(hd), True)
        h = kernels.gemm(att, wo.detach(), residual=x)  # x + attention block: the residual is added in the GEMM's epilogue
        n2, rstd2 = kernels.rmsnorm_fwd(h, w_n2.detach(), dims.eps)
        gu = kernels.gemm(n2, w_gu)
        a = kernels.swiglu_fwd(gu)
        out = kernels.gemm(a, wd.detach(), residual=h)
        ctx.save_for_backward(x, rstd1, n1, qkv, att, lse, h, rstd2, n2, gu, a, cos_sin)
        ctx.weights = (w_n1, wq, wk, wv, wo, w_n2, wg, wu, wd)
        ctx.dims = dims
        return out

    @staticmethod
    def backward(ctx: Any, dout: torch.Tensor) -> Any:  # type: ignore[override]
        x, rstd1, n1, qkv, att, lse, h, rstd2, n2, gu, a, cos_sin = ctx.saved_tensors
        w_n1, wq, wk, wv, wo, w_n2, wg, wu, wd = ctx.weights
        dims: LayerDims = ctx.dims
        hd, hq, hkv = dims.head_dim, dims.n_heads, dims.n_kv_heads
        dout = _c(dout)
        # the weights are views of a rotating gather buffer: read them now, as gathered for this backward
        w_qkv = fuse_adjacent([wq, wk, wv])
        w_gu = fuse_adjacent([wg, wu])
        # ---- MLP
        pushed: list[tuple[Any, ...]] = []  # push mode: the four weight-gradient GEMMs run as one grouped launch at the end
        da = kernels.gemm(dout, wd.detach(), b_mn_major=True)
        (g_wd,) = _WeightGrad([wd]).run(dout, a, pushed)
        dgu = kernels.swiglu_bwd(gu, da)
        del da
        dn2 = kernels.gemm(dgu, w_gu, b_mn_major=True)
        g_wg, g_wu = _WeightGrad([wg, wu]).run(dgu, n2, pushed)
        del dgu
        box: list[torch.Tensor] = []
        g_n2 = _norm_weight_grad(w_n2, lambda dw, z: box.append(kernels.rmsnorm_bwd(h, w_n2.detach(), dn2, rstd2, dw, dres=dout, zero_dw=z)), True)
        dh = box.pop()
        # ---- attention
        datt = kernels.gemm(dh, wo.detach(), b_mn_major=True)
        (g_wo,) = _WeightGrad([wo]).run(dh, att, pushed)
        dqkv = torch.empty_like(qkv)
        q, k, v = qkv[:, : hq * hd], qkv[:, hq * hd : (hq + hkv) * hd], qkv[:, (hq + hkv) * hd :]
        kernels.attn_bwd(q, k, v, att, datt, lse, dqkv[:, : hq * hd], dqkv[:, hq * hd : (hq + hkv) * hd],
                         dqkv[:, (hq + hkv) * hd :], dims.batch, dims.seq, hq, hkv, 1.0 / math.sqrt(hd), True)
        kernels.rope_(dqkv, cos_sin, dims.seq, 0, hq + hkv, hd, backward=True)
        dn1 = kernels.gemm(dqkv, w_qkv, b_mn_major=True)
        g_wq, g_wk, g_wv = _WeightGrad([wq, wk, wv]).run(dqkv, n1, pushed)
        g_n1 = _norm_weight_grad(w_n1, lambda dw, z: box.append(kernels.rmsnorm_bwd(x, w_n1.detach(), dn1, rstd1, dw, dres=dh, zero_dw=z)), True)
        dx = box.pop()
        flush_pushed(pushed)
        return dx, g_n1, g_wq, g_wk, g_wv, g_wo, g_n2, g_wg, g_wu, g_wd, None, None


# ------------------------------------------------------------------------------------- final norm + head + loss
class HeadLossFn(torch.autograd.Function):
    """mean cross-entropy of ``lm_head(RMSNorm(h))`` against ``labels`` (``-100`` rows ignored).  The logits are
    overwritten by their own gradient in the forward pass, so the ``[T, vocab]`` tensor exists once."""

    @staticmethod
    def forward(ctx: Any, h: torch.Tensor, w_norm: torch.Tensor, w_head: torch.Tensor, labels: torch.Tensor, eps: float) -> torch.Tensor:  # type: ignore[override]
        h = _c(h)
        n, rstd = kernels.rmsnorm_fwd(h, w_norm.detach(), eps)
        logits = kernels.gemm(n, w_head.detach())
        # the mean's 1 / (number of valid labels) goes into the gradient that the loss kernel leaves in place of the logits
        inv_valid = (labels >= 0).sum().clamp_(min=1).to(torch.float32).reciprocal_().reshape(1)
        loss_rows = kernels.cross_entropy_(logits, labels, 1.0, write_grad=True, scale=inv_valid)
        ctx.save_for_backward(h, rstd, n, logits)
        ctx.weights = (w_norm, w_head)
        return (loss_rows.sum() * inv_valid).reshape(())

    @staticmethod
    def backward(ctx: Any, dloss: torch.Tensor) -> Any:  # type: ignore[override]
        h, rstd, n, dlogits = ctx.saved_tensors
        w_norm, w_head = ctx.weights
        # the incoming gradient of the loss (a device scalar) scales the two small [T, d] operands instead of a pass over
        # the [T, vocab] gradient: dn = dloss * (dlogits W), dW = dlogits^T (dloss * n)
        dn = kernels.gemm(dlogits, w_head.detach(), b_mn_major=True)
        dn.mul_(dloss.to(dn.dtype))
        (g_head,) = _WeightGrad([w_head]).run(dlogits, n * dloss.to(n.dtype))
        box: list[torch.Tensor] = []
        g_norm = _norm_weight_grad(w_norm, lambda dw, z: box.append(kernels.rmsnorm_bwd(h, w_norm.detach(), dn, rstd, dw, zero_dw=z)), True)
        return box.pop(), g_norm, g_head, None, None


class HeadLogitsFn(torch.autograd.Function):
    """logits = lm_head(RMSNorm(h)) (inference / evaluation path)."""

    @staticmethod
    def forward(ctx: Any, h: torch.Tensor, w_norm: torch.Tensor, w_head: torch.Tensor, eps: float) -> torch.Tensor:  # type: ignore[override]
        h = _c(h)
        n, rstd = kernels.rmsnorm_fwd(h, w_norm.detach(), eps)
        ctx.save_for_backward(h, rstd, n)
        ctx.weights = (w_norm, w_head)
        return kernels.gemm(n, w_head.detach())

    @staticmethod
    def backward(ctx: Any, dlogits: torch.Tensor) -> Any:  # type: ignore[override]
        h, rstd, n = ctx.saved_tensors
        w_norm, w_head = ctx.weights
        dlogits = _c(dlogits)
        dn = kernels.gemm(dlogits, w_head.detach(), b_mn_major=True)
        (g_head,) = _WeightGrad([w_head]).run(dlogits, n)
        box: list[torch.Tensor] = []
        g_norm = _norm_weight_grad(w_norm, lambda dw, z: box.append(kernels.rmsnorm_bwd(h, w_norm.detach(), dn, rstd, dw, zero_dw=z)), True)
        return box.pop(), g_norm, g_head, None


# ------------------------------------------------------------------------------------- CPU restatements
def rmsnorm_ref(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def rope_ref(t: torch.Tensor, cos_sin: torch.Tensor) -> torch.Tensor:
    """t: [B, S, H, D]; rotate-half convention."""
    half = t.shape[-1] // 2
    cos = cos_sin[: t.shape[1], :, 0].view(1, t.shape[1], 1, half).to(torch.float32)
    sin = cos_sin[: t.shape[1], :, 1].view(1, t.shape[1], 1, half).to(torch.float32)
    t1, t2 = t[..., :half].float(), t[..., half:].float()
    return torch.cat([t1 * cos - t2 * sin, t2 * cos + t1 * sin], dim=-1).to(t.dtype)


def decoder_layer_ref(x: torch.Tensor, w_n1: torch.Tensor, wq: torch.Tensor, wk: torch.Tensor, wv: torch.Tensor, wo: torch.Tensor,
                      w_n2: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor, cos_sin: torch.Tensor,
                      dims: LayerDims) -> torch.Tensor:
    b, s, hq, hkv, hd = dims.batch, dims.seq, dims.n_heads, dims.n_kv_heads, dims.head_dim
    n1 = rmsnorm_ref(x, w_n1, dims.eps)
    q = F.linear(n1, wq).view(b, s, hq, hd)
    k = F.linear(n1, wk).view(b, s, hkv, hd)
    v = F.linear(n1, wv).view(b, s, hkv, hd)
    q, k = rope_ref(q, cos_sin), rope_ref(k, cos_sin)
    att = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                         enable_gqa=hq != hkv)
    att = att.transpose(1, 2).reshape(b * s, hq * hd)
    h = x + F.linear(att, wo)
    n2 = rmsnorm_ref(h, w_n2, dims.eps)
    return h + F.linear(F.silu(F.linear(n2, wg)) * F.linear(n2, wu), wd)


def decoder_layer(x: torch.Tensor, *weights_and_table: Any) -> torch.Tensor:
    """``x [B*S, d]`` through one decoder layer (arguments as ``DecoderLayerFn.forward``)."""
    if x.is_cuda:
        return DecoderLayerFn.apply(x, *weights_and_table)
    return decoder_layer_ref(x, *weights_and_table)


def head_loss(h: torch.Tensor, w_norm: torch.Tensor, w_head: torch.Tensor, labels: torch.Tensor, eps: float) -> torch.Tensor:
    if h.is_cuda:
        return HeadLossFn.apply(h, w_norm, w_head, labels, eps)
    logits = F.linear(rmsnorm_ref(h, w_norm, eps), w_head)
    return F.cross_entropy(logits.float(), labels, ignore_index=-100)


def head_logits(h: torch.Tensor, w_norm: torch.Tensor, w_head: torch.Tensor, eps: float) -> torch.Tensor:
    if h.is_cuda:
        return HeadLogitsFn.apply(h, w_norm, w_head, eps)
    return F.linear(rmsnorm_ref(h, w_norm, eps), w_head)
