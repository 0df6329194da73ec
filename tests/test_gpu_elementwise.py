"""Memory-bound sm_100a kernels vs fp32 PyTorch restatements."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, rtol=2e-2, atol=2e-2):
    assert torch.allclose(a.float(), b.float(), rtol=rtol, atol=atol), (a.float() - b.float()).abs().max().item()


@pytest.mark.parametrize("t,d", [(64, 256), (300, 4096), (17, 8192), (33, 1000 * 8), (2049, 2048), (130, 5120), (5, 2056)])
def test_rmsnorm_fwd_bwd(t, d):
    from yafsdp_b200.ops import kernels

    torch.manual_seed(0)
    x = torch.randn(t, d, device="cuda", dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
    dy = torch.randn(t, d, device="cuda", dtype=torch.bfloat16)
    y, rstd = kernels.rmsnorm_fwd(x, w, 1e-5)
    xf = x.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    yr = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    _close(y, yr)
    yr.backward(dy.float())
    dw = torch.zeros(d, device="cuda", dtype=torch.float32)
    dres = torch.randn(t, d, device="cuda", dtype=torch.bfloat16)
    dx = kernels.rmsnorm_bwd(x, w, dy, rstd, dw, dres)
    _close(dx, xf.grad + dres.float(), rtol=3e-2, atol=3e-2)
    assert torch.allclose(dw, wf.grad, rtol=2e-2, atol=5e-2 * math.sqrt(t))
    # without the residual gradient, and with the weight gradient cleared by the kernel itself
    dw2 = torch.full((d,), 7.0, device="cuda", dtype=torch.float32)
    dx2 = kernels.rmsnorm_bwd(x, w, dy, rstd, dw2, zero_dw=True)
    _close(dx2, xf.grad, rtol=3e-2, atol=3e-2)
    assert torch.allclose(dw2, wf.grad, rtol=2e-2, atol=5e-2 * math.sqrt(t))


def test_rope_roundtrip_and_reference():
    from yafsdp_b200.ops import kernels
    from yafsdp_b200.ops.functional import rope_table

    torch.manual_seed(0)
    seq, b, h, hd = 128, 2, 4, 128
    t = seq * b
    qkv = torch.randn(t, 3 * h * hd, device="cuda", dtype=torch.bfloat16)
    orig = qkv.clone()
    cs = rope_table(seq, hd, 10000.0, qkv.device)
    kernels.rope_(qkv, cs, seq, 0, h, hd)
    q = orig[:, : h * hd].float().view(b, seq, h, hd)
    cos = cs[..., 0].view(1, seq, 1, hd // 2)
    sin = cs[..., 1].view(1, seq, 1, hd // 2)
    q1, q2 = q[..., : hd // 2], q[..., hd // 2 :]
    ref = torch.cat([q1 * cos - q2 * sin, q2 * cos + q1 * sin], -1).view(t, h * hd)
    _close(qkv[:, : h * hd], ref)
    assert torch.equal(qkv[:, h * hd :], orig[:, h * hd :])
    kernels.rope_(qkv, cs, seq, 0, h, hd, backward=True)
    _close(qkv, orig, rtol=3e-2, atol=3e-2)


def test_swiglu():
    from yafsdp_b200.ops import kernels

    torch.manual_seed(0)
    t, f = 130, 688
    gu = torch.randn(t, 2 * f, device="cuda", dtype=torch.bfloat16)
    dh = torch.randn(t, f, device="cuda", dtype=torch.bfloat16)
    h = kernels.swiglu_fwd(gu)
    guf = gu.float().requires_grad_(True)
    ref = torch.nn.functional.silu(guf[:, :f]) * guf[:, f:]
    _close(h, ref)
    ref.backward(dh.float())
    dgu = kernels.swiglu_bwd(gu, dh)
    _close(dgu, guf.grad, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("v", [1024, 32000, 1003])
def test_cross_entropy(v):
    from yafsdp_b200.ops import kernels

    torch.manual_seed(0)
    t = 96
    vp = (v + 7) // 8 * 8
    buf = torch.randn(t, vp, device="cuda", dtype=torch.bfloat16) * 3
    logits = buf[:, :v]
    labels = torch.randint(0, v, (t,), device="cuda")
    labels[5] = -100
    lf = logits.float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lf, labels, ignore_index=-100, reduction="sum")
    ref.backward()
    loss_rows = kernels.cross_entropy_(logits, labels, 1.0)
    assert abs(loss_rows.sum().item() - ref.item()) <= 2e-3 * abs(ref.item()) + 1e-2
    assert torch.allclose(logits.float(), lf.grad, rtol=2e-2, atol=4e-3)
    # the gradient scale as host value x device scalar (what the mean over valid labels uses)
    buf2 = torch.zeros_like(buf)
    logits2 = buf2[:, :v]
    logits2.copy_(lf.detach())
    dev_scale = torch.tensor([0.25], device="cuda")
    kernels.cross_entropy_(logits2, labels, 0.5, scale=dev_scale)
    assert torch.allclose(logits2.float(), lf.grad * 0.125, rtol=2e-2, atol=1e-3)


def test_embedding():
    from yafsdp_b200.ops import kernels

    torch.manual_seed(0)
    v, d, t = 500, 256, 777
    table = torch.randn(v, d, device="cuda", dtype=torch.bfloat16)
    ids = torch.randint(0, v, (t,), device="cuda")
    out = kernels.embedding_fwd(table, ids)
    assert torch.equal(out, table[ids])
    dout = torch.randn(t, d, device="cuda", dtype=torch.bfloat16)
    dt = torch.zeros(v, d, device="cuda", dtype=torch.float32)
    kernels.embedding_bwd_(dout, ids, dt)
    ref = torch.zeros_like(dt).index_add_(0, ids, dout.float())
    assert torch.allclose(dt, ref, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("n", [1024, 1000003])
def test_adamw_matches_torch(n):
    from yafsdp_b200.ops import kernels

    torch.manual_seed(0)
    p = torch.randn(n, device="cuda")
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m = torch.zeros_like(p)
    v = torch.zeros_like(p)
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    for step in range(1, 4):
        g = torch.randn(n, device="cuda")
        ref_p.grad = g.clone()
        opt.step()
        kernels.adamw_(p, g, m, v, pb, None, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
    assert torch.allclose(p, ref_p.detach(), rtol=1e-5, atol=1e-6)
    assert torch.equal(pb, p.bfloat16())


def test_sumsq_clip_and_casts():
    from yafsdp_b200.ops import kernels

    torch.manual_seed(0)
    g = torch.randn(3 * 1000 * 1000 + 3, device="cuda")
    acc = torch.zeros(1, device="cuda")
    kernels.sumsq_(g, acc)
    assert abs(acc.item() - g.double().pow(2).sum().item()) <= 1e-4 * acc.item()
    coef = torch.empty(1, device="cuda")
    nrm = torch.empty(1, device="cuda")
    kernels.clip_coef_(acc, 1.0, coef, nrm)
    assert abs(nrm.item() - math.sqrt(acc.item())) < 1e-2 and abs(coef.item() - 1.0 / nrm.item()) < 1e-5
    dst = torch.empty(g.numel(), device="cuda", dtype=torch.bfloat16)
    kernels.cast_f32_to_bf16_(g, dst)
    assert torch.equal(dst, g.bfloat16())
    back = torch.ones_like(g)
    kernels.accum_bf16_to_f32_(dst, back, scale=0.5, accumulate=True)
    assert torch.allclose(back, 1 + 0.5 * dst.float())
    s = kernels.add_bf16(dst, dst)
    assert torch.equal(s, (dst.float() * 2).bfloat16())
