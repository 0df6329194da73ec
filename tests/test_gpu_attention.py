"""tcgen05 flash attention forward/backward vs an fp32 PyTorch restatement."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(q, k, v, causal):
    # q: [B,S,Hq,D], k/v: [B,S,Hkv,D] fp32
    b, s, hq, d = q.shape
    hkv = k.shape[2]
    k = k.repeat_interleave(hq // hkv, dim=2)
    v = v.repeat_interleave(hq // hkv, dim=2)
    att = torch.einsum("bqhd,bkhd->bhqk", q, k) / math.sqrt(d)
    if causal:
        mask = torch.ones(s, s, device=q.device, dtype=torch.bool).tril()
        att = att.masked_fill(~mask, float("-inf"))
    p = att.softmax(-1)
    return torch.einsum("bhqk,bkhd->bqhd", p, v)


@pytest.mark.parametrize("b,s,hq,hkv", [(1, 128, 1, 1), (2, 384, 4, 4), (1, 512, 8, 2), (2, 200, 2, 1), (1, 2048, 2, 2),
                                         (1, 4096, 32, 8), (1, 4096, 16, 2), (2, 1000, 8, 1), (1, 8192, 8, 1)])
@pytest.mark.parametrize("causal", [True, False])
def test_attention_fwd_bwd(b, s, hq, hkv, causal):
    from yafsdp_b200.ops import kernels

    if not causal and s >= 4096:
        pytest.skip("long sequences are checked in the causal form the models use")
    torch.manual_seed(0)
    d = 128
    t = b * s
    width = (hq + 2 * hkv) * d
    qkv = torch.randn(t, width, device="cuda", dtype=torch.bfloat16)
    q = qkv[:, : hq * d]
    k = qkv[:, hq * d : (hq + hkv) * d]
    v = qkv[:, (hq + hkv) * d :]
    scale = 1.0 / math.sqrt(d)
    out, lse = kernels.attn_fwd(q, k, v, b, s, hq, hkv, scale, causal)
    qf = q.float().view(b, s, hq, d).detach().requires_grad_(True)
    kf = k.float().view(b, s, hkv, d).detach().requires_grad_(True)
    vf = v.float().view(b, s, hkv, d).detach().requires_grad_(True)
    ref = _ref(qf, kf, vf, causal)
    torch.cuda.synchronize()
    kernels.check_status()
    err = (out.float().view(b, s, hq, d) - ref).abs().max().item()
    assert err < 2e-2, f"forward max err {err}"
    dout = torch.randn(t, hq * d, device="cuda", dtype=torch.bfloat16)
    ref.backward(dout.float().view(b, s, hq, d))
    dqkv = torch.zeros_like(qkv)
    kernels.attn_bwd(q, k, v, out, dout, lse, dqkv[:, : hq * d], dqkv[:, hq * d : (hq + hkv) * d], dqkv[:, (hq + hkv) * d :],
                     b, s, hq, hkv, scale, causal)
    torch.cuda.synchronize()
    kernels.check_status()
    for name, got, want in (
        ("dq", dqkv[:, : hq * d], qf.grad.reshape(t, -1)),
        ("dk", dqkv[:, hq * d : (hq + hkv) * d], kf.grad.reshape(t, -1)),
        ("dv", dqkv[:, (hq + hkv) * d :], vf.grad.reshape(t, -1)),
    ):
        e = (got.float() - want).abs().max().item()
        ref_scale = want.abs().max().item()
        assert e <= 2e-2 * ref_scale + 2e-2, f"{name} max err {e} (scale {ref_scale})"


def test_attention_forward_with_growing_scores():
    """Scores that keep growing along the key axis force the forward kernel to move its reference maximum many times
    (the output then is rescaled in TMEM); a large constant offset exercises the exponent range."""
    from yafsdp_b200.ops import kernels

    torch.manual_seed(1)
    b, s, hq, hkv, d = 1, 1024, 2, 1, 128
    t = b * s
    qkv = torch.randn(t, (hq + 2 * hkv) * d, device="cuda", dtype=torch.bfloat16)
    ramp = torch.linspace(0.0, 6.0, s, device="cuda").view(s, 1)
    qkv[:, hq * d : (hq + hkv) * d] = (qkv[:, hq * d : (hq + hkv) * d].float() * (1.0 + ramp)).to(torch.bfloat16)  # later keys score higher
    q, k, v = qkv[:, : hq * d], qkv[:, hq * d : (hq + hkv) * d], qkv[:, (hq + hkv) * d :]
    out, lse = kernels.attn_fwd(q, k, v, b, s, hq, hkv, 1.0 / math.sqrt(d), True)
    ref = _ref(q.float().view(b, s, hq, d), k.float().view(b, s, hkv, d), v.float().view(b, s, hkv, d), True)
    torch.cuda.synchronize()
    kernels.check_status()
    assert (out.float().view(b, s, hq, d) - ref).abs().max().item() < 3e-2
    att = torch.einsum("bqhd,bkhd->bhqk", q.float().view(b, s, hq, d), k.float().view(b, s, hkv, d).repeat_interleave(hq // hkv, dim=2)) / math.sqrt(d)
    att = att.masked_fill(~torch.ones(s, s, device="cuda", dtype=torch.bool).tril(), float("-inf"))
    assert torch.allclose(lse, att.logsumexp(-1), atol=2e-2, rtol=1e-3)
