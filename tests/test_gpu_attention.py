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


@pytest.mark.parametrize("b,s,hq,hkv", [(1, 128, 1, 1), (2, 384, 4, 4), (1, 512, 8, 2), (2, 200, 2, 1), (1, 2048, 2, 2)])
@pytest.mark.parametrize("causal", [True, False])
def test_attention_fwd_bwd(b, s, hq, hkv, causal):
    from yafsdp_b200.ops import kernels

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
