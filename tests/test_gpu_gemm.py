"""tcgen05 GEMM family vs an fp32 PyTorch restatement, every operand-major combination."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    af = a.float().t() if a_mn else a.float()
    bf = b.float().t() if b_mn else b.float()
    return af @ bf.t()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (256, 512, 256), (384, 640, 192), (200, 328, 136), (2048, 1024, 2048),
                                   (448, 1000, 136), (2304, 512, 64), (512, 2304, 4096)])
def test_gemm_matches_fp32(m, n, k, a_mn, b_mn):
    from yafsdp_b200.ops import kernels

    torch.manual_seed(0)
    a = torch.randn((k, m) if a_mn else (m, k), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((k, n) if b_mn else (n, k), device="cuda", dtype=torch.bfloat16)
    out = kernels.gemm(a, b, a_mn_major=a_mn, b_mn_major=b_mn)
    ref = _ref(a, b, a_mn, b_mn)
    torch.cuda.synchronize()
    kernels.check_status()
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, f"max err {err} vs scale {scale}"


def test_gemm_fp32_out_accumulate_alpha():
    from yafsdp_b200.ops import kernels

    torch.manual_seed(1)
    m, n, k = 512, 768, 320
    a = torch.randn(k, m, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(k, n, device="cuda", dtype=torch.bfloat16)
    out = torch.randn(m, n, device="cuda", dtype=torch.float32)
    ref = out + 0.5 * (a.float().t() @ b.float())
    kernels.gemm(a, b, a_mn_major=True, b_mn_major=True, out=out, accumulate=True, alpha=0.5)
    torch.cuda.synchronize()
    kernels.check_status()
    assert torch.allclose(out, ref, rtol=1e-3, atol=1e-2)


def test_gemm_strided_views():
    """Operands and output that are column slices of wider buffers (row pitch > row length)."""
    from yafsdp_b200.ops import kernels

    torch.manual_seed(2)
    big_a = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16)
    big_b = torch.randn(384, 512, device="cuda", dtype=torch.bfloat16)
    big_c = torch.zeros(256, 1024, device="cuda", dtype=torch.bfloat16)
    a = big_a[:, 128:384]
    b = big_b[:, 256:512]
    c = big_c[:, 256:640]
    kernels.gemm(a, b, out=c)
    torch.cuda.synchronize()
    kernels.check_status()
    ref = a.float() @ b.float().t()
    assert (c.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-2
    assert big_c[:, :256].abs().max().item() == 0 and big_c[:, 640:].abs().max().item() == 0


def test_gemm_fused_sum_of_squares():
    """The fp32 epilogue can add the squared norm of what it writes to a device scalar (gradient-norm fusion)."""
    from yafsdp_b200.ops import kernels

    torch.manual_seed(3)
    m, n, k = 640, 1000, 256  # n not a multiple of the tile: clipped columns must not contribute
    a = torch.randn(k, m, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(k, n, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(m, n, device="cuda", dtype=torch.float32)
    acc = torch.full((1,), 5.0, device="cuda")
    kernels.gemm(a, b, a_mn_major=True, b_mn_major=True, out=out, sumsq=acc)
    torch.cuda.synchronize()
    kernels.check_status()
    want = 5.0 + out.double().pow(2).sum().item()
    assert abs(acc.item() - want) <= 1e-4 * want


@pytest.mark.parametrize("m,n,k", [(256, 512, 256), (200, 328, 136), (2048, 4096, 1024), (448, 1000, 136), (130, 136, 64)])
def test_gemm_residual_epilogue(m, n, k):
    """out = A @ B^T + R with the bf16 residual added in fp32 inside the epilogue (single-CTA and CTA-pair tiles, ragged
    edges, a residual with a row pitch, and in place on the residual)."""
    from yafsdp_b200.ops import kernels

    torch.manual_seed(3)
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    wide = (8 * torch.randn(m, n + 24, device="cuda")).bfloat16()
    res = wide[:, 8 : 8 + n]  # 16-byte aligned view with a pitch of n + 24
    ref = a.float() @ b.float().t() + res.float()
    out = kernels.gemm(a, b, residual=res)
    torch.cuda.synchronize()
    kernels.check_status()
    scale = ref.abs().max().item()
    assert (out.float() - ref).abs().max().item() <= 1e-2 * scale + 1e-2
    # one rounding only: no worse than rounding the exact sum to bf16, up to the accumulation order
    assert (out.float() - ref).abs().max().item() <= (ref.bfloat16().float() - ref).abs().max().item() + 1e-3 * scale
    inplace = res.contiguous()
    kernels.gemm(a, b, residual=inplace, out=inplace)
    torch.cuda.synchronize()
    assert torch.equal(inplace, out)
