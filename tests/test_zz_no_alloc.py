"""The allocation-free attention backward (``yf_attn_bwd_noalloc``), called through its exported C symbol.

Some users of the native library cannot hand it scratch memory: a C/C++ host that binds the symbols without a
tensor framework, or a job whose own memory pool already owns the whole GPU so that a later ``cudaMalloc`` fails.
For them the library keeps the backward's scratch (delta and the fp32 dQ accumulator) in a fixed device array and
exports an entry point that takes inputs and outputs only.  This test drives that entry point the way such a
caller would (``ctypes`` on the shared object, raw pointers) and checks it against the regular entry point, twice
in a row with different inputs, because every call reuses the same scratch and must clear what has to start at zero.
This file sorts last so that a run stopping at the first failure has already run every other test.
"""

import ctypes
import math
import pathlib

import pytest
import torch

pytestmark = pytest.mark.gpu

_P, _I, _L, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def _load():
    path = pathlib.Path(__file__).resolve().parent.parent / "yafsdp_b200" / "lib" / "libyafsdp_b200.so"
    if not path.exists():
        from yafsdp_b200 import _native

        _native.build()
    lib = ctypes.CDLL(str(path))
    lib.yf_attn_fwd.argtypes = [_P, _P, _P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _F, _I, _P]
    lib.yf_attn_bwd.argtypes = [_P] * 11 + [_I] * 4 + [_L] * 6 + [_F, _I, _P]
    lib.yf_attn_bwd_noalloc.argtypes = [_P] * 9 + [_I] * 4 + [_L] * 6 + [_F, _I, _P]
    for fn in (lib.yf_attn_fwd, lib.yf_attn_bwd, lib.yf_attn_bwd_noalloc):
        fn.restype = _I
    return lib


def _fp32_oracle(qkv, dout, b, s, hq, hkv):
    """Gradients of causal softmax attention with respect to the packed q/k/v, by autograd on an fp32 restatement."""
    d = 128
    x = qkv.float().detach().requires_grad_(True)
    q = x[:, : hq * d].view(b, s, hq, d)
    k = x[:, hq * d : (hq + hkv) * d].view(b, s, hkv, d).repeat_interleave(hq // hkv, dim=2)
    v = x[:, (hq + hkv) * d :].view(b, s, hkv, d).repeat_interleave(hq // hkv, dim=2)
    att = torch.einsum("bqhd,bkhd->bhqk", q, k) / math.sqrt(d)
    att = att.masked_fill(~torch.ones(s, s, device=x.device, dtype=torch.bool).tril(), float("-inf"))
    o = torch.einsum("bhqk,bkhd->bqhd", att.softmax(-1), v).reshape(b * s, hq * d)
    o.backward(dout.float())
    return x.grad


def _case(lib, seed, b, s, hq, hkv, oracle=True):
    d = 128
    t = b * s
    width = (hq + 2 * hkv) * d
    torch.manual_seed(seed)
    qkv = torch.randn(t, width, device="cuda", dtype=torch.bfloat16)
    q, k, v = qkv[:, : hq * d], qkv[:, hq * d : (hq + hkv) * d], qkv[:, (hq + hkv) * d :]
    out = torch.empty(t, hq * d, device="cuda", dtype=torch.bfloat16)
    lse = torch.empty(b, hq, s, device="cuda", dtype=torch.float32)
    dout = torch.randn(t, hq * d, device="cuda", dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.yf_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), b, s, hq, hkv, width, width,
                           hq * d, scale, 1, stream) == 0
    # regular entry point: scratch comes from the caller
    delta = torch.empty(b, hq, s, device="cuda", dtype=torch.float32)
    acc = torch.empty(t, hq * d, device="cuda", dtype=torch.float32)
    ref = torch.zeros_like(qkv)
    rq, rk, rv = ref[:, : hq * d], ref[:, hq * d : (hq + hkv) * d], ref[:, (hq + hkv) * d :]
    assert lib.yf_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
                           delta.data_ptr(), acc.data_ptr(), rq.data_ptr(), rk.data_ptr(), rv.data_ptr(), b, s, hq, hkv,
                           width, width, hq * d, hq * d, width, width, scale, 1, stream) == 0
    # allocation-free entry point: inputs and outputs only
    got = torch.zeros_like(qkv)
    gq, gk, gv = got[:, : hq * d], got[:, hq * d : (hq + hkv) * d], got[:, (hq + hkv) * d :]
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]  # cudaMemGetInfo: what the driver has left on the device
    rc = lib.yf_attn_bwd_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
                                 gq.data_ptr(), gk.data_ptr(), gv.data_ptr(), b, s, hq, hkv, width, width, hq * d, hq * d,
                                 width, width, scale, 1, stream)
    assert rc == 0, rc
    torch.cuda.synchronize()
    if seed != 0:  # the very first call on a device may map the library's status page; later calls must not move the needle
        assert torch.cuda.mem_get_info()[0] == free_before, "the allocation-free entry point changed the device's free memory"
    if oracle:
        want = _fp32_oracle(qkv, dout, b, s, hq, hkv)
        err32 = (got.float() - want).abs().max().item()
        assert err32 <= 2e-2 * want.abs().max().item() + 2e-2, f"against the fp32 restatement: max err {err32}"
    err = (got.float() - ref.float()).abs().max().item()
    scale_ref = ref.float().abs().max().item()
    # same kernels and same math; only the order of the fp32 dQ reductions may differ between two runs
    assert err <= 2e-2 * scale_ref + 2e-2, f"max err {err} (scale {scale_ref})"
    assert scale_ref > 0


def test_noalloc_backward_matches_regular_entry_point_twice():
    lib = _load()
    _case(lib, 0, 2, 384, 4, 2)      # first call on this device also resolves the scratch address
    _case(lib, 1, 1, 1024, 8, 8)     # different shape and data: stale scratch from the first call must not leak in
    # exactly at the limit of the built-in scratch: B * S * Hq = 32768 rows (the fp32 restatement would need S^2 memory)
    _case(lib, 2, 1, 4096, 8, 2, oracle=False)
    code, site = ctypes.c_int(0), ctypes.c_int(0)
    lib.yf_status_read.argtypes = [_P, _P, _I]
    assert lib.yf_status_read(ctypes.byref(code), ctypes.byref(site), 1) == 0 and code.value == 0


def test_noalloc_backward_refuses_oversized_problem():
    lib = _load()
    dummy = torch.zeros(64, device="cuda", dtype=torch.bfloat16)
    p = dummy.data_ptr()
    rc = lib.yf_attn_bwd_noalloc(p, p, p, p, p, p, p, p, p, 4, 4096, 32, 32, 12288, 12288, 4096, 4096, 12288, 12288, 0.1, 1,
                                 torch.cuda.current_stream().cuda_stream)
    assert rc == -3
