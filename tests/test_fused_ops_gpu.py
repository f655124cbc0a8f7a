"""GPU tests of the element-wise neighbours of the linears (ns_rmsnorm, ns_rope, ns_swiglu) and of the decode
helpers, against plain PyTorch fp32 references of the same ops (the reference project's own *_ref functions follow the
same formulas, python/nanoserve/ops.py:101-142).  Bound: 3e-2 relative to |ref| + 1, the reference's fused-op gate
(bench/bench_fused.cu:70-77)."""
import ctypes

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def close(a, ref, tol=3e-2):
    return bool(torch.all((a.float() - ref.float()).abs() <= tol * (ref.float().abs() + 1)))


@pytest.mark.parametrize("T,H", [(1, 3584), (8, 256), (5, 8192)])
def test_rmsnorm(kernels, T, H):
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    r = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).to(torch.bfloat16)
    for res in (None, r):
        xi = x.clone()
        y = kernels.rmsnorm(xi, res, w, 1e-6)
        xs = (x.float() + res.float()).to(torch.bfloat16) if res is not None else x
        h = xs.float()
        ref = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
        assert close(y, ref)
        assert torch.equal(xi, xs)  # the residual stream is updated in place, rounded to bf16


def test_rope_and_swiglu(kernels):
    g = torch.Generator(device="cuda").manual_seed(2)
    T, Hq, Hk, D = 6, 4, 2, 128
    q = torch.randn(T, Hq * D, device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn(T, Hk * D, device="cuda", generator=g).to(torch.bfloat16)
    inv = 1.0 / (1e4 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    q0, k0 = q.clone().float(), k.clone().float()
    kernels.rope(q, k, inv, Hq, Hk, D, 7)
    fr = torch.outer(torch.arange(7, 7 + T, device="cuda").float(), inv)
    cos, sin = torch.cat([fr, fr], -1).cos()[:, None], torch.cat([fr, fr], -1).sin()[:, None]
    for got, src, H in ((q, q0, Hq), (k, k0, Hk)):
        v = src.view(T, H, D)
        ref = v * cos + torch.cat([-v[..., D // 2:], v[..., :D // 2]], -1) * sin
        assert close(got.view(T, H, D), ref)
    a = torch.randn(3, 512, device="cuda", generator=g).to(torch.bfloat16)
    b = torch.randn(3, 512, device="cuda", generator=g).to(torch.bfloat16)
    assert close(kernels.swiglu(a, b), F.silu(a.float()) * b.float())
    with pytest.raises(RuntimeError, match="ns_swiglu failed with code -1"):
        kernels.swiglu(a[:1, :4].contiguous(), b[:1, :4].contiguous())  # T*I % 8 (csrc/nanoserve_ops.cu:39)


def test_flash_fwd_is_reported_as_not_implemented(kernels):
    q = torch.zeros(64, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="ns_flash_fwd failed with code -3"):
        kernels.flash_attention(q, q, q, 1, 1, 128)


def test_decode_attention_and_rope_kv_store(kernels):
    lib = kernels.lib
    g = torch.Generator(device="cuda").manual_seed(3)
    Hq, Hk, D, L, pos = 8, 2, 128, 64, 37
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ck = torch.randn(Hk, L, D, device="cuda", generator=g).to(torch.bfloat16)
    cv = torch.randn(Hk, L, D, device="cuda", generator=g).to(torch.bfloat16)
    qkv = torch.randn((Hq + 2 * Hk) * D, device="cuda", generator=g).to(torch.bfloat16)
    bias = (0.1 * torch.randn((Hq + 2 * Hk) * D, device="cuda", generator=g)).to(torch.bfloat16)
    inv = 1.0 / (1e4 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    p = torch.tensor([pos], dtype=torch.int32, device="cuda")
    src = (qkv.float() + bias.float()).to(torch.bfloat16).float().view(Hq + 2 * Hk, D)
    assert lib.b2_rope_kv_store(qkv.data_ptr(), bias.data_ptr(), inv.data_ptr(), p.data_ptr(), ck.data_ptr(),
                                cv.data_ptr(), Hq, Hk, D, L, st) == 0
    fr = pos * inv
    cos, sin = torch.cat([fr, fr]).cos(), torch.cat([fr, fr]).sin()
    rot = src * cos + torch.cat([-src[:, D // 2:], src[:, :D // 2]], -1) * sin
    ref = torch.cat([rot[:Hq + Hk], src[Hq + Hk:]])
    got = qkv.view(Hq + 2 * Hk, D)
    assert close(got, ref)
    assert torch.equal(ck[:, pos], got[Hq:Hq + Hk]) and torch.equal(cv[:, pos], got[Hq + Hk:])
    out = torch.empty(Hq * D, dtype=torch.bfloat16, device="cuda")
    ws = torch.empty(int(lib.b2_decode_workspace_bytes(Hq, D)), dtype=torch.uint8, device="cuda")
    assert lib.b2_decode_attention(qkv.data_ptr(), ck.data_ptr(), cv.data_ptr(), p.data_ptr(), out.data_ptr(),
                                   ws.data_ptr(), Hq, Hk, D, L, st) == 0
    qh = got[:Hq].float()[None, :, None, :]
    ref_o = F.scaled_dot_product_attention(qh, ck[None, :, :pos + 1].float(), cv[None, :, :pos + 1].float(),
                                           enable_gqa=True)
    assert close(out.view(Hq, D), ref_o[0, :, 0])


def test_greedy_next(kernels):
    lib = kernels.lib
    V, H = 152064, 64
    g = torch.Generator(device="cuda").manual_seed(4)
    logits = torch.randn(V, device="cuda", generator=g).to(torch.bfloat16)
    logits[777] = 50.0
    logits[90000] = 50.0  # tie: the lower index wins, as torch.argmax on the first occurrence
    embed = torch.randn(V, H, device="cuda", generator=g).to(torch.bfloat16)
    pos = torch.tensor([11], dtype=torch.int32, device="cuda")
    step = torch.tensor([2], dtype=torch.int32, device="cuda")
    toks = torch.zeros(8, dtype=torch.int64, device="cuda")
    x = torch.zeros(H, dtype=torch.bfloat16, device="cuda")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ws = torch.empty(int(lib.b2_decode_workspace_bytes(28, 128)), dtype=torch.uint8, device="cuda")
    assert lib.b2_greedy_next(logits.data_ptr(), V, embed.data_ptr(), H, pos.data_ptr(), toks.data_ptr(),
                              step.data_ptr(), x.data_ptr(), ws.data_ptr(), st) == 0
    torch.cuda.synchronize()
    assert int(toks[2]) == 777 and int(pos) == 12 and int(step) == 3 and torch.equal(x, embed[777])
