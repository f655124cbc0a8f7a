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


def _reference_kernels():
    """The reference's own library (its C-ABI source built unchanged for sm_100a by oracle/Makefile) behind this
    repository's binding class: the live checker for the three element-wise operators."""
    import os
    import oracle
    from nanoserve_b200.ops import Kernels
    if not os.path.exists(oracle.REF_LIB_PATH):
        pytest.skip("reference library not built (oracle/_ref/libnanoserve_ref.so)")
    return Kernels(oracle.REF_LIB_PATH)


@pytest.mark.parametrize("T,H", [(1, 3584), (7, 512), (3, 8192)])
def test_rmsnorm_rope_swiglu_against_the_reference_kernels(kernels, T, H):
    """Same inputs through the reference's ns_rmsnorm / ns_rope / ns_swiglu (kernels/fused/*.cuh behind
    csrc/nanoserve_ops.cu:21-45) and through this library's.  Both compute in fp32 and round once to bf16; the
    summation order of the norm's sum of squares differs, so the bound is one bf16 ulp of the value plus 1e-3 absolute;
    the residual stream (bf16(x + r), an exact operation) must be bit-identical."""
    ref = _reference_kernels()
    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    r = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).to(torch.bfloat16)

    def near(a, b):
        a, b = a.float(), b.float()
        return bool(torch.all((a - b).abs() <= torch.maximum(a.abs(), b.abs()) * 2.0**-7 + 1e-3))

    for res in (None, r):
        xa, xb = x.clone(), x.clone()
        ya, yb = kernels.rmsnorm(xa, res, w, 1e-6), ref.rmsnorm(xb, res, w, 1e-6)
        assert near(ya, yb) and torch.equal(xa, xb)
    D, Hq, Hk = 128, H // 128, max(1, H // 512)
    if H % 128 == 0:
        q = torch.randn(T, Hq * D, device="cuda", generator=g).to(torch.bfloat16)
        k = torch.randn(T, Hk * D, device="cuda", generator=g).to(torch.bfloat16)
        inv = 1.0 / (1e6 ** (torch.arange(0, D, 2, device="cuda").float() / D))
        qa, ka, qb, kb = q.clone(), k.clone(), q.clone(), k.clone()
        kernels.rope(qa, ka, inv, Hq, Hk, D, 37)
        ref.rope(qb, kb, inv, Hq, Hk, D, 37)
        assert near(qa, qb) and near(ka, kb)
    a = (3 * torch.randn(T, H, device="cuda", generator=g)).to(torch.bfloat16)
    b = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    assert near(kernels.swiglu(a, b), ref.swiglu(a, b))
    torch.cuda.synchronize()


def test_misaligned_pointers_are_refused_not_faulted(kernels):
    """The element-wise kernels move 16 bytes at a time: a view that starts in the middle of a row is refused with -4
    on the host (nothing is launched) instead of faulting on the device."""
    lib = kernels.lib
    t = torch.zeros(4096, dtype=torch.bfloat16, device="cuda")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = t.data_ptr()
    assert lib.ns_rmsnorm(p + 2, None, p, p, 1, 64, 1e-6, st) == -4
    assert lib.ns_rmsnorm(p, p + 4, p, p, 1, 64, 1e-6, st) == -4
    assert lib.ns_swiglu(p, p + 8, p, 1, 64, st) == -4
    assert lib.ns_rope(p + 2, p, p, 1, 1, 1, 64, 0, 64, 64, st) == -4
    assert lib.b2_decode_attention(p + 2, p, p, p, p, p, 4, 2, 128, 16, st) == -4
    torch.cuda.synchronize()
    assert kernels.device_status() == 0


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


@pytest.mark.parametrize("Hq,Hk,D,L,pos", [(8, 2, 128, 64, 37), (28, 4, 128, 1024, 0), (28, 4, 128, 1024, 599),
                                            (28, 4, 128, 1024, 1023), (16, 2, 64, 300, 131), (4, 4, 128, 96, 95),
                                            (8, 1, 128, 40, 40)])
def test_fused_attention_equals_the_two_calls(kernels, Hq, Hk, D, L, pos):
    """b2_decode_attention_fused against b2_rope_kv_store + b2_decode_attention on the same inputs: the attention
    output and the appended cache rows must be bit-identical, qkv must be left as it was, and the arrival counters
    must be back at zero (the launch is repeated).  pos == L: the cache is full, nothing is appended."""
    lib = kernels.lib
    g = torch.Generator(device="cuda").manual_seed(100 + pos)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ck = torch.randn(Hk, L, D, device="cuda", generator=g).to(torch.bfloat16)
    cv = torch.randn(Hk, L, D, device="cuda", generator=g).to(torch.bfloat16)
    qkv = torch.randn((Hq + 2 * Hk) * D, device="cuda", generator=g).to(torch.bfloat16)
    bias = (0.1 * torch.randn((Hq + 2 * Hk) * D, device="cuda", generator=g)).to(torch.bfloat16)
    inv = 1.0 / (1e4 ** (torch.arange(0, D, 2, device="cuda").float() / D))
    p = torch.tensor([pos], dtype=torch.int32, device="cuda")
    # the two-call form on copies
    qkv2, ck2, cv2 = qkv.clone(), ck.clone(), cv.clone()
    out2 = torch.empty(Hq * D, dtype=torch.bfloat16, device="cuda")
    ws2 = torch.empty(int(lib.b2_decode_workspace_bytes(Hq, D)), dtype=torch.uint8, device="cuda")
    assert lib.b2_rope_kv_store(qkv2.data_ptr(), bias.data_ptr(), inv.data_ptr(), p.data_ptr(), ck2.data_ptr(),
                                cv2.data_ptr(), Hq, Hk, D, L, st) == 0
    assert lib.b2_decode_attention(qkv2.data_ptr(), ck2.data_ptr(), cv2.data_ptr(), p.data_ptr(), out2.data_ptr(),
                                   ws2.data_ptr(), Hq, Hk, D, L, st) == 0
    # the fused form, twice
    ws = torch.zeros(int(lib.b2_decode_attention_fused_workspace_bytes(Hq, Hk, D)), dtype=torch.uint8, device="cuda")
    keep = qkv.clone()
    for flags in (1, 1, 0, 2, 3):
        ck1, cv1 = ck.clone(), cv.clone()
        out = torch.full((Hq * D,), 7.0, dtype=torch.bfloat16, device="cuda")
        assert lib.b2_decode_attention_fused(qkv.data_ptr(), bias.data_ptr(), inv.data_ptr(), p.data_ptr(),
                                             ck1.data_ptr(), cv1.data_ptr(), out.data_ptr(), ws.data_ptr(), Hq, Hk, D,
                                             L, None, flags, st) == 0
        torch.cuda.synchronize()
        assert torch.equal(out, out2)
        assert torch.equal(ck1, ck2) and torch.equal(cv1, cv2)
        assert torch.equal(qkv, keep)
        assert int(ws[-4 * Hk:].view(torch.int32).abs().sum()) == 0
    assert kernels.device_status() == 0


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
