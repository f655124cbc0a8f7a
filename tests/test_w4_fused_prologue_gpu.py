"""GPU tests of b2_w4_linear_fused: the GEMV with the preceding operator folded in must equal the two-kernel sequence
(ns_rmsnorm or ns_swiglu, then ns_w4_linear) up to the rounding of the norm's sum of squares, and must match the CPU
oracle applied to the operator's bf16 output."""
import numpy as np
import pytest
import torch

import oracle
from nanoserve_b200 import ops
from tests.util import bits_to_torch, check_bf16_output, torch_to_bits, u32_to_torch

pytestmark = pytest.mark.gpu


def agree(a, b, scale_slack=2e-3):
    a, b = a.float(), b.float()
    tol = torch.maximum(a.abs(), b.abs()) * 2.0**-7 + scale_slack * b.abs().max()
    return bool(torch.all((a - b).abs() <= tol))


@pytest.mark.parametrize("M,N,K", [(1, 4608, 3584), (1, 512, 3584), (3, 256, 1024), (16, 448, 3584), (8, 64, 18944)])
@pytest.mark.parametrize("with_residual", [True, False])
def test_add_rmsnorm_prologue(kernels, M, N, K, with_residual):
    G = 128
    _, Wq, S = oracle.synth_inputs(1, N, K, G, seed=41)
    wq, s = u32_to_torch(Wq), bits_to_torch(S)
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    r = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16) if with_residual else None
    wn = (1 + 0.1 * torch.randn(K, device="cuda", generator=g)).to(torch.bfloat16)
    eps = 1e-6
    # two-kernel sequence of the reference flow
    x_seq = x.clone()
    h = kernels.rmsnorm(x_seq, r, wn, eps)
    y_seq = kernels.w4_linear(h, wq, s, G)
    # fused
    x_out = torch.full_like(x, 3.0) if with_residual else None
    y = kernels.w4_linear_fused(x, wq, s, G, prologue=1, r=r, wn=wn, eps=eps, x_out=x_out)
    torch.cuda.synchronize()
    if with_residual:
        assert torch.equal(x_out, x_seq)  # the updated residual stream, bit for bit
    assert agree(y, y_seq)
    # the norm output differs from the separate kernel's by at most a bf16 ulp where the factor rounds differently;
    # against the oracle on the separate kernel's output the product stays within that plus the GEMV's own bound
    ref = oracle.w4_linear_f32(torch_to_bits(h), Wq, S, G, threads=oracle.max_threads())
    check_bf16_output(torch_to_bits(y), ref, 4e-3)
    assert kernels.device_status() == 0


@pytest.mark.parametrize("M,N,K", [(1, 3584, 18944), (4, 256, 512), (16, 448, 2304)])
def test_swiglu_prologue(kernels, M, N, K):
    G = 128
    _, Wq, S = oracle.synth_inputs(1, N, K, G, seed=43)
    wq, s = u32_to_torch(Wq), bits_to_torch(S)
    g = torch.Generator(device="cuda").manual_seed(M + K)
    gu = torch.randn(M, 2 * K, device="cuda", generator=g).to(torch.bfloat16)
    act = kernels.swiglu(gu[:, :K].contiguous(), gu[:, K:].contiguous())
    # the CTA shape and K split come from the cost model here, so that both calls sum in the same order; X converted in
    # every CTA, or once by the kernel in front of the GEMV
    for flags in (ops.FLAG_NO_AUTOTUNE, ops.FLAG_NO_AUTOTUNE | ops.FLAG_PRE_STAGE_X,
                  ops.FLAG_NO_AUTOTUNE | ops.FLAG_NO_PRE_STAGE_X):
        # (a plain launch of several tokens would go to the many-token kernel, which has no prologues: keep both
        # calls on the same kernel)
        y_seq = kernels.w4_linear(act, wq, s, G, flags=flags | ops.FLAG_NO_MID_KERNEL)
        y = kernels.w4_linear_fused(gu, wq, s, G, prologue=2, flags=flags)
        torch.cuda.synchronize()
        assert torch.equal(y, y_seq), flags  # same element-wise arithmetic, same product: identical
    # SwiGLU outputs have heavy tails: the 16-bit fixed-point staging of X is coarser where a chunk holds an outlier
    check_bf16_output(torch_to_bits(y), oracle.w4_linear_f32(torch_to_bits(act), Wq, S, G, threads=oracle.max_threads()),
                      5e-5)


def test_prologue_error_codes(kernels):
    x = torch.zeros(1, 256, dtype=torch.bfloat16, device="cuda")
    wq = torch.zeros(8, 32, dtype=torch.int32, device="cuda")
    s = torch.ones(8, 8, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="code -3"):   # G = 32: prologues are fast-path only
        kernels.w4_linear_fused(x, wq, s, 32, prologue=1, wn=x[0])
    s = torch.ones(8, 2, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="code -4"):   # norm weights missing
        kernels.w4_linear_fused(x, wq, s, 128, prologue=1)
    with pytest.raises(RuntimeError, match="code -1"):
        kernels.w4_linear_fused(x, wq, s, 128, prologue=7)


def _pairs(a, b, blk=16):
    """`blk` rows of a, the same rows of b, the next `blk` of a ..."""
    n = a.shape[0]
    return torch.stack([a.view(n // blk, blk, -1), b.view(n // blk, blk, -1)], 1).reshape(2 * n, -1).contiguous()


@pytest.mark.parametrize("I,K,norm", [(18944, 3584, True), (18944, 3584, False), (2048, 1024, False), (160, 512, True)])
def test_swiglu_pairs_epilogue(kernels, I, K, norm):
    """gate|up with SwiGLU in its epilogue (rows in blocks of 16 gate + 16 up) against the plain launch on the
    row-concatenated matrix followed by ns_swiglu: the same rows, the same arithmetic, so bit-identical."""
    G = 128
    _, Wq, S = oracle.synth_inputs(1, 2 * I, K, G, seed=47)
    wq, s = u32_to_torch(Wq), bits_to_torch(S)
    g = torch.Generator(device="cuda").manual_seed(I + K)
    x = torch.randn(1, K, device="cuda", generator=g).to(torch.bfloat16)
    r = torch.randn(1, K, device="cuda", generator=g).to(torch.bfloat16) if norm else None
    wn = (1 + 0.1 * torch.randn(K, device="cuda", generator=g)).to(torch.bfloat16) if norm else None
    pro = 1 if norm else 0
    # one warp per row block along K in the plain launch too (bits 20-23 of the flags), so that both sum in one order
    gu = kernels.w4_linear_fused(x, wq, s, G, prologue=pro, r=r, wn=wn, eps=1e-6, flags=1 << 20)
    ref = kernels.swiglu(gu[:, :I].contiguous(), gu[:, I:].contiguous())
    wq2, s2 = _pairs(wq[:I], wq[I:]), _pairs(s[:I], s[I:])
    act = kernels.w4_linear_fused(x, wq2, s2, G, prologue=pro, r=r, wn=wn, eps=1e-6, epilogue=ops.EPI_SWIGLU_PAIRS)
    # the same with row blocks of 8 (16 rows per warp)
    wq3, s3 = _pairs(wq[:I], wq[I:], 8), _pairs(s[:I], s[I:], 8)
    act8 = kernels.w4_linear_fused(x, wq3, s3, G, prologue=pro, r=r, wn=wn, eps=1e-6, epilogue=ops.EPI_SWIGLU_PAIRS8)
    torch.cuda.synchronize()
    assert act.shape == (1, I)
    assert torch.equal(act, ref)
    assert torch.equal(act8, ref)
    assert kernels.device_status() == 0


def test_swiglu_pairs_epilogue_is_refused_where_it_cannot_run(kernels):
    """More than one token, a row count that is not whole blocks, or a group size the streaming kernel does not take:
    code -3, nothing launched; the caller runs the plain launch and the SwiGLU prologue of the next one instead."""
    G = 128
    for M, N, K, grp in [(2, 256, 512, G), (1, 240, 512, G), (1, 256, 512, 64)]:
        _, Wq, S = oracle.synth_inputs(1, N, K, grp, seed=5)
        x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        with pytest.raises(RuntimeError, match="code -3"):
            kernels.w4_linear_fused(x, u32_to_torch(Wq), bits_to_torch(S), grp, epilogue=ops.EPI_SWIGLU_PAIRS)
    assert kernels.device_status() == 0


@pytest.mark.parametrize("I,K,H", [(18944, 3584, 3584), (1024, 512, 320)])
def test_staged_handover_between_two_gemvs(kernels, I, K, H):
    """gate|up writes silu(gate) * up in the converted form (epilogue 2), the down projection copies it into its
    shared memory instead of converting (prologue 3): the down output must equal, bit for bit, the one computed from
    the bf16 activations of epilogue 1."""
    G = 128
    _, Wa, Sa = oracle.synth_inputs(1, 2 * I, K, G, seed=51)
    _, Wb, Sb = oracle.synth_inputs(1, H, I, G, seed=52)
    wa, sa, wb, sb = u32_to_torch(Wa), bits_to_torch(Sa), u32_to_torch(Wb), bits_to_torch(Sb)
    wa, sa = _pairs(wa[:I], wa[I:]), _pairs(sa[:I], sa[I:])
    g = torch.Generator(device="cuda").manual_seed(I)
    x = torch.randn(1, K, device="cuda", generator=g).to(torch.bfloat16)
    act = kernels.w4_linear_fused(x, wa, sa, G, epilogue=ops.EPI_SWIGLU_PAIRS)
    want = kernels.w4_linear(act, wb, sb, G)
    staged = kernels.w4_linear_fused(x, wa, sa, G, epilogue=ops.EPI_SWIGLU_STAGED)
    assert staged.dtype == torch.uint8 and staged.numel() == ops.staged_x_bytes(I)
    got = kernels.w4_linear_fused(staged, wb, sb, G, prologue=ops.PRO_STAGED)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    # an inf among the activations poisons its chunk in both forms alike
    x2 = x.clone()
    x2[0, 3] = float("inf")
    a2 = kernels.w4_linear_fused(x2, wa, sa, G, epilogue=ops.EPI_SWIGLU_PAIRS)
    w2 = kernels.w4_linear(a2, wb, sb, G)
    s2 = kernels.w4_linear_fused(x2, wa, sa, G, epilogue=ops.EPI_SWIGLU_STAGED)
    g2 = kernels.w4_linear_fused(s2, wb, sb, G, prologue=ops.PRO_STAGED)
    torch.cuda.synchronize()
    assert torch.equal(torch.isnan(g2), torch.isnan(w2))
    assert torch.equal(torch.nan_to_num(g2.float()), torch.nan_to_num(w2.float()))
    assert kernels.device_status() == 0
