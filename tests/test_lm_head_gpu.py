"""GPU tests of b2_lm_head (bf16 vocabulary projection with the greedy argmax in its epilogue) and b2_greedy_pick.

This is a floating-point kernel without a counterpart in the reference library (the reference calls F.linear and
argmax, python/nanoserve/qwen.py:164,174-177), so the checker is a plain PyTorch fp32 product of the same bf16
operands: every logit within one bf16 rounding of it plus 1e-5 of the largest logit for the fp32 summation order;
the (value, index) pairs must equal the block-wise argmax of the kernel's own bf16 logits exactly."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref_logits(x, W):
    return x.float() @ W.float().T


@pytest.mark.parametrize("M,V,K", [(1, 1000, 256), (1, 4096, 3584), (3, 777, 512), (8, 130, 128), (1, 128, 64), (2, 152064 // 8, 3584)])
def test_logits_and_block_argmax(kernels, M, V, K):
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(M * 1000 + V)
    x = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
    W = (torch.randn(V, K, device=dev, generator=gen) * 0.05).to(torch.bfloat16)
    nblk = kernels.lm_head_blocks(V)
    assert nblk == (V + 127) // 128
    logits = torch.empty(M, V, dtype=torch.bfloat16, device=dev)
    pv = torch.empty(nblk, dtype=torch.float32, device=dev)
    pi = torch.empty(nblk, dtype=torch.int32, device=dev)
    kernels.lm_head(x, W, logits=logits, part_max=pv, part_idx=pi, idx_offset=5000)
    torch.cuda.synchronize()
    ref = _ref_logits(x, W)
    scale = ref.abs().max()
    err = (logits.float() - ref).abs()
    assert torch.all(err <= ref.abs() * 2.0**-8 + 1e-5 * scale), float((err / scale).max())
    l0 = logits[0].float()
    for b in range(nblk):
        blk = l0[b * 128:(b + 1) * 128]
        assert pv[b].item() == blk.max().item()
        first = int((blk == blk.max()).nonzero()[0])  # lowest index on ties
        assert pi[b].item() == 5000 + b * 128 + first


def test_ragged_k_is_refused(kernels):
    """A ring slot is 64 values of K: other K are refused on the host, nothing is launched."""
    x = torch.ones(1, 96, dtype=torch.bfloat16, device="cuda")
    W = torch.ones(128, 96, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="code -1"):
        kernels.lm_head(x, W, logits=torch.empty(1, 128, dtype=torch.bfloat16, device="cuda"))
    assert kernels.device_status() == 0


def test_argmax_only_and_ties(kernels):
    """No logits buffer; all-equal logits: the lowest index wins in every block."""
    dev = torch.device("cuda")
    V, K = 300, 64
    x = torch.ones(1, K, dtype=torch.bfloat16, device=dev)
    W = torch.ones(V, K, dtype=torch.bfloat16, device=dev)
    nblk = kernels.lm_head_blocks(V)
    pv = torch.empty(nblk, dtype=torch.float32, device=dev)
    pi = torch.empty(nblk, dtype=torch.int32, device=dev)
    kernels.lm_head(x, W, logits=None, part_max=pv, part_idx=pi)
    torch.cuda.synchronize()
    assert pv.tolist() == [64.0] * nblk
    assert pi.tolist() == [0, 128, 256]


def test_final_norm_prologue_matches_two_kernels(kernels):
    """add + RMSNorm folded into the projection against ns_rmsnorm followed by the plain projection."""
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(9)
    V, K = 2000, 1024
    x = torch.randn(1, K, device=dev, generator=gen).to(torch.bfloat16)
    r = torch.randn(1, K, device=dev, generator=gen).to(torch.bfloat16)
    wn = (1 + 0.1 * torch.randn(K, device=dev, generator=gen)).to(torch.bfloat16)
    W = (torch.randn(V, K, device=dev, generator=gen) * 0.05).to(torch.bfloat16)
    fused = torch.empty(1, V, dtype=torch.bfloat16, device=dev)
    kernels.lm_head(x, W, logits=fused, r=r, wn=wn, eps=1e-6)
    h = kernels.rmsnorm(x.clone(), r, wn, 1e-6)
    plain = torch.empty(1, V, dtype=torch.bfloat16, device=dev)
    kernels.lm_head(h, W, logits=plain)
    torch.cuda.synchronize()
    # the two paths round the norm's sum of squares in different orders: a normalised value may differ by one bf16 ulp
    scale = plain.float().abs().max()
    assert (fused.float() - plain.float()).abs().max() <= 2e-2 * scale


def test_greedy_pick_over_rank_partials(kernels):
    """The pick over the (value, index) pairs of several vocabulary slices equals argmax over the whole row, and the
    device-side state advances as b2_greedy_next advances it."""
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(3)
    V, K, H, P = 1024, 256, 64, 4
    x = torch.randn(1, K, device=dev, generator=gen).to(torch.bfloat16)
    W = (torch.randn(V, K, device=dev, generator=gen) * 0.05).to(torch.bfloat16)
    embed = torch.randn(V, H, device=dev, generator=gen).to(torch.bfloat16)
    vl = V // P
    nblk = kernels.lm_head_blocks(vl)
    pv = torch.empty(P, nblk, dtype=torch.float32, device=dev)
    pi = torch.empty(P, nblk, dtype=torch.int32, device=dev)
    full = torch.empty(1, V, dtype=torch.bfloat16, device=dev)
    for rnk in range(P):
        kernels.lm_head(x, W[rnk * vl:(rnk + 1) * vl], logits=full[:, rnk * vl:(rnk + 1) * vl].contiguous(),
                        part_max=pv[rnk], part_idx=pi[rnk], idx_offset=rnk * vl)
    kernels.lm_head(x, W, logits=full)
    pos = torch.tensor([7], dtype=torch.int32, device=dev)
    step = torch.tensor([2], dtype=torch.int32, device=dev)
    toks = torch.zeros(8, dtype=torch.int64, device=dev)
    xn = torch.zeros(1, H, dtype=torch.bfloat16, device=dev)
    rc = kernels.lib.b2_greedy_pick(pv.data_ptr(), pi.data_ptr(), P * nblk, V, embed.data_ptr(), H, pos.data_ptr(),
                                    toks.data_ptr(), step.data_ptr(), xn.data_ptr(),
                                    ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    l = full[0].float()
    want = int((l == l.max()).nonzero()[0])
    assert toks[2].item() == want and pos.item() == 8 and step.item() == 3
    assert torch.equal(xn[0], embed[want])


def test_error_codes_launch_nothing(kernels):
    lib = kernels.lib
    t = torch.zeros(4096, dtype=torch.bfloat16, device="cuda")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = t.data_ptr()
    assert lib.b2_lm_head(p, p, p, 9, 64, 64, 0, None, None, 0.0, None, None, None, 0, st) == -2
    assert lib.b2_lm_head(p, p, p, 1, 64, 48, 0, None, None, 0.0, None, None, None, 0, st) == -1
    assert lib.b2_lm_head(p + 2, p, p, 1, 64, 64, 0, None, None, 0.0, None, None, None, 0, st) == -4
    assert lib.b2_lm_head(p, p, p, 1, 64, 64, 0, None, None, 0.0, None, p, None, 0, st) == -4
    assert lib.b2_lm_head(p, p, p, 1, 64, 64, 1, None, None, 0.0, None, None, None, 0, st) == -4
