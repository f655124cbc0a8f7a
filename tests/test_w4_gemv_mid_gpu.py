"""GPU parity tests of the many-token decode GEMV (2 <= M <= 16 -- by default from five tokens, from two where K is
long --, G == 128, K % 256 == 0; plain launches), through the C ABI, against the CPU oracle.

The kernel carries X as 16-bit block fixed point per (token, 128-chunk), like the ring kernel: the int4 unpack must be
bit-exact; bf16 outputs are within one correct rounding plus 2e-5 of the largest output on N(0,1) inputs (each element
is off by at most 2^-16 of its chunk's largest magnitude) and 5e-4 on heavy-tailed ones.  A CTA cuts its rows x K into sixteen equal runs, one per warp,
so tiles are shared between warps in every possible way as N and K vary: the shapes below cover runs shorter than a
tile, longer than several tiles, ragged last tiles and CTAs with unequal tile counts.
"""
import numpy as np
import pytest
import torch

import oracle
from nanoserve_b200 import ops
from tests.util import bits_to_torch, check_bf16_output, torch_to_bits, u32_to_torch

pytestmark = pytest.mark.gpu

SLACK_DEFAULT, SLACK_HEAVY = 2e-5, 5e-4


def run(k, X, Wq, S, G=128, flags=0):
    if not flags & ops.FLAG_NO_MID_KERNEL:
        flags |= ops.FLAG_MID_KERNEL
    y = k.w4_linear(bits_to_torch(X), u32_to_torch(Wq), bits_to_torch(S), G, flags=flags)
    torch.cuda.synchronize()
    return torch_to_bits(y)


def served(k, M, N, K, flags=ops.FLAG_MID_KERNEL):
    return k.gemv_describe(M, N, K, 128, flags).startswith("many-token kernel")


def test_dispatch(kernels):
    assert served(kernels, 8, 18944, 3584) and served(kernels, 16, 18944, 3584) and served(kernels, 5, 2368, 256)
    assert served(kernels, 8, 28672, 8192, 0) and served(kernels, 16, 18944, 3584, 0) and served(kernels, 9, 37888, 3584, 0)
    assert served(kernels, 8, 37888, 3584, 0) and served(kernels, 5, 3584, 3584, 0)
    assert not served(kernels, 4, 18944, 3584, 0)
    plan = kernels.gemv_describe(8, 512, 3584, 128, 0)  # few rows: K in slices that fill the SMs
    assert plan.startswith("many-token kernel") and "K slices across CTAs 4 (sum kernel)" in plan
    assert served(kernels, 2, 3584, 18944, 0) and served(kernels, 4, 28672, 8192, 0) and not served(kernels, 1, 3584, 18944)
    plan = kernels.gemv_describe(16, 3584, 18944, 128, 0)  # the converted X fits in slices of K only
    assert plan.startswith("many-token kernel") and "K slices across CTAs 5 (sum kernel)" in plan
    assert "K slices across CTAs 1," in kernels.gemv_describe(16, 18944, 3584, 128, 0)
    assert not served(kernels, 16, 3584, 18944, ops.FLAG_MID_KERNEL | ops.FLAG_NO_SPLIT_K)
    assert not kernels.gemv_describe(8, 18944, 3584, 128, ops.FLAG_NO_MID_KERNEL).startswith("many-token")


def test_unpack_is_bit_exact(kernels):
    """S == 1 and one-hot X rows make Y[m, n] = q[n, k_m] - 8: every nibble value in every in-word position."""
    N, K = 2400, 512
    rng = np.random.default_rng(7)
    Wq = rng.integers(0, 2**32, size=(N, K // 8), dtype=np.uint32)
    for v in range(16):
        Wq[v, :] = np.uint32(v * 0x11111111)
    Wq[16, :] = 0x76543210
    Wq[17, :] = 0xFEDCBA98
    S = np.full((N, K // 128), 0x3F80, dtype=np.uint16)
    Q = oracle.w4_unpack(Wq)
    assert served(kernels, 16, N, K)
    for k0 in range(0, K, 16):
        X = np.zeros((16, K), dtype=np.float32)
        X[np.arange(16), k0 + np.arange(16)] = 1.0
        y = oracle.bf16_bits_to_f32(run(kernels, oracle.f32_to_bf16_bits(X), Wq, S))
        assert np.array_equal(y, Q[:, k0:k0 + 16].T.astype(np.float32)), k0
    assert kernels.device_status() == 0


@pytest.mark.parametrize("N,K", [(2368, 256), (2399, 256), (2400, 512), (5000, 768), (9001, 256), (40000, 256),
                                 (3000, 3584), (7777, 1024), (2368, 8192), (1, 256), (17, 512), (100, 3584), (513, 1024),
                                 (64, 18944), (1184, 3584)])
def test_every_token_count(kernels, N, K):
    for M in range(2, 17):
        if not served(kernels, M, N, K):
            assert K == 8192 and M > 8
            continue
        X, Wq, S = oracle.synth_inputs(M, N, K, 128, seed=M + N % 13)
        ref = oracle.w4_linear_f32(X, Wq, S, 128, threads=oracle.max_threads())
        a = run(kernels, X, Wq, S)
        check_bf16_output(a, ref, SLACK_DEFAULT)
        assert np.array_equal(a, run(kernels, X, Wq, S)), "two identical launches differ"
        assert np.array_equal(a, run(kernels, X, Wq, S, flags=ops.FLAG_NO_PDL))
    assert kernels.device_status() == 0


@pytest.mark.parametrize("rows", [16, 32])
@pytest.mark.parametrize("N,K", [(2368, 512), (4736, 256), (4750, 1024), (9001, 768), (20000, 256), (6000, 3584)])
def test_both_tile_heights(kernels, rows, N, K):
    """Tiles of 16 and of 32 rows (two row blocks share the B fragments; twelve warps instead of sixteen above eight
    tokens), forced: the default takes 32 where every SM gets a tile and the rings fit."""
    force = (rows // 16) << 10
    for M in (5, 8, 9, 13, 16):
        plan = kernels.gemv_describe(M, N, K, 128, ops.FLAG_MID_KERNEL | force)
        if not plan.startswith("many-token kernel"):
            continue  # (32-row slots of twelve warps do not fit beside sixteen tokens of a long K)
        assert f"tiles of {rows} rows" in plan
        X, Wq, S = oracle.synth_inputs(M, N, K, 128, seed=M + rows)
        ref = oracle.w4_linear_f32(X, Wq, S, 128, threads=oracle.max_threads())
        a = run(kernels, X, Wq, S, flags=force)
        check_bf16_output(a, ref, SLACK_DEFAULT)
        assert np.array_equal(a, run(kernels, X, Wq, S, flags=force))
    assert kernels.device_status() == 0


@pytest.mark.parametrize("N,K,slices", [(2400, 2048, 2), (2400, 2048, 4), (3000, 1792, 3), (5000, 768, 3),
                                        (3584, 18944, 0), (2399, 18944, 0)])
def test_k_slices_across_ctas(kernels, N, K, slices):
    """K cut into slices across CTAs (fp32 partial sums, added in slice order by the kernel behind): forced on short
    K, chosen by the plan where the converted X of the whole K does not fit in shared memory."""
    force = slices << 24
    for M in (5, 8, 11, 16):
        plan = kernels.gemv_describe(M, N, K, 128, ops.FLAG_MID_KERNEL | force)
        assert plan.startswith("many-token kernel"), plan
        if slices:
            assert f"K slices across CTAs {slices} " in plan
        else:
            assert "(sum kernel)" in plan
        X, Wq, S = oracle.synth_inputs(M, N, K, 128, seed=M + slices)
        ref = oracle.w4_linear_f32(X, Wq, S, 128, threads=oracle.max_threads())
        a = run(kernels, X, Wq, S, flags=force)
        check_bf16_output(a, ref, SLACK_DEFAULT)
        assert np.array_equal(a, run(kernels, X, Wq, S, flags=force)), "two identical launches differ"
    assert kernels.device_status() == 0


@pytest.mark.parametrize("depth", [2, 3, 6])
def test_ring_depths(kernels, depth):
    M, N, K = 12, 4000, 2048
    X, Wq, S = oracle.synth_inputs(M, N, K, 128, seed=5)
    ref = oracle.w4_linear_f32(X, Wq, S, 128, threads=oracle.max_threads())
    check_bf16_output(run(kernels, X, Wq, S, flags=depth << 4), ref, SLACK_DEFAULT)
    assert kernels.device_status() == 0


@pytest.mark.parametrize("M", [8, 16])
@pytest.mark.parametrize("N,K", [(18944, 3584), (28672, 8192)])
def test_benchmark_shapes_sampled_rows(kernels, M, N, K):
    """Full benchmark shapes: every output of 4096 sampled rows against the oracle, and linearity on all of them."""
    if not served(kernels, M, N, K):
        pytest.skip("not served at this token count")
    X, Wq, S = oracle.synth_inputs(M, N, K, 128, seed=17)
    y = run(kernels, X, Wq, S)
    rows = np.sort(np.random.default_rng(1).choice(N, size=4096, replace=False))
    rows[:32] = np.arange(32)
    rows[-32:] = np.arange(N - 32, N)
    ref = oracle.w4_linear_f32(X, Wq[rows], S[rows], 128, threads=oracle.max_threads())
    check_bf16_output(y[:, rows], ref, SLACK_DEFAULT)
    # doubling X doubles Y bit for bit (block fixed point: the digits do not change, the exponent does)
    X2 = oracle.f32_to_bf16_bits(2.0 * oracle.bf16_bits_to_f32(X))
    y2 = run(kernels, X2, Wq, S)
    assert np.array_equal(oracle.bf16_bits_to_f32(y2), 2.0 * oracle.bf16_bits_to_f32(y))
    assert kernels.device_status() == 0


def test_heavy_tailed_and_nan(kernels):
    M, N, K = 9, 3000, 1024
    X, Wq, S = oracle.synth_inputs(M, N, K, 128, seed=23)
    x = oracle.bf16_bits_to_f32(X)
    rng = np.random.default_rng(3)
    idx = rng.choice(x.size, size=40, replace=False)
    x.reshape(-1)[idx] *= 1000.0
    Xh = oracle.f32_to_bf16_bits(x)
    ref = oracle.w4_linear_f32(Xh, Wq, S, 128, threads=oracle.max_threads())
    check_bf16_output(run(kernels, Xh, Wq, S), ref, SLACK_HEAVY)
    x[4, 300] = np.nan
    x[7, 5] = np.inf
    y = oracle.bf16_bits_to_f32(run(kernels, oracle.f32_to_bf16_bits(x), Wq, S))
    assert np.isnan(y[4]).all() and np.isnan(y[7]).all()
    ok = [m for m in range(M) if m not in (4, 7)]
    assert np.isfinite(y[ok]).all()
    check_bf16_output(oracle.f32_to_bf16_bits(y[ok]), ref[ok], SLACK_HEAVY)
    assert kernels.device_status() == 0


def test_agrees_with_the_ring_kernel(kernels):
    M, N, K = 16, 18944, 3584
    X, Wq, S = oracle.synth_inputs(M, N, K, 128, seed=29)
    a = oracle.bf16_bits_to_f32(run(kernels, X, Wq, S))
    b = oracle.bf16_bits_to_f32(run(kernels, X, Wq, S, flags=ops.FLAG_NO_MID_KERNEL))
    scale = np.abs(b).max()
    assert np.abs(a - b).max() <= 2 ** -7 * scale


def test_random_shapes_property(kernels):
    """Property test over random token counts, ragged row counts from one row to a few thousand, K = 256 j, forced K
    slices, ring depths and both tile heights: the bf16 output is within one rounding plus 2e-5 of the largest output of
    the oracle, and two launches agree bit for bit."""
    from hypothesis import given, settings, strategies as st_

    @settings(max_examples=60, deadline=None, derandomize=True)
    @given(M=st_.integers(2, 16), N=st_.one_of(st_.integers(1, 400), st_.integers(2300, 5200)), j=st_.integers(1, 12),
           slices=st_.sampled_from([0, 0, 2, 3]), depth=st_.sampled_from([0, 2, 4]), rows=st_.sampled_from([0, 0, 1, 2]),
           seed=st_.integers(0, 1000))
    def prop(M, N, j, slices, depth, rows, seed):
        K = 256 * j
        flags = ops.FLAG_MID_KERNEL | (slices << 24) | (depth << 4) | (rows << 10)
        if not kernels.gemv_describe(M, N, K, 128, flags).startswith("many-token kernel"):
            return  # (a forced combination that does not fit, e.g. more slices than super-chunks)
        X, Wq, S = oracle.synth_inputs(M, N, K, 128, seed=seed)
        ref = oracle.w4_linear_f32(X, Wq, S, 128, threads=oracle.max_threads())
        a = run(kernels, X, Wq, S, flags=flags)
        # few rows make the largest output a small yardstick: the reference's own gate (1e-2) below 64 rows
        check_bf16_output(a, ref, SLACK_DEFAULT if N >= 64 else 1e-2)
        assert np.array_equal(a, run(kernels, X, Wq, S, flags=flags))

    prop()
    assert kernels.device_status() == 0
