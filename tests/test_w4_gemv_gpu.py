"""GPU parity tests of the decode GEMV (M <= 16) through the C ABI, against the CPU oracle.

Three kernels serve the GEMV.  The streaming kernel (default for one token, and up to four on tall matrices, when
G % 128 == 0 and K % 256 == 0; every M <= 16 with FLAG_STREAM_KERNEL) carries X as block fixed point per (token,
128-chunk): 32 bits for one and two tokens, 15 bits plus sign above.  The many-token kernel (five to sixteen tokens, two
to four on a long K; its own tests are in test_w4_gemv_mid_gpu.py) and the ring kernel (everything else, or
FLAG_RING_KERNEL) carry it as 16-bit block fixed point (ring kernel: 24 bits with FLAG_WIDE_X, or, with FLAG_FLOAT_X,
in fp16 on the floating-point mma).

Integer work (the int4 unpack) must be bit-exact.  Floating-point outputs are bf16: the bound is one correct
rounding (2^-8 relative) plus slack relative to the largest output:
3e-6 for one token on the default path (32-bit fixed point: fp32 summation order is all that is left), on any input;
2e-5 for the 15/16-bit forms on N(0,1) inputs (each element is off by at most 2^-15 / 2^-16 of its chunk's largest
magnitude; measured 1e-5 / 3e-6), 5e-4 on heavy-tailed inputs (a 1000x outlier sets its chunk's exponent);
3e-6 with FLAG_WIDE_X (24-bit fixed point) and with FLAG_FLOAT_X (X in fp16 on the floating-point mma),
2e-4 with FLAG_FLOAT_X | FLAG_FOLD_ZERO_POINT (fp32 cancellation of the +1024 bias of the fp16 unpack),
2e-3 for G < 128 where each weight is rounded to bf16 as the reference's tensor-core path does.
"""
import ctypes
import os

import numpy as np
import pytest
import torch

import oracle
from nanoserve_b200 import ops
from tests.util import bits_to_torch, check_bf16_output, torch_to_bits, u32_to_torch

pytestmark = pytest.mark.gpu

SLACK_DEFAULT, SLACK_EXACT, SLACK_FOLD, SLACK_SMALL_G, SLACK_HEAVY = 2e-5, 3e-6, 2e-4, 2e-3, 5e-4
FLOAT_FOLD = ops.FLAG_FLOAT_X | ops.FLAG_FOLD_ZERO_POINT
RING, STREAM = ops.FLAG_RING_KERNEL, ops.FLAG_STREAM_KERNEL


def run(k, X, Wq, S, G, flags=0):
    y = k.w4_linear(bits_to_torch(X), u32_to_torch(Wq), bits_to_torch(S), G, flags=flags)
    torch.cuda.synchronize()
    return torch_to_bits(y)


def slack_for(G, flags):
    if G % 128:
        return SLACK_SMALL_G
    if flags & ops.FLAG_FLOAT_X:
        return SLACK_FOLD if flags & ops.FLAG_FOLD_ZERO_POINT else SLACK_EXACT
    return SLACK_EXACT if (flags & ops.FLAG_WIDE_X) and (flags & RING) else SLACK_DEFAULT


@pytest.mark.parametrize("flags", [0, STREAM, RING, RING | ops.FLAG_WIDE_X, ops.FLAG_FLOAT_X, FLOAT_FOLD,
                                   RING | ops.FLAG_NARROW_CTA, RING | ops.FLAG_PRE_STAGE_X, RING | ops.FLAG_NO_PRE_STAGE_X,
                                   RING | ops.FLAG_PRE_STAGE_X | ops.FLAG_WIDE_X])
@pytest.mark.parametrize("G", [128, 32])
def test_unpack_is_bit_exact(kernels, flags, G):
    """S == 1 and one-hot X rows make Y[m, n] = q[n, k_m] - 8: every nibble value in every in-word
    position, in the first and last word of a group and of a row, must come back as that integer."""
    N, K = 48, 256
    rng = np.random.default_rng(7)
    Wq = rng.integers(0, 2**32, size=(N, K // 8), dtype=np.uint32)
    for v in range(16):  # rows 0..15: constant nibble v everywhere
        Wq[v, :] = np.uint32(v * 0x11111111)
    Wq[16, :] = 0x76543210  # ascending nibbles in every word
    Wq[17, :] = 0xFEDCBA98
    S = np.full((N, K // G), 0x3F80, dtype=np.uint16)
    Q = oracle.w4_unpack(Wq)  # [N, K] int8
    for k0 in range(0, K, 16):
        X = np.zeros((16, K), dtype=np.float32)
        X[np.arange(16), k0 + np.arange(16)] = 1.0
        y = oracle.bf16_bits_to_f32(run(kernels, oracle.f32_to_bf16_bits(X), Wq, S, G, flags))
        want = Q[:, k0:k0 + 16].T.astype(np.float32)
        assert np.array_equal(y, want), (k0, flags, G)
    # M = 1 goes through the other kernel variant
    for k0 in (0, 7, 127, 128, 255):
        X = np.zeros((1, K), dtype=np.float32)
        X[0, k0] = 1.0
        y = oracle.bf16_bits_to_f32(run(kernels, oracle.f32_to_bf16_bits(X), Wq, S, G, flags))
        assert np.array_equal(y[0], Q[:, k0].astype(np.float32))
    assert kernels.device_status() == 0


SMALL_SHAPES = [(64, 128, 128), (96, 256, 128), (100, 384, 128), (33, 1024, 128), (1, 128, 128), (1, 256, 128),
                (31, 256, 256), (257, 512, 128), (130, 768, 256), (17, 1024, 512), (64, 32, 32), (40, 160, 32),
                (72, 192, 64), (50, 96, 96)]


@pytest.mark.parametrize("N,K,G", SMALL_SHAPES)
@pytest.mark.parametrize("flags", [0, STREAM, STREAM | ops.FLAG_NO_PDL, RING, RING | ops.FLAG_WIDE_X, ops.FLAG_FLOAT_X,
                                   FLOAT_FOLD, RING | ops.FLAG_NO_PDL, RING | ops.FLAG_PRE_STAGE_X,
                                   RING | ops.FLAG_NO_PRE_STAGE_X, RING | ops.FLAG_PRE_STAGE_X | ops.FLAG_WIDE_X,
                                   RING | ops.FLAG_PRE_STAGE_X | ops.FLAG_NO_PDL, RING | ops.FLAG_SPLIT_SUM_KERNEL,
                                   RING | ops.FLAG_SPLIT_SUM_KERNEL | ops.FLAG_NO_AUTOTUNE | ops.FLAG_PRE_STAGE_X])
def test_small_shapes_all_m(kernels, N, K, G, flags):
    for M in range(1, 17):
        X, Wq, S = oracle.synth_inputs(M, N, K, G, seed=11)
        ref = oracle.w4_linear_f32(X, Wq, S, G)
        y = run(kernels, X, Wq, S, G, flags)
        check_bf16_output(y, ref, slack_for(G, flags))
    assert kernels.device_status() == 0


# the linears of a Qwen2.5-7B-shaped layer, their 8-way tensor-parallel shards, and a 70B-class shape
LAYER_SHAPES = [(3584, 3584), (512, 3584), (18944, 3584), (3584, 18944), (448, 3584), (64, 3584),
                (2368, 3584), (448, 18944), (1024, 8192)]


@pytest.mark.parametrize("N,K", LAYER_SHAPES)
@pytest.mark.parametrize("M", [1, 2, 4, 8, 16])
def test_layer_shapes(kernels, N, K, M):
    G = 128
    X, Wq, S = oracle.synth_inputs(M, N, K, G, seed=3)
    ref = oracle.w4_linear_f32(X, Wq, S, G, threads=oracle.max_threads())
    for flags in (0, STREAM, RING, RING | ops.FLAG_WIDE_X, ops.FLAG_FLOAT_X, FLOAT_FOLD):
        y = run(kernels, X, Wq, S, G, flags)
        _, rel = check_bf16_output(y, ref, SLACK_EXACT if (M == 1 and flags in (0, STREAM)) else slack_for(G, flags))
        assert rel < 1e-2  # the reference's own gate (bench/bench_w4a16.cu:120,174-180)
    assert kernels.device_status() == 0


@pytest.mark.parametrize("N,K", [(3584, 18944), (512, 3584), (18944, 3584)])
def test_split_k_matches_single_pass_and_is_deterministic(kernels, N, K):
    G, M = 128, 4
    X, Wq, S = oracle.synth_inputs(M, N, K, G, seed=21)
    ref = oracle.w4_linear_f32(X, Wq, S, G, threads=oracle.max_threads())
    a = run(kernels, X, Wq, S, G, 0)
    b = run(kernels, X, Wq, S, G, 0)
    c = run(kernels, X, Wq, S, G, ops.FLAG_NO_SPLIT_K)
    assert np.array_equal(a, b), "two identical launches differ: the K reduction is not deterministic"
    check_bf16_output(a, ref, SLACK_DEFAULT)
    check_bf16_output(c, ref, SLACK_DEFAULT)
    # the slices added up by the last CTA to arrive or by the kernel behind: same order, same bits (split pinned)
    pin = RING | ops.FLAG_NO_AUTOTUNE | (4 << 24)
    d = run(kernels, X, Wq, S, G, pin | ops.FLAG_NO_SPLIT_SUM_KERNEL)
    for _ in range(2):
        e = run(kernels, X, Wq, S, G, pin | ops.FLAG_SPLIT_SUM_KERNEL)
        assert np.array_equal(d, e)
    check_bf16_output(d, ref, SLACK_DEFAULT)
    assert kernels.device_status() == 0


@pytest.mark.parametrize("N,K", [(96, 4096), (512, 3584), (18944, 3584), (100, 384)])  # K that fits one CTA unsplit
@pytest.mark.parametrize("M", [1, 3, 8, 16])
def test_x_staged_in_front_gives_the_same_bits(kernels, N, K, M):
    """The kernel in front of the GEMV writes the bytes a CTA would have produced itself: with the CTA shape and the
    K split pinned, the outputs are bit-identical, launch after launch (the staging area is reused)."""
    G = 128
    pin = RING | ops.FLAG_NO_SPLIT_K | (4 << 4) | 0x800  # ring kernel, 8 consumer warps, one chunk per warp and stage
    for wide in (0, ops.FLAG_WIDE_X):
        if wide and M * K * 3 > 150000:
            continue  # three bytes per value of X: the unsplit K no longer fits one CTA's shared memory
        X, Wq, S = oracle.synth_inputs(M, N, K, G, seed=31)
        a = run(kernels, X, Wq, S, G, pin | wide | ops.FLAG_NO_PRE_STAGE_X)
        for _ in range(3):
            b = run(kernels, X, Wq, S, G, pin | wide | ops.FLAG_PRE_STAGE_X)
            assert np.array_equal(a, b)
        X2, _, _ = oracle.synth_inputs(M, N, K, G, seed=32)  # another X through the same staging area
        a2 = run(kernels, X2, Wq, S, G, pin | wide | ops.FLAG_NO_PRE_STAGE_X)
        assert np.array_equal(a2, run(kernels, X2, Wq, S, G, pin | wide | ops.FLAG_PRE_STAGE_X))
    assert kernels.device_status() == 0


def test_scaling_x_by_two_is_exact(kernels):
    """Linearity at full size: doubling X doubles every partial sum exactly, so outputs double bit for bit."""
    M, N, K, G = 2, 18944, 3584, 128
    X, Wq, S = oracle.synth_inputs(M, N, K, G, seed=4)
    X2 = oracle.f32_to_bf16_bits(2.0 * oracle.bf16_bits_to_f32(X))
    y1 = oracle.bf16_bits_to_f32(run(kernels, X, Wq, S, G))
    y2 = oracle.bf16_bits_to_f32(run(kernels, X2, Wq, S, G))
    assert np.array_equal(y2, 2.0 * y1)


def test_row_permutation_equivariance(kernels):
    """Permuting the rows of (Wq, S) permutes the output columns and changes nothing else."""
    M, N, K, G = 3, 3584, 3584, 128
    X, Wq, S = oracle.synth_inputs(M, N, K, G, seed=6)
    perm = np.random.default_rng(0).permutation(N)
    y = run(kernels, X, Wq, S, G)
    yp = run(kernels, X, Wq[perm], S[perm], G)
    assert np.array_equal(yp, y[:, perm])


def test_output_is_fully_overwritten_and_nothing_else(kernels):
    M, N, K, G = 5, 100, 384, 128
    X, Wq, S = oracle.synth_inputs(M, N, K, G, seed=8)
    buf = torch.full((M * N + 64,), 7.0, dtype=torch.bfloat16, device="cuda")
    out = buf[32:32 + M * N].view(M, N)
    kernels.w4_linear(bits_to_torch(X), u32_to_torch(Wq), bits_to_torch(S), G, out=out)
    torch.cuda.synchronize()
    assert torch.all(buf[:32] == 7.0) and torch.all(buf[32 + M * N:] == 7.0)
    check_bf16_output(torch_to_bits(out), oracle.w4_linear_f32(X, Wq, S, G), SLACK_EXACT)


def _heavy_tailed(M, K, kind, seed):
    """bf16 bit patterns of X for the adversarial cases: planted outliers, a chunk of denormals, SwiGLU-shaped values."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K)).astype(np.float32)
    if kind == "outliers":
        x[:, 5] *= 1000.0
        x[:, K // 2 + 3] *= 300.0
        x[:, K - 1] *= -1000.0
    elif kind == "denormal_chunk":
        x[:, 128:256] = 1e-39 * rng.standard_normal((M, 128)).astype(np.float32)
        x[:, 256:384] = 0.0
    elif kind == "swiglu":
        g, u = rng.standard_normal((M, K)).astype(np.float32) * 3, rng.standard_normal((M, K)).astype(np.float32) * 3
        x = g / (1 + np.exp(-g)) * u
    return oracle.f32_to_bf16_bits(x)


@pytest.mark.parametrize("kind", ["outliers", "denormal_chunk", "swiglu"])
@pytest.mark.parametrize("M", [1, 2, 4, 8, 16])
def test_heavy_tailed_activations(kernels, M, kind):
    """The fixed-point forms of X depend on the dynamic range inside a 128-chunk.  One token (32-bit form) stays at
    fp32-summation accuracy on any input; the 15/16-bit forms are bounded by 5e-4 of the largest output with 1000x
    outliers planted (2^-15 of the outlier per element of its chunk) and with SwiGLU-shaped products, which are
    heavy-tailed by themselves."""
    N, K, G = 1024, 2048, 128
    _, Wq, S = oracle.synth_inputs(M, N, K, G, seed=41)
    X = _heavy_tailed(M, K, kind, 43)
    ref = oracle.w4_linear_f32(X, Wq, S, G, threads=oracle.max_threads())
    for flags in (0, STREAM, RING):
        y = run(kernels, X, Wq, S, G, flags)
        exact = M == 1 and flags in (0, STREAM)
        check_bf16_output(y, ref, SLACK_EXACT if exact else (SLACK_DEFAULT if kind == "denormal_chunk" else SLACK_HEAVY))
    assert kernels.device_status() == 0


@pytest.mark.parametrize("flags", [0, STREAM, RING])
def test_inf_and_nan_poison_their_outputs_only(kernels, flags):
    """A chunk of X that holds an inf or a nan makes that token's outputs nan (its fixed-point form is meaningless);
    the other tokens are untouched."""
    M, N, K, G = 3, 256, 512, 128
    X, Wq, S = oracle.synth_inputs(M, N, K, G, seed=47)
    ref = oracle.w4_linear_f32(X, Wq, S, G)
    Xb = X.copy()
    Xb[0, 130] = 0x7F80  # +inf
    Xb[2, 300] = 0x7FC0  # nan
    y = oracle.bf16_bits_to_f32(run(kernels, Xb, Wq, S, G, flags))
    assert np.all(np.isnan(y[0])) and np.all(np.isnan(y[2]))
    check_bf16_output(oracle.f32_to_bf16_bits(y[1:2]), ref[1:2], SLACK_DEFAULT)


# the 70B-class linears at full size: rows sampled for the oracle (the whole matrix is 117 MB of nibbles)
@pytest.mark.parametrize("N,K", [(28672, 8192), (8192, 28672)])
@pytest.mark.parametrize("M", [1, 16])
def test_70b_class_shapes_sampled_rows(kernels, N, K, M):
    G = 128
    X, Wq, S = oracle.synth_inputs(M, N, K, G, seed=5)
    y = run(kernels, X, Wq, S, G)
    rows = np.unique(np.concatenate([np.arange(0, 48), np.arange(N - 48, N),
                                     np.random.default_rng(1).integers(0, N, 160)]))
    ref = oracle.w4_linear_f32(X, Wq[rows], S[rows], G, threads=oracle.max_threads())
    check_bf16_output(y[:, rows], ref, SLACK_EXACT if M == 1 else SLACK_DEFAULT)
    assert kernels.device_status() == 0


# one-token launches whose plan departs from one warp per row tile and a whole K: twice the warps per tile where the CTAs
# leave SMs idle (16384 x 4096, 28672 x 4096 with 32 rows per warp, 8192 x 8192), K slices across CTAs for a long K with
# few rows (3584 x 18944, 5120 x 13824), even shares of the tiles (20000 x 4096)
@pytest.mark.parametrize("N,K,what", [(16384, 4096, "2 warp(s) per row tile"), (28672, 4096, "2 warp(s) per row tile"),
                                      (8192, 8192, "4 warp(s) per row tile"), (3584, 18944, "K slices across CTAs 10 (sum kernel)"),
                                      (5120, 13824, "K slices across CTAs"), (20000, 4096, "shared evenly"),
                                      (14200, 1024, "2 warp(s) per row tile")])
def test_one_token_plans_sampled_rows(kernels, N, K, what):
    G = 128
    assert what in kernels.gemv_describe(1, N, K, G, 0), kernels.gemv_describe(1, N, K, G, 0)
    X, Wq, S = oracle.synth_inputs(1, N, K, G, seed=N % 89)
    y = run(kernels, X, Wq, S, G)
    rows = np.unique(np.concatenate([np.arange(0, 64), np.arange(N - 64, N),
                                     np.random.default_rng(2).integers(0, N, 512)]))
    ref = oracle.w4_linear_f32(X, Wq[rows], S[rows], G, threads=oracle.max_threads())
    check_bf16_output(y[:, rows], ref, SLACK_EXACT)
    assert np.array_equal(y, run(kernels, X, Wq, S, G)), "two identical launches differ"
    # K slices added up by the last CTA of a row group instead of the kernel behind: the same sums in the same order
    assert np.array_equal(y, run(kernels, X, Wq, S, G, ops.FLAG_NO_SPLIT_SUM_KERNEL))
    assert np.array_equal(y, run(kernels, X, Wq, S, G, ops.FLAG_NO_SPLIT_SUM_KERNEL))
    assert kernels.device_status() == 0


def test_random_large_shapes_one_token_property(kernels):
    """Random row counts from a few to tens of thousands and K = 256 j at one token: whatever plan the library picks
    (warps per row tile, K slices across CTAs, even tile shares, rows per warp), sampled rows agree with the oracle to
    the one-token bound and two launches agree bit for bit."""
    from hypothesis import given, settings, strategies as st_

    @settings(max_examples=30, deadline=None, derandomize=True)
    @given(N=st_.integers(300, 60000), j=st_.sampled_from([1, 2, 3, 4, 7, 8, 14, 16, 20, 32, 54, 74]),
           seed=st_.integers(0, 1000))
    def prop(N, j, seed):
        K, G = 256 * j, 128
        if N * K > 300 << 20:
            N = (300 << 20) // K
        X, Wq, S = oracle.synth_inputs(1, N, K, G, seed=seed)
        y = run(kernels, X, Wq, S, G)
        rows = np.unique(np.concatenate([np.arange(0, min(N, 40)), np.arange(max(0, N - 40), N),
                                         np.random.default_rng(seed).integers(0, N, 256)]))
        ref = oracle.w4_linear_f32(X, Wq[rows], S[rows], G, threads=oracle.max_threads())
        check_bf16_output(y[:, rows], ref, SLACK_EXACT)
        assert np.array_equal(y, run(kernels, X, Wq, S, G))

    prop()
    assert kernels.device_status() == 0


def test_random_shapes_property(kernels):
    """Property test over random M, ragged N >= 16 (the slack is relative to the largest output), K = G j, G in {32, 64, 128, 256}, every kernel choice: the bf16 output is
    within one rounding plus the path's slack of the oracle."""
    from hypothesis import given, settings, strategies as st_

    @settings(max_examples=40, deadline=None, derandomize=True)
    @given(M=st_.integers(1, 16), N=st_.integers(16, 300), G=st_.sampled_from([32, 64, 128, 256]), j=st_.integers(1, 10),
           which=st_.sampled_from([0, STREAM, RING]), seed=st_.integers(0, 1000))
    def prop(M, N, G, j, which, seed):
        K = G * j
        X, Wq, S = oracle.synth_inputs(M, N, K, G, seed=seed)
        ref = oracle.w4_linear_f32(X, Wq, S, G)
        # G < 128: every weight is rounded to bf16 first (as on the reference's tensor-core path); with few rows the
        # largest output is a small yardstick, so the reference's own gate (1e-2, bench/bench_w4a16.cu:120) applies
        check_bf16_output(run(kernels, X, Wq, S, G, which), ref, 1e-2 if G % 128 else slack_for(G, which))

    prop()
    assert kernels.device_status() == 0


def test_error_codes(kernels):
    lib = kernels.lib
    x = torch.zeros(1, 256, dtype=torch.bfloat16, device="cuda")
    wq = torch.zeros(8, 32, dtype=torch.int32, device="cuda")
    s = torch.ones(8, 2, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(1, 8, dtype=torch.bfloat16, device="cuda")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    P = lambda t: t.data_ptr()
    assert lib.ns_w4_linear(P(x), P(wq), P(s), P(y), 1, 8, 256, 128, st) == 0
    assert lib.ns_w4_linear(P(x), P(wq), P(s), P(y), 0, 8, 256, 128, st) == -2   # reference: -2, nanoserve_ops.cu:86-88
    assert lib.ns_w4_linear(P(x), P(wq), P(s), P(y), 1, 8, 256, 96, st) == -1    # K % G
    assert lib.ns_w4_linear(P(x), P(wq), P(s), P(y), 1, 8, 256, 16, st) == -1    # G % 32
    assert lib.ns_w4_linear(P(x), P(wq), P(s), P(y), 1, 8, 40, 8, st) == -1      # K % 32
    assert lib.ns_w4_linear(None, P(wq), P(s), P(y), 1, 8, 256, 128, st) == -4
    assert lib.ns_w4_linear(P(x) + 2, P(wq), P(s), P(y), 1, 8, 256, 128, st) == -4
    with pytest.raises(RuntimeError, match="ns_w4_linear failed with code -1"):
        kernels.w4_linear(x, wq, s, 96)
    torch.cuda.synchronize()
    assert kernels.device_status() == 0


def _ref_lib():
    path = oracle.REF_LIB_PATH
    if not os.path.exists(path):
        pytest.skip("reference library not built (oracle/_ref/libnanoserve_ref.so)")
    lib = ctypes.CDLL(path)
    vp, i32 = ctypes.c_void_p, ctypes.c_int
    lib.ns_w4_linear.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, vp]
    lib.ns_w4_linear.restype = i32
    return lib


@pytest.mark.parametrize("N,K", [(18944, 3584), (3584, 18944), (512, 3584)])
@pytest.mark.parametrize("M", [1, 2, 4, 8])
def test_against_reference_kernels(kernels, N, K, M):
    """Same inputs through the reference's own GEMV (kernels/quant/w4a16.cuh:42-115, built unchanged for
    sm_100a): both round an fp32 sum once to bf16, so they agree to one bf16 ulp, and almost always exactly."""
    ref = _ref_lib()
    G = 128
    X, Wq, S = oracle.synth_inputs(M, N, K, G, seed=13)
    x, wq, s = bits_to_torch(X), u32_to_torch(Wq), bits_to_torch(S)
    y_ref = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    rc = ref.ns_w4_linear(x.data_ptr(), wq.data_ptr(), s.data_ptr(), y_ref.data_ptr(), M, N, K, G,
                          ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    y = kernels.w4_linear(x, wq, s, G)
    torch.cuda.synchronize()
    a, b = y.float(), y_ref.float()
    # one bf16 ulp of the value, plus fp32 summation-order noise relative to the largest output
    # (outputs near zero come from cancellation and carry the absolute error of the large terms)
    tol = torch.maximum(a.abs(), b.abs()) * 2.0**-7 + 1e-5 * b.abs().max()
    assert torch.all((a - b).abs() <= tol)
    assert (a != b).float().mean().item() < 0.02


def test_cluster_shared_staging_in_a_child_process():
    """B2_GEMV_CLUSTER is read once per process, so the cluster variant of the streaming kernel (CTAs of a cluster
    convert X in turns and write into each other's shared memory) is exercised in a child: same outputs as the
    plain variant, bit for bit, on a shape with several conversion rounds and on a ragged one."""
    import os
    import subprocess
    import sys
    code = r'''
import sys, torch
sys.path.insert(0, %r)
from nanoserve_b200.ops import Kernels, FLAG_STREAM_KERNEL
k = Kernels(); k.init()
g = torch.Generator(device="cuda").manual_seed(7)
out = []
for M, N, K in [(1, 3584, 18944), (8, 4000, 3584), (3, 72, 1024)]:
    Wq = torch.randint(-2**31, 2**31 - 1, (N, K // 8), dtype=torch.int32, device="cuda", generator=g)
    S = (0.005 + (torch.randn(N, K // 128, device="cuda", generator=g) * 0.01).abs()).to(torch.bfloat16)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    y = k.w4_linear(x, Wq, S, 128, flags=FLAG_STREAM_KERNEL)
    torch.cuda.synchronize()
    out.append(y.view(torch.int16).cpu())
assert k.device_status() == 0
torch.save(out, sys.argv[1])
''' % os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    import tempfile
    res = {}
    with tempfile.TemporaryDirectory() as tmp:
        for c in ("1", "4", "2"):
            path = os.path.join(tmp, f"y{c}.pt")
            env = dict(os.environ, B2_GEMV_CLUSTER=c)
            subprocess.run([sys.executable, "-c", code, path], check=True, env=env, timeout=600)
            res[c] = torch.load(path)
    for c in ("4", "2"):
        for a, b in zip(res["1"], res[c]):
            assert torch.equal(a, b)


@pytest.mark.parametrize("N,K", [(20000, 512), (22000, 1024), (19700, 256), (45000, 8192)])
def test_row_counts_between_one_and_two_ctas_per_sm(kernels, N, K):
    """Row counts for which the streaming kernel launches whole waves of CTAs and gives each its even share of the row
    tiles (some warps of a CTA idle): every row must still be computed exactly once -- against the oracle, all rows."""
    G = 128
    X, Wq, S = oracle.synth_inputs(1, N, K, G, seed=N % 97)
    y = kernels.w4_linear(bits_to_torch(X), u32_to_torch(Wq), bits_to_torch(S), G)
    torch.cuda.synchronize()
    check_bf16_output(torch_to_bits(y), oracle.w4_linear_f32(X, Wq, S, G, threads=oracle.max_threads()), 3e-6)
    assert kernels.device_status() == 0
