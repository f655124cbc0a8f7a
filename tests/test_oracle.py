"""CPU tests of the oracle itself: it must reproduce the reference's known answers before it is trusted.

Citations are paths inside the reference project.
"""
import json
import os

import numpy as np
import pytest

import oracle

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _ref_case():
    # bench/bench_w4a16.cu:142-155: N=256, K=512, G=128; W = fill(seed 11, scale 0.05), X = fill(seed 12, 1)
    N, K, M, G = 256, 512, 128, 128
    W = oracle.fill_bf16(N * K, 11, 0.05).reshape(N, K)
    X = oracle.fill_bf16(M * K, 12, 1.0).reshape(M, K)
    return N, K, M, G, W, X


def test_known_answer_quantization_error():
    """results/ncu/w4_gemv_m8.txt:11 records 7.05 % for bench_w4a16.cu:192-196 on the seeded inputs."""
    N, K, M, G, W, X = _ref_case()
    Wq, S = oracle.w4_quantize(W, G)
    Y = oracle.w4_linear_f32(X, Wq, S, G)
    Yd = oracle.dense_linear_f32(X, W)
    pct = 100.0 * oracle.rel_fro(Y, Yd)
    assert f"{pct:.2f}" == "7.05", pct


def test_fill_generator_properties():
    # bench_w4a16.cu:32-40: u in [-1,1) scaled by 1.732*scale, rounded to bf16
    v = oracle.bf16_bits_to_f32(oracle.fill_bf16(1 << 16, 12, 1.0))
    assert np.abs(v).max() <= 1.7344  # bf16(1.732) rounds up to 1.734375
    assert abs(v.mean()) < 0.02 and abs(v.std() - 1.0) < 0.02  # uniform on [-sqrt3, sqrt3) has unit variance
    # element 0, seed 0: h = 0 -> u = -1 -> bf16(-1.732)
    assert oracle.fill_bf16(1, 0, 1.0)[0] == oracle.f32_to_bf16_bits(np.float32(-1.732))[()]


def test_c_and_numpy_quantizer_agree_bitwise():
    N, K, M, G, W, X = _ref_case()
    for g in (32, 64, 128, 256):
        a = oracle.w4_quantize(W, g)
        b = oracle.np_quantize(W, g)
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_quantizer_edge_cases():
    G = 32
    W = np.zeros((2, 64), dtype=np.uint16)  # all-zero groups: scale 1.0, q = 8 (w4a16.cuh:288)
    Wq, S = oracle.w4_quantize(W, G)
    assert np.all(S == 0x3F80) and np.all(Wq == 0x88888888)
    # extremes clamp to [0, 15]: +max -> 7+8 = 15, -max -> -7+8 = 1
    vals = np.zeros((1, 32), dtype=np.float32)
    vals[0, 0], vals[0, 1], vals[0, 2] = 7.0, -7.0, 3.5  # 3.5/1.0 ties-to-even -> 4
    Wq, S = oracle.w4_quantize(oracle.f32_to_bf16_bits(vals), G)
    assert S[0, 0] == 0x3F80
    q = oracle.w4_unpack(Wq)[0]
    assert q[0] == 7 and q[1] == -7 and q[2] == 4 and np.all(q[3:] == 0)
    with pytest.raises(ValueError):  # csrc/nanoserve_ops.cu:67: K % G or G % 32 -> -1
        oracle.w4_quantize(np.zeros((1, 96), dtype=np.uint16), 64)
    with pytest.raises(ValueError):
        oracle.w4_quantize(np.zeros((1, 48), dtype=np.uint16), 48)


def test_nibble_order():
    # w4a16.cuh:6: value k = 8j+i sits in bits 4i..4i+3 of word j
    Wq = np.array([[0x76543210, 0xFEDCBA98]], dtype=np.uint32)
    assert list(oracle.w4_unpack(Wq)[0]) == [i - 8 for i in range(16)]
    assert np.array_equal(oracle.np_unpack(Wq)[0], np.arange(16) - 8)


def test_c_linear_matches_numpy_twin():
    for (M, N, K, G) in [(1, 64, 256, 128), (3, 40, 384, 64), (16, 33, 512, 32), (5, 7, 128, 128)]:
        X, Wq, S = oracle.synth_inputs(M, N, K, G, seed=5)
        Y = oracle.w4_linear_f32(X, Wq, S, G)
        Yn = oracle.np_linear_f64(X, Wq, S, G)
        assert np.abs(Y - Yn).max() <= 2e-7 * np.abs(Yn).max() + 1e-12
        assert np.array_equal(oracle.w4_dequant(Wq, S, G), oracle.np_dequant(Wq, S, G))
        Y8 = oracle.w4_linear_f32(X, Wq, S, G, threads=4)
        assert np.array_equal(Y, Y8)


def test_dequant_bf16_is_single_rounding():
    X, Wq, S = oracle.synth_inputs(1, 16, 256, 128, seed=1)
    a = oracle.w4_dequant_bf16(Wq, S, 128)
    b = oracle.f32_to_bf16_bits(oracle.w4_dequant(Wq, S, 128))
    assert np.array_equal(a, b)


def test_linearity_property():
    # the path is linear in X: f(a) + f(b) == f applied to rows stacked, and f(2x) == 2 f(x) exactly
    X, Wq, S = oracle.synth_inputs(2, 48, 256, 128, seed=9)
    Y = oracle.w4_linear_f32(X, Wq, S, 128)
    X2 = oracle.f32_to_bf16_bits(2.0 * oracle.bf16_bits_to_f32(X))
    Y2 = oracle.w4_linear_f32(X2, Wq, S, 128)
    assert np.array_equal(Y2, 2.0 * Y)


def _golden_files():
    return sorted(f for f in os.listdir(GOLDEN) if f.endswith(".npz")) if os.path.isdir(GOLDEN) else []


@pytest.mark.parametrize("name", _golden_files())
def test_oracle_against_reference_kernel_outputs(name):
    """Fixtures captured from the reference's own library (ns_w4_quantize / ns_w4_linear built unchanged
    for sm_100a) on a B200 by tests/golden/make_golden.py."""
    z = np.load(os.path.join(GOLDEN, name))
    meta = json.loads(str(z["meta"]))
    G = meta["G"]
    if "W" in z:
        Wq, S = oracle.w4_quantize(z["W"], G)
        assert np.array_equal(Wq, z["Wq"]), "quantizer words differ from the reference kernel"
        assert np.array_equal(S, z["S"]), "quantizer scales differ from the reference kernel"
    Yo = oracle.w4_linear_f32(z["X"], z["Wq"], z["S"], G)
    scale = np.abs(Yo).max()
    y_ref = oracle.bf16_bits_to_f32(z["Y_ref"])
    # reference output = fp32 accumulation rounded once to bf16: half an ulp plus accumulation noise
    tol = meta.get("tol", 2.0**-8)
    assert np.all(np.abs(y_ref - Yo) <= np.abs(Yo) * tol + meta.get("slack", 1e-5) * scale), name
