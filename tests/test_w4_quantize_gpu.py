"""GPU parity tests of the quantizer through the C ABI: bit-exact against the CPU oracle."""
import ctypes
import os

import numpy as np
import pytest
import torch

import oracle
from tests.util import bits_to_torch, torch_to_bits, torch_to_u32

pytestmark = pytest.mark.gpu


def quant(k, W_bits, G):
    Wq, S = k.w4_quantize(bits_to_torch(W_bits), G)
    torch.cuda.synchronize()
    return torch_to_u32(Wq), torch_to_bits(S)


@pytest.mark.parametrize("N,K,G", [(256, 512, 128), (64, 256, 32), (33, 384, 64), (8, 1024, 256), (5, 96, 96),
                                   (3584, 3584, 128)])
def test_bit_exact_against_oracle(kernels, N, K, G):
    rng = np.random.default_rng([N, K, G])
    cases = {
        "reference fill (bench_w4a16.cu:32-40, seed 11)": oracle.fill_bf16(N * K, 11, 0.05).reshape(N, K),
        "normal": oracle.f32_to_bf16_bits(rng.standard_normal((N, K), dtype=np.float32) * 0.02),
        "wide dynamic range": oracle.f32_to_bf16_bits(
            (rng.standard_normal((N, K)) * np.exp(rng.uniform(-20, 20, size=(N, 1)))).astype(np.float32)),
    }
    z = cases["normal"].copy()
    z[0, :G] = 0          # an all-zero group: scale 1, q = 8
    z[-1, -G:] = 0x8000   # negative zeros
    cases["zero groups"] = z
    for name, W in cases.items():
        Wq, S = quant(kernels, W, G)
        Wq_o, S_o = oracle.w4_quantize(W, G)
        assert np.array_equal(S, S_o), name
        assert np.array_equal(Wq, Wq_o), name


def test_ties_round_to_even(kernels):
    G = 32
    vals = np.zeros((1, 32), dtype=np.float32)
    vals[0, :8] = [7.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 3.5]
    Wq, S = quant(kernels, oracle.f32_to_bf16_bits(vals), G)
    q = oracle.w4_unpack(Wq)[0][:8]
    assert list(q) == [7, 0, 2, 2, 0, -2, -2, 4]


def test_error_codes(kernels):
    W = torch.zeros(4, 96, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="ns_w4_quantize failed with code -1"):
        kernels.w4_quantize(W, 64)   # K % G  (csrc/nanoserve_ops.cu:67)
    with pytest.raises(RuntimeError, match="ns_w4_quantize failed with code -1"):
        kernels.w4_quantize(W, 48)   # G % 32


def test_round_trip_then_linear_matches_oracle(kernels):
    """quantize -> linear on the GPU equals quantize -> linear in the oracle (the reference's own check,
    bench/bench_w4a16.cu:142-180, on its own seeded inputs)."""
    from tests.util import check_bf16_output, u32_to_torch
    N, K, G = 256, 512, 128
    W = oracle.fill_bf16(N * K, 11, 0.05).reshape(N, K)
    Wq, S = kernels.w4_quantize(bits_to_torch(W), G)
    for M in (1, 8, 16):
        X = oracle.fill_bf16(M * K, 12, 1.0).reshape(M, K)
        y = kernels.w4_linear(bits_to_torch(X), Wq, S, G)
        torch.cuda.synchronize()
        ref = oracle.w4_linear_f32(X, torch_to_u32(Wq), torch_to_bits(S), G)
        check_bf16_output(torch_to_bits(y), ref, 3e-6)


def test_against_reference_quantizer(kernels):
    path = oracle.REF_LIB_PATH
    if not os.path.exists(path):
        pytest.skip("reference library not built (oracle/_ref/libnanoserve_ref.so)")
    ref = ctypes.CDLL(path)
    vp, i32 = ctypes.c_void_p, ctypes.c_int
    ref.ns_w4_quantize.argtypes = [vp, vp, vp, i32, i32, i32, vp]
    ref.ns_w4_quantize.restype = i32
    N, K, G = 1024, 3584, 128
    W = bits_to_torch(oracle.fill_bf16(N * K, 11, 0.05).reshape(N, K))
    Wq_r = torch.empty(N, K // 8, dtype=torch.int32, device="cuda")
    S_r = torch.empty(N, K // G, dtype=torch.bfloat16, device="cuda")
    assert ref.ns_w4_quantize(W.data_ptr(), Wq_r.data_ptr(), S_r.data_ptr(), N, K, G,
                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    Wq, S = kernels.w4_quantize(W, G)
    torch.cuda.synchronize()
    assert torch.equal(Wq, Wq_r) and torch.equal(S.view(torch.int16), S_r.view(torch.int16))
