"""The calibrated (GPTQ) quantizer: same packed format as the reference's round-to-nearest quantizer, lower output error.

CPU tests: the PyTorch restatement of round-to-nearest against the oracle (bit-exact), GPTQ with uncorrelated inputs ==
round-to-nearest (bit-exact: nothing to spread), GPTQ with correlated inputs beats round-to-nearest on the layer's
outputs, every stored value lies on the int4 grid of its group, the container round trip.  A GPU test runs the
calibrated weights through ns_w4_linear.
"""
import numpy as np
import pytest
import torch

import oracle
from nanoserve_b200 import calibrate, weights_io


def _weights(N, K, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)


def _correlated_inputs(T, K, seed, rank=24, samples=0):
    """Activations with a few dominant directions and a handful of large channels, like a transformer's.  `seed` fixes
    the directions (the layer's input distribution), `samples` the draws from it."""
    basis = torch.randn(rank, K, generator=torch.Generator().manual_seed(seed))
    g = torch.Generator().manual_seed(1000 + samples)
    x = torch.randn(T, rank, generator=g) @ basis + 0.3 * torch.randn(T, K, generator=g)
    x[:, ::97] *= 8.0
    return x.to(torch.bfloat16)


def _bits(t):
    return t.view(torch.int16).numpy().view(np.uint16)


@pytest.mark.parametrize("N,K,G", [(48, 256, 128), (33, 384, 64), (16, 512, 32), (7, 1024, 256)])
def test_round_to_nearest_matches_the_oracle(N, K, G):
    W = _weights(N, K, seed=K + G)
    W[0, :G] = 0  # an all-zero group: scale 1
    Wq, S = calibrate.rtn_quantize(W, G)
    Wq_o, S_o = oracle.np_quantize(_bits(W), G)
    assert np.array_equal(Wq.numpy().view(np.uint32), Wq_o)
    assert np.array_equal(_bits(S), S_o)


@pytest.mark.parametrize("N,K,G", [(40, 512, 128), (24, 384, 64)])
def test_uncorrelated_inputs_give_round_to_nearest(N, K, G):
    W = _weights(N, K, seed=3)
    H = torch.diag(torch.rand(K, generator=torch.Generator().manual_seed(1)) + 0.5)
    Wq, S = calibrate.gptq_quantize(W, H, G)
    Wq_r, S_r = calibrate.rtn_quantize(W, G)
    assert torch.equal(Wq, Wq_r) and torch.equal(S.view(torch.int16), S_r.view(torch.int16))


@pytest.mark.parametrize("N,K,G,block", [(96, 512, 128, 128), (64, 768, 128, 256), (48, 512, 64, 128)])
def test_correlated_inputs_beat_round_to_nearest(N, K, G, block):
    W = _weights(N, K, seed=11)
    X = _correlated_inputs(2048, K, seed=5)
    X_held_out = _correlated_inputs(1024, K, seed=5, samples=1)  # the same distribution, other draws
    Wq, S = calibrate.gptq_quantize(W, calibrate.hessian(X), G, block=block)
    Wq_r, S_r = calibrate.rtn_quantize(W, G)
    e_gptq, e_rtn = calibrate.output_error(W, Wq, S, X, G), calibrate.output_error(W, Wq_r, S_r, X, G)
    assert e_gptq < 0.8 * e_rtn, (e_gptq, e_rtn)
    h_gptq, h_rtn = calibrate.output_error(W, Wq, S, X_held_out, G), calibrate.output_error(W, Wq_r, S_r, X_held_out, G)
    assert h_gptq < 0.9 * h_rtn, (h_gptq, h_rtn)
    # the format: the oracle's unpack sees nibbles, and dequantised values sit on the group's grid
    deq = oracle.np_dequant(Wq.numpy().view(np.uint32), _bits(S), G)
    assert np.array_equal(deq, calibrate.dequantize(Wq, S, G).numpy())


def test_dead_input_channels_and_container_round_trip(tmp_path):
    N, K, G = 32, 256, 128
    W = _weights(N, K, seed=2)
    X = _correlated_inputs(512, K, seed=9)
    X[:, 5] = 0  # a channel that never fires: its weights are free and must not break the factorisation
    packed = calibrate.quantize_linears({"a": W, "b": W}, inputs={"a": X}, group=G)
    assert packed["a"][0].dtype == np.uint32 and packed["a"][1].dtype == np.uint16
    Wq_r, S_r = calibrate.rtn_quantize(W, G)  # "b" had no inputs: round to nearest
    assert np.array_equal(packed["b"][0], Wq_r.numpy().view(np.uint32)) and np.array_equal(packed["b"][1], _bits(S_r))
    path = str(tmp_path / "w.nsw4")
    weights_io.save(path, packed, meta={"quantizer": "gptq"})
    pw = weights_io.PackedWeights(path, verify=True)
    wq, s, g = pw.linear("a")
    assert g == G and np.array_equal(np.asarray(wq), packed["a"][0]) and np.array_equal(np.asarray(s), packed["a"][1])
    assert pw.meta["quantizer"] == "gptq"


@pytest.mark.gpu
def test_calibrated_weights_run_through_the_kernels(kernels):
    from tests.util import check_bf16_output, torch_to_bits
    N, K, G = 4608, 1024, 128
    W = _weights(N, K, seed=21).cuda()
    X = _correlated_inputs(4096, K, seed=6).cuda()
    Wq, S = calibrate.gptq_quantize(W, calibrate.hessian(X), G)
    Wq_r, S_r = calibrate.rtn_quantize(W, G)
    assert calibrate.output_error(W, Wq, S, X, G) < 0.8 * calibrate.output_error(W, Wq_r, S_r, X, G)
    for M in (1, 8):
        x = X[:M].contiguous()
        y = kernels.w4_linear(x, Wq, S, G)
        torch.cuda.synchronize()
        ref = oracle.w4_linear_f32(torch_to_bits(x), Wq.cpu().numpy().view(np.uint32), _bits(S.cpu()), G,
                                   threads=oracle.max_threads())
        check_bf16_output(torch_to_bits(y), ref, 5e-4)  # (heavy-tailed inputs: the large channels)
    assert kernels.device_status() == 0
