"""The reference's own Python binding (python/nanoserve/ops.py of the reference checkout) against this library.

The checkout's location comes from the environment variable NANOSERVE_REFERENCE_ROOT; without it the tests are
skipped (a GPU box does not carry the checkout).  The CPU test constructs the reference's ``Kernels`` class on
build/libnanoserve.so unchanged -- its constructor resolves the six ``ns_*`` symbols and sets their signatures -- and
the GPU test runs ``w4_quantize`` + ``w4_linear`` through it and compares with the CPU oracle.
"""
import importlib.util
import os

import numpy as np
import pytest


def _reference_ops():
    root = os.environ.get("NANOSERVE_REFERENCE_ROOT")
    if not root:
        pytest.skip("NANOSERVE_REFERENCE_ROOT is not set")
    path = os.path.join(root, "python", "nanoserve", "ops.py")
    if not os.path.exists(path):
        pytest.skip(f"{path} not found")
    spec = importlib.util.spec_from_file_location("reference_nanoserve_ops", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_kernels_class_loads_this_library(lib_path):
    ops = _reference_ops()
    k = ops.Kernels(lib_path)  # AttributeError here if a symbol of the reference ABI were missing
    for name in ("ns_rmsnorm", "ns_rope", "ns_swiglu", "ns_flash_fwd", "ns_w4_quantize", "ns_w4_linear"):
        assert getattr(k.lib, name).restype is not None


@pytest.mark.gpu
def test_reference_kernels_class_runs_the_quantized_linear(lib_path):
    import torch
    import oracle
    from tests.util import bits_to_torch, check_bf16_output, torch_to_bits, torch_to_u32
    ops = _reference_ops()
    k = ops.Kernels(lib_path)
    G = 128
    W = oracle.fill_bf16(256 * 512, 11, 0.05).reshape(256, 512)
    Wq, S = k.w4_quantize(bits_to_torch(W), G)
    Wq_o, S_o = oracle.w4_quantize(W, G)
    torch.cuda.synchronize()
    assert np.array_equal(torch_to_u32(Wq), Wq_o) and np.array_equal(torch_to_bits(S), S_o)
    for M in (1, 8, 128):  # what the reference's own library serves: its wrapper pads other M to these
        X = oracle.synth_inputs(M, 256, 512, G, seed=3)[0]
        y = k.w4_linear(bits_to_torch(X), Wq, S, G)
        torch.cuda.synchronize()
        check_bf16_output(torch_to_bits(y), oracle.w4_linear_f32(X, Wq_o, S_o, G), 2e-5 if M <= 16 else 1e-2)
