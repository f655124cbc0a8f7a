"""GPU test of b2_w4_gemv_noalloc, the GEMV entry point that allocates nothing.

It exists for hosts that cannot call cudaMalloc where they call the GEMV (a process whose device memory is
all handed to a pool at start-up, a plugin inside another runtime's capture region): its split-K scratch is
a fixed array in the library's device image.  The test calls it through the C ABI twice in a row -- the second
call finds the array as the first left it -- and compares with ns_w4_linear on the same inputs, on shapes
that do split K (so the scratch is really used) and one that does not.  This file sorts last on purpose:
a run that stops at the first failure has then already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from tests.util import bits_to_torch, check_bf16_output, torch_to_bits, u32_to_torch

pytestmark = pytest.mark.gpu


def _call(lib, name, x, wq, s, M, N, K, G, y=None):
    if y is None:
        y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    rc = getattr(lib, name)(x.data_ptr(), wq.data_ptr(), s.data_ptr(), y.data_ptr(), M, N, K, G,
                            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, (name, rc)
    return y


@pytest.mark.parametrize("M,N,K", [(4, 512, 3584), (1, 64, 3584), (16, 448, 18944), (1, 2368, 3584)])
def test_matches_existing_entry_point_twice_in_a_row(kernels, M, N, K):
    G = 128
    lib = kernels.lib
    X, Wq, S = oracle.synth_inputs(M, N, K, G, seed=77)
    x, wq, s = bits_to_torch(X), u32_to_torch(Wq), bits_to_torch(S)
    want = _call(lib, "ns_w4_linear", x, wq, s, M, N, K, G)
    # outputs allocated up front and one untimed call made (kernel images load on first use), so that the free
    # device memory can be compared across the two calls proper: the entry point itself must not allocate
    out1, out2 = torch.empty_like(want), torch.empty_like(want)
    _call(lib, "b2_w4_gemv_noalloc", x, wq, s, M, N, K, G, y=out1)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    first = _call(lib, "b2_w4_gemv_noalloc", x, wq, s, M, N, K, G, y=out1)
    second = _call(lib, "b2_w4_gemv_noalloc", x, wq, s, M, N, K, G, y=out2)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before, "device memory was allocated or freed during the calls"
    assert lib.b2_device_status() == 0  # reads the fixed array's own status word, without allocating either
    assert torch.cuda.mem_get_info()[0] == free_before
    a = want.float()
    for got in (first, second):
        b = got.float()
        # the tolerance of the other GEMV tests: one bf16 ulp of the value plus fp32 summation-order noise
        tol = torch.maximum(a.abs(), b.abs()) * 2.0**-7 + 1e-5 * a.abs().max()
        assert torch.all((a - b).abs() <= tol)
    assert torch.equal(first, second), "the second call saw state left by the first"
    check_bf16_output(torch_to_bits(second), oracle.w4_linear_f32(X, Wq, S, G, threads=oracle.max_threads()), 2e-5)


def test_rejects_sizes_beyond_the_fixed_scratch(kernels):
    lib = kernels.lib
    t = torch.zeros(4096, dtype=torch.int32, device="cuda")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = t.data_ptr()
    # M * N > 2^20 outputs, and N > 131072 rows: refused before anything is launched
    assert lib.b2_w4_gemv_noalloc(p, p, p, p, 16, 70000, 128, 128, st) == -6
    assert lib.b2_w4_gemv_noalloc(p, p, p, p, 1, 131073 + 31, 128, 128, st) == -6
    assert lib.b2_w4_gemv_noalloc(p, p, p, p, 17, 64, 128, 128, st) == -2
    assert lib.b2_w4_gemv_noalloc(p, p, p, p, 1, 64, 128, 96, st) == -1
