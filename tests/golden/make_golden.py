"""Captures outputs of the REFERENCE library on a GPU and writes them as golden fixtures.

Run on a CUDA box where oracle/_ref/libnanoserve_ref.so exists (built from the reference checkout by
`make -C oracle ref`; the built file travels with the repository snapshot, the checkout does not):

    python tests/golden/make_golden.py [out_dir]

Each .npz holds the inputs as raw bit patterns (bf16 as uint16, packed words as uint32), the reference
library's ns_w4_quantize / ns_w4_linear outputs, and a JSON `meta` string with the shape and the
tolerance tests/test_oracle.py applies (GEMV: one bf16 rounding of an fp32 sum; GEMM: the reference
rounds every dequantised weight to bf16 first, kernels/quant/w4a16.cuh:196-197, so 1e-2 of the largest
output, its own gate).  Only shapes the reference serves are used: M in {1,2,4,8} or M % 128 == 0 with
N % 128 == 0 (csrc/nanoserve_ops.cu:82-88).
"""
import ctypes
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402
from tests.util import bits_to_torch, torch_to_bits, torch_to_u32, u32_to_torch  # noqa: E402


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <output directory>")
    out_dir = sys.argv[1]
    os.makedirs(out_dir, exist_ok=True)
    ref = ctypes.CDLL(oracle.REF_LIB_PATH)
    vp, i32 = ctypes.c_void_p, ctypes.c_int
    ref.ns_w4_quantize.argtypes = [vp, vp, vp, i32, i32, i32, vp]
    ref.ns_w4_quantize.restype = i32
    ref.ns_w4_linear.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, vp]
    ref.ns_w4_linear.restype = i32
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def linear(x, wq, s, M, N, K, G):
        y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        rc = ref.ns_w4_linear(x.data_ptr(), wq.data_ptr(), s.data_ptr(), y.data_ptr(), M, N, K, G, st)
        assert rc == 0, rc
        torch.cuda.synchronize()
        return torch_to_bits(y)

    # 1. the reference's own correctness case (bench/bench_w4a16.cu:142-191): hash-filled W and X,
    #    device quantizer, GEMV M = 1, 8 and GEMM M = 128
    N, K, G = 256, 512, 128
    W = oracle.fill_bf16(N * K, 11, 0.05).reshape(N, K)
    w = bits_to_torch(W)
    wq = torch.empty(N, K // 8, dtype=torch.int32, device="cuda")
    s = torch.empty(N, K // G, dtype=torch.bfloat16, device="cuda")
    assert ref.ns_w4_quantize(w.data_ptr(), wq.data_ptr(), s.data_ptr(), N, K, G, st) == 0
    torch.cuda.synchronize()
    for M in (1, 8, 128):
        X = oracle.fill_bf16(M * K, 12, 1.0).reshape(M, K)
        Y = linear(bits_to_torch(X), wq, s, M, N, K, G)
        meta = {"case": "reference bench [1]", "M": M, "N": N, "K": K, "G": G,
                "tol": 2.0**-8, "slack": 1e-5 if M < 128 else 1e-2}
        np.savez_compressed(os.path.join(out_dir, f"refbench_m{M}.npz"), W=W, X=X, Wq=torch_to_u32(wq),
                            S=torch_to_bits(s), Y_ref=Y, meta=json.dumps(meta))

    # 2. synthetic inputs with the benchmark's distributions, small shapes
    for (M, N, K, G) in [(1, 512, 1024, 128), (2, 96, 2048, 128), (4, 40, 512, 64), (8, 256, 3584, 128),
                         (128, 128, 256, 32)]:
        X, Wq, S = oracle.synth_inputs(M, N, K, G, seed=17)
        Y = linear(bits_to_torch(X), u32_to_torch(Wq), bits_to_torch(S), M, N, K, G)
        meta = {"case": "synthetic", "M": M, "N": N, "K": K, "G": G, "tol": 2.0**-8,
                "slack": 1e-5 if M < 128 else 1e-2}
        np.savez_compressed(os.path.join(out_dir, f"synth_m{M}_n{N}_k{K}_g{G}.npz"), X=X, Wq=Wq, S=S,
                            Y_ref=Y, meta=json.dumps(meta))
    print("wrote", sorted(os.listdir(out_dir)))


if __name__ == "__main__":
    main()
