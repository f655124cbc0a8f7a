"""Seeded synthetic inputs with the shapes and value distributions the benchmark configurations name.

X: bf16 from N(0,1).  Weights: iid uniform 4-bit nibbles packed 8 per uint32 along K (value k = 8j+i in bits
4i..4i+3 of word j).  Scales: bf16 of 0.005 + |N(0, 0.01)| per (row, group).  The zero-point is the constant 8.
Everything is returned as raw bit patterns in numpy arrays (bf16 as uint16, packed words as uint32).
"""
import numpy as np

# name -> (N out features, K in features) of one Qwen2.5-7B-shaped decoder layer
QWEN25_7B_LAYER = {
    "q": (3584, 3584), "k": (512, 3584), "v": (512, 3584), "o": (3584, 3584),
    "gate": (18944, 3584), "up": (18944, 3584), "down": (3584, 18944),
}
# 70B-class shapes: hidden 8192, intermediate 28672
CLASS_70B_LAYER = {
    "q": (8192, 8192), "k": (1024, 8192), "v": (1024, 8192), "o": (8192, 8192),
    "gate": (28672, 8192), "up": (28672, 8192), "down": (8192, 28672),
}


def f32_to_bf16_bits(x):
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[(u & 0x7FFFFFFF) > 0x7F800000] = 0x7FFF
    return r


def synth_x(M, K, seed=0):
    rng = np.random.default_rng([seed, 1, M, K])
    return f32_to_bf16_bits(rng.standard_normal((M, K), dtype=np.float32))


def synth_weight(N, K, G=128, seed=0):
    rng = np.random.default_rng([seed, 2, N, K, G])
    Wq = rng.integers(0, 2**32, size=(N, K // 8), dtype=np.uint32)
    S = f32_to_bf16_bits((0.005 + np.abs(rng.normal(0.0, 0.01, size=(N, K // G)))).astype(np.float32))
    return Wq, S


def synth_inputs(M, N, K, G=128, seed=0):
    """(X [M,K] u16, Wq [N,K/8] u32, S [N,K/G] u16)."""
    Wq, S = synth_weight(N, K, G, seed)
    return synth_x(M, K, seed), Wq, S


def gemv_bytes(M, N, K, G=128):
    """Algorithmic bytes of one linear: packed weights + scales + X + bf16 Y (the reference's byte model,
    bench/bench_w4a16.cu:239, with the 2-byte output the C ABI writes)."""
    return N * K // 2 + N * (K // G) * 2 + M * K * 2 + M * N * 2


def shard_rows(N, rank, world):
    """Row range [lo, hi) of an N-row matrix owned by `rank` of `world` (contiguous, sizes differ by <= 1)."""
    lo = (N * rank) // world
    hi = (N * (rank + 1)) // world
    return lo, hi
