"""CPU oracle for the W4A16 quantized-linear path -- TEST INFRASTRUCTURE, not product code.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of ``bench.py``
may import this package.  It wraps ``oracle/w4_oracle.c`` (a plain-C restatement of the reference's
host check, quantizer and input generator; each C function cites the reference lines it follows) and
offers a numpy twin used to cross-check the C code.

Parity status: pinned -- see the header of ``w4_oracle.c`` and ``tests/test_oracle.py``.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libw4oracle.so")
REF_LIB_PATH = os.path.join(_HERE, "_ref", "libnanoserve_ref.so")
_lib = None


def build(with_ref: bool = False, ref_root: str = "") -> None:
    """Compile the C oracle and, if asked, the reference's own library from the checkout at `ref_root` (or at
    NANOSERVE_REFERENCE_ROOT in the environment)."""
    subprocess.check_call(["make", "-s", "-C", _HERE])
    if with_ref:
        root = ref_root or os.environ.get("NANOSERVE_REFERENCE_ROOT", "")
        if not root:
            raise RuntimeError("the reference checkout's location is not given (NANOSERVE_REFERENCE_ROOT)")
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref", f"REF_ROOT={root}"])


def lib():
    global _lib
    if _lib is None:
        src = os.path.join(_HERE, "w4_oracle.c")
        if not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        vp, i32, f32, sz, u32 = (ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t,
                                 ctypes.c_uint32)
        L.orc_fill_bf16.argtypes = [vp, sz, u32, f32]
        L.orc_fill_bf16.restype = None
        L.orc_w4_quantize.argtypes = [vp, vp, vp, i32, i32, i32]
        L.orc_w4_quantize.restype = i32
        L.orc_w4_dequant.argtypes = [vp, vp, i32, i32, i32, vp]
        L.orc_w4_dequant.restype = None
        L.orc_w4_dequant_bf16.argtypes = [vp, vp, i32, i32, i32, vp]
        L.orc_w4_dequant_bf16.restype = None
        L.orc_w4_unpack.argtypes = [vp, i32, i32, vp]
        L.orc_w4_unpack.restype = None
        L.orc_w4_linear_f32.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i32]
        L.orc_w4_linear_f32.restype = i32
        L.orc_w4_linear_bf16.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i32]
        L.orc_w4_linear_bf16.restype = i32
        L.orc_dense_linear_f32.argtypes = [vp, vp, vp, i32, i32, i32]
        L.orc_dense_linear_f32.restype = None
        L.orc_max_rel_err.argtypes = [vp, vp, sz]
        L.orc_max_rel_err.restype = f32
        L.orc_rel_fro.argtypes = [vp, vp, sz]
        L.orc_rel_fro.restype = f32
        L.orc_max_threads.argtypes = []
        L.orc_max_threads.restype = i32
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype):
    a = np.ascontiguousarray(a)
    assert a.dtype == dtype, (a.dtype, dtype)
    return a


# ------------------------------------------------------------------ bf16 helpers (numpy, uint16 bits)
def f32_to_bf16_bits(x):
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r[nan] = 0x7FFF
    return r


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ------------------------------------------------------------------ C oracle wrappers
def fill_bf16(n, seed, scale):
    """Reference test-input generator (bench/bench_w4a16.cu:32-40); returns uint16 bf16 bits."""
    out = np.empty(n, dtype=np.uint16)
    lib().orc_fill_bf16(_p(out), n, seed, scale)
    return out


def w4_quantize(W_bits, G=128):
    """RTN quantizer (kernels/quant/w4a16.cuh:274-297). W_bits: [N,K] uint16 -> (Wq [N,K/8] u32, S [N,K/G] u16)."""
    W_bits = _c(W_bits, np.uint16)
    N, K = W_bits.shape
    Wq = np.empty((N, K // 8), dtype=np.uint32)
    S = np.empty((N, K // G), dtype=np.uint16)
    rc = lib().orc_w4_quantize(_p(W_bits), _p(Wq), _p(S), N, K, G)
    if rc != 0:
        raise ValueError(f"orc_w4_quantize rejected N={N} K={K} G={G} (rc={rc})")
    return Wq, S


def w4_dequant(Wq, S, G=128):
    Wq, S = _c(Wq, np.uint32), _c(S, np.uint16)
    N, K = Wq.shape[0], Wq.shape[1] * 8
    Wd = np.empty((N, K), dtype=np.float32)
    lib().orc_w4_dequant(_p(Wq), _p(S), N, K, G, _p(Wd))
    return Wd


def w4_dequant_bf16(Wq, S, G=128):
    Wq, S = _c(Wq, np.uint32), _c(S, np.uint16)
    N, K = Wq.shape[0], Wq.shape[1] * 8
    Wd = np.empty((N, K), dtype=np.uint16)
    lib().orc_w4_dequant_bf16(_p(Wq), _p(S), N, K, G, _p(Wd))
    return Wd


def w4_unpack(Wq):
    Wq = _c(Wq, np.uint32)
    N, K = Wq.shape[0], Wq.shape[1] * 8
    Q = np.empty((N, K), dtype=np.int8)
    lib().orc_w4_unpack(_p(Wq), N, K, _p(Q))
    return Q


def w4_linear_f32(X_bits, Wq, S, G=128, threads=1):
    """Dequant-then-double-accumulate check (bench/bench_w4a16.cu:156-173). Returns fp32 [M,N]."""
    X_bits, Wq, S = _c(X_bits, np.uint16), _c(Wq, np.uint32), _c(S, np.uint16)
    M, K = X_bits.shape
    N = Wq.shape[0]
    assert Wq.shape[1] * 8 == K and S.shape == (N, K // G)
    Y = np.empty((M, N), dtype=np.float32)
    rc = lib().orc_w4_linear_f32(_p(X_bits), _p(Wq), _p(S), _p(Y), M, N, K, G, threads)
    if rc < 0:
        raise MemoryError("orc_w4_linear_f32")
    return Y


def w4_linear_bf16(X_bits, Wq, S, G=128, threads=1):
    """Same, rounded once to bf16 bits: the value ns_w4_linear stores."""
    return f32_to_bf16_bits(w4_linear_f32(X_bits, Wq, S, G, threads))


def dense_linear_f32(X_bits, W_bits):
    X_bits, W_bits = _c(X_bits, np.uint16), _c(W_bits, np.uint16)
    M, K = X_bits.shape
    N = W_bits.shape[0]
    Y = np.empty((M, N), dtype=np.float32)
    lib().orc_dense_linear_f32(_p(X_bits), _p(W_bits), _p(Y), M, N, K)
    return Y


def max_rel_err(a, ref):
    a, ref = _c(a, np.float32), _c(ref, np.float32)
    return float(lib().orc_max_rel_err(_p(a), _p(ref), a.size))


def rel_fro(a, ref):
    a, ref = _c(a, np.float32), _c(ref, np.float32)
    return float(lib().orc_rel_fro(_p(a), _p(ref), a.size))


def max_threads():
    return int(lib().orc_max_threads())


# ------------------------------------------------------------------ numpy twin (cross-check of the C code)
def np_unpack(Wq):
    """q - 8 for every (n, k): value k = 8j+i sits in bits 4i..4i+3 of word j (w4a16.cuh:6)."""
    Wq = np.ascontiguousarray(Wq, dtype=np.uint32)
    sh = (4 * np.arange(8, dtype=np.uint32))[None, None, :]
    q = (Wq[:, :, None] >> sh) & 0xF
    return q.reshape(Wq.shape[0], -1).astype(np.int32) - 8


def np_dequant(Wq, S, G=128):
    q = np_unpack(Wq).astype(np.float32)
    s = np.repeat(bf16_bits_to_f32(S), G, axis=1)
    return q * s


def np_linear_f64(X_bits, Wq, S, G=128):
    """fp64 matmul on the dequantised weights (pairwise summation; compare with a tolerance)."""
    return bf16_bits_to_f32(X_bits).astype(np.float64) @ np_dequant(Wq, S, G).astype(np.float64).T


def np_quantize(W_bits, G=128):
    W = bf16_bits_to_f32(W_bits)
    N, K = W.shape
    Wg = W.reshape(N, K // G, G)
    mx = np.abs(Wg).max(axis=2)
    s32 = np.where(mx > 0, (mx / np.float32(7.0)).astype(np.float32), np.float32(1.0)).astype(np.float32)
    S = f32_to_bf16_bits(s32)
    sf = bf16_bits_to_f32(S)
    r = (Wg / sf[:, :, None]).astype(np.float32)
    q = np.clip(np.rint(r).astype(np.int64) + 8, 0, 15).astype(np.uint32)
    q = q.reshape(N, K // 8, 8)
    sh = (4 * np.arange(8, dtype=np.uint32))[None, None, :]
    Wq = np.bitwise_or.reduce(q << sh, axis=2).astype(np.uint32)
    return Wq, S


# ------------------------------------------------------------------ seeded synthetic inputs of the benchmark shapes
from nanoserve_b200.synth import synth_inputs  # noqa: E402,F401  (one generator for tests, bench and oracle)
