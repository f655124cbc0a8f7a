"""ctypes binding to build/libnanoserve.so: the host-side mirror of the reference's operator interface.

``Kernels`` has the same constructor, method names, argument meaning and error behaviour as the
reference's ``python/nanoserve/ops.py`` (class ``Kernels``, lines 15-97): torch tensors in and out on the
current CUDA stream, ``RuntimeError("<symbol> failed with code <rc>")`` on a non-zero return code.  The one
deliberate difference is that ``w4_linear`` no longer pads M (reference ops.py:89-91): the B200 library
serves every M >= 1 natively.

There is no CPU path: if the shared library is missing or a tensor is not on a CUDA device the call
raises.
"""
import ctypes
import os

import torch

_LIB_DEFAULT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "build", "libnanoserve.so")

FLAG_FOLD_ZERO_POINT = 1
FLAG_NO_SPLIT_K = 2
FLAG_NARROW_CTA = 4
FLAG_NO_PDL = 8
FLAG_FLOAT_X = 256
FLAG_WIDE_X = 512
FLAG_NO_AUTOTUNE = 4096
FLAG_PRE_STAGE_X = 8192
FLAG_NO_PRE_STAGE_X = 16384
FLAG_SPLIT_SUM_KERNEL = 32768
FLAG_NO_SPLIT_SUM_KERNEL = 65536
FLAG_RING_KERNEL = 131072    # decode GEMV: the shared-memory ring kernel even where the streaming kernel applies
PRO_STAGED = 3        # prologue of b2_w4_linear_fused: x is the converted form EPI_SWIGLU_STAGED left (uint8 buffer)
EPI_SWIGLU_STAGED = 2  # like EPI_SWIGLU_PAIRS, but the output is the converted form the next GEMV takes with PRO_STAGED
EPI_SWIGLU_PAIRS8 = 3  # EPI_SWIGLU_PAIRS with row blocks of 8 gate + 8 up rows (the kernel then gives a warp 16 rows)
EPI_SWIGLU_PAIRS = 1  # epilogue of b2_w4_linear_fused: silu(gate) * up over row blocks of 16 gate + 16 up rows
FLAG_GEMM_NO_PAIRS = 1 << 29  # prefill GEMM: one CTA per tile unpacks the whole weight tile (no clusters of two)
FLAG_GEMM_WHOLE_TILES = 1 << 30  # prefill GEMM: every CTA takes whole output tiles (no fp32 part-tiles)
FLAG_NO_MID_KERNEL = 262144  # decode GEMV: never the many-token kernel (2 <= M <= 16 on plain launches)
FLAG_MID_KERNEL = 131072 | 524288  # decode GEMV (both kernel flags): the many-token kernel for every shape it can serve
FLAG_STREAM_KERNEL = 524288  # decode GEMV: the streaming kernel for every M <= 16 it can serve (default: M <= 2)

# Every symbol include/nanoserve_b200.h declares, with its ctypes signature.
_vp, _i32, _f32, _i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
SIGNATURES = {
    # the six symbols of the reference library (python/nanoserve/ops.py:19-26)
    "ns_rmsnorm": ([_vp, _vp, _vp, _vp, _i32, _i32, _f32, _vp], _i32),
    "ns_rope": ([_vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i64, _i64, _vp], _i32),
    "ns_swiglu": ([_vp, _vp, _vp, _i32, _i32, _vp], _i32),
    "ns_flash_fwd": ([_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i64, _i64, _i64, _i32, _i32, _vp], _i32),
    "ns_w4_quantize": ([_vp, _vp, _vp, _i32, _i32, _i32, _vp], _i32),
    "ns_w4_linear": ([_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp], _i32),
    # additions
    "b2_init": ([], _i32),
    "b2_w4_linear": ([_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp], _i32),
    "b2_w4_linear_fused": ([_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _f32, _vp, _i32, _vp], _i32),
    "b2_device_status": ([], _i32),
    "b2_clear_status": ([], _i32),
    "b2_w4_gemv_scratch_bytes": ([_i32, _i32, _i32, _i32, _i32], ctypes.c_size_t),
    "b2_w4_gemv_noalloc": ([_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp], _i32),
    "b2_rope_kv_store": ([_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp], _i32),
    "b2_decode_attention": ([_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp], _i32),
    "b2_greedy_next": ([_vp, _i32, _vp, _i32, _vp, _vp, _vp, _vp, _vp, _vp], _i32),
    "b2_decode_workspace_bytes": ([_i32, _i32], ctypes.c_size_t),
    "b2_lm_head_blocks": ([_i32], _i32),
    "b2_lm_head": ([_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _f32, _vp, _vp, _vp, _i32, _vp], _i32),
    "b2_greedy_pick": ([_vp, _vp, _i32, _i32, _vp, _i32, _vp, _vp, _vp, _vp, _vp], _i32),
    "b2_w4_linear_tp": ([_vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _f32, _vp, _vp, _i32, _vp], _i32),
    "b2_w4_gemv_grid": ([_i32, _i32, _i32, _i32, _i32], ctypes.c_size_t),
    "b2_decode_attention_fused": ([_vp] * 8 + [_i32, _i32, _i32, _i32, _vp, _i32, _vp], _i32),
    "b2_tp_wait_desc": ([_vp, _i32, _vp], _i32),
    "b2_w4_gemv_describe": ([_i32, _i32, _i32, _i32, _i32, ctypes.c_char_p, _i32], _i32),
    "b2_decode_attention_fused_workspace_bytes": ([_i32, _i32, _i32], ctypes.c_size_t),
    "b2_rope_kv_store_tp": ([_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp, ctypes.c_uint, _vp], _i32),
    "b2_tp_wait": ([_vp, _vp, ctypes.c_uint, _vp], _i32),
    "b2_version": ([], ctypes.c_char_p),
}


class TpDesc(ctypes.Structure):
    """struct b2_tp_desc of include/nanoserve_b200.h."""
    _fields_ = [("world", _i32), ("y_peer", _vp * 8), ("sig_peer", _vp * 8), ("ld", _i64), ("seg_end", _i32 * 2),
                ("seg_dst", _i32 * 3), ("y_local", _vp), ("wait_sig", _vp), ("epoch", _vp),
                ("wait_per_epoch", ctypes.c_uint), ("defer_signal", _i32), ("announce_world", _i32),
                ("announce_peer", _vp * 8)]


def staged_x_bytes(K: int) -> int:
    """Bytes of one token's activations in the converted form EPI_SWIGLU_STAGED writes and PRO_STAGED reads."""
    return 4 * K + (K // 128) * 32


def make_tp_desc(y_peers=(), sig_peers=(), ld=0, pieces=None, y_local=None, wait_sig=None, epoch=None,
                 wait_per_epoch=0, defer=False, announce_peers=()) -> TpDesc:
    """pieces: [(local_width, gathered_column), ...] of the row-concatenated local shard (at most three).
    defer: the producer only stores; announce_peers: the counters (one per rank) this call adds one to once the kernel
    in front of it on the stream has completed (see struct b2_tp_desc)."""
    d = TpDesc()
    d.world = len(y_peers)
    for r, y in enumerate(y_peers):
        d.y_peer[r] = y
    for r, sg in enumerate(sig_peers):
        d.sig_peer[r] = sg
    d.defer_signal = 1 if defer else 0
    d.announce_world = len(announce_peers)
    for r, a in enumerate(announce_peers):
        d.announce_peer[r] = a
    d.ld = ld
    ends, dst, acc = [0x7FFFFFFF, 0x7FFFFFFF], [0, 0, 0], 0
    for i, (w, col) in enumerate(pieces or []):
        acc += w
        dst[i] = col
        if i < 2 and i + 1 < len(pieces):
            ends[i] = acc
    d.seg_end[0], d.seg_end[1] = ends
    d.seg_dst[0], d.seg_dst[1], d.seg_dst[2] = dst
    d.y_local, d.wait_sig, d.epoch, d.wait_per_epoch = y_local, wait_sig, epoch, wait_per_epoch
    return d


def load_library(path: str = _LIB_DEFAULT) -> ctypes.CDLL:
    """Loads the C-ABI library and sets the signature of every exported entry point."""
    path = os.path.abspath(path)
    if not os.path.exists(path):
        raise FileNotFoundError(
            f"{path} not found: build it with `python -m nanoserve_b200.build` (needs nvcc); "
            "there is no CPU fallback")
    lib = ctypes.CDLL(path)
    for name, (args, res) in SIGNATURES.items():
        if not hasattr(lib, name):
            continue  # optional additions may be absent in an older build; required ones fail on use
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = res
    return lib


class Kernels:
    def __init__(self, path: str = _LIB_DEFAULT):
        self.lib = load_library(path)
        for name in ("ns_rmsnorm", "ns_rope", "ns_swiglu", "ns_flash_fwd", "ns_w4_quantize", "ns_w4_linear"):
            getattr(self.lib, name)  # AttributeError if the library is not a drop-in

    @staticmethod
    def _stream():
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    @staticmethod
    def _check(rc: int, name: str):
        if rc != 0:
            raise RuntimeError(f"{name} failed with code {rc}")

    @staticmethod
    def _cuda(*tensors):
        for t in tensors:
            if t is not None and not t.is_cuda:
                raise RuntimeError("nanoserve_b200 operators take CUDA tensors only (no CPU path)")

    # x: [T, H] residual stream, updated in place when r is given. Returns rmsnorm(x) * w.
    def rmsnorm(self, x, r, w, eps):
        self._cuda(x, r, w)
        assert x.is_contiguous() and x.dtype == torch.bfloat16
        y = torch.empty_like(x)
        rc = self.lib.ns_rmsnorm(x.data_ptr(), None if r is None else r.data_ptr(), w.data_ptr(),
                                 y.data_ptr(), x.shape[0], x.shape[1], eps, self._stream())
        self._check(rc, "ns_rmsnorm")
        return y

    # In place on q [T, Hq*D] and k [T, Hk*D] (row stride may exceed Hq*D / Hk*D).
    def rope(self, q, k, inv_freq, n_heads, n_kv_heads, head_dim, pos0):
        self._cuda(q, k, inv_freq)
        rc = self.lib.ns_rope(q.data_ptr(), k.data_ptr(), inv_freq.data_ptr(), q.shape[0], n_heads,
                              n_kv_heads, head_dim, pos0, q.stride(0), k.stride(0), self._stream())
        self._check(rc, "ns_rope")

    def swiglu(self, gate, up):
        self._cuda(gate, up)
        assert gate.is_contiguous() and up.is_contiguous()
        out = torch.empty_like(gate)
        rc = self.lib.ns_swiglu(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.shape[0],
                                gate.shape[1], self._stream())
        self._check(rc, "ns_swiglu")
        return out

    def flash_attention(self, q, k, v, n_heads, n_kv_heads, head_dim, causal=True):
        # Attention is outside the quantized-linear path; the library exports the symbol and reports
        # "not implemented" (-3), which surfaces here as the reference's RuntimeError.
        N = q.shape[0]
        o = torch.empty((N, n_heads * head_dim), dtype=q.dtype, device=q.device)
        rc = self.lib.ns_flash_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), N, n_heads,
                                   n_kv_heads, head_dim, q.stride(0), k.stride(0), o.stride(0),
                                   int(causal), 1, self._stream())
        self._check(rc, "ns_flash_fwd")
        return o

    def w4_quantize(self, W, group=128):
        self._cuda(W)
        N, K = W.shape
        Wq = torch.empty((N, K // 8), dtype=torch.int32, device=W.device)
        S = torch.empty((N, K // group), dtype=torch.bfloat16, device=W.device)
        rc = self.lib.ns_w4_quantize(W.contiguous().data_ptr(), Wq.data_ptr(), S.data_ptr(), N, K,
                                     group, self._stream())
        self._check(rc, "ns_w4_quantize")
        return Wq, S

    # x [M, K] -> [M, N] for any M >= 1 (decode GEMV for M <= 16, tensor-core GEMM above).
    def w4_linear(self, x, Wq, S, group=128, flags=0, out=None):
        """`out` may also be a pinned host tensor: the kernel then stores its outputs straight into host memory
        (unified addressing), which saves a copy node when the outputs are wanted on the host anyway."""
        self._cuda(x, Wq, S, None if out is not None and not out.is_cuda and out.is_pinned() else out)
        M, K = x.shape
        N = Wq.shape[0]
        x = x.contiguous()
        y = out if out is not None else torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        if flags:
            rc = self.lib.b2_w4_linear(x.data_ptr(), Wq.data_ptr(), S.data_ptr(), y.data_ptr(), M, N, K,
                                       group, flags, self._stream())
        else:
            rc = self.lib.ns_w4_linear(x.data_ptr(), Wq.data_ptr(), S.data_ptr(), y.data_ptr(), M, N, K,
                                       group, self._stream())
        self._check(rc, "ns_w4_linear")
        return y

    # ---- additions
    def w4_linear_fused(self, x, Wq, S, group=128, prologue=0, r=None, wn=None, eps=0.0, x_out=None, flags=0,
                        epilogue=0):
        """Decode GEMV with the neighbouring operators folded in: prologue 1 = add + RMSNorm (x + r normalised with
        weights wn; the sum goes to x_out), prologue 2 = SwiGLU (x is [M, 2K] gate | up); epilogue EPI_SWIGLU_PAIRS =
        the rows of Wq are 16 gate rows, their 16 up rows, the next 16 gate rows ... and the output is
        silu(gate) * up, [M, N / 2] (one token; raises with code -3 where the kernel cannot serve it)."""
        self._cuda(x, Wq, S, r, wn, x_out)
        N, K = Wq.shape[0], Wq.shape[1] * 8
        if prologue == PRO_STAGED:  # one token; x: four digit planes of K bytes + 32 bytes per 128-chunk
            M = 1
            assert x.is_contiguous() and x.dtype == torch.uint8 and x.numel() == staged_x_bytes(K)
        else:
            M = x.shape[0]
            assert x.is_contiguous() and x.shape[1] == (2 * K if prologue == 2 else K)
        if epilogue == EPI_SWIGLU_STAGED:
            y = torch.empty(staged_x_bytes(N // 2), dtype=torch.uint8, device=x.device)
        else:
            y = torch.empty((M, N // 2 if epilogue in (EPI_SWIGLU_PAIRS, EPI_SWIGLU_PAIRS8) else N), dtype=torch.bfloat16,
                            device=x.device)
        p = lambda t: None if t is None else t.data_ptr()
        rc = self.lib.b2_w4_linear_fused(x.data_ptr(), Wq.data_ptr(), S.data_ptr(), y.data_ptr(), M, N, K, group,
                                         prologue | (epilogue << 8), p(r), p(wn), eps, p(x_out), flags, self._stream())
        self._check(rc, "b2_w4_linear_fused")
        return y

    def w4_linear_tp(self, x, Wq, S, desc: "TpDesc", group=128, prologue=0, r=None, wn=None, eps=0.0, x_out=None,
                     flags=0, epilogue=0):
        """Decode GEMV of a tensor-parallel shard with the all-gather fused in (see b2_w4_linear_tp); the outputs
        go where `desc` says."""
        self._cuda(x, Wq, S, r, wn, x_out)
        M = x.shape[0]
        N, K = Wq.shape[0], Wq.shape[1] * 8
        assert x.is_contiguous() and x.shape[1] == (2 * K if prologue == 2 else K)
        p = lambda t: None if t is None else t.data_ptr()
        rc = self.lib.b2_w4_linear_tp(x.data_ptr(), Wq.data_ptr(), S.data_ptr(), M, N, K, group,
                                      prologue | (epilogue << 8), p(r), p(wn), eps, p(x_out), ctypes.byref(desc), flags,
                                      self._stream())
        self._check(rc, "b2_w4_linear_tp")

    def lm_head(self, x, W, logits=None, part_max=None, part_idx=None, idx_offset=0, r=None, wn=None, eps=0.0):
        """bf16 vocabulary projection (x [M, K] . W [V, K]^T) with the per-128-row argmax of token 0 in its epilogue
        and, when `wn` is given, the final add + RMSNorm in its prologue.  Returns the logits tensor (or None)."""
        self._cuda(x, W, logits, part_max, part_idx, r, wn)
        M, K = x.shape
        V = W.shape[0]
        assert x.is_contiguous() and W.is_contiguous()
        p = lambda t: None if t is None else t.data_ptr()
        rc = self.lib.b2_lm_head(x.data_ptr(), W.data_ptr(), p(logits), M, V, K, 1 if wn is not None else 0, p(r),
                                 p(wn), eps, None, p(part_max), p(part_idx), idx_offset, self._stream())
        self._check(rc, "b2_lm_head")
        return logits

    def lm_head_blocks(self, V) -> int:
        return int(self.lib.b2_lm_head_blocks(V))

    def tp_wait(self, wait_sig: int, epoch: int, wait_per_epoch: int):
        self._check(self.lib.b2_tp_wait(wait_sig, epoch, wait_per_epoch, self._stream()), "b2_tp_wait")

    def tp_wait_desc(self, desc: "TpDesc", advance_epoch: bool = False):
        """The consumer side of a descriptor as a kernel of its own: announce, wait, optionally *epoch += 1."""
        self._check(self.lib.b2_tp_wait_desc(ctypes.byref(desc), 1 if advance_epoch else 0, self._stream()),
                    "b2_tp_wait_desc")

    def gemv_describe(self, M, N, K, group=128, flags=0) -> str:
        """Which kernel and launch shape a decode GEMV of this shape gets on the current device."""
        buf = ctypes.create_string_buffer(512)
        self._check(self.lib.b2_w4_gemv_describe(M, N, K, group, flags, buf, 512), "b2_w4_gemv_describe")
        return buf.value.decode()

    def gemv_grid(self, M, N, K, group=128, flags=0) -> int:
        return int(self.lib.b2_w4_gemv_grid(M, N, K, group, flags))

    def init(self):
        self._check(self.lib.b2_init(), "b2_init")

    def device_status(self) -> int:
        return int(self.lib.b2_device_status())

    def clear_status(self):
        self._check(self.lib.b2_clear_status(), "b2_clear_status")

    def gemv_scratch_bytes(self, M, N, K, group=128, flags=0) -> int:
        return int(self.lib.b2_w4_gemv_scratch_bytes(M, N, K, group, flags))

    def version(self) -> str:
        return self.lib.b2_version().decode()
