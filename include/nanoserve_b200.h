/*
 * C ABI of libnanoserve.so for NVIDIA B200 (sm_100a): the W4A16 quantized-linear path.
 *
 * The first group of entry points has the exact names, argument lists and return conventions of the
 * reference library's C ABI (csrc/nanoserve_ops.cu of the reference project), so the reference's own
 * ctypes binding (python/nanoserve/ops.py:19-30) loads this library unchanged.  All pointers are device
 * pointers owned and allocated by the caller; `stream` is a raw cudaStream_t; every call is asynchronous
 * and returns right after the launch.  Return value: 0 on success, a positive CUDA error code, or one of
 * the negative codes below.
 *
 * Weight format (reference kernels/quant/w4a16.cuh:5-9):
 *   Wq [N, K/8] uint32  word j of row n packs k = 8j..8j+7, value k = 8j+i in bits 4i..4i+3
 *   S  [N, K/G] bf16    w[n,k] = (q - 8) * S[n, k/G], q in [0, 15]; the zero-point is the constant 8
 */
#ifndef NANOSERVE_B200_H_
#define NANOSERVE_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B2_OK 0
#define B2_ERR_BAD_SHAPE (-1)       /* K % G, G % 32 or K % 32 violated (reference: -1) */
#define B2_ERR_UNSUPPORTED_M (-2)   /* M < 1 (reference: -2 for M it cannot serve) */
#define B2_ERR_NOT_IMPLEMENTED (-3) /* operator outside the W4A16 path */
#define B2_ERR_BAD_POINTER (-4)     /* null or misaligned pointer (X, Wq: 16 bytes) */
#define B2_ERR_WORKSPACE (-5)       /* per-device scratch could not be set up */
#define B2_ERR_TOO_LARGE (-6)       /* size beyond a documented maximum */
#define B2_ERR_DEVICE (-7)          /* a kernel recorded a device-side time-out */

/* ---- drop-in entry points (same symbols as the reference library) ------------------------------ */

/*
 * Y[M,N] (bf16) = X[M,K] (bf16) . dequant(Wq, S)^T, fp32 accumulation, one rounding to bf16 at the store.
 * Replaces ns_w4_linear, csrc/nanoserve_ops.cu:75-90.  The reference serves M in {1,2,4,8} (GEMV) and
 * M % 128 == 0 with N % 128 == 0 (GEMM) and returns -2 otherwise; this library serves every M >= 1 and
 * every N >= 1: M <= 16 runs the decode GEMV, larger M the tensor-core GEMM.  Needs K % 32 == 0,
 * G % 32 == 0, K % G == 0 (the reference calls exit() on these inside w4a16.cuh:100-103; this library
 * returns -1 instead).
 */
int ns_w4_linear(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int G,
                 void* stream);

/*
 * W[N,K] (bf16) -> Wq[N,K/8] (uint32) + S[N,K/G] (bf16): round-to-nearest symmetric group quantizer,
 * bit-identical to the reference's.  Replaces ns_w4_quantize, csrc/nanoserve_ops.cu:66-71.
 * Returns -1 if K % G or G % 32.
 */
int ns_w4_quantize(const void* W, void* Wq, void* S, int N, int K, int G, void* stream);

/*
 * The reference's Python binding resolves these four symbols when it loads the library
 * (python/nanoserve/ops.py:19-30), so they are exported.  They lie outside the W4A16 path.
 * ns_rmsnorm / ns_rope / ns_swiglu replace csrc/nanoserve_ops.cu:21-45 with the same semantics;
 * ns_flash_fwd (csrc/nanoserve_ops.cu:47-63) returns B2_ERR_NOT_IMPLEMENTED.
 */
int ns_rmsnorm(void* x, const void* r, const void* w, void* y, int T, int H, float eps, void* stream);
int ns_rope(void* q, void* k, const void* inv_freq, int T, int Hq, int Hk, int D, int pos0,
            long long q_stride, long long k_stride, void* stream);
int ns_swiglu(const void* gate, const void* up, void* out, int T, int I, void* stream);
int ns_flash_fwd(const void* q, const void* k, const void* v, void* o, int N, int Hq, int Hk, int D,
                 long long q_t, long long kv_t, long long o_t, int causal, int variant, void* stream);

/* ---- additions (no counterpart in the reference library) --------------------------------------- */

/*
 * Flags for b2_w4_linear.  Three kernels serve the decode GEMV (M <= 16).  The streaming kernel (G % 128 == 0,
 * K % 256 == 0, Wq 16-byte aligned) runs one token always and two to four tokens on tall matrices with K < 8192; it
 * carries X as block fixed point per (token, 128-wide chunk of K) -- 32 bits for M <= 2 (exact to fp32 summation
 * order), 15 bits + sign above -- on an 8-bit integer mma.  The many-token kernel (G == 128, K % 256 == 0, plain
 * launches) runs five to sixteen tokens, and two to four where K >= 8192, with X as 16-bit block
 * fixed point.  The ring kernel runs everything else, with X as 16-bit block fixed point (every element off by at most
 * 2^-16 of its chunk's largest magnitude) or as the flags below say.  No kernel measures anything or synchronises:
 * every call is asynchronous.  A K that is cut into slices across CTAs (long K, few rows) is followed by a small
 * kernel that adds the slices' fp32 partial sums in fixed order; B2_FLAG_NO_SPLIT_K forbids that.
 */
#define B2_FLAG_FOLD_ZERO_POINT 1 /* ring kernel with B2_FLAG_FLOAT_X: apply the -8 as one fp32 correction per 128-wide chunk */
#define B2_FLAG_NO_SPLIT_K 2      /* GEMV: never split K across CTAs (uses no scratch memory) */
#define B2_FLAG_NARROW_CTA 4      /* ring kernel: 8 consumer warps per CTA instead of 16 */
#define B2_FLAG_FLOAT_X 256       /* GEMV, G % 128 == 0: keep X in floating point (fp16 operands of a floating-point mma, ring
                                     kernel) instead of block fixed point */
#define B2_FLAG_WIDE_X 512        /* ring kernel, G % 128 == 0: 24-bit instead of 16-bit block fixed point for X */
#define B2_FLAG_NO_AUTOTUNE 4096  /* ring kernel: never time CTA shapes.  (Timing is off unless B2_GEMV_AUTOTUNE=1 is set in the
                                     environment: it synchronises the stream on the first call of a shape, which a drop-in
                                     for an asynchronous call must not do.  The built-in cost model decides otherwise.) */
#define B2_FLAG_PRE_STAGE_X 8192  /* ring kernel, integer path: convert X to its fixed-point form once, in a small kernel launched
                                     in front of the GEMV, and let every CTA copy its slice (default from M = 8 on, from M = 4
                                     where K >= 8192); ignored where it does not apply (RMSNorm prologue, tensor-parallel
                                     consumer, B2_FLAG_FLOAT_X, M * K beyond the staging area) */
#define B2_FLAG_NO_PRE_STAGE_X 16384 /* ring kernel: every CTA converts the slice of X it needs itself, at every M */
#define B2_FLAG_SPLIT_SUM_KERNEL 32768   /* GEMV with K split across CTAs: a small kernel behind the GEMV adds up the slices'
                                           partial sums (the default; never for tensor-parallel producers) */
#define B2_FLAG_NO_SPLIT_SUM_KERNEL 65536 /* GEMV: the last CTA of a row group to arrive adds them up (a hand-shake of
                                           three L2 round trips per tile, but no second kernel) */
#define B2_FLAG_RING_KERNEL 131072 /* GEMV: the ring kernel even where the streaming kernel would run */
#define B2_FLAG_NO_MID_KERNEL 262144 /* GEMV: never the many-token kernel (2 <= M <= 16, G == 128, K % 256 == 0, plain launches) */
#define B2_FLAG_MID_KERNEL (131072 | 524288) /* GEMV (both kernel flags): the many-token kernel for every shape it can serve */
#define B2_FLAG_STREAM_KERNEL 524288 /* GEMV: the streaming kernel for every M <= 16 it can serve */
#define B2_FLAG_GEMM_NO_PAIRS 536870912 /* prefill GEMM: no clusters of two CTAs (by default two CTAs on neighbouring token
                                           tiles unpack half of the weight tile each, for both) */
#define B2_FLAG_GEMM_WHOLE_TILES 1073741824 /* prefill GEMM (M > 16): every CTA takes whole output tiles; by default the CTAs
                                           take equal shares of the (tile, K block) pairs and tiles that several CTAs cover
                                           are finished from fp32 part-tiles in the scratch */
#define B2_FLAG_NO_PDL 8          /* GEMV: plain launch.  By default the GEMV is launched with programmatic stream
                                     serialization: it may begin (weight prefetch only) while the previous kernel of
                                     the stream is still running, and touches X, Y and scratch only after that kernel
                                     has completed */

/*
 * Sets up the calling thread's current device: queries the SM count and allocates the per-device scratch
 * (split-K partial sums, arrival counters, the staged X of a launch, a status word; 100 MiB + 256 KiB).  ns_w4_linear does this on
 * its first call on a device; call b2_init first when that first call would fall inside a CUDA-graph
 * capture.  Launches on different streams of one device share the scratch: launches that use it (split-K GEMVs, GEMMs whose
 * tile count is not a multiple of the SM count) race when they overlap in time.
 */
int b2_init(void);

/* ns_w4_linear with flags (0 = the defaults ns_w4_linear uses). */
int b2_w4_linear(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int G,
                 int flags, void* stream);

/*
 * Decode GEMV (1 <= M <= 16, G % 128 == 0) with the operator that precedes the linear folded into the kernel, so a
 * decoder layer needs fewer launches.  No counterpart in the reference library (it runs ns_rmsnorm / ns_swiglu
 * as separate kernels before ns_w4_linear, python/nanoserve/qwen.py:158-161).  Results equal the two-kernel
 * sequence up to the rounding of the norm's sum of squares.
 *   prologue 0: none (same as b2_w4_linear).
 *   prologue 1: add + RMSNorm (semantics of ns_rmsnorm): the product's input is rmsnorm(bf16(X + R)) * Wn with
 *               X, R [M, K], Wn [K]; R may be NULL (plain norm).  If Xout is not NULL, bf16(X + R) is stored there
 *               (Xout must not alias X: other CTAs are still reading X).
 *   prologue 2: SwiGLU (semantics of ns_swiglu): X is [M, 2K] = gate | up; the input is bf16(silu(gate) * up).
 *   prologue 3: X is one token's activations already in the kernel's converted form, as epilogue 2 of the producing
 *               launch left them (4 K + K / 4 bytes, 16-byte aligned; M = 1; streaming kernel only, else -3).
 * An epilogue may be added to the prologue as (epilogue << 8); one token, streaming kernel only (else -3):
 *   epilogue 1: the rows of Wq / S are 16 gate rows, their 16 up rows, the next 16 gate rows ...; Y [M, N / 2] =
 *               bf16(silu(gate) * up), each half rounded to bf16 first: bit-identical to the plain launch on the
 *               row-concatenated matrix followed by ns_swiglu.  N % 32 == 0.
 *   epilogue 3: epilogue 1 with row blocks of 8 gate + 8 up rows (the kernel then gives a warp 16 rows).  N % 16 == 0.
 *   epilogue 2: the same values, written in the converted form that a following launch takes with prologue 3 (so that
 *               launch need not convert 18944 activations in every CTA): Y is 4 (N/2) + (N/2) / 4 bytes.  N % 256 == 0.
 */
#define B2_PROLOGUE_NONE 0
#define B2_PROLOGUE_ADD_RMSNORM 1
#define B2_PROLOGUE_SWIGLU 2
#define B2_PROLOGUE_STAGED 3
#define B2_EPILOGUE_SWIGLU_PAIRS (1 << 8)
#define B2_EPILOGUE_SWIGLU_STAGED (2 << 8)
#define B2_EPILOGUE_SWIGLU_PAIRS8 (3 << 8)
int b2_w4_linear_fused(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int G, int prologue,
                       const void* R, const void* Wn, float eps, void* Xout, int flags, void* stream);

/*
 * Synchronises the current device and returns its status word: 0, or B2_ERR_DEVICE if a kernel gave up
 * on a bounded wait since the last b2_clear_status (an mbarrier of its pipeline, or a tensor-parallel arrival
 * counter).  The outputs of that launch are undefined.  While the word is set, GEMM launches return at once on the
 * device; b2_clear_status also clears arrival counters a time-out may have left half counted.
 */
int b2_device_status(void);
int b2_clear_status(void);

/* Scratch bytes the GEMV would use for this shape on the current device (0 = no split-K). */
size_t b2_w4_gemv_scratch_bytes(int M, int N, int K, int G, int flags);

/*
 * No counterpart in the reference library.  The decode GEMV (1 <= M <= 16, same operands and result as
 * ns_w4_linear) for callers that cannot allocate device memory at the point of the call -- a process whose
 * memory budget is handed to a pool at start-up, a plugin inside another runtime's capture or callback.
 * It calls no cudaMalloc / cudaFree and no allocating library routine: the split-K scratch is a fixed
 * array inside the library's device image (8 MiB + 16.25 KiB per GPU that loads the library, held until
 * exit).  Limits: M * N <= 1048576 and N <= 131072, otherwise B2_ERR_TOO_LARGE.  All calls on a device
 * share the array: calls whose kernels overlap in time race, so keep them on one stream.  The first call
 * on a device looks up the array's address, and the first call of a shape loads its kernel image; make those
 * calls before any stream capture.  A device-side time-out of such a call is recorded in a status word inside the
 * array; b2_device_status reports it (and b2_clear_status clears it) without allocating anything either.
 */
int b2_w4_gemv_noalloc(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int G,
                       void* stream);

/*
 * Batch-1 decode helpers that read the current position from device memory, so one captured CUDA graph serves
 * every decode step.  No counterpart in the reference library: the reference does these steps with PyTorch ops and
 * a host-side position (python/nanoserve/qwen.py:119-133,147-151,174-177).
 *   b2_rope_kv_store: qkv [(Hq+2Hk)*D] bf16 of the new token, in place: += bias (may be NULL), rotate-half RoPE on
 *     the q and k heads at position *pos, k and v written to cache_k / cache_v [Hk, max_len, D] at that position.
 *   b2_decode_attention: out [Hq*D] = softmax(q K^T / sqrt(D)) V over cache positions 0..*pos (D = 64 or 128);
 *     two launches (32 key slices per KV head, then a merge).
 *   b2_decode_attention_fused: both of the above with the RoPE / KV-store launch folded into the attention pass.
 *     qkv is read, not modified: every CTA rotates the query heads it serves in registers; the CTA whose key slice
 *     holds position *pos builds the new k and v rows, stores them to the caches and uses them from shared memory.
 *     flags 0: the merge of the key slices is a second launch (two launches in all; the faster form: 9.0 -> about
 *     7 us per layer at 600 positions).  flags 1: ONE launch; the last CTA of a KV head to finish merges the slices
 *     (an arrival counter per KV head; nobody waits), which puts a fence, an atomic and the merge's two L2 round
 *     trips behind the slowest CTA.  flags 2 (may be added to either): the caller promises that the kernel launched
 *     in front of this one on the stream writes neither *pos nor cached rows below *pos (true for a decode step, where
 *     that kernel is the q|k|v projection); the first tile of cached rows is then requested before that kernel has
 *     completed.  Results are bit-identical to the two calls above in every form.
 *     workspace: b2_decode_attention_fused_workspace_bytes(Hq, Hk, D) bytes, ZEROED once by the caller (the counters
 *     at its end return to zero after every launch).  tp: NULL, or the consumer side (wait_sig, epoch,
 *     wait_per_epoch, announce_peer) of the tensor-parallel GEMV that produced qkv (see b2_tp_desc).
 *   b2_greedy_next: token = argmax(logits[0..V)) (lowest index on ties); out_tokens[*step] = token; *step += 1;
 *     *pos += 1; x_next[0..H) = embed[token].  pos, step: int32 on the device; out_tokens: int64 on the device.
 */
int b2_rope_kv_store(void* qkv, const void* bias, const void* inv_freq, const void* pos, void* cache_k, void* cache_v,
                     int Hq, int Hk, int D, int max_len, void* stream);
int b2_decode_attention(const void* q, const void* cache_k, const void* cache_v, const void* pos, void* out,
                        void* workspace, int Hq, int Hk, int D, int max_len, void* stream);
typedef struct b2_tp_desc b2_tp_desc; /* defined below, with the tensor-parallel entry points */
size_t b2_decode_attention_fused_workspace_bytes(int Hq, int Hk, int D);
int b2_decode_attention_fused(const void* qkv, const void* bias, const void* inv_freq, const void* pos, void* cache_k,
                              void* cache_v, void* out, void* workspace, int Hq, int Hk, int D, int max_len,
                              const b2_tp_desc* tp, int flags, void* stream);
int b2_greedy_next(const void* logits, int V, const void* embed, int H, void* pos, void* out_tokens, void* step,
                   void* x_next, void* workspace, void* stream);
/*
 * The bf16 vocabulary projection of a decode step with the greedy argmax in its epilogue.  No counterpart in the
 * reference library: the reference runs F.linear on the bf16 lm_head and argmax over the logits on the host side of
 * the step (python/nanoserve/qwen.py:164,174-177).
 *   b2_lm_head: logits[M, V] (bf16; may be NULL when only the argmax is wanted) = X[M, K] . W[V, K]^T, fp32
 *     accumulation, 1 <= M <= 8, K % 64 == 0.  prologue / R / Wn / eps / Xout as in b2_w4_linear_fused (0 or 1: the
 *     model's final add + RMSNorm folded in).  If part_max / part_idx are not NULL, entry b of them receives the
 *     largest bf16 logit of token 0 among rows [128 b, 128 b + 128) and its row index + idx_offset (lowest index on
 *     ties); b2_lm_head_blocks(V) entries each.  A rank that holds a slice of the vocabulary passes its first row
 *     as idx_offset.
 *   b2_greedy_pick: b2_greedy_next starting from such (value, index) pairs instead of the logits.
 */
int b2_lm_head_blocks(int V);
int b2_lm_head(const void* X, const void* W, void* logits, int M, int V, int K, int prologue, const void* R,
               const void* Wn, float eps, void* Xout, void* part_max, void* part_idx, int idx_offset, void* stream);
int b2_greedy_pick(const void* part_max, const void* part_idx, int nparts, int V, const void* embed, int H, void* pos,
                   void* out_tokens, void* step, void* x_next, void* stream);

/* Bytes of caller-owned device scratch (`workspace`) the two calls above need (split partials; Hq / Hk <= 8). */
size_t b2_decode_workspace_bytes(int Hq, int D);

/*
 * Tensor parallelism over the output rows of a linear, one process per GPU, with the all-gather of the outputs fused
 * into the decode GEMV.  No counterpart in the reference library (it has no multi-GPU code).  Rank r holds rows
 * [r N/P, (r+1) N/P) of Wq and S (a zero-copy slice of the reference layout); X is replicated.
 *   Producer side (world > 0): the GEMV stores every output value straight into the gathered row [M, ld] (bf16) of
 *     EVERY rank through peer-mapped device pointers y_peer[0..world) (the caller maps them: CUDA IPC, symmetric
 *     memory; its own rank included), and the launch, after its last store, adds one to the arrival counter
 *     sig_peer[r] (uint32, peer-mapped) of every rank.  The local shard may be up to three row-concatenated pieces (q | k | v,
 *     gate | up) ending at local columns seg_end[0], seg_end[1], N; piece i lands at gathered column seg_dst[i].
 *   Consumer side (wait_sig != NULL): before it reads X the GEMV waits until this rank's counter wait_sig has reached
 *     (*epoch + 1) * wait_per_epoch: wait_per_epoch = ranks x producing launches per use, *epoch (int32 on the
 *     device) = completed uses of the counter, e.g. the decode step.  Counters only grow; zero them (all ranks,
 *     with a host barrier) whenever *epoch restarts.  The wait is bounded (about half a second); a time-out shows in
 *     b2_device_status().
 * A call may be producer, consumer or both; with world == 0 the output goes to y_local.  The other arguments are those
 * of b2_w4_linear_fused.  b2_rope_kv_store_tp is b2_rope_kv_store with the same wait in front.
 */
typedef struct b2_tp_desc {
  int world;
  void* y_peer[8];
  void* sig_peer[8];
  long long ld;
  int seg_end[2];
  int seg_dst[3];
  void* y_local;
  const void* wait_sig;
  const void* epoch;
  unsigned wait_per_epoch;
  /* Deferred signal (the cheaper protocol: a producer that signals for itself pays a fence per CTA and a release per
   * launch, about 4.5 us, before it may end).  A producer with defer_signal set stores its outputs and ends; sig_peer
   * is not used.  The NEXT kernel of the same stream -- the consumer of some other gathered row, as a rule -- has
   * seen that producer complete when it starts reading, and then adds one to announce_peer[0..announce_world): the
   * arrival counters, one per rank, that the producer would have signalled.  wait_per_epoch of such a counter is the
   * number of ranks (x producing launches per use). */
  int defer_signal;
  int announce_world;
  void* announce_peer[8];
} b2_tp_desc;
int b2_w4_linear_tp(const void* X, const void* Wq, const void* S, int M, int N, int K, int G, int prologue,
                    const void* R, const void* Wn, float eps, void* Xout, const b2_tp_desc* tp, int flags,
                    void* stream);
/* The consumer side of a descriptor as a small kernel of its own (announce, wait, and with advance_epoch != 0 add one
 * to *epoch afterwards): behind the last producer of a step, or in front of a consumer that is not a GEMV. */
int b2_tp_wait_desc(const b2_tp_desc* tp, int advance_epoch, void* stream);
/* CTAs the decode GEMV launches for this shape on the current device (0: not served by the GEMV). */
size_t b2_w4_gemv_grid(int M, int N, int K, int G, int flags);
/* One line of text into buf: which kernel and launch shape a decode GEMV of this shape gets (benchmark records). */
int b2_w4_gemv_describe(int M, int N, int K, int G, int flags, char* buf, int buflen);
int b2_rope_kv_store_tp(void* qkv, const void* bias, const void* inv_freq, const void* pos, void* cache_k,
                        void* cache_v, int Hq, int Hk, int D, int max_len, const void* wait_sig, const void* epoch,
                        unsigned wait_per_epoch, void* stream);

/* The consumer-side wait of b2_w4_linear_tp as a one-thread kernel of its own, for consumers that are not a GEMV
 * (a norm, a sampler): kernels after it on the stream see the gathered rows complete. */
int b2_tp_wait(const void* wait_sig, const void* epoch, unsigned wait_per_epoch, void* stream);

/* Library identification: "nanoserve-b200 <version> sm_100a". */
const char* b2_version(void);

#ifdef __cplusplus
}
#endif
#endif /* NANOSERVE_B200_H_ */
