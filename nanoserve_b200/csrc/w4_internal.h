// Host-side declarations shared by the C-ABI layer and the kernel translation units.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda_runtime.h>

namespace b2 {

// Return codes of the C ABI.  0 and positive values follow the reference library
// (csrc/nanoserve_ops.cu:3: 0 on success, else a CUDA error code); -1 / -2 keep its meaning
// (-1 bad shape for the quantizer :67, -2 unsupported M for the linear :86-88); the rest are new.
enum : int {
  kOk = 0,
  kErrBadShape = -1,     // K % G, G % 32 or K % 32 violated
  kErrUnsupportedM = -2, // M < 1
  kErrNotImplemented = -3,
  kErrBadPointer = -4,   // null or misaligned pointer
  kErrWorkspace = -5,    // workspace missing or too small
  kErrTooLarge = -6,     // size beyond a documented maximum
  kErrDevice = -7,       // a kernel reported a device-side time-out in the status word
};

// Device status word values written by kernels (0 = fine).
enum : int {
  kStatusOk = 0,
  kStatusGemvTimeout = 1,
  kStatusGemmTimeout = 2,
};

// Scratch memory a launch may use.  `partial` holds split-K partial sums, `counters` one arrival
// counter per 32-row group (zero between launches: the last arriver resets it), `status` one int.
struct Workspace {
  float* partial = nullptr;
  size_t partial_bytes = 0;
  int* counters = nullptr;
  int n_counters = 0;
  int* status = nullptr;
  unsigned char* xstage = nullptr;  // GEMV: X of a launch staged once for all CTAs (optional)
  size_t xstage_bytes = 0;
};

// Flags for the linear launches.
enum : int {
  kFlagFoldZeroPoint = 1,  // GEMV: fold the zero-point into one correction per group instead of a
                           // bf16x2 subtract per weight pair (fewer ALU ops, fp32-level cancellation)
  kFlagForceNoSplitK = 2,  // GEMV: never use split-K (no scratch needed)
  kFlagNarrowCta = 4,      // GEMV: use the 8-consumer-warp CTA even when the 16-warp one applies
  kFlagFloatX = 256,       // GEMV: keep X in floating point (fp16 mma path) instead of 16-bit block fixed point
  kFlagNoAutotune = 4096,  // GEMV: never time CTA shapes on the first launch of a shape; the cost model decides
  kFlagWideX = 512,        // GEMV: 24-bit instead of 16-bit block fixed point for X (three byte planes)
  kFlagPreStageX = 8192,   // GEMV, integer path: convert X once in a small kernel in front and let every CTA copy its
                           // slice, instead of converting in every CTA (default: for M >= 4)
  kFlagNoPreStageX = 16384,  // GEMV: never do that
  kFlagSplitSumKernel = 32768,    // GEMV, split K: the slices' partial sums are added up by a small kernel behind the GEMV
                                  // instead of by the last CTA of a row group to arrive (not for tensor-parallel producers)
  kFlagNoSplitSumKernel = 65536,  // GEMV: never do that
  kFlagRingKernel = 131072,  // GEMV: run the shared-memory ring kernel (w4_gemv.cu) even where the register-streaming
                             // kernel (w4_gemv_stream.cu) applies; bits 20-23: force that kernel's warps per row block
  kFlagNoMidKernel = 262144,  // GEMV: never run the many-token kernel (w4_gemv_mid.cu, 2 <= M <= 16)
  kFlagMidKernel = 131072 | 524288,  // (ring | streaming, both) GEMV: the many-token kernel for every shape it can
                                     // serve (by default not where another kernel measured faster)
  kFlagStreamKernel = 262144 * 2,  // GEMV: run the streaming kernel for every M <= 16 it can serve (by default M <= 2)
  kFlagGemmNoPairs = 1 << 29,     // GEMM: one CTA per tile unpacks the whole weight tile (no clusters of two)
  kFlagGemmWholeTiles = 1 << 30,  // GEMM: every CTA takes whole output tiles (no part-tiles, no scratch)
  kFlagNoPdl = 8,          // GEMV: do NOT launch with programmatic stream serialization (by default the kernel may
                           // begin -- weight prefetch only -- while the previous kernel of the stream still runs)
};

// Optional prologue of the GEMV (G % 128 == 0 only): the operator that precedes the linear, folded into the
// kernel's staging of X.  kind 0: none; 1: X <- bf16(X + R) (R may be null), input = RMSNorm(X) * Wn, X + R stored to
// Xout (may be null); 2: X is a [M, 2K] gate|up row, input = silu(gate) * up.
struct GemvPrologue {
  int kind = 0;
  int epilogue = 0;  // kEpi*
  const void* R = nullptr;
  const void* Wn = nullptr;
  void* Xout = nullptr;
  float eps = 0.f;
};

// Tensor parallelism over the output rows, with the all-gather fused into the GEMV (all fields zero: off).
// Producer side (world > 0): every output value is stored into the gathered row [M, ld] of EVERY rank through
// peer-mapped pointers -- local column n goes to column seg_dst[i] + (n - start of piece i), the local shard being up
// to three row-concatenated pieces ending at seg_end[0], seg_end[1], N -- and the launch, after its last store, adds
// one to an arrival counter on every rank (release, system scope).
// Consumer side (wait_sig != null): before it reads X the kernel waits (bounded; a time-out sets the device status)
// until its own rank's counter has reached (*epoch + 1) * wait_per_epoch, where wait_per_epoch is the number of
// signals per use of the counter -- ONE per producing launch and rank, sent by the launch's last CTA after every CTA
// has counted itself in on a device-scope counter -- and *epoch counts completed uses (the decode step).
// Counters only ever grow.
constexpr int kMaxTpRanks = 8;
struct GemvTp {
  int world = 0;
  void* y_peer[kMaxTpRanks] = {};
  unsigned* sig_peer[kMaxTpRanks] = {};
  long long ld = 0;
  int seg_end[2] = {0x7fffffff, 0x7fffffff};
  int seg_dst[3] = {0, 0, 0};
  const unsigned* wait_sig = nullptr;
  const int* epoch = nullptr;
  unsigned wait_per_epoch = 0;
  int* local_count = nullptr;
  // Deferred signal: a producer with `defer` set stores its outputs and does nothing else; the NEXT kernel of the
  // same stream, once it has seen that producer complete, adds one to announce_peer[0..announce_world) before it
  // waits for its own input.
  int defer = 0;
  unsigned* announce_peer[kMaxTpRanks] = {};
  int announce_world = 0;
};

int gemv_launch_ex(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int G,
                   const GemvPrologue& pro, const Workspace& ws, int flags, int sm_count, cudaStream_t stream,
                   const GemvTp* tp = nullptr);
// CTAs gemv_launch_ex launches for this shape (what a consumer of its fused all-gather has to wait for, per rank).
size_t gemv_grid(int M, int N, int K, int G, int flags, int sm_count, size_t partial_cap, int counters_cap);
int gemv_launch(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int G,
                const Workspace& ws, int flags, int sm_count, cudaStream_t stream);
int gemm_launch(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int G,
                const Workspace& ws, int flags, int sm_count, cudaStream_t stream);
int quantize_launch(const void* W, void* Wq, void* S, int N, int K, int G, cudaStream_t stream);

int decode_attention_fused_launch(const void* qkv, const void* bias, const void* inv_freq, const void* pos,
                                  void* cache_k, void* cache_v, void* out, void* workspace, int Hq, int Hk, int D,
                                  int max_len, const GemvTp* tp, int flags, int* status, cudaStream_t stream);
// The status word of the current device's scratch (created on first use); rc receives 0 or an error code.
int* device_status_word(int* rc);
int tp_wait_launch(const void* wait_sig, const void* epoch, unsigned wait_per_epoch, int* status, cudaStream_t stream,
                   const GemvTp* announce = nullptr, int advance_epoch = 0);
int rope_kv_store_launch(void* qkv, const void* bias, const void* inv_freq, const void* pos, void* cache_k,
                         void* cache_v, int Hq, int Hk, int D, int max_len, const void* wait_sig, const void* epoch,
                         unsigned wait_per_epoch, int* status, cudaStream_t stream);

// The register-streaming GEMV (w4_gemv_stream.cu): G % 128 == 0, K % 128 == 0, Wq 16-byte aligned, no kFlagFloatX.
// gemv_stream_launch returns kStreamNotApplicable when no plan fits (the staged X does not fit in shared memory and
// K may not be split): the caller falls back to the ring kernel.  Arguments are validated by the caller.
constexpr int kStreamNotApplicable = 0x40000000;
bool gemv_stream_applies(const void* Wq, int M, int N, int K, int G, int flags);
int gemv_stream_launch(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int G,
                       const GemvPrologue& pro, const Workspace& ws, int flags, int sm_count, cudaStream_t stream,
                       const GemvTp* tp);
size_t gemv_stream_grid(int M, int N, int K, int G, int flags, int sm_count, size_t partial_cap);
int gemv_stream_describe(int M, int N, int K, int G, int flags, int sm_count, size_t partial_cap, int counters_cap,
                         char* buf, int buflen);
int gemv_describe(int M, int N, int K, int G, int flags, int sm_count, size_t partial_cap, int counters_cap, char* buf,
                  int buflen);
size_t gemv_stream_scratch_bytes(int M, int N, int K, int G, int flags, int sm_count, size_t partial_cap);

// The many-token GEMV (w4_gemv_mid.cu): 2 <= M <= 16, G == 128, K % 256 == 0, a converted X
// that fits in shared memory -- whole, or, with split-K scratch, in up to eight slices of K across CTAs; plain launches only
// (no prologue, epilogue or tensor-parallel form).
bool gemv_mid_applies(const void* X, const void* Wq, const void* S, int M, int N, int K, int G, int flags,
                      int sm_count, size_t partial_cap);
int gemv_mid_launch(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, const Workspace& ws,
                    int flags, int sm_count, cudaStream_t stream);
int gemv_mid_describe(int M, int N, int K, int flags, int sm_count, size_t partial_cap, char* buf, int buflen);
size_t gemv_mid_scratch_bytes(int M, int N, int K, int flags, int sm_count, size_t partial_cap);

// Status word of b2_w4_gemv_noalloc's fixed scratch array (w4_gemv_noalloc.cu); false when that entry point has not
// run on the device.
bool noalloc_status_word(int dev, int* word);
bool noalloc_clear(int dev);

// Scratch bytes gemv_launch would use for this shape (0 when it runs without split-K).
size_t gemv_scratch_bytes(int M, int N, int K, int G, int flags, int sm_count, size_t partial_cap);

}  // namespace b2
