// Device-side pieces shared by the two decode-GEMV kernels (the shared-memory ring kernel in w4_gemv.cu and the
// register-streaming kernel in w4_gemv_stream.cu): the parameter block, the integer mma wrappers, the loads of X
// with the optional prologue operators, the tensor-parallel epilogue and the split-K sums.
#pragma once
#include <cuda_fp16.h>

#include "ptx.cuh"
#include "w4_common.cuh"
#include "w4_internal.h"

namespace b2 {

// What the kernel does to its input before the product (the operators that precede a linear in a decoder layer)
// kProStaged: X is not activations but their converted form, as the kEpiSwigluStaged epilogue of the producing GEMV left
// it: four digit planes of K bytes, then one 32-byte info block per 128-chunk (streaming kernel, one token).
enum : int { kProNone = 0, kProAddRmsNorm = 1, kProSwiglu = 2, kProStaged = 3 };
// Epilogues (bits above the prologue kind in the `prologue` argument of the fused entry points).
// kEpiSwigluPairs8: as kEpiSwigluPairs with row blocks of 8 gate + 8 up rows (16 rows per warp instead of 32).
enum : int { kEpiNone = 0, kEpiSwigluPairs = 1, kEpiSwigluStaged = 2, kEpiSwigluPairs8 = 3, kEpiShift = 8 };

struct GemvParams {
  const __nv_bfloat16* X;
  const __nv_bfloat16* S;
  __nv_bfloat16* Y;
  int M, N, K, G;
  int KG;           // K / G
  int gdiv;         // chunks per quantization group (G / 128), 1 when G < 128
  int nchunks;      // ceil(K / 128)
  int nrg;          // ceil(N / 32)
  int nslices;      // CTAs sharing one row group along K
  int cps;          // chunks per slice
  int ntiles;       // nrg * nslices
  int nstages;
  int xs_m_stride;  // bytes between tokens of the staged X
  int sc_async;     // 0, or the width in bytes (4, 8, 16) of the cp.async copies with which the producer warp
                    // stages the scales of every ring stage in shared memory
  float* partial;   // [nslices][M][N]
  int* counters;    // [nrg]
  int* status;
  // prologue (fast path only)
  int pro;                    // kPro*
  const __nv_bfloat16* R;     // add + RMSNorm: residual to add to X first (may be null)
  const __nv_bfloat16* Wn;    // add + RMSNorm: norm weights [K]
  __nv_bfloat16* Xout;        // add + RMSNorm: where X + R is stored (may be null)
  float eps;
  GemvTp tp;                  // tensor-parallel epilogue / input wait (all zero: off)
  // integer path, optional: X staged once by w4_stage_x_kernel ([M][nchunks] chunks of 128 L bytes, and the
  // per-(token, chunk) info) instead of by every CTA; null = every CTA converts its own slice
  const unsigned char* pre_x;
  const int4* pre_info;
  int sum_kernel;  // split-K: the partial sums are added up by w4_sum_slices_kernel behind this kernel, not by the last CTA
};

__device__ __forceinline__ void consumer_sync(int nthreads) {
  asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
}

// D[16x8] = A[16x32] * B[32x8] + C, 8-bit integer inputs, 32-bit accumulate.  A is unsigned (nibbles, or nibbles
// times 16); B is unsigned (a low byte of X) or signed (its top byte).
// d = A * B + {c0, c1, c0, c1}: the first product of a chain takes its initial value without register moves.
__device__ __forceinline__ void imma_16832_init(bool b_signed, int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                uint32_t a3, uint32_t b0, uint32_t b1, int c0, int c1) {
  if (b_signed)
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%10,%11};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c0), "r"(c1));
  else
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%10,%11};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c0), "r"(c1));
}
__device__ __forceinline__ void imma_16832(bool b_signed, int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                           uint32_t a3, uint32_t b0, uint32_t b1) {
  if (b_signed)  // a compile-time constant at every call site after unrolling
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  else
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Loads of activations, scales and norm weights go to L2 (ld.global.cg), never through the non-coherent path: a
// kernel launched with programmatic stream serialization becomes resident while earlier kernels still run, so the
// SM's L1 is not invalidated between the producer of the data and this load, and a cached line can be stale
// (observed: wrong scales after a library GEMV that triggers its dependents early).
template <typename T>
__device__ __forceinline__ T ld_l2(const T* p) {
  return __ldcg(p);
}

__device__ __forceinline__ void unpack8_bf16(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ uint4 pack8_bf16(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

// The eight input values x[m, k0..k0+8) as the product sees them, as bf16 bits.  With a prologue they are
// what the separate operator would have stored in bf16: RMSNorm of the (bf16-rounded) sum X + R times the norm
// weight (semantics of ns_rmsnorm), or silu(gate) * up of a [M, 2K] gate|up row (semantics of ns_swiglu).
__device__ __forceinline__ uint4 load_x_unit(const GemvParams& p, int m, int k0, const float* inv) {
  if (p.pro == kProNone) return ld_l2(reinterpret_cast<const uint4*>(p.X + (size_t)m * p.K + k0));
  float a[8], b[8];
  if (p.pro == kProSwiglu) {
    unpack8_bf16(ld_l2(reinterpret_cast<const uint4*>(p.X + (size_t)m * 2 * p.K + k0)), a);
    unpack8_bf16(ld_l2(reinterpret_cast<const uint4*>(p.X + (size_t)m * 2 * p.K + p.K + k0)), b);
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = a[e] / (1.f + __expf(-a[e])) * b[e];
    return pack8_bf16(a);
  }
  unpack8_bf16(ld_l2(reinterpret_cast<const uint4*>(p.X + (size_t)m * p.K + k0)), a);
  if (p.R != nullptr) {
    unpack8_bf16(ld_l2(reinterpret_cast<const uint4*>(p.R + (size_t)m * p.K + k0)), b);
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = __bfloat162float(__float2bfloat16(a[e] + b[e]));
  }
  unpack8_bf16(ld_l2(reinterpret_cast<const uint4*>(p.Wn + k0)), b);
  const float s = inv[m];
#pragma unroll
  for (int e = 0; e < 8; ++e) a[e] = a[e] * s * b[e];
  return pack8_bf16(a);
}

// add + RMSNorm prologue, first pass: every CTA computes 1 / rms of each token's full row of X + R (the row is a
// few KB; recomputing it per CTA is cheaper than another launch); CTA 0 also stores X + R to Xout.
template <int CT>
__device__ __forceinline__ void rmsnorm_factors(const GemvParams& p, float* ss, float* inv, int ctid) {
  const int warp = ctid >> 5, lane = ctid & 31, nw = CT / 32;
  const int units = p.K / 8;
  for (int m = 0; m < p.M; ++m) {
    float acc = 0.f;
    for (int u = ctid; u < units; u += CT) {
      float a[8], b[8];
      unpack8_bf16(ld_l2(reinterpret_cast<const uint4*>(p.X + (size_t)m * p.K + u * 8)), a);
      if (p.R != nullptr) {
        unpack8_bf16(ld_l2(reinterpret_cast<const uint4*>(p.R + (size_t)m * p.K + u * 8)), b);
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = __bfloat162float(__float2bfloat16(a[e] + b[e]));
        if (blockIdx.x == 0 && p.Xout != nullptr)
          *reinterpret_cast<uint4*>(p.Xout + (size_t)m * p.K + u * 8) = pack8_bf16(a);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) acc += a[e] * a[e];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) ss[m * 16 + warp] = acc;
  }
  consumer_sync(CT);
  if (ctid < p.M) {
    float t = 0.f;
    for (int w = 0; w < nw; ++w) t += ss[ctid * 16 + w];
    inv[ctid] = rsqrtf(t / p.K + p.eps);
  }
  consumer_sync(CT);
}

// ---- tensor parallelism: the all-gather of Y fused into the epilogue -------------------------------------
// Global column of local output column n: the local shard is up to three row-concatenated pieces (q | k | v,
// gate | up), each of which lands at its own offset of the gathered row.
__device__ __forceinline__ int tp_column(const GemvTp& tp, int n) {
  int c = tp.seg_dst[0] + n;
  if (n >= tp.seg_end[0]) c = tp.seg_dst[1] + (n - tp.seg_end[0]);
  if (n >= tp.seg_end[1]) c = tp.seg_dst[2] + (n - tp.seg_end[1]);
  return c;
}
// One output value into the gathered row of every rank (plain stores through peer-mapped pointers).
__device__ __forceinline__ void tp_store(const GemvTp& tp, int tok, int n, __nv_bfloat16 v) {
  const size_t at = (size_t)tok * tp.ld + tp_column(tp, n);
  for (int r = 0; r < tp.world; ++r) static_cast<__nv_bfloat16*>(tp.y_peer[r])[at] = v;
}
// Four consecutive outputs of one token (n0 a multiple of 4) rounded to bf16: into Y or, tensor parallel, into the
// gathered row of every rank.  One 8-byte store where the four land side by side on an 8-byte boundary.
__device__ __forceinline__ void store_out4(const GemvParams& p, int tok, int n0, const float4& v) {
  if (n0 >= p.N) return;
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  const uint2 pk = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
  const __nv_bfloat16 e[4] = {lo.x, lo.y, hi.x, hi.y};
  const bool whole = n0 + 3 < p.N;
  if (p.tp.world) {
    const int c0 = tp_column(p.tp, n0);
    const size_t at = (size_t)tok * p.tp.ld + c0;
    const bool side_by_side = whole && tp_column(p.tp, n0 + 3) == c0 + 3;
    for (int r = 0; r < p.tp.world; ++r) {
      __nv_bfloat16* y = static_cast<__nv_bfloat16*>(p.tp.y_peer[r]);
      if (side_by_side && (reinterpret_cast<uintptr_t>(y + at) & 7) == 0) {
        *reinterpret_cast<uint2*>(y + at) = pk;
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (n0 + i < p.N) y[(size_t)tok * p.tp.ld + tp_column(p.tp, n0 + i)] = e[i];
      }
    }
    return;
  }
  __nv_bfloat16* y = p.Y + (size_t)tok * p.N + n0;
  if (whole && (reinterpret_cast<uintptr_t>(y) & 7) == 0) {
    *reinterpret_cast<uint2*>(y) = pk;
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (n0 + i < p.N) y[i] = e[i];
  }
}
// Split-K: the partial sums of all slices for four consecutive outputs of one token, added in slice order.
__device__ __forceinline__ float4 sum_slices4(const GemvParams& p, int tok, int n0) {
  const float* s0 = p.partial + (size_t)tok * p.N + n0;
  const size_t qstride = (size_t)p.M * p.N;
  float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
  if ((p.N & 3) == 0 && n0 + 3 < p.N) {
    // sixteen slices' loads in flight together (an L2 round trip takes a microsecond under the weight stream, and
    // this kernel is nothing but round trips: with four at a time ten slices took three of them)
    constexpr int kInFlight = 16;
    for (int q0 = 0; q0 < p.nslices; q0 += kInFlight) {
      float4 v[kInFlight];
#pragma unroll
      for (int i = 0; i < kInFlight; ++i)
        if (q0 + i < p.nslices) v[i] = __ldcg(reinterpret_cast<const float4*>(s0 + (q0 + i) * qstride));
#pragma unroll
      for (int i = 0; i < kInFlight; ++i)
        if (q0 + i < p.nslices) {
          sum.x += v[i].x;
          sum.y += v[i].y;
          sum.z += v[i].z;
          sum.w += v[i].w;
        }
    }
  } else {
    float f[4] = {0.f, 0.f, 0.f, 0.f};
    for (int q = 0; q < p.nslices; ++q)
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (n0 + i < p.N) f[i] += __ldcg(s0 + q * qstride + i);
    sum = make_float4(f[0], f[1], f[2], f[3]);
  }
  return sum;
}
// Called by one warp of every CTA when all of the CTA's outputs have been stored.  System-scope releases are dear
// (a release per CTA cost 6 us per launch, an explicit system fence on top of it 13 us), so the CTAs first count
// themselves in on a device-scope counter of their own GPU; the last one to arrive -- which has thereby observed the
// stores of all the others -- resets that counter and adds one, with release at system scope, to the arrival counter
// of every rank: one signal per launch and rank.
__device__ __forceinline__ void tp_signal(const GemvTp& tp, int lane) {
  __syncwarp();
  int last = 0;
  if (lane == 0) {
    __threadfence();
    last = atomicAdd(tp.local_count, 1) == (int)gridDim.x - 1;
    if (last) {
      *tp.local_count = 0;  // ready for the next launch (launches sharing the counter are stream-ordered)
      __threadfence();
    }
  }
  last = __shfl_sync(0xffffffffu, last, 0);
  if (last && lane < tp.world) {
    asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(tp.sig_peer[lane]) : "memory");
  }
}
// Deferred signal, consumer side: called by one warp of one CTA after the kernel has seen the previous kernel of its
// stream complete (programmatic wait or plain stream order).  That kernel's stores into the peers' memory happen
// before this release in causality order, so a peer that acquires the counter sees them.
__device__ __forceinline__ void tp_announce(const GemvTp& tp, int lane) {
  if (lane < tp.announce_world)
    asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(tp.announce_peer[lane]) : "memory");
}
// Waits (bounded) until every producing launch of every rank has counted itself in on this rank's counter for the
// current epoch.  One thread polls; the caller synchronises the rest.  Returns false on time-out.
__device__ __forceinline__ bool tp_wait(const GemvTp& tp, volatile int* abort_flag) {
  const unsigned target = ((unsigned)*reinterpret_cast<const volatile int*>(tp.epoch) + 1u) * tp.wait_per_epoch;
  const long long t0 = clock64();
  for (;;) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(tp.wait_sig) : "memory");
    if ((int)(v - target) >= 0) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitLimitCycles) {
      *abort_flag = 1;
      return false;
    }
    __nanosleep(40);
  }
}

// Launches w4_sum_slices_kernel behind a split-K GEMV whose CTAs left their partial sums in p.partial.
int launch_sum_slices(const GemvParams& p, int sm_count, bool pdl, cudaStream_t stream);

}  // namespace b2
