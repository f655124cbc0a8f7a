// W4A16 decode GEMV for sm_100a:  Y[M,N] (bf16) = X[M,K] (bf16) . dequant(Wq, S)^T,  1 <= M <= 16.
//
// Replaces the reference's w4a16_gemv_kernel / w4a16_gemv (kernels/quant/w4a16.cuh:42-115), which
// serves M in {1,2,4,8} only on CUDA cores.  Same operands, same weight format, fp32 accumulation.
//
// Structure (HBM-bound: every weight byte is read exactly once, X is tiny and lives in shared memory):
//   * Persistent CTAs: two half-SM CTAs per SM where they fit (8 consumer warps + producer + reducer), else one wide
//     CTA (14 or 16 consumer warps); the host picks with a cost model.  Lane 0 of the producer warp streams the
//     packed weights of a 32-row group into a shared-memory ring with tiled TMA loads through a tensor map over Wq:
//     boxes of 32 rows x 128 bytes (two K chunks) with the 128-byte swizzle, NCW/2 boxes per stage, completion counted
//     on an mbarrier; several stages are in flight from the first instruction.  (Per-row untiled bulk copies were
//     measured first: the TMA unit retires about one copy per 70 cycles whatever its size, so 1 KB row segments cap
//     near 4 TB/s; tiled boxes reach the copy-kernel bandwidth.)  The other producer lanes copy the stage's scales
//     with cp.async (8 or 16 bytes per copy) onto the same mbarrier: under the weight stream a dependent global load
//     costs a microsecond or more, so the consumers never issue one.
//   * NCW consumer warps each take one 128-wide K chunk of the stage for both 16-row blocks.  A lane reads 16 bytes
//     (32 nibbles) per row with one 128-bit shared load; the swizzle plus a fixed permutation of which tile row feeds
//     which mma row makes those loads bank-conflict free.
//   * Launched with programmatic stream serialization: the weight stream starts while the previous kernel of the
//     stream drains; X, Y and scratch are touched only after griddepcontrol.wait.  Every load of activations, scales
//     and norm weights goes to L2 (ld.global.cg): under such a launch the SM's L1 is not invalidated between the
//     producer of the data and the load.
//   * K reduction: inside the mma across the four lanes of a quad, then across warps through shared memory: the
//     consumer warps drop their partial sums of a finished row group into one of two buffers and move on, a reducer
//     warp sums them and stores Y (mbarrier hand-off, nobody blocks).  Only when K is split across CTAs to fill the
//     machine, fp32 partials go through scratch memory and are summed in fixed order by the last CTA to arrive (an
//     atomic counter per row group; nobody waits on anybody, the result is deterministic).
//   * Optional prologue: the operator that precedes the linear (add + RMSNorm, SwiGLU) is evaluated while X is staged.
//   * Optional tensor-parallel epilogue: outputs go straight into the gathered row of every rank (peer stores), one
//     arrival signal per launch and rank; the consumer side waits on its rank's counter before it reads X.
//
// Arithmetic, by mode:
//   * integer (default for G % 128 == 0): (w & 0x0F0F0F0F) holds the four even-k nibbles of a word as bytes,
//     (w & 0xF0F0F0F0) the four odd-k nibbles times 16: ready-made unsigned A fragments of mma.sync.m16n8k32 (s32
//     accumulate), two LOP3 per eight weights, no shift, no conversion.  X is staged as block fixed point: per
//     (token, 128-chunk) scaled by a power of two so that the largest magnitude lands in [2^14, 2^15) (or [2^22, 2^23)),
//     rounded to an integer and split into 2 (or 3) byte planes, the low ones unsigned, the top one signed.  Every
//     plane has its own accumulators, even and odd nibbles apart; one combination per chunk gives
//     16 sum_k (q_k - 8) v_k exactly -- the zero-point is the initial value of an accumulator -- then one
//     int-to-float conversion, times group scale and the chunk's power of two, fp32 accumulation over the chunks.
//   * fp16 (kFlagFloatX): one shift and four LOP3 per word turn eight nibbles into four fp16x2 registers
//     {1024 + q[p], 1024 + q[p+4]} / {1024 + 16 q[p], 1024 + 16 q[p+4]}; one packed-half FMA per register gives q - 8
//     exactly; mma.sync.m16n8k16 (f16 inputs, fp32 accumulate).  X is staged as fp16 after an exact power-of-two
//     normalisation per (token, chunk).  With kFlagFoldZeroPoint the -8 is one fp32 correction per chunk instead.
//     The contraction index of an mma is a dummy, so the pairing {p, p+4} the unpack produces is matched by permuting
//     X when it is staged; the weights are never shuffled.
//   * generic (G < 128): each lane scales its own words in bf16 (the rounding the reference's tensor-core path
//     applies) on a bf16 mma.
//   Tokens sit on the n-side of the mma (8 per tile, two tiles for M > 8).  The integer/logic pipe runs at half rate
//   on this SM and a warp issues about one instruction per ten cycles at the occupancy this kernel reaches, so the
//   instruction count on a warp's path, not the issue-slot utilisation, sets the run time.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>
#include <type_traits>
#include <cuda_fp16.h>

#include "ptx.cuh"
#include "tensor_map.h"
#include "w4_common.cuh"
#include "w4_gemv_shared.cuh"
#include "w4_internal.h"

namespace b2 {

namespace {

constexpr int kRowsPerGroup = 32;      // rows of W per stage / tile
constexpr int kChunkK = 128;           // K elements per consumer-warp work item
constexpr int kRedPitch = 36;          // floats per (warp, token) row of the reduction buffer: 32 + 4 pad
constexpr int kMaxStages = 8;
constexpr int kSmemLimit = 232448;     // 227 KB opt-in maximum per CTA on sm_100
constexpr int kHeaderBytes = 2048;     // flags + barriers (256 B), 512 B of zeros, RMSNorm partial sums and factors
constexpr int kZeroOffset = 256;       // 512 bytes of zeros: the staged X and info of padding tokens
constexpr int kNormSsOffset = 768;     // float [16 tokens][16 warps]
constexpr int kNormInvOffset = 1792;   // float [16 tokens]
constexpr int kBoxBytes = kRowsPerGroup * 128;  // 32 rows x 128 B (two chunks), swizzled

enum : int { kModeGeneric = 0, kModeExact = 1, kModeFold = 2, kModeI8x2 = 3, kModeI8x3 = 4 };
// bytes of one staged (token, 128-chunk) of X and of its info record
__host__ __device__ constexpr int mode_limbs(int mode) { return mode == kModeI8x2 ? 2 : (mode == kModeI8x3 ? 3 : 0); }
__host__ __device__ constexpr int x_chunk_bytes(int mode) { return mode_limbs(mode) ? 128 * mode_limbs(mode) : 256; }
__host__ __device__ constexpr int x_info_bytes(int mode) { return mode_limbs(mode) ? 16 : 8; }

// two buffers of [consumer warp][token < M][kRedPitch] floats
__host__ __device__ constexpr int red_bytes(int ncw, int m) { return (2 * ncw * m * kRedPitch * 4 + 127) & ~127; }


// (a & b) | c in one LOP3 with both constants held in registers.
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t hadd2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// D[16x8] (+)= A[16x16] * B[16x8], fp16 inputs, fp32 accumulate.
__device__ __forceinline__ void mma_16816_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_16816_f16_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                   uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
  unsigned short v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}

// ---- staging of X -------------------------------------------------------------------------------
// Every 16-byte unit holds the 8 values x[b..b+8) of one token as four pairs {x[b+p], x[b+p+4]},
// p = 0..3 -- the pairing the unpack produces.  Unit (j, t) of a chunk (k = 128 c + 32 t + 8 j) sits at
// byte (j*4 + t) * 16 of the chunk's 256 bytes.  16 consecutive units (one half-warp) make up one
// (token, chunk).

// bf16 staging for the generic path: values are only permuted.
template <int CT>
__device__ __forceinline__ void stage_x_bf16(const GemvParams& p, uint32_t xs_base, int cb, int ce, int ctid) {
  const int nch = ce - cb;
  const int units = p.M * nch * 16;
  for (int u = ctid; u < units; u += CT) {
    const int m = u / (nch * 16);
    const int r = u - m * nch * 16;
    const int ch = r >> 4, jt = r & 15;
    const int j = jt >> 2, t = jt & 3;
    const int k0 = (cb + ch) * kChunkK + 32 * t + 8 * j;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (k0 < p.K) v = ld_l2(reinterpret_cast<const uint4*>(p.X + (size_t)m * p.K + k0));
    uint4 o;
    o.x = __byte_perm(v.x, v.z, 0x5410);  // {x0, x4}
    o.y = __byte_perm(v.x, v.z, 0x7632);  // {x1, x5}
    o.z = __byte_perm(v.y, v.w, 0x5410);  // {x2, x6}
    o.w = __byte_perm(v.y, v.w, 0x7632);  // {x3, x7}
    sts128(xs_base + m * p.xs_m_stride + ch * 256 + jt * 16, o);
  }
}


// fp16 staging for the fast path.  Per (token, chunk): e = biased exponent of the largest |x| (clamped),
// x is multiplied by 2^(141 - e) (largest magnitude lands in [2^14, 2^15)) and converted to fp16;
// xinfo[token][chunk] = { 2^(e - 141), correction }.  FOLD: the odd in-word positions are stored
// divided by 16 (their weights arrive as 1024 + 16 q) and correction = sum of offset * stored value.
template <int CT, bool FOLD>
__device__ __forceinline__ void stage_x_f16(const GemvParams& p, uint32_t xs_base, float2* xinfo, const float* inv,
                                            int cb, int ce, int ctid) {
  const int nch = ce - cb;
  const int units = p.M * nch * 16;
  const int units_pad = (units + 31) & ~31;
  for (int u = ctid; u < units_pad; u += CT) {
    const bool valid = u < units;
    int m = 0, ch = 0, jt = 0;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (valid) {
      m = u / (nch * 16);
      const int r = u - m * nch * 16;
      ch = r >> 4;
      jt = r & 15;
      const int k0 = (cb + ch) * kChunkK + 32 * (jt & 3) + 8 * (jt >> 2);
      if (k0 < p.K) v = load_x_unit(p, m, k0, inv);
    }
    // largest magnitude of the chunk: bf16 magnitudes order like their 15-bit patterns
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t mx = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) mx = max(mx, max(w[i] & 0x7FFFu, (w[i] >> 16) & 0x7FFFu));
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    uint32_t eb = mx >> 7;
    eb = eb == 255u ? 141u : min(254u, max(15u, eb));  // inf/nan: convert unscaled; tiny: clamp
    const float down = __uint_as_float((268u - eb) << 23);
    const float up = __uint_as_float((eb - 14u) << 23);
    float f[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16) * down;
      f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u) * down;
    }
    if (FOLD) {
#pragma unroll
      for (int i = 1; i < 8; i += 2) f[i] *= 0.0625f;
    }
    __half h[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) h[i] = __float2half_rn(f[i]);
    float corr = 0.f;
    if (FOLD) {
#pragma unroll
      for (int i = 0; i < 8; ++i) corr = fmaf((i & 1) ? 1152.f : 1032.f, __half2float(h[i]), corr);
      corr += __shfl_xor_sync(0xffffffffu, corr, 8);
      corr += __shfl_xor_sync(0xffffffffu, corr, 4);
      corr += __shfl_xor_sync(0xffffffffu, corr, 2);
      corr += __shfl_xor_sync(0xffffffffu, corr, 1);
    }
    if (valid) {
      auto pack = [&](int a, int b) {
        return (uint32_t)__half_as_ushort(h[a]) | ((uint32_t)__half_as_ushort(h[b]) << 16);
      };
      sts128(xs_base + m * p.xs_m_stride + ch * 256 + jt * 16,
             make_uint4(pack(0, 4), pack(1, 5), pack(2, 6), pack(3, 7)));
      if ((u & 15) == 0) xinfo[m * nch + ch] = make_float2(up, corr);
    }
  }
}

// 8-bit staging for the integer path (L = 2 or 3 bytes per value).  Per (token, chunk): e = biased exponent of the
// largest |x| (clamped); every x is multiplied by 2^(8L - 2 - (e - 127)) -- the largest magnitude lands in
// [2^(8L-2), 2^(8L-1)) -- and rounded to an integer v of 8L bits (exact for every x within 2^(8L-9) of the largest:
// bf16 has 8 significant bits).  Byte l of v's two's complement is "limb" l: the low limbs are unsigned, the top one
// is signed, v = sum of 256^l limb_l.  A work item is 16 consecutive k of one token (two packed weight words of a
// lane); it stores, per limb, one 16-byte unit { even k of word 0, even k of word 1, odd k of word 0, odd k of
// word 1 }, four bytes each: the B fragments of one even-nibble and one odd-nibble mma.  Unit (jj, t)
// (k = 128 c + 32 t + 16 jj) of limb l sits at byte l * 128 + (jj * 4 + t) * 16 of the chunk's 128 L bytes.
// xinfo[token][chunk] = { bits of 2^(e - 127 - (8L - 2)) / 16, -128 * sum_k limb_l(v_k) for l = 0, 1, 2 }: the
// zero-point 8, times the 16 that the nibble products carry, as the initial value of an accumulator.  A chunk that
// holds an inf or a nan gets a nan factor (its integers are meaningless), so the outputs become nan.
// GLOBAL: the same bytes go to global memory (gx: [M][nch] chunks of 128 L bytes, xinfo: [M][nch]) for every CTA of a
// later kernel to copy; `ctid` / `nthreads` are then grid-wide.
template <int L, bool GLOBAL>
__device__ __forceinline__ void stage_x_i8(const GemvParams& p, uint32_t xs_base, int4* xinfo, const float* inv,
                                           int cb, int ce, int ctid, int nthreads, unsigned char* gx = nullptr) {
  constexpr int B = 8 * L;
  // items in flight per thread: a load from L2 takes a microsecond under the weight stream, so the loads of several
  // items are issued before the first is converted
  constexpr int UN = GLOBAL ? 1 : 4;
  const int nch = ce - cb;
  const int items = p.M * nch * 8;
  const int items_pad = (items + 31) & ~31;
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  for (int it0 = ctid; it0 < items_pad; it0 += nthreads * UN) {
    uint4 va[UN], vb[UN];
#pragma unroll
    for (int q = 0; q < UN; ++q) {
      va[q] = zero4;
      vb[q] = zero4;
      const int it = it0 + q * nthreads;
      if (it < items) {
        const int m = it / (nch * 8);
        const int r = it - m * nch * 8;
        const int k0 = (cb + (r >> 3)) * kChunkK + 32 * (r & 3) + 16 * ((r & 7) >> 2);
        if (k0 < p.K) {
          va[q] = load_x_unit(p, m, k0, inv);
          vb[q] = load_x_unit(p, m, k0 + 8, inv);
        }
      }
    }
#pragma unroll
    for (int q = 0; q < UN; ++q) {
      const int it = it0 + q * nthreads;
      if (it >= items_pad) break;  // whole warps leave together: the shuffles below stay converged
      const bool valid = it < items;
      int m = 0, ch = 0, u = 0;
      if (valid) {
        m = it / (nch * 8);
        const int r = it - m * nch * 8;
        ch = r >> 3;
        u = r & 7;
      }
      const uint32_t w[8] = {va[q].x, va[q].y, va[q].z, va[q].w, vb[q].x, vb[q].y, vb[q].z, vb[q].w};
      uint32_t mx = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) mx = max(mx, max(w[i] & 0x7FFFu, (w[i] >> 16) & 0x7FFFu));
      mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      uint32_t eb = mx >> 7;
      const bool bad = eb == 255u;
      eb = min(254u, max(40u, eb));
      const float down = __uint_as_float((uint32_t)(B + 252 - (int)eb) << 23);
      const uint32_t up_bits = bad ? 0x7FC00000u : (uint32_t)((int)eb - B - 2) << 23;
      int v[16];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[2 * i] = __float2int_rn(__uint_as_float(w[i] << 16) * down);
        v[2 * i + 1] = __float2int_rn(__uint_as_float(w[i] & 0xFFFF0000u) * down);
      }
      int csum[3] = {0, 0, 0};
#pragma unroll
      for (int l = 0; l < L; ++l) {
        const uint32_t sel = (uint32_t)l | ((uint32_t)(4 + l) << 4);
        auto pack = [&](int a, int b, int c, int d) {
          return __byte_perm(__byte_perm((uint32_t)v[a], (uint32_t)v[b], sel),
                             __byte_perm((uint32_t)v[c], (uint32_t)v[d], sel), 0x5410);
        };
        const uint4 o = make_uint4(pack(0, 2, 4, 6), pack(8, 10, 12, 14), pack(1, 3, 5, 7), pack(9, 11, 13, 15));
        int c;
        if (l == L - 1) {
          c = __dp4a((int)o.x, 0x01010101, 0);
          c = __dp4a((int)o.y, 0x01010101, c);
          c = __dp4a((int)o.z, 0x01010101, c);
          c = __dp4a((int)o.w, 0x01010101, c);
        } else {
          uint32_t cu = __dp4a(o.x, 0x01010101u, 0u);
          cu = __dp4a(o.y, 0x01010101u, cu);
          cu = __dp4a(o.z, 0x01010101u, cu);
          cu = __dp4a(o.w, 0x01010101u, cu);
          c = (int)cu;
        }
        c += __shfl_xor_sync(0xffffffffu, c, 4);
        c += __shfl_xor_sync(0xffffffffu, c, 2);
        c += __shfl_xor_sync(0xffffffffu, c, 1);
        csum[l] = -128 * c;
        if constexpr (GLOBAL) {
          if (valid) __stcg(reinterpret_cast<uint4*>(gx + ((size_t)m * nch + ch) * (128 * L) + l * 128 + u * 16), o);
        } else {
          if (valid) sts128(xs_base + m * p.xs_m_stride + ch * (128 * L) + l * 128 + u * 16, o);
        }
      }
      if (valid && u == 0) {
        const int4 info = make_int4((int)up_bits, csum[0], csum[1], csum[2]);
        if constexpr (GLOBAL)
          __stcg(xinfo + m * nch + ch, info);
        else
          xinfo[m * nch + ch] = info;
      }
    }
  }
}

// Copy of a slice [cb, ce) of the pre-staged X and its info into the CTA's shared memory with 16-byte asynchronous
// copies through L2 (the staging kernel may have finished only just before, under programmatic launch).
template <int L>
__device__ __forceinline__ void copy_staged_x(const GemvParams& p, uint32_t xs_base, uint32_t xinfo_base, int cb, int ce,
                                              int ctid, int nthreads) {
  const int nch = ce - cb;
  const int nx = nch * (8 * L);  // 16-byte units of X per token
  const int per = nx + nch;      // ... plus one unit of info per chunk
  const int total = p.M * per;
  const uint4* gx = reinterpret_cast<const uint4*>(p.pre_x);
  const uint4* gi = reinterpret_cast<const uint4*>(p.pre_info);
  for (int it = ctid; it < total; it += nthreads) {
    const int m = it / per, r = it - m * per;
    const bool is_x = r < nx;
    const uint4* src = is_x ? gx + ((size_t)m * p.nchunks + cb) * (8 * L) + r : gi + (size_t)m * p.nchunks + cb + (r - nx);
    const uint32_t dst = is_x ? xs_base + m * p.xs_m_stride + r * 16 : xinfo_base + (m * nch + (r - nx)) * 16;
    cp_async_cg16(dst, src);  // all copies of a thread are in flight together
  }
  cp_async_wait_all();
}


// X of a launch staged once for all CTAs (integer path, M >= 2 or so: converting M x K values in every CTA costs more
// than one small kernel in front).  One thread per 16 values; launched in front of the GEMV on the same stream.
constexpr int kStageXThreads = 128;
template <int L>
__global__ void __launch_bounds__(kStageXThreads) w4_stage_x_kernel(const GemvParams p) {
  pdl_launch_dependents();  // the GEMV behind may start its weight stream
  pdl_wait_prior_grid();    // X is the previous kernel's output; the staging area may still be read by the previous GEMV
  stage_x_i8<L, true>(p, 0u, const_cast<int4*>(p.pre_info), nullptr, 0, p.nchunks,
                      blockIdx.x * kStageXThreads + threadIdx.x, gridDim.x * kStageXThreads,
                      const_cast<unsigned char*>(p.pre_x));
}

// Split-K without the per-tile hand-shake: behind a GEMV launched with `sum_kernel` set, adds up the partial sums of
// the slices and stores the outputs.  (In the GEMV itself a split tile costs the reducer warp a store, a fence and an
// atomic whose answer it needs: three L2 round trips, 3.5 us per tile measured, one after the other.)
// Small CTAs: launched programmatically, they become resident beside the GEMV's CTAs (which leave few registers
// free) and only then let the next kernel of the stream start its weight stream.
constexpr int kSumThreads = 64;
__global__ void __launch_bounds__(kSumThreads) w4_sum_slices_kernel(const GemvParams p) {
  pdl_launch_dependents();
  pdl_wait_prior_grid();  // all partial sums are in memory once the GEMV has completed
  const int quads = (p.N + 3) >> 2;
  const int total = p.M * quads;
  for (int u = blockIdx.x * kSumThreads + threadIdx.x; u < total; u += gridDim.x * kSumThreads) {
    const int tok = u / quads, n0 = (u - tok * quads) * 4;
    store_out4(p, tok, n0, sum_slices4(p, tok, n0));
  }
}

// MT: token tiles of 8 (1 or 2).  NCW: consumer warps (= chunks per stage, even).  MODE: see kMode*.
// CPW: K chunks a consumer warp takes per ring stage (2: a whole 128-byte box; integer modes with staged scales only).
// An iteration of the consumer loop costs about a quarter of a microsecond of latency whatever it contains, so
// fewer, fatter iterations are cheaper.
template <int MT, int NCW, int MODE, int CPW>
__global__ void __launch_bounds__((NCW + 2) * 32, (MT == 1 && NCW <= 12) ? 2 : 1)
    w4_gemv_kernel(const __grid_constant__ CUtensorMap tmap_w, const GemvParams p) {
  constexpr int kSC = NCW * CPW;  // chunks per stage
  constexpr int kStageBytes = (kSC / 2) * kBoxBytes;
  constexpr int kConsumerThreads = NCW * 32;
  constexpr bool kHalf = MODE != kModeGeneric;  // a chunk lies in one group: its sum is scaled once, in fp32
  constexpr int L = mode_limbs(MODE);           // bytes per staged value of X on the integer path, else 0
  constexpr bool kI8 = L > 0;
  static_assert(CPW == 1 || (CPW == 2 && kI8), "two chunks per warp: integer modes only");
  constexpr int kXChunk = x_chunk_bytes(MODE);
  extern __shared__ __align__(1024) unsigned char smem[];
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem);
  const uint32_t bar_full = smem_u32(smem + 64);
  const uint32_t bar_empty = bar_full + 8 * kMaxStages;
  const uint32_t bar_red_full = bar_empty + 8 * kMaxStages;  // [2] partial sums of a tile are in shared memory
  const uint32_t bar_red_empty = bar_red_full + 16;           // [2] the reducer has consumed them
  const uint32_t zero_base = smem_u32(smem + kZeroOffset);
  float* red = reinterpret_cast<float*>(smem + kHeaderBytes);
  float2* xinfo = reinterpret_cast<float2*>(smem + kHeaderBytes + red_bytes(NCW, p.M));
  const int xinfo_bytes = (p.M * p.cps * x_info_bytes(MODE) + 127) & ~127;
  const uint32_t xs_base = smem_u32(smem + kHeaderBytes + red_bytes(NCW, p.M) + xinfo_bytes);
  const int xs_bytes = (p.M * p.xs_m_stride + 127) & ~127;
  // scales of each ring stage: [32 rows][NCW chunks] bf16, filled by the producer warp with cp.async
  constexpr int kScStage = kHalf ? kRowsPerGroup * kSC * 2 : 0;
  const uint32_t ring_base = (xs_base + xs_bytes + 1023) & ~1023u;  // swizzled boxes: 1024-byte aligned
  const uint32_t sc_base = ring_base + p.nstages * kStageBytes;
  const bool sc_async = kHalf && p.sc_async;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    *abort_flag = 0;
    for (int s = 0; s < p.nstages; ++s) {
      mbar_init(bar_full + 8 * s, sc_async ? 33 : 1);  // the TMA issuer, and each lane's scale copies
      mbar_init(bar_empty + 8 * s, NCW);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_red_full + 8 * b, NCW);
      mbar_init(bar_red_empty + 8 * b, 1);
    }
    fence_mbar_init();
  }
  __syncthreads();
  pdl_launch_dependents();  // let the next kernel in the stream begin its own prologue as SMs free up

  if (warp == NCW) {
    // ------------------------------------------------------------ producer warp
    // Lane 0 issues the TMA boxes of a stage; every lane copies the scales of one row of the stage (cp.async, two
    // bf16 per copy), so the consumers never wait on a global load.
    if (lane == 0) tma_prefetch_desc(&tmap_w);
    int s = 0;
    uint32_t ph = 0;
    for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x) {
      const int sl = tile / p.nrg, rg = tile - sl * p.nrg;
      const int cb = sl * p.cps, ce = min(p.nchunks, cb + p.cps);
      const int row0 = rg * kRowsPerGroup;
      const bool s_ok = row0 + lane < p.N;
      const __nv_bfloat16* s_lane = p.S + (size_t)(s_ok ? row0 + lane : 0) * p.KG;
      for (int c0 = cb; c0 < ce; c0 += kSC) {
        const int nbox = (min(kSC, ce - c0) + 1) >> 1;
        if (lane == 0) mbar_wait_backoff<100>(bar_empty + 8 * s, ph ^ 1, abort_flag);
        __syncwarp();
        if (lane == 0) {
          // out-of-range rows and K columns are zero-filled and still counted in the transaction bytes
          mbar_arrive_expect_tx(bar_full + 8 * s, (uint32_t)(nbox * kBoxBytes));
          for (int b = 0; b < nbox; ++b)
            tma_load_2d(ring_base + s * kStageBytes + b * kBoxBytes, &tmap_w, (c0 + 2 * b) * 16, row0,
                        bar_full + 8 * s);
        }
        if (sc_async) {
          const uint32_t dst = sc_base + s * kScStage + lane * (kSC * 2);
          auto copy_row = [&](auto width) {  // the lane's NCW scales of this stage in copies of `width` bytes
            constexpr int W = decltype(width)::value;
#pragma unroll
            for (int i = 0; i < kSC * 2 / W; ++i) {
              const int c = c0 + i * (W / 2);
              const int left = s_ok ? (ce - c) * 2 : 0;  // valid source bytes from this chunk on
              cp_async<W>(dst + W * i, s_lane + (left > 0 ? c : cb), (uint32_t)min(W, max(0, left)));
            }
          };
          if (p.sc_async == 16) {
            if constexpr (kSC % 8 == 0) copy_row(std::integral_constant<int, 16>{});
          } else if (p.sc_async == 8) {
            if constexpr (kSC % 4 == 0) copy_row(std::integral_constant<int, 8>{});
          } else {
            copy_row(std::integral_constant<int, 4>{});
          }
          cp_async_mbar_arrive_noinc(bar_full + 8 * s);
        }
        if (++s == p.nstages) {
          s = 0;
          ph ^= 1;
        }
      }
    }
    __syncwarp();
  } else if (warp == NCW + 1) {
    // ------------------------------------------------------------ reducer warp
    // Sums the per-warp partial sums of a finished tile while the consumer warps are already on the
    // next one; owns the output stores and the cross-CTA (split-K) reduction.
    constexpr int kRedUnits = 2 * MT;  // (token, four rows) units per lane: 8 MT tokens x 8 row quads / 32 lanes
    int tcount = 0;
    pdl_wait_prior_grid();  // Y, the scratch and the counters may still be in use by the previous kernel
    for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x, ++tcount) {
      const int sl = tile / p.nrg, rg = tile - sl * p.nrg;
      const int row0 = rg * kRowsPerGroup;
      const int b = tcount & 1;
      const float* rbuf = red + b * (NCW * p.M * kRedPitch);
      if (lane == 0) mbar_wait_backoff<100>(bar_red_full + 8 * b, (tcount >> 1) & 1, abort_flag);
      __syncwarp();
      if (p.M == 1) {
        // one token: a row per lane is the shortest instruction sequence
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < NCW; ++w) sum += rbuf[w * kRedPitch + lane];
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_red_empty + 8 * b);
        const int n = row0 + lane;
        if (n < p.N) {
          if (p.nslices > 1)
            __stcg(p.partial + (size_t)sl * p.N + n, sum);
          else if (p.tp.world)
            tp_store(p.tp, 0, n, __float2bfloat16(sum));
          else
            p.Y[n] = __float2bfloat16(sum);
        }
        if (p.nslices > 1 && !p.sum_kernel) {
          __threadfence();
          __syncwarp();
          int last = 0;
          if (lane == 0) {
            const int old = atomicAdd(p.counters + rg, 1);
            last = old == p.nslices - 1;
            if (last) p.counters[rg] = 0;  // ready for the next launch
          }
          last = __shfl_sync(0xffffffffu, last, 0);
          if (last) {
            __threadfence();
            if (n < p.N) {
              float total = 0.f;
              for (int q = 0; q < p.nslices; ++q) total += __ldcg(p.partial + (size_t)q * p.N + n);
              if (p.tp.world)
                tp_store(p.tp, 0, n, __float2bfloat16(total));
              else
                p.Y[n] = __float2bfloat16(total);
            }
          }
        }
        continue;
      }
      // A unit is four consecutive rows of one token; lane takes units lane, lane + 32, ...  The warp competes for
      // issue slots with all the consumer warps (an instruction every ten cycles or so), so what counts is its
      // instruction count: 16-byte loads, paired adds, 8-byte stores.  Sums run over the warps in ascending order.
      const int nunits = p.M * 8;
      float4 acc[kRedUnits];
      const float* src[kRedUnits];
#pragma unroll
      for (int j = 0; j < kRedUnits; ++j) {
        const int u = min(lane + 32 * j, nunits - 1);
        acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        src[j] = rbuf + (u >> 3) * kRedPitch + (u & 7) * 4;
      }
      const int wstride = p.M * kRedPitch;
#pragma unroll
      for (int w = 0; w < NCW; ++w)
#pragma unroll
        for (int j = 0; j < kRedUnits; ++j)
          if (j == 0 || lane + 32 * j < nunits) {
            const float4 v = *reinterpret_cast<const float4*>(src[j] + w * wstride);
            const float2 lo = add_f32x2(make_float2(acc[j].x, acc[j].y), make_float2(v.x, v.y));
            const float2 hi = add_f32x2(make_float2(acc[j].z, acc[j].w), make_float2(v.z, v.w));
            acc[j] = make_float4(lo.x, lo.y, hi.x, hi.y);
          }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_red_empty + 8 * b);  // the sums are in registers: the buffer is free again
      const bool rows_aligned = (p.N & 3) == 0;
#pragma unroll
      for (int j = 0; j < kRedUnits; ++j) {
        const int u = lane + 32 * j;
        if (u < nunits) {
          const int tok = u >> 3, n0 = row0 + (u & 7) * 4;
          if (p.nslices > 1) {
            float* d = p.partial + ((size_t)sl * p.M + tok) * p.N + n0;
            const float f[4] = {acc[j].x, acc[j].y, acc[j].z, acc[j].w};
            if (rows_aligned && n0 + 3 < p.N) {
              __stcg(reinterpret_cast<float4*>(d), acc[j]);
            } else {
#pragma unroll
              for (int i = 0; i < 4; ++i)
                if (n0 + i < p.N) __stcg(d + i, f[i]);
            }
          } else {
            store_out4(p, tok, n0, acc[j]);
          }
        }
      }
      if (p.nslices > 1 && !p.sum_kernel) {
        // the last slice of this row group to arrive sums all partials in slice order
        __threadfence();
        __syncwarp();
        int last = 0;
        if (lane == 0) {
          const int old = atomicAdd(p.counters + rg, 1);
          last = old == p.nslices - 1;
          if (last) p.counters[rg] = 0;  // ready for the next launch
        }
        last = __shfl_sync(0xffffffffu, last, 0);
        if (last) {
          __threadfence();
#pragma unroll
          for (int j = 0; j < kRedUnits; ++j) {
            const int u = lane + 32 * j;
            const int tok = u >> 3, n0 = row0 + (u & 7) * 4;
            if (u < nunits && n0 < p.N) store_out4(p, tok, n0, sum_slices4(p, tok, n0));
          }
        }
      }
    }
    if (p.tp.world && !p.tp.defer) tp_signal(p.tp, lane);  // every CTA counts itself in once, after its last store
  } else {
    // ------------------------------------------------------------ consumer warps
    const int g = lane >> 2, t = lane & 3;
    // tile row fed to mma row g: neighbouring g get rows 4 apart, so that the eight lanes of one shared-
    // memory access phase land in opposite halves of the swizzled 128-byte rows (no bank conflicts)
    const int gr = (g >> 1) | ((g & 1) << 2);
    const int ctid = tid;  // consumer warps are warps 0..NCW-1
    // chunk j of a stage sits in box j / 2, 64-byte half j % 2; 16-byte unit index XOR (row % 8 = gr).  With one
    // chunk per warp j = warp; with two, the warp owns box `warp` and takes half 0 then half 1.
    const uint32_t w_lane_addr = ring_base + (CPW == 2 ? warp : (warp >> 1)) * kBoxBytes + gr * 128;
    const uint32_t w_unit0 = (uint32_t(((CPW == 2 ? 0 : (warp & 1)) << 2) | t) ^ uint32_t(gr)) << 4;
    const uint32_t w_unit1 = (uint32_t(4 | t) ^ uint32_t(gr)) << 4;  // second half of the box (CPW == 2)
    // unpack constants, pinned in registers so that every (x & mask) | magic is a single LOP3
    uint32_t k_mask_lo = 0x000F000Fu, k_mask_hi = 0x00F000F0u, k_magic = 0x64006400u;
    uint32_t k_n1032 = 0xE408E408u;  // fp16 -1032 twice
    uint32_t k_n72 = 0xD480D480u;    // fp16 -72 twice
    uint32_t k_r16 = 0x2C002C00u;    // fp16 1/16 twice
    asm volatile("" : "+r"(k_mask_lo), "+r"(k_mask_hi), "+r"(k_magic), "+r"(k_n1032), "+r"(k_n72), "+r"(k_r16));
    uint32_t k_nib_lo = 0x0F0F0F0Fu, k_nib_hi = 0xF0F0F0F0u;  // integer path: even / odd nibbles of a word as bytes
    asm volatile("" : "+r"(k_nib_lo), "+r"(k_nib_hi));
    const bool multi_token = p.M > 1;
    // this lane's scales of a stage: rows gr (+8, +16, +24) of the stage's [32][chunks] block, column = its chunk
    const uint32_t sc_lane = sc_base + gr * (kSC * 2) + (CPW * warp) * 2;
    const int nstages = p.nstages, gdiv = p.gdiv;
    // Launched with programmatic stream serialization this kernel may start while the previous one is still
    // running: the weight stream (constant data) is already flowing; X, produced upstream, is touched only
    // after the previous grid has completed and flushed.
    pdl_wait_prior_grid();
    if (p.tp.announce_world && blockIdx.x == 0 && ctid < 32) tp_announce(p.tp, ctid);
    if (p.tp.wait_sig != nullptr) {
      // the input is the gathered output of the producing kernels of every rank: wait until all their CTAs have
      // counted themselves in (their stores are visible by then)
      if (ctid == 0) tp_wait(p.tp, abort_flag);
      consumer_sync(kConsumerThreads);
    }

    int s = 0;
    uint32_t ph = 0;
    int staged_slice = -1, tcount = 0;
    for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x, ++tcount) {
      const int sl = tile / p.nrg, rg = tile - sl * p.nrg;
      const int cb = sl * p.cps, ce = min(p.nchunks, cb + p.cps);
      const int nch = ce - cb;
      const int row0 = rg * kRowsPerGroup;
      if (sl != staged_slice) {
        if (staged_slice >= 0) consumer_sync(kConsumerThreads);  // all done with the old slice
        if constexpr (kHalf) {
          float* inv = reinterpret_cast<float*>(smem + kNormInvOffset);
          if (p.pro == kProAddRmsNorm && staged_slice < 0)
            rmsnorm_factors<kConsumerThreads>(p, reinterpret_cast<float*>(smem + kNormSsOffset), inv, ctid);
          if constexpr (kI8) {
            if (p.pre_x != nullptr)
              copy_staged_x<L>(p, xs_base, smem_u32(xinfo), cb, ce, ctid, kConsumerThreads);
            else
              stage_x_i8<L, false>(p, xs_base, reinterpret_cast<int4*>(xinfo), inv, cb, ce, ctid, kConsumerThreads);
          } else
            stage_x_f16<kConsumerThreads, MODE == kModeFold>(p, xs_base, xinfo, inv, cb, ce, ctid);
        }
        if constexpr (!kHalf) stage_x_bf16<kConsumerThreads>(p, xs_base, cb, ce, ctid);
        if (ctid < 32) sts128(zero_base + ctid * 16, make_uint4(0u, 0u, 0u, 0u));
        consumer_sync(kConsumerThreads);
        staged_slice = sl;
      }
      // B-fragment source of this lane: its token's staged X, or a block of zeros for padding tokens
      uint32_t xaddr[MT], xstep[MT];
      bool xreal[MT];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int m = mt * 8 + g;
        const bool real = m < p.M;
        xreal[mt] = real;
        xaddr[mt] = real ? xs_base + m * p.xs_m_stride + (CPW * warp) * kXChunk + t * 16 : zero_base + t * 16;
        xstep[mt] = real ? kSC * kXChunk : 0;
      }
      // per-(token, chunk) info of the two accumulator columns (tokens mt*8 + 2t, +1) of this lane;
      // padding tokens read a zero pair (their accumulators are zero anyway)
      const float2* xi[MT][2];
      const int4* xi8[MT][2];
      int xi_step[MT][2];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const int m = mt * 8 + 2 * t + q;
          const bool real = m < p.M;
          xi[mt][q] = real ? xinfo + m * nch + CPW * warp : reinterpret_cast<const float2*>(smem + kZeroOffset);
          xi8[mt][q] = real ? reinterpret_cast<const int4*>(xinfo) + m * nch + CPW * warp
                            : reinterpret_cast<const int4*>(smem + kZeroOffset);
          xi_step[mt][q] = real ? kSC : 0;
        }
      // fast path: lane i fetches the scale of row row0 + i; the quad layout is rebuilt with shuffles
      const int n_lane = row0 + lane;
      const bool s_valid = n_lane < p.N;
      const __nv_bfloat16* s_lane = p.S + (size_t)(s_valid ? n_lane : 0) * p.KG;

      float fin[2][MT][4];
#pragma unroll
      for (int rb = 0; rb < 2; ++rb)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int i = 0; i < 4; ++i) fin[rb][mt][i] = 0.f;

      uint32_t srow_next = 0u;
      if constexpr (kHalf) {
        const int cf = cb + warp;
        if (!sc_async && s_valid && cf < ce)
          srow_next = ld_l2(reinterpret_cast<const unsigned short*>(s_lane) + (gdiv == 1 ? cf : cf / gdiv));
      }
      for (int c0 = cb; c0 < ce; c0 += kSC) {
        const int c = c0 + CPW * warp;  // this warp's (first) chunk of the stage
        const bool active = c < ce;

        // scales: the fast path fetched this stage's scale one stage ago and now fetches the next one, so
        // the L2 round trip never sits between the math and the accumulate
        uint32_t sc2[2][2] = {{0u, 0u}, {0u, 0u}};
        const uint32_t srow = srow_next;
        if constexpr (kHalf) {
          const int cn = c + kSC;
          srow_next = 0u;
          if (!sc_async && s_valid && cn < ce)
            srow_next = ld_l2(reinterpret_cast<const unsigned short*>(s_lane) + (gdiv == 1 ? cn : cn / gdiv));
        }
        if (active) {
          if constexpr (!kHalf) {
            const int k_lane = c * kChunkK + 32 * t;
            const int grp = k_lane < p.K ? k_lane / p.G : -1;
#pragma unroll
            for (int rb = 0; rb < 2; ++rb)
#pragma unroll
              for (int hh = 0; hh < 2; ++hh) {
                const int n = row0 + rb * 16 + gr + 8 * hh;
                __nv_bfloat16 sv = __float2bfloat16(0.f);
                if (n < p.N && grp >= 0)
                  sv = __ushort_as_bfloat16(ld_l2(reinterpret_cast<const unsigned short*>(p.S) + (size_t)n * p.KG + grp));
                sc2[rb][hh] = bf16_dup(sv);
              }
          }
        }

        if (lane == 0) mbar_wait(bar_full + 8 * s, ph, abort_flag);
        __syncwarp();

#pragma unroll
        for (int h = 0; h < CPW; ++h)
        if (c + h < ce) {
          if constexpr (kI8) {
          // ---- integer path: nibbles stay integers.  (w & 0x0F0F0F0F) holds the four even-k nibbles of a word as
          // bytes, (w & 0xF0F0F0F0) the four odd-k nibbles times 16: both are ready-made u8 A fragments of
          // mma.m16n8k32, so the unpack is two LOP3 per eight weights and no shift.  X arrives as L byte planes
          // ("limbs"); every plane gets its own s32 accumulators, even and odd nibbles apart (the odd ones carry the
          // factor 16), all combined once per chunk: T = sum_l 256^l (16 even_l + odd_l) = 16 sum_k (q_k - 8) v_k.
          uint32_t xb[MT][L][8];
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int l = 0; l < L; ++l)
#pragma unroll
              for (int jj = 0; jj < 2; ++jj) {
                uint4 v = make_uint4(0u, 0u, 0u, 0u);  // padding tokens: no load at all (fewer wavefronts)
                if (xreal[mt]) v = lds128(xaddr[mt] + h * kXChunk + l * 128 + jj * 64);
                xb[mt][l][4 * jj + 0] = v.x;
                xb[mt][l][4 * jj + 1] = v.y;
                xb[mt][l][4 * jj + 2] = v.z;
                xb[mt][l][4 * jj + 3] = v.w;
              }
          const uint32_t wa = w_lane_addr + s * kStageBytes + (h ? w_unit1 : w_unit0);
          uint4 wv[2][2];
#pragma unroll
          for (int rb = 0; rb < 2; ++rb) {
            wv[rb][0] = lds128(wa + rb * 2048);
            wv[rb][1] = lds128(wa + rb * 2048 + 1024);
          }
          int4 info[MT][2];
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            info[mt][0] = *(xi8[mt][0] + (xi_step[mt][0] ? h : 0));
            info[mt][1] = *(xi8[mt][1] + (xi_step[mt][1] ? h : 0));
          }
          uint32_t scr[4] = {0u, 0u, 0u, 0u};  // scales of rows gr, gr + 8, gr + 16, gr + 24 of the stage
          if (sc_async) {
#pragma unroll
            for (int i = 0; i < 4; ++i) scr[i] = lds_u16(sc_lane + h * 2 + s * kScStage + i * (8 * kSC * 2));
          }
#pragma unroll
          for (int rb = 0; rb < 2; ++rb) {
            const uint32_t wl[4] = {wv[rb][0].x, wv[rb][0].y, wv[rb][0].z, wv[rb][0].w};
            const uint32_t wh[4] = {wv[rb][1].x, wv[rb][1].y, wv[rb][1].z, wv[rb][1].w};
            int ae[MT][L][4], ao[MT][L][4];
#pragma unroll
            for (int jj = 0; jj < 2; ++jj) {
              const uint32_t e0 = wl[2 * jj] & k_nib_lo, e1 = wh[2 * jj] & k_nib_lo;
              const uint32_t e2 = wl[2 * jj + 1] & k_nib_lo, e3 = wh[2 * jj + 1] & k_nib_lo;
              const uint32_t o0 = wl[2 * jj] & k_nib_hi, o1 = wh[2 * jj] & k_nib_hi;
              const uint32_t o2 = wl[2 * jj + 1] & k_nib_hi, o3 = wh[2 * jj + 1] & k_nib_hi;
#pragma unroll
              for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int l = 0; l < L; ++l) {
                  if (jj == 0) {
                    // the odd chain starts from the zero-point term of its limb, the even chain from zero
                    const int c0 = l == 0 ? info[mt][0].y : (l == 1 ? info[mt][0].z : info[mt][0].w);
                    const int c1 = l == 0 ? info[mt][1].y : (l == 1 ? info[mt][1].z : info[mt][1].w);
                    imma_16832_init(l == L - 1, ae[mt][l], e0, e1, e2, e3, xb[mt][l][0], xb[mt][l][1], 0, 0);
                    imma_16832_init(l == L - 1, ao[mt][l], o0, o1, o2, o3, xb[mt][l][2], xb[mt][l][3], c0, c1);
                  } else {
                    imma_16832(l == L - 1, ae[mt][l], e0, e1, e2, e3, xb[mt][l][4 * jj], xb[mt][l][4 * jj + 1]);
                    imma_16832(l == L - 1, ao[mt][l], o0, o1, o2, o3, xb[mt][l][4 * jj + 2], xb[mt][l][4 * jj + 3]);
                  }
                }
            }
            float s_lo, s_hi;
            if (sc_async) {
              s_lo = __uint_as_float(scr[2 * rb] << 16);
              s_hi = __uint_as_float(scr[2 * rb + 1] << 16);
            } else {
              s_lo = __uint_as_float(__shfl_sync(0xffffffffu, srow, rb * 16 + gr) << 16);
              s_hi = __uint_as_float(__shfl_sync(0xffffffffu, srow, rb * 16 + gr + 8) << 16);
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              const float up0 = __int_as_float(info[mt][0].x), up1 = __int_as_float(info[mt][1].x);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                if ((i & 1) && !multi_token) continue;  // one token: accumulator columns 1.. are padding
                float f;
                if constexpr (L == 2) {
                  f = (float)((16 * ae[mt][1][i] + ao[mt][1][i]) * 256 + (16 * ae[mt][0][i] + ao[mt][0][i]));
                } else {
                  const int th = (16 * ae[mt][2][i] + ao[mt][2][i]) * 256 + (16 * ae[mt][1][i] + ao[mt][1][i]);
                  f = fmaf((float)th, 256.f, (float)(16 * ae[mt][0][i] + ao[mt][0][i]));
                }
                fin[rb][mt][i] = fmaf((i < 2 ? s_lo : s_hi) * ((i & 1) ? up1 : up0), f, fin[rb][mt][i]);
              }
            }
          }
          } else {
          // all shared-memory loads of the stage first, then the math: the loads are ordered after the
          // barrier wait, the math is free to be scheduled around them
          uint32_t xf[MT][16];
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint4 v = lds128(xaddr[mt] + j * 64);
              xf[mt][4 * j + 0] = v.x;
              xf[mt][4 * j + 1] = v.y;
              xf[mt][4 * j + 2] = v.z;
              xf[mt][4 * j + 3] = v.w;
            }
          }
          const uint32_t wa = w_lane_addr + s * kStageBytes + w_unit0;
          uint4 wv[2][2];
#pragma unroll
          for (int rb = 0; rb < 2; ++rb) {
            wv[rb][0] = lds128(wa + rb * 2048);
            wv[rb][1] = lds128(wa + rb * 2048 + 1024);
          }
          float2 info[MT][2];
          if constexpr (kHalf) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              info[mt][0] = *xi[mt][0];
              info[mt][1] = *xi[mt][1];
            }
          }
          uint32_t scr[4] = {0u, 0u, 0u, 0u};
          if (sc_async) {
#pragma unroll
            for (int i = 0; i < 4; ++i) scr[i] = lds_u16(sc_lane + s * kScStage + i * (8 * kSC * 2));
          }
#pragma unroll
          for (int rb = 0; rb < 2; ++rb) {
            const uint32_t wl[4] = {wv[rb][0].x, wv[rb][0].y, wv[rb][0].z, wv[rb][0].w};
            const uint32_t wh[4] = {wv[rb][1].x, wv[rb][1].y, wv[rb][1].z, wv[rb][1].w};
            if constexpr (kHalf) {
              float acc[MT][2][4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint32_t rl[4], rh[4];
                const uint32_t ul = wl[j] >> 8, uh = wh[j] >> 8;
                rl[0] = and_or(wl[j], k_mask_lo, k_magic);
                rl[1] = and_or(wl[j], k_mask_hi, k_magic);
                rl[2] = and_or(ul, k_mask_lo, k_magic);
                rl[3] = and_or(ul, k_mask_hi, k_magic);
                rh[0] = and_or(wh[j], k_mask_lo, k_magic);
                rh[1] = and_or(wh[j], k_mask_hi, k_magic);
                rh[2] = and_or(uh, k_mask_lo, k_magic);
                rh[3] = and_or(uh, k_mask_hi, k_magic);
                if constexpr (MODE == kModeExact) {
#pragma unroll
                  for (int q = 0; q < 4; q += 2) {
                    rl[q] = hadd2_u32(rl[q], k_n1032);
                    rh[q] = hadd2_u32(rh[q], k_n1032);
                    rl[q + 1] = hfma2_u32(rl[q + 1], k_r16, k_n72);
                    rh[q + 1] = hfma2_u32(rh[q + 1], k_r16, k_n72);
                  }
                }
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                  for (int mt = 0; mt < MT; ++mt) {
                    if (j == 0)
                      mma_16816_f16_zero(acc[mt][h], rl[2 * h], rh[2 * h], rl[2 * h + 1], rh[2 * h + 1],
                                         xf[mt][4 * j + 2 * h], xf[mt][4 * j + 2 * h + 1]);
                    else
                      mma_16816_f16(acc[mt][h], rl[2 * h], rh[2 * h], rl[2 * h + 1], rh[2 * h + 1],
                                    xf[mt][4 * j + 2 * h], xf[mt][4 * j + 2 * h + 1]);
                  }
              }
              // scale of rows gr and gr + 8 of this block, from the lanes that fetched them
              float s_lo, s_hi;
              if (sc_async) {
                s_lo = __uint_as_float(scr[2 * rb] << 16);
                s_hi = __uint_as_float(scr[2 * rb + 1] << 16);
              } else {
                s_lo = __uint_as_float(__shfl_sync(0xffffffffu, srow, rb * 16 + gr) << 16);
                s_hi = __uint_as_float(__shfl_sync(0xffffffffu, srow, rb * 16 + gr + 8) << 16);
              }
#pragma unroll
              for (int mt = 0; mt < MT; ++mt) {
                float v0 = acc[mt][0][0] + acc[mt][1][0], v1 = acc[mt][0][1] + acc[mt][1][1];
                float v2 = acc[mt][0][2] + acc[mt][1][2], v3 = acc[mt][0][3] + acc[mt][1][3];
                if constexpr (MODE == kModeFold) {
                  v0 -= info[mt][0].y;
                  v1 -= info[mt][1].y;
                  v2 -= info[mt][0].y;
                  v3 -= info[mt][1].y;
                }
                fin[rb][mt][0] = fmaf(s_lo * info[mt][0].x, v0, fin[rb][mt][0]);
                fin[rb][mt][1] = fmaf(s_lo * info[mt][1].x, v1, fin[rb][mt][1]);
                fin[rb][mt][2] = fmaf(s_hi * info[mt][0].x, v2, fin[rb][mt][2]);
                fin[rb][mt][3] = fmaf(s_hi * info[mt][1].x, v3, fin[rb][mt][3]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint32_t rl[4], rh[4];
                unpack_w4_biased(wl[j], rl);
                unpack_w4_biased(wh[j], rh);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  rl[q] = mul_bf16x2(sub136_bf16x2(rl[q]), sc2[rb][0]);
                  rh[q] = mul_bf16x2(sub136_bf16x2(rh[q]), sc2[rb][1]);
                }
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                  for (int mt = 0; mt < MT; ++mt)
                    mma_16816_bf16(fin[rb][mt], rl[2 * h], rh[2 * h], rl[2 * h + 1], rh[2 * h + 1],
                                   xf[mt][4 * j + 2 * h], xf[mt][4 * j + 2 * h + 1]);
              }
            }
          }
          }  // !kI8
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty + 8 * s);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          xaddr[mt] += xstep[mt];
          xi[mt][0] += xi_step[mt][0];
          xi[mt][1] += xi_step[mt][1];
          xi8[mt][0] += xi_step[mt][0];
          xi8[mt][1] += xi_step[mt][1];
        }
        if (++s == nstages) {
          s = 0;
          ph ^= 1;
        }
      }

      // ---- hand the per-warp partial sums of this tile to the reducer warp (two buffers in rotation)
      const int b = tcount & 1;
      float* rbuf = red + b * (NCW * p.M * kRedPitch);
      if (lane == 0) mbar_wait(bar_red_empty + 8 * b, ((tcount >> 1) & 1) ^ 1, abort_flag);
      __syncwarp();
#pragma unroll
      for (int rb = 0; rb < 2; ++rb)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const int tok = mt * 8 + 2 * t;  // accumulator columns 2t, 2t+1 of this tile; padding tokens are dropped
          float* r0 = rbuf + (warp * p.M + tok) * kRedPitch + rb * 16 + gr;
          if (tok < p.M) {
            r0[0] = fin[rb][mt][0];
            r0[8] = fin[rb][mt][2];
          }
          if (tok + 1 < p.M) {
            r0[kRedPitch] = fin[rb][mt][1];
            r0[kRedPitch + 8] = fin[rb][mt][3];
          }
        }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_red_full + 8 * b);
    }
  }

  __syncthreads();
  if (*abort_flag) {
    if (tid == 0) atomicCAS(p.status, kStatusOk, kStatusGemvTimeout);
    // give copies that may still be in flight time to land before the shared memory is released
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
}

// ------------------------------------------------------------------ host side
struct GemvPlan {
  int mt, ncw, cpw, mode, nslices, cps, nstages, grid;
  bool pdl, prestage, sum_kernel;
  int ctas_per_sm;
  size_t smem;
  int xs_m_stride;
  double cost;
};

size_t smem_without_ring(int M, int mode, int ncw, int cps) {
  const int xs_m_stride = cps * x_chunk_bytes(mode) + 64;
  const size_t xinfo_bytes = ((size_t)M * cps * x_info_bytes(mode) + 127) & ~(size_t)127;
  const size_t xs_bytes = ((size_t)M * xs_m_stride + 127) & ~(size_t)127;
  return kHeaderBytes + red_bytes(ncw, M) + xinfo_bytes + xs_bytes + 1024;
}

// Plan for a fixed CTA width.  Cost model in units of "one chunk of one row group" (2 KB of weights): a
// tile costs its chunk count rounded up to whole stages (idle warps in a short last stage are lost
// time), plus a fixed reduction overhead; split-K tiles pay the scratch round trip as well.  The slice
// count with the smallest makespan over the persistent CTAs wins.
bool plan_for_width(int M, int N, int K, int ncw, int cpw, int mt, int mode, int flags, bool prestage, int sm_count,
                    size_t partial_cap, int counters_cap, GemvPlan* out) {
  GemvPlan pl{};
  pl.prestage = prestage;
  pl.mt = mt;
  pl.mode = mode;
  pl.ncw = ncw;
  pl.cpw = cpw;
  const int sc = ncw * cpw;  // chunks per stage
  const int nchunks = (K + kChunkK - 1) / kChunkK;
  const int nrg = (N + kRowsPerGroup - 1) / kRowsPerGroup;
  // a ring stage: the weight boxes plus (fast paths) the stage's scales, [32 rows][ncw] bf16
  const int stage_bytes = (sc / 2) * kBoxBytes + (mode == kModeGeneric ? 0 : kRowsPerGroup * sc * 2);
  const int grid = std::max(1, sm_count);
  // Two CTAs per SM when both fit (shared memory: half of 227 KB minus the per-CTA reserve; registers: the narrow
  // MT == 1 kernels are compiled for it): more warps to hide latency, and one CTA's tail overlaps the other's
  // streaming.  Otherwise one CTA with a deeper ring.
  constexpr size_t kHalfSmem = 113 * 1024;
  double best = 1e30;
  int best_ns = 0, best_cps = 0, best_ctas = 1;
  const int max_ns = (flags & kFlagForceNoSplitK) ? 1 : std::min(nchunks, 64);
  const int forced_ns = (flags >> 24) & 0x3F;  // bits 24-29 of the flags: this many K slices or none (diagnostics)
  for (int ns = 1; ns <= max_ns; ++ns) {
    if (forced_ns && ns != forced_ns) continue;
    const int cps = (nchunks + ns - 1) / ns;
    if ((nchunks + cps - 1) / cps != ns) continue;
    if (cpw == 2 && ns > 1 && (cps & 1)) continue;  // slices start on a box boundary, scale copies stay aligned
    if (ns > 1) {
      if ((size_t)ns * M * N * sizeof(float) > partial_cap) continue;
      if (nrg > counters_cap) continue;
    }
    const size_t fixed = smem_without_ring(M, mode, ncw, cps);
    const long tiles = (long)nrg * ns;
    const int iters = (cps + sc - 1) / sc;  // ring stages per tile
    const int stage_chunks = iters * sc;
    // the memory system moves only real bytes, the warps pay for padded stages: weigh them equally
    // fixed cost of a tile (hand-off to the reducer) and of a split-K tile (scratch round trip, measured to be
    // dear: splitting the 3584 x 18944 projection five ways was slower than leaving 36 SMs idle)
    // ... and of an iteration of the consumer loop (wait, release, bookkeeping: 0.23 us measured, just under three
    // chunks), which is what two chunks per warp and stage save
    // split-K tiles pay the scratch round trip, the counter and the final sum (1 to 3 us measured; whether a split pays
    // is one of the things the first-launch measurement settles)
    // (with the sums left to the kernel behind, a split tile costs a 16-byte store more than a whole one, and the
    // launch pays for that kernel once)
    const bool sum_kernel = (flags & kFlagSplitSumKernel) != 0;
    const double tile_cost = 0.5 * (cps + stage_chunks) + 2.85 * iters + 3.0 + (ns > 1 ? (sum_kernel ? 1.0 : 12.0) : 0.0);
    const double launch_cost = ns > 1 && sum_kernel ? 20.0 : 0.0;
    // staging of X: once per CTA and slice, spread over the consumer threads
    // (pre-staged X: a plain copy of the slice, about a tenth of the conversion)
    const double stage_cost = (prestage ? 0.05 : 0.5) * M * cps * (8.0 / ncw);
    for (int ctas = 2; ctas >= 1; --ctas) {
      if (ctas == 2 && !(mt == 1 && ncw <= 12 && fixed + 2 * (size_t)stage_bytes <= kHalfSmem)) continue;
      if (ctas == 1 && fixed + 2 * (size_t)stage_bytes > (size_t)kSmemLimit) continue;
      const long slots = (long)grid * ctas;
      const long rounds = (tiles + slots - 1) / slots;
      const long active = std::min<long>(ctas, (tiles + grid - 1) / grid);  // CTAs that share the busiest SM
      double cost = (rounds * tile_cost + stage_cost * std::min<long>(rounds, ns)) * active;
      if (active == 2) cost *= 0.78;  // measured: one CTA's staging and tail overlap the other's streaming
      cost += launch_cost;
      // a ring of two stages lets the producer run only one stage ahead
      const size_t cap = ctas == 2 ? kHalfSmem : (size_t)kSmemLimit;
      if ((cap - fixed) / stage_bytes < 3) cost *= 1.25;
      if (active == 1 && ncw <= 12) cost *= 1.0 + (16 - ncw) / 20.0;  // measured: too few warps on the SM
      if (cost < best) {
        best = cost;
        best_ns = ns;
        best_cps = cps;
        best_ctas = ctas;
      }
    }
  }
  if (best_ns == 0) return false;
  pl.nslices = best_ns;
  pl.cps = best_cps;
  pl.xs_m_stride = pl.cps * x_chunk_bytes(mode) + 64;
  pl.cost = best;
  const size_t fixed = smem_without_ring(M, mode, ncw, pl.cps);
  const long tiles = (long)nrg * pl.nslices;
  int stages;
  if (best_ctas == 2) {
    stages = std::min<int>(4, (int)((kHalfSmem - fixed) / stage_bytes));
  } else {
    stages = (int)(((size_t)kSmemLimit - fixed) / stage_bytes);
    stages = std::min(stages, ncw >= 14 ? 5 : kMaxStages);
  }
  if (stages < 2) return false;
  pl.nstages = stages;
  pl.smem = fixed + (size_t)stages * stage_bytes;
  pl.grid = (int)std::min<long>((long)grid * best_ctas, tiles);
  pl.ctas_per_sm = best_ctas;
  *out = pl;
  return true;
}

bool make_plan(int M, int N, int K, int G, int flags, int sm_count, size_t partial_cap, int counters_cap,
               GemvPlan* out) {
  // split K: the slices are summed by a kernel behind the GEMV unless the caller (or a tensor-parallel launch) says no
  flags = (flags & kFlagNoSplitSumKernel) ? (flags & ~kFlagSplitSumKernel) : (flags | kFlagSplitSumKernel);
  const int mt = M > 8 ? 2 : 1;
  // G % 128 == 0: the integer path with two bytes per value of X, or three (kFlagWideX), or X in floating point on
  // the fp16 mma (kFlagFloatX; with kFlagFoldZeroPoint its cheaper variant)
  int mode = kModeGeneric;
  if (G % 128 == 0) {
    if (flags & kFlagFloatX)
      mode = (flags & kFlagFoldZeroPoint) ? kModeFold : kModeExact;
    else
      mode = (flags & kFlagWideX) ? kModeI8x3 : kModeI8x2;
  }
  // X staged by a kernel in front: integer modes; by default from eight tokens on, from four where K is long
  const bool prestage = mode_limbs(mode) > 0 && !(flags & kFlagNoPreStageX) &&
                        ((flags & kFlagPreStageX) || M >= 8 || (M >= 4 && K >= 8192));
  GemvPlan best{};
  bool have = false;
  // One token tile: candidates are the wide CTAs (16 or 14 consumer warps, one per SM) and the narrow one
  // (8 consumer warps, two per SM when they fit); the cost model picks.  Bits 4-7 of the flags force a
  // width (diagnostics).  Two token tiles need the registers of the 8-warp CTA.
  const int forced = ((flags >> 4) & 0xF) * 2;
  // Two chunks per warp and stage: integer modes whose scales can be staged with aligned copies (one scale per chunk,
  // an even number of scales per row).  Bits 10 / 11 of the flags force two / one (diagnostics).
  const bool cpw2_ok = mode_limbs(mode) > 0 && G == 128 && (K / G) % 2 == 0 && !(flags & 0x800);
  if (mt == 1 && !(flags & kFlagNarrowCta)) {
    const int widths[3] = {16, 14, 8};
    for (int w : widths) {
      if (forced && w != forced) continue;
      for (int cpw = cpw2_ok ? 2 : 1; cpw >= 1; --cpw) {
        if (cpw == 1 && cpw2_ok && (flags & 0x400)) continue;
        if (cpw == 2 && w == 16) continue;  // not instantiated: 14 x 2 covers the wide case
        GemvPlan pl;
        if (plan_for_width(M, N, K, w, cpw, mt, mode, flags, prestage, sm_count, partial_cap, counters_cap, &pl) &&
            (!have || pl.cost < best.cost)) {
          best = pl;
          have = true;
        }
      }
    }
  }
  if (!have && mt == 2) {  // two token tiles: the 8-warp CTA, two chunks per warp and stage or one
    for (int cpw = cpw2_ok ? 2 : 1; cpw >= 1; --cpw) {
      if (cpw == 1 && cpw2_ok && (flags & 0x400)) continue;
      GemvPlan pl;
      if (plan_for_width(M, N, K, 8, cpw, mt, mode, flags, prestage, sm_count, partial_cap, counters_cap, &pl) &&
          (!have || pl.cost < best.cost)) {
        best = pl;
        have = true;
      }
    }
  }
  if (!have) have = plan_for_width(M, N, K, 8, 1, mt, mode, flags, prestage, sm_count, partial_cap, counters_cap, &best);
  if (!have) return false;
  best.mode = mode;
  best.sum_kernel = best.nslices > 1 && (flags & kFlagSplitSumKernel);
  best.pdl = (flags & kFlagNoPdl) == 0;
  *out = best;
  return true;
}

template <int MT, int NCW, int MODE, int CPW>
int launch_variant(const CUtensorMap& tmap, const GemvParams& p, const GemvPlan& pl, cudaStream_t stream) {
  auto kernel = w4_gemv_kernel<MT, NCW, MODE, CPW>;
  // Raising the dynamic shared-memory limit is idempotent and cheap; doing it on every launch keeps
  // the call correct on every device of a multi-GPU process without per-device bookkeeping.
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem);
  if (e != cudaSuccess) return (int)e;
  // ask for the largest shared-memory carve-out so that two CTAs of ~100 KB can be resident together
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(pl.grid);
  cfg.blockDim = dim3((NCW + 2) * 32);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pl.pdl ? 1 : 0;
  e = cudaLaunchKernelEx(&cfg, kernel, tmap, p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

template <int MT, int NCW>
int launch_mode(const CUtensorMap& tmap, const GemvParams& p, const GemvPlan& pl, cudaStream_t stream) {
  switch (pl.mode) {
    case kModeExact: return launch_variant<MT, NCW, kModeExact, 1>(tmap, p, pl, stream);
    case kModeFold: return launch_variant<MT, NCW, kModeFold, 1>(tmap, p, pl, stream);
    case kModeI8x2:
      if constexpr (NCW != 16)
        if (pl.cpw == 2) return launch_variant<MT, NCW, kModeI8x2, 2>(tmap, p, pl, stream);
      return launch_variant<MT, NCW, kModeI8x2, 1>(tmap, p, pl, stream);
    case kModeI8x3:
      if constexpr (NCW != 16)
        if (pl.cpw == 2) return launch_variant<MT, NCW, kModeI8x3, 2>(tmap, p, pl, stream);
      return launch_variant<MT, NCW, kModeI8x3, 1>(tmap, p, pl, stream);
    default: return launch_variant<MT, NCW, kModeGeneric, 1>(tmap, p, pl, stream);
  }
}

}  // namespace

// Plain launches of five to sixteen tokens whose converted X fits in shared memory run the many-token kernel.
// (Pointers: null = "assume aligned", for the queries that have no operands.)
static bool mid_serves(const void* X, const void* Wq, const void* S, int M, int N, int K, int G, const GemvPrologue& pro,
                       const Workspace& ws, int flags, int sm_count, const GemvTp* tp) {
  if (pro.kind != kProNone || pro.epilogue != kEpiNone) return false;
  if (tp != nullptr && (tp->world > 0 || tp->wait_sig != nullptr || tp->announce_world > 0)) return false;
  return gemv_mid_applies(X, Wq, S, M, N, K, G, flags, sm_count, ws.partial ? ws.partial_bytes : 0);
}

size_t gemv_scratch_bytes(int M, int N, int K, int G, int flags, int sm_count, size_t partial_cap) {
  if (gemv_mid_applies(nullptr, nullptr, nullptr, M, N, K, G, flags, sm_count, partial_cap))
    return gemv_mid_scratch_bytes(M, N, K, flags, sm_count, partial_cap);
  if (gemv_stream_applies(nullptr, M, N, K, G, flags)) {
    // (0 also when no streaming plan fits and the ring kernel runs: its own answer follows)
    const size_t b = gemv_stream_scratch_bytes(M, N, K, G, flags, sm_count, partial_cap);
    if (b || gemv_stream_grid(M, N, K, G, flags, sm_count, partial_cap)) return b;
  }
  GemvPlan pl;
  if (!make_plan(M, N, K, G, flags, sm_count, partial_cap, 1 << 30, &pl)) return 0;
  return pl.nslices > 1 ? (size_t)pl.nslices * M * N * sizeof(float) : 0;
}

int gemv_launch(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int G,
                const Workspace& ws, int flags, int sm_count, cudaStream_t stream) {
  return gemv_launch_ex(X, Wq, S, Y, M, N, K, G, GemvPrologue{}, ws, flags, sm_count, stream);
}

size_t gemv_grid(int M, int N, int K, int G, int flags, int sm_count, size_t partial_cap, int counters_cap) {
  if (gemv_stream_applies(nullptr, M, N, K, G, flags)) {
    const size_t g = gemv_stream_grid(M, N, K, G, flags, sm_count, partial_cap);
    if (g) return g;
  }
  GemvPlan pl;
  if (!make_plan(M, N, K, G, flags, sm_count, partial_cap, counters_cap, &pl)) return 0;
  return (size_t)pl.grid;
}

// One line of text saying which kernel and launch shape a decode GEMV of this shape gets (for benchmark records).
int gemv_describe(int M, int N, int K, int G, int flags, int sm_count, size_t partial_cap, int counters_cap, char* buf,
                  int buflen) {
  if (!buf || buflen < 1) return kErrBadPointer;
  if (gemv_mid_applies(nullptr, nullptr, nullptr, M, N, K, G, flags, sm_count, partial_cap) &&
      gemv_mid_describe(M, N, K, flags, sm_count, partial_cap, buf, buflen) > 0)
    return 0;
  if (gemv_stream_applies(nullptr, M, N, K, G, flags)) {
    const int n = gemv_stream_describe(M, N, K, G, flags, sm_count, partial_cap, counters_cap, buf, buflen);
    if (n > 0) return 0;
  }
  GemvPlan pl;
  if (!make_plan(M, N, K, G, flags, sm_count, partial_cap, counters_cap, &pl)) {
    snprintf(buf, buflen, "not served by the GEMV");
    return 0;
  }
  snprintf(buf, buflen,
           "ring kernel: %d persistent CTAs (%d per SM), %d consumer warps x %d chunk(s) per stage, %d stages, %d token "
           "tile(s) of 8, X %s, K slices %d%s%s, %zu KB smem",
           pl.grid, pl.ctas_per_sm, pl.ncw, pl.cpw, pl.nstages, pl.mt,
           pl.mode == kModeI8x2   ? "16-bit fixed point"
           : pl.mode == kModeI8x3 ? "24-bit fixed point"
           : pl.mode == kModeGeneric ? "bf16 (groups below 128)"
                                     : "fp16",
           pl.nslices,
           pl.nslices > 1 ? (pl.sum_kernel ? " (sum kernel)" : " (last CTA sums)") : "", pl.prestage ? ", X pre-staged" : "",
           pl.smem >> 10);
  return 0;
}

namespace {

// ---- choice of the CTA shape by measurement ---------------------------------------------------------------
// The cost model ranks the five CTA shapes (8, 14 or 16 consumer warps x one or two chunks per warp and stage) well
// enough for the shapes it was fitted on and misses by 20-60 % elsewhere (long K with few rows, tensor-parallel
// shards, M = 4..8).  So the first launch of a shape on a device, when the stream is not being captured, times
// every shape of CTA on the caller's own operands (a few launches each with the matrix pushed out of L2 in between,
// about a millisecond in all, a handful of stream synchronisations) and remembers the fastest; later launches, and launches under capture, use the remembered
// choice or, failing that, the model.  Trial launches are plain GEMVs: they never signal a tensor-parallel counter
// and, for a tensor-parallel call, write to the tail of the scratch area instead of the gathered rows.
constexpr int kShapeFlagMask = 0xCF0;         // forced width (bits 4-7), forced chunks per warp (bits 10, 11)
// (a remembered choice may also carry kFlagForceNoSplitK)
constexpr size_t kTrialBytes = 2u << 20;      // tail of the split-K scratch kept for trial outputs (>= 16 x 65536 bf16)
struct TuneKey {
  int dev, M, N, K, G, flags, pro;
  bool operator<(const TuneKey& o) const {
    return std::tie(dev, M, N, K, G, flags, pro) < std::tie(o.dev, o.M, o.N, o.K, o.G, o.flags, o.pro);
  }
};
std::map<TuneKey, int> g_tuned;  // -> shape flags of the fastest candidate
std::mutex g_tune_mu;

int gemv_launch_planned(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int G,
                        const GemvPrologue& pro, const Workspace& ws, int flags, int sm_count, cudaStream_t stream,
                        const GemvTp* tp);

bool autotune_enabled() {
  static const bool on = [] {
    const char* e = getenv("B2_GEMV_AUTOTUNE");
    return e && e[0] == '1';  // opt-in: the drop-in entry points never measure, never synchronise
  }();
  return on;
}

}  // namespace

int gemv_launch_ex(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int G,
                   const GemvPrologue& pro, const Workspace& ws_in, int flags, int sm_count, cudaStream_t stream,
                   const GemvTp* tp) {
  Workspace ws = ws_in;
  // a tensor-parallel producer sums its slices in the kernel (its CTAs signal the peers after their stores): plans and
  // trial launches must assume that too
  if (tp != nullptr && tp->world > 0) flags |= kFlagNoSplitSumKernel;
  const bool tunable = !mid_serves(X, Wq, S, M, N, K, G, pro, ws, flags, sm_count, tp) &&
                       !gemv_stream_applies(Wq, M, N, K, G, flags) &&
                       !(flags & (kShapeFlagMask | kFlagNarrowCta | kFlagNoAutotune)) && autotune_enabled() &&
                       ws.partial && ws_in.partial_bytes > 2 * kTrialBytes && (size_t)M * N * 2 <= kTrialBytes;
  if (!tunable) return gemv_launch_planned(X, Wq, S, Y, M, N, K, G, pro, ws, flags, sm_count, stream, tp);
  ws.partial_bytes -= kTrialBytes;  // trial outputs live in the tail of the scratch while shapes are being timed
  int dev = 0;
  cudaGetDevice(&dev);
  const TuneKey key{dev, M, N, K, G, flags, pro.kind};
  {
    std::lock_guard<std::mutex> lock(g_tune_mu);
    auto it = g_tuned.find(key);
    if (it != g_tuned.end())
      return gemv_launch_planned(X, Wq, S, Y, M, N, K, G, pro, ws, flags | it->second, sm_count, stream, tp);
  }
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone)
    return gemv_launch_planned(X, Wq, S, Y, M, N, K, G, pro, ws, flags, sm_count, stream, tp);

  // ---- time the candidates
  const bool is_tp = tp != nullptr && (tp->world > 0 || tp->wait_sig != nullptr);
  void* y_trial = is_tp ? static_cast<void*>(reinterpret_cast<unsigned char*>(ws_in.partial) + ws.partial_bytes) : Y;
  if (!is_tp && !Y) return kErrBadPointer;
  // candidates: the CTA shapes (one token tile; two token tiles have one shape), each with the model's K split and,
  // where the model splits, without a split
  const int shapes[5] = {(4 << 4) | 0x800, (7 << 4) | 0x800, (8 << 4) | 0x800, (4 << 4) | 0x400, (7 << 4) | 0x400};
  // ... and, from two tokens on, with X converted in every CTA or once by a kernel in front (a caller's flag for
  // either stands; launches that cannot use the kernel in front ignore the flag)
  int cand[32], ncand = 0;
  const bool pre_open = M >= 2 && G % 128 == 0 && !(flags & (kFlagFloatX | kFlagPreStageX | kFlagNoPreStageX)) &&
                        pro.kind != kProAddRmsNorm && !(tp != nullptr && tp->wait_sig != nullptr);
  // ... and, where K is split, with the slices added up by the last CTA to arrive or by a kernel behind (which may
  // change the split the model picks)
  const bool sum_open = !(flags & (kFlagSplitSumKernel | kFlagNoSplitSumKernel | kFlagForceNoSplitK)) &&
                        !(tp != nullptr && tp->world > 0);
  const int shapes2[2] = {0x800, 0x400};  // two token tiles: 8 consumer warps, one or two chunks per warp and stage
  for (int c = 0; c < (M > 8 ? 2 : 5); ++c) {
    for (int pre = 0; pre < (pre_open ? 2 : 1); ++pre) {
      const int shape = (M > 8 ? shapes2[c] : shapes[c]) | (pre_open ? (pre ? kFlagPreStageX : kFlagNoPreStageX) : 0);
      GemvPlan pl;
      const int in_kernel = sum_open ? kFlagNoSplitSumKernel : 0;
      if (!make_plan(M, N, K, G, flags | shape | in_kernel, sm_count, ws.partial_bytes, ws.n_counters - 1, &pl)) continue;
      cand[ncand++] = shape | in_kernel;
      if (pl.nslices > 1) cand[ncand++] = shape | kFlagForceNoSplitK;
      if (sum_open && make_plan(M, N, K, G, flags | shape | kFlagSplitSumKernel, sm_count, ws.partial_bytes,
                                ws.n_counters - 1, &pl) && pl.nslices > 1)
        cand[ncand++] = shape | kFlagSplitSumKernel;
    }
  }
  cudaEvent_t e0, e1;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess)
    return gemv_launch_planned(X, Wq, S, Y, M, N, K, G, pro, ws, flags, sm_count, stream, tp);
  // score of a candidate in milliseconds (1e30 if a launch failed)
  auto measure = [&](int f) -> float {
    if (gemv_launch_planned(X, Wq, S, y_trial, M, N, K, G, pro, ws, f, sm_count, stream, nullptr) != 0) return 1e30f;
    // In use the weights come from HBM (a model's matrices do not fit the 126 MB L2 together), so every timed launch
    // is preceded by a write over the scratch area that pushes the matrix out of L2.
    bool ok = true;
    float cold[6];
    for (int i = 0; i < 6 && ok; ++i) {
      cudaMemsetAsync(ws.partial, 0, ws.partial_bytes, stream);
      cudaEventRecord(e0, stream);
      ok = gemv_launch_planned(X, Wq, S, y_trial, M, N, K, G, pro, ws, f, sm_count, stream, nullptr) == 0;
      cudaEventRecord(e1, stream);
      cold[i] = 0.f;
      ok = ok && cudaEventSynchronize(e1) == cudaSuccess && cudaEventElapsedTime(&cold[i], e0, e1) == cudaSuccess;
    }
    if (!ok) return 1e30f;
    std::sort(cold, cold + 6);  // the three fastest count: other work on the GPU only ever adds time
    // ... and a dependent chain of launches, as in a decode step, where one launch's fixed costs overlap the weight
    // stream of its neighbours (the matrix may sit in L2 here; the sum of the two views ranks the shapes best)
    float chain = 1e30f;
    for (int rep = 0; rep < 2 && ok; ++rep) {
      cudaEventRecord(e0, stream);
      for (int i = 0; i < 8 && ok; ++i)
        ok = gemv_launch_planned(X, Wq, S, y_trial, M, N, K, G, pro, ws, f, sm_count, stream, nullptr) == 0;
      cudaEventRecord(e1, stream);
      float t = 0.f;
      ok = ok && cudaEventSynchronize(e1) == cudaSuccess && cudaEventElapsedTime(&t, e0, e1) == cudaSuccess;
      chain = std::min(chain, t);
    }
    if (!ok) return 1e30f;
    return (cold[0] + cold[1] + cold[2]) / 3.f + chain / 8.f;
  };
  float score[32];
  int order[32];
  for (int c = 0; c < ncand; ++c) {
    score[c] = measure(flags | cand[c]);
    order[c] = c;
  }
  std::sort(order, order + ncand, [&](int a, int b) { return score[a] < score[b]; });
  // the leaders are often within the noise of one another: a second look at the best three
  for (int r = 0; r < std::min(3, ncand); ++r) {
    const int c = order[r];
    if (score[c] < 1e29f) score[c] = std::min(score[c], measure(flags | cand[c])) ;
  }
  int best = 0;
  float best_ms = 1e30f;
  for (int r = 0; r < std::min(3, ncand); ++r)
    if (score[order[r]] < best_ms) {
      best_ms = score[order[r]];
      best = cand[order[r]];
    }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  {
    std::lock_guard<std::mutex> lock(g_tune_mu);
    g_tuned[key] = best;  // 0 if every trial failed: the model decides
  }
  return gemv_launch_planned(X, Wq, S, Y, M, N, K, G, pro, ws, flags | best, sm_count, stream, tp);
}

namespace {

int gemv_launch_planned(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int G,
                        const GemvPrologue& pro, const Workspace& ws, int flags, int sm_count, cudaStream_t stream,
                        const GemvTp* tp) {
  if (M < 1 || M > 16) return kErrUnsupportedM;
  if (tp != nullptr && tp->world > 0) {
    // (with the SwiGLU epilogue a launch delivers N / 2 columns)
    if (tp->world > kMaxTpRanks || tp->ld < (pro.epilogue != kEpiNone ? N / 2 : N) || tp->seg_end[0] < 0 ||
        tp->seg_end[1] < tp->seg_end[0])
      return kErrBadShape;
    for (int r = 0; r < tp->world; ++r)
      if (!tp->y_peer[r] ||
          (!tp->defer && (!tp->sig_peer[r] || (reinterpret_cast<uintptr_t>(tp->sig_peer[r]) & 3))))
        return kErrBadPointer;
    Y = tp->y_peer[0];  // the plain output pointer is not used
  }
  if (tp != nullptr && tp->wait_sig != nullptr && !tp->epoch) return kErrBadPointer;
  if (pro.kind != kProNone) {
    if (pro.kind != kProAddRmsNorm && pro.kind != kProSwiglu && pro.kind != kProStaged) return kErrBadShape;
    if (G % 128) return kErrNotImplemented;  // prologues live in the fp16 staging of the fast path
    if (pro.kind == kProAddRmsNorm) {
      if (!pro.Wn) return kErrBadPointer;
      if ((reinterpret_cast<uintptr_t>(pro.Wn) & 15) || (reinterpret_cast<uintptr_t>(pro.R) & 15) ||
          (reinterpret_cast<uintptr_t>(pro.Xout) & 15))
        return kErrBadPointer;
    }
  }
  if (N < 1 || K < 32 || G < 32 || K % 32 || G % 32 || K % G) return kErrBadShape;
  if (!X || !Wq || !S || !Y) return kErrBadPointer;
  if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(Wq) & 15) ||
      (reinterpret_cast<uintptr_t>(S) & 1) || (reinterpret_cast<uintptr_t>(Y) & 1))
    return kErrBadPointer;
  if (!ws.status) return kErrWorkspace;
  if (mid_serves(X, Wq, S, M, N, K, G, pro, ws, flags, sm_count, tp))
    return gemv_mid_launch(X, Wq, S, Y, M, N, K, ws, flags, sm_count, stream);
  if (gemv_stream_applies(Wq, M, N, K, G, flags)) {
    const int rc = gemv_stream_launch(X, Wq, S, Y, M, N, K, G, pro, ws, flags, sm_count, stream, tp);
    if (rc != kStreamNotApplicable) return rc;
  }
  // epilogues and the pre-converted X exist in the streaming kernel only
  if (pro.epilogue != kEpiNone || pro.kind == kProStaged) return kErrNotImplemented;
  const bool have_scratch = ws.partial && ws.counters;
  GemvPlan pl;
  if (reinterpret_cast<uintptr_t>(S) & 3) flags |= 0x800;  // scale copies need a 4-byte aligned base: one chunk per warp
  // X staged by a kernel in front: not with the RMSNorm prologue (its factors need the whole row first), not for a
  // tensor-parallel consumer (the wait on the arrival counter happens inside the GEMV), and only while it fits
  const int nchunks_all = (K + kChunkK - 1) / kChunkK;
  const size_t pre_x_bytes = ((size_t)M * nchunks_all * 128 * ((flags & kFlagWideX) ? 3 : 2) + 255) & ~(size_t)255;
  const size_t pre_bytes = pre_x_bytes + (size_t)M * nchunks_all * sizeof(int4);
  if (pro.kind == kProAddRmsNorm || (tp != nullptr && tp->wait_sig != nullptr) || !ws.xstage ||
      pre_bytes > ws.xstage_bytes)
    flags = (flags & ~kFlagPreStageX) | kFlagNoPreStageX;
  // split-K sums by a kernel behind (the default): not for a tensor-parallel producer, whose CTAs signal the peers
  // after their stores
  if (tp != nullptr && tp->world > 0) flags |= kFlagNoSplitSumKernel;
  // the last counter is kept for the tensor-parallel epilogue's CTA count
  if (!make_plan(M, N, K, G, have_scratch ? flags : (flags | kFlagForceNoSplitK), sm_count,
                 ws.partial_bytes, ws.n_counters - 1, &pl))
    return kErrTooLarge;

  // Wq as a 2-D tensor of 32-bit words [N rows, K/8 columns]; boxes of 32 words (two chunks) x 32 rows
  CUtensorMap tmap;
  if (!make_tensor_map_2d(&tmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, Wq, (uint64_t)N, (uint64_t)K / 8, kRowsPerGroup,
                          32, CU_TENSOR_MAP_SWIZZLE_128B))
    return kErrDevice;

  GemvParams p{};
  p.X = static_cast<const __nv_bfloat16*>(X);
  p.S = static_cast<const __nv_bfloat16*>(S);
  p.Y = static_cast<__nv_bfloat16*>(Y);
  p.M = M; p.N = N; p.K = K; p.G = G;
  p.KG = K / G;
  p.gdiv = (G % 128) ? 1 : G / 128;
  p.nchunks = (K + kChunkK - 1) / kChunkK;
  p.nrg = (N + kRowsPerGroup - 1) / kRowsPerGroup;
  p.nslices = pl.nslices;
  p.cps = pl.cps;
  p.ntiles = p.nrg * p.nslices;
  p.nstages = pl.nstages;
  p.xs_m_stride = pl.xs_m_stride;
  // two scales per 4-byte copy: needs one scale per chunk, even element offsets and a 4-byte aligned base
  p.sc_async = 0;
  if (pl.mode != kModeGeneric && p.gdiv == 1) {
    // every copy starts at element n * KG + slice * cps + i * ncw + j * (width / 2) of S: the widest width that
    // keeps all of them aligned
    for (int w = 16; w >= 4 && !p.sc_async; w >>= 1) {
      const int e = w / 2;
      if ((reinterpret_cast<uintptr_t>(S) % w) == 0 && p.KG % e == 0 && (pl.ncw * pl.cpw) % e == 0 &&
          (pl.nslices == 1 || pl.cps % e == 0))
        p.sc_async = w;
    }
  }
  p.partial = ws.partial;
  p.counters = ws.counters;
  p.status = ws.status;
  p.pro = pro.kind;
  p.R = static_cast<const __nv_bfloat16*>(pro.R);
  p.Wn = static_cast<const __nv_bfloat16*>(pro.Wn);
  p.Xout = static_cast<__nv_bfloat16*>(pro.Xout);
  p.eps = pro.eps;
  if (tp != nullptr) {
    p.tp = *tp;
    if (tp->world > 0 && !tp->defer) {
      if (!ws.counters || ws.n_counters < 2) return kErrWorkspace;
      p.tp.local_count = ws.counters + ws.n_counters - 1;  // the last counter is never used by split-K (see make_plan)
    }
  }

  if (pl.prestage) {
    p.pre_x = ws.xstage;
    p.pre_info = reinterpret_cast<const int4*>(ws.xstage + pre_x_bytes);
    const int items = M * p.nchunks * 8;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((items + kStageXThreads - 1) / kStageXThreads);
    cfg.blockDim = dim3(kStageXThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pl.pdl ? 1 : 0;
    const cudaError_t e = pl.mode == kModeI8x3 ? cudaLaunchKernelEx(&cfg, w4_stage_x_kernel<3>, p)
                                               : cudaLaunchKernelEx(&cfg, w4_stage_x_kernel<2>, p);
    if (e != cudaSuccess) return (int)e;
  }

  p.sum_kernel = pl.sum_kernel ? 1 : 0;
  int rc;
  if (pl.mt == 2) {
    rc = launch_mode<2, 8>(tmap, p, pl, stream);
  } else {
    switch (pl.ncw) {
      case 16: rc = launch_mode<1, 16>(tmap, p, pl, stream); break;
      case 14: rc = launch_mode<1, 14>(tmap, p, pl, stream); break;
      default: rc = launch_mode<1, 8>(tmap, p, pl, stream); break;
    }
  }
  if (rc != 0 || !p.sum_kernel) return rc;
  return launch_sum_slices(p, sm_count, pl.pdl, stream);
}

}  // namespace

int launch_sum_slices(const GemvParams& p, int sm_count, bool pdl, cudaStream_t stream) {
  const int units = p.M * ((p.N + 3) / 4);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(std::min((units + kSumThreads - 1) / kSumThreads, 4 * sm_count));
  cfg.blockDim = dim3(kSumThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, w4_sum_slices_kernel, p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

}  // namespace b2
