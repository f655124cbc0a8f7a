// W4A16 decode GEMV for sm_100a, several tokens (five to sixteen; two to four where K is long):
// Y[M,N] (bf16) = X[M,K] (bf16) . dequant(Wq, S)^T.
//
// Replaces the reference's w4a16_gemv_kernel / w4a16_gemv (kernels/quant/w4a16.cuh:42-115) for the token counts at
// which its own analysis (README.md:137-146) finds it compute-bound.  G == 128, K % 256 == 0, a staged X that fits in
// shared memory; other shapes run the ring kernel of w4_gemv.cu.  Same operands, same weight format.
//
// The arithmetic is that of the streaming kernel's one-group layout (w4_gemv_stream.cu): nibble masks of the packed
// words are the A fragments of mma.sync.m16n8k32, X is block fixed point per (token, 128-chunk) -- here the two bytes of
// a 16-bit two's complement integer: an unsigned low plane and a signed high plane -- and the planes of the tokens are
// the columns of B.  What differs is everything around it, because with many tokens the launch is bound by shared
// memory bandwidth and instruction issue, not by start-up:
//   * One CTA of sixteen warps per SM (four per scheduler) instead of two CTAs of eight: the converted X of all
//     tokens (2 M (K + 16) bytes) is held once per SM, and every thread converts a 512th of it while the weight ring
//     fills.  (Converting once, in a small kernel in front, and fetching the result with bulk copies was measured:
//     the second launch and its completion cost more than the conversion, 7.5 us fixed per GEMV against 4.)
//   * The nibbles reach the mma as SIGNED bytes 16 (q - 8): (w & 0xF0F0F0F0) ^ 0x80808080 is one LOP3, and the
//     zero-point needs no term of its own (no per-chunk digit sums, no accumulator start values).  Shared-memory
//     bandwidth bounds the loop (the B fragments of 32 mma per 2 KB of weights), so what a lane reads besides them is
//     one float per (chunk, token).
//   * The work of a CTA -- its even share of the 16-row tiles times the 256-wide super-chunks of K -- is cut into
//     sixteen equal contiguous runs, one per warp, whatever the row count: a warp streams the end of one tile, whole
//     tiles, and the beginning of another.  Whole tiles go from registers to Y; the at most two partial tiles of a
//     warp are summed per tile, in warp order (deterministic), through shared memory at the end.
//   * Eight tokens are two column tiles: their low planes (mma s8 x u8) and their high planes (s8 x s8).  A lane holds
//     the same (row, token) of both, so they are combined as integers (lo + 256 hi) before ONE int-to-float
//     conversion and one fused multiply-add per (row, token, chunk);
//     the even nibbles are shifted up (x16, like the odd ones come out of their mask), so the four mma of a chunk
//     chain through one accumulator.
//   * Every warp is its own producer (cp.async ring with one mbarrier per slot, as in the streaming kernel); a slot
//     also carries the 16 rows' two scales of the super-chunk, so no scale table is staged.
#include <algorithm>
#include <cstdio>

#include "w4_gemv_shared.cuh"

namespace b2 {

namespace {

constexpr int kMaxDepth = 6;
constexpr int kBarOffset = 64;    // mbarriers [warp][slot], 8 bytes each
constexpr int kHeader = 1024;
constexpr int kBlockBytes = 2048 + 128;  // 16 rows x 128 bytes of packed weights (swizzled), 16 x 4 bytes of scales
constexpr int kSmemMax = 227 * 1024;

struct MidParams {
  const unsigned char* Wq;
  const __nv_bfloat16* S;
  const __nv_bfloat16* X;
  __nv_bfloat16* Y;
  int* status;
  int M, N, K;
  int nsc;      // 256-wide super-chunks of K
  int n_tiles;  // row tiles of the matrix (16 or 32 rows)
  int depth;    // ring slots per warp
  int pstride;  // bytes between digit planes of the staged X: K + 16 (the eight lanes of a shared-memory phase, two
                // planes x four 32-byte pieces, then cover all banks)
  int off_x;          // the converted X in shared memory: digit planes, then the factors
  int info_off;       // offset of the factors inside it
  int scps;           // super-chunks of K per slice (blockIdx.y); nsc when K is not cut
  float* partial;     // K cut into slices: fp32 partial sums [slice][M][N], added up by the kernel behind; else null
};

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts32f(uint32_t addr, float v) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ float lds32f(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
// d = A (s8) * B (+ d); B unsigned (the low plane) or signed (the high plane).  The accumulators are tied operands:
// written as separate inputs and outputs they cost a register move each.
template <bool BSIGNED>
__device__ __forceinline__ void imma_first(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
  if constexpr (BSIGNED)
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
  else
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
template <bool BSIGNED>
__device__ __forceinline__ void imma_acc(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  if constexpr (BSIGNED)
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  else
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float2 lds64f(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
  return v;
}

// Converts X into the B operand, all threads of the CTA, while the first weights are in flight.  An item is 16
// consecutive k of one token; the eight items of a 128-chunk sit in eight consecutive lanes.  Per (token, chunk): e =
// biased exponent of the largest |x| (clamped), every x is multiplied by 2^(14 - (e - 127)) -- the largest becomes at
// most 255 * 2^7: a bf16 value has eight significant bits -- and rounded to a 16-bit two's complement integer
// v = d0 + 256 d1, d0 its unsigned low byte, d1 its signed high byte.  The rounding is one fused multiply-add with
// 1.5 * 2^23, which leaves v in the low mantissa bits (round to nearest even, like cvt.rni, at the full rate of the
// fma pipe instead of the quarter rate of the conversion unit).  Plane p of the item: 16 bytes { d_p of k = 0,2,4,6 |
// 8,10,12,14 | 1,3,5,7 | 9,11,13,15 } -- the B fragments of one even-nibble and one odd-nibble mma (the contraction
// index is a dummy: this order is what the nibble masks produce).  factor[chunk][token] = 2^(e - 127 - 14) / 16 (the 16
// every nibble product carries).  Tokens beyond M (the token count is padded to eight or sixteen) convert zeros.  A
// chunk with an inf or a nan gets a nan factor.  Layout: planes [2][Mp][K + 16], then the factors [K / 128][Mp].
template <typename F>
__device__ __forceinline__ void convert_x(const MidParams& q, uint32_t xs, uint32_t info, int Mp, int tid,
                                          int nthreads, int k0, int klen, F&& after_first_loads) {
  // All of a thread's loads (up to UN items) are in flight before the first conversion, and AHEAD of the weight
  // stream, which `after_first_loads` starts: behind the ring's first fill (a third of the matrix) they took 2 us.
  constexpr int UN = 8;
  const int items_tok = klen >> 4;   // the CTA's slice of K: [k0, k0 + klen)
  const int items = Mp * items_tok;  // a multiple of 32: whole warps stay together for the shuffles
  // (token, item in token) of the thread's items advance by a fixed step: two divisions per thread, not two per item
  const int step_m = nthreads / items_tok, step_r = nthreads - step_m * items_tok;
  int m0 = tid / items_tok, r0 = tid - m0 * items_tok;
  for (int it0 = tid; it0 == tid || it0 < items; it0 += nthreads * UN) {  // (at least once: the callback)
    uint4 va[UN], vb[UN];
    int ms[UN], rs[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int it = it0 + u * nthreads;
      ms[u] = m0;
      rs[u] = r0;
      va[u] = make_uint4(0u, 0u, 0u, 0u);
      vb[u] = va[u];
      if (it < items && m0 < q.M) {
        const uint4* src = reinterpret_cast<const uint4*>(q.X + (size_t)m0 * q.K + k0 + r0 * 16);
        va[u] = ld_l2(src);
        vb[u] = ld_l2(src + 1);
      }
      m0 += step_m;
      r0 += step_r;
      if (r0 >= items_tok) {
        r0 -= items_tok;
        ++m0;
      }
    }
    if (it0 == tid) after_first_loads();
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int it = it0 + u * nthreads;
      if (it < items) {  // (warp-uniform)
        const int m = ms[u], r = rs[u];
        const uint32_t w[8] = {va[u].x, va[u].y, va[u].z, va[u].w, vb[u].x, vb[u].y, vb[u].z, vb[u].w};
        uint32_t mx2 = 0;  // bf16 magnitudes order like their bit patterns; both halves of a word at once
#pragma unroll
        for (int i = 0; i < 8; ++i) mx2 = __vmaxu2(mx2, w[i] & 0x7FFF7FFFu);
        uint32_t mx = max(mx2 & 0xFFFFu, mx2 >> 16);
        mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        uint32_t eb = mx >> 7;
        const bool bad = eb == 255u;
        eb = min(254u, max(40u, eb));
        const float down = __uint_as_float((uint32_t)(16 + 252 - (int)eb) << 23);
        uint32_t v[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          v[2 * i] = __float_as_uint(fmaf(__uint_as_float(w[i] << 16), down, 12582912.f));
          v[2 * i + 1] = __float_as_uint(fmaf(__uint_as_float(w[i] & 0xFFFF0000u), down, 12582912.f));
        }
#pragma unroll
        for (int p = 0; p < 2; ++p) {
          uint32_t pl[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int b = (j & 1) * 8 + (j >> 1);  // first k of the word: 0, 8, 1, 9; then every second one
            const uint32_t t0 = __byte_perm(v[b], v[b + 2], 0x5140), t1 = __byte_perm(v[b + 4], v[b + 6], 0x5140);
            pl[j] = __byte_perm(t0, t1, p ? 0x7632 : 0x5410);
          }
          sts128(xs + (uint32_t)(p * Mp + m) * q.pstride + r * 16, make_uint4(pl[0], pl[1], pl[2], pl[3]));
        }
        if ((r & 7) == 0)
          sts32f(info + (uint32_t)((r >> 3) * Mp + m) * 4,
                 __uint_as_float(bad ? 0x7FC00000u : (uint32_t)((int)eb - 18) << 23));
      }
    }
  }
}

// NP: groups of eight tokens (M <= 8 NP), two column tiles each: the low planes and the high planes.
// RB: 16-row blocks per tile.  With two, the B fragments of a chunk serve both blocks: shared memory moves 69 (eight
// tokens) or 87 (sixteen) 128-byte wavefronts per 2 KB of weights instead of 120 or 156 -- fills included, which take
// two per 128 bytes -- and the loop stops being bound by it.
// W: warps.  Sixteen, or twelve where the converted X leaves no room for sixteen rings of two 32-row slots.
template <int NP, int RB, int W>
__global__ void __launch_bounds__(W * 32, 1) w4_gemv_mid_kernel(const MidParams q) {
  extern __shared__ __align__(1024) unsigned char smem[];
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  constexpr int Mp = NP * 8, kRows = RB * 16, kSlotBytes = RB * kBlockBytes, kThreads = W * 32;
  constexpr int kSegBytes = Mp * kRows * 4;  // a partial tile parked in shared memory: [token][row] floats

  // ---- the CTA's tiles and the warp's run of (tile, super-chunk) units
  const int T0 = (int)(((long)blockIdx.x * q.n_tiles) / gridDim.x);
  const int T1 = (int)(((long)(blockIdx.x + 1) * q.n_tiles) / gridDim.x);
  const int scb = blockIdx.y * q.scps, nscl = min(q.nsc, scb + q.scps) - scb;  // the CTA's slice of K
  const int U = (T1 - T0) * nscl;
  const int u0 = (int)(((long)warp * U) / W), u1 = (int)(((long)(warp + 1) * U) / W);
  const int n = u1 - u0;
  const uint32_t bar0 = smem_u32(smem + kBarOffset) + warp * (8 * kMaxDepth);
  const uint32_t ring0 = smem_u32(smem + kHeader) + warp * q.depth * kSlotBytes;
  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < W * kMaxDepth; ++i) mbar_init(smem_u32(smem + kBarOffset) + 8 * i, 32);
    fence_mbar_init();
  }
  __syncthreads();
  pdl_launch_dependents();

  // ---- weight stream.  Lane l copies 16 bytes of rows (l >> 3) + 4 j of every 16-row block: a warp instruction
  // covers four rows x 128 bytes, whole lines.  Rows beyond N are zero-filled.
  // Running source pointers (the next unit to feed): row l >> 3 of the tile for the weights, row l of the tile for the
  // scales; they advance by one super-chunk per unit and by fifteen rows more at the end of a tile.
  int ftile = T0 + u0 / nscl, fsc = u0 % nscl;
  const int r4 = lane >> 3, c16 = lane & 7;
  const size_t row_bytes = (size_t)q.K >> 1;
  const int KG = q.K >> 7;
  const unsigned char* wsrc = q.Wq + ((size_t)ftile * kRows + r4) * row_bytes + (size_t)(scb + fsc) * 128 + c16 * 16;
  const __nv_bfloat16* ssrc = q.S + ((size_t)ftile * kRows + lane) * KG + 2 * (scb + fsc);
  const uint32_t dst_lane = r4 * 128;  // + the swizzled 16-byte column, per row
  auto rows_mask = [&](int tile) {  // bit j: row r4 + 4 j of the tile exists; bit 31: row `lane` exists (scales)
    const int left = q.N - tile * kRows;
    uint32_t m = lane < left ? 0x80000000u : 0u;
#pragma unroll
    for (int j = 0; j < 4 * RB; ++j)
      if (r4 + 4 * j < left) m |= 1u << j;
    return m;
  };
  uint32_t fvalid = rows_mask(ftile);
  constexpr uint32_t kAllRows = (1u << (4 * RB)) - 1u;
  auto feed = [&](uint32_t slot, uint32_t bar) {
    if ((fvalid & kAllRows) == kAllRows) {
#pragma unroll
      for (int j = 0; j < 4 * RB; ++j) {
        const int row = r4 + 4 * (j & 3);
        asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16;" ::"r"(slot + (j >> 2) * kBlockBytes + dst_lane +
                                                                              (j & 3) * 512 +
                                                                              ((uint32_t)(c16 ^ (row & 7)) << 4)),
                     "l"(wsrc + (size_t)(4 * j) * row_bytes)
                     : "memory");
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4 * RB; ++j) {
        const int row = r4 + 4 * (j & 3);
        const bool ok = (fvalid >> j) & 1u;
        asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16, %2;" ::"r"(slot + (j >> 2) * kBlockBytes +
                                                                                  dst_lane + (j & 3) * 512 +
                                                                                  ((uint32_t)(c16 ^ (row & 7)) << 4)),
                     "l"(ok ? wsrc + (size_t)(4 * j) * row_bytes : q.Wq), "r"(ok ? 16u : 0u)
                     : "memory");
      }
    }
    if (lane < kRows) {  // the two scales of the super-chunk, a row per lane
      const bool ok = fvalid >> 31;
      cp_async<4>(slot + (lane >> 4) * kBlockBytes + 2048 + (lane & 15) * 4, ok ? ssrc : q.S, ok ? 4u : 0u);
    }
    cp_async_mbar_arrive_noinc(bar);
    wsrc += 128;
    ssrc += 2;
    if (++fsc == nscl) {
      fsc = 0;
      ++ftile;
      wsrc += (size_t)kRows * row_bytes - (size_t)nscl * 128;
      ssrc += (size_t)kRows * KG - 2 * nscl;
      fvalid = rows_mask(ftile);
    }
  };

  // ---- X: every thread converts its share once the previous kernel's output is visible; the ring's first fill is
  // issued between the loads of X and their use
  pdl_wait_prior_grid();
  const uint32_t xs = smem_u32(smem + q.off_x), info = xs + q.info_off;
  convert_x(q, xs, info, Mp, tid, kThreads, scb * 256, nscl * 256, [&]() {
    const int pre = min(q.depth, n);
    for (int i = 0; i < pre; ++i) feed(ring0 + i * kSlotBytes, bar0 + 8 * i);
  });
  __syncthreads();

  // ---- main loop.  mma row g is slot row rho(g) (and rho + 8): the eight lanes of a shared-memory phase then land in
  // opposite halves of the swizzled 128-byte rows.
  const int rho = (g >> 1) | ((g & 1) << 2);
  const uint32_t a_u0 = rho * 128 + ((uint32_t)(t ^ rho) << 4), a_u1 = rho * 128 + ((uint32_t)((4 + t) ^ rho) << 4);
  // B column g of group j is token 8 j + g: its low plane at plane row 8 j + g, its high plane Mp rows further;
  // accumulator columns 2t, 2t + 1 are tokens 8 j + 2t, + 1
  const uint32_t xlane = xs + (uint32_t)g * q.pstride + t * 32, xhigh = (uint32_t)Mp * q.pstride;
  const uint32_t ilane = info + (uint32_t)(2 * t) * 4;
  const int first_tile = T0 + u0 / nscl, last_tile = n > 0 ? T0 + (u1 - 1) / nscl : first_tile;
  float fin[RB][NP][4], first[RB][NP][4];  // [token 2t | 2t + 1][row rho | rho + 8]: index 2 * row half + token
#pragma unroll
  for (int b = 0; b < RB; ++b)
#pragma unroll
    for (int j = 0; j < NP; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) fin[b][j][e] = first[b][j][e] = 0.f;
  // an output: bf16 into Y, or -- K cut into slices -- the slice's fp32 partial sum
  float* const part = q.partial ? q.partial + (size_t)blockIdx.y * q.M * q.N : nullptr;
  auto out = [&](int tok, int r, float v) {
    if (part)
      part[(size_t)tok * q.N + r] = v;
    else
      q.Y[(size_t)tok * q.N + r] = __float2bfloat16(v);
  };
  auto store_tile = [&](int tile, const float (&v)[RB][NP][4]) {
#pragma unroll
    for (int b = 0; b < RB; ++b)
#pragma unroll
      for (int j = 0; j < NP; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tok = j * 8 + 2 * t + (e & 1), r = tile * kRows + b * 16 + rho + (e >> 1) * 8;
          if (tok < q.M && r < q.N) out(tok, r, v[b][j][e]);
        }
  };
  auto park = [&](uint32_t base, const float (&v)[RB][NP][4]) {
#pragma unroll
    for (int b = 0; b < RB; ++b)
#pragma unroll
      for (int j = 0; j < NP; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e)
          sts32f(base + (uint32_t)((j * 8 + 2 * t + (e & 1)) * kRows + b * 16 + rho + (e >> 1) * 8) * 4, v[b][j][e]);
  };
  int tile = first_tile, sc = u0 % nscl, sc_start = sc;
  uint32_t slot = ring0, bar = bar0, ph = 0;
  int d = 0;
  for (int i = 0; i < n; ++i) {
    mbar_wait(bar, ph, abort_flag);
    uint4 wl[RB][2], wh[RB][2];  // rows rho / rho + 8 of every block; even chunk, odd chunk
    uint32_t s2_lo[RB], s2_hi[RB];
    uint32_t all = 0;
#pragma unroll
    for (int b = 0; b < RB; ++b) {
      const uint32_t blk = slot + b * kBlockBytes;
      wl[b][0] = lds128(blk + a_u0);
      wh[b][0] = lds128(blk + 1024 + a_u0);
      wl[b][1] = lds128(blk + a_u1);
      wh[b][1] = lds128(blk + 1024 + a_u1);
      s2_lo[b] = lds32(blk + 2048 + rho * 4);
      s2_hi[b] = lds32(blk + 2048 + 32 + rho * 4);
    }
#pragma unroll
    for (int b = 0; b < RB; ++b)
#pragma unroll
      for (int c = 0; c < 2; ++c)
        all ^= (wl[b][c].x ^ wl[b][c].y ^ wl[b][c].z) ^ (wl[b][c].w ^ wh[b][c].x ^ wh[b][c].y) ^
               (wh[b][c].z ^ wh[b][c].w ^ (c ? s2_hi[b] : s2_lo[b]));
    // The slot is free as soon as every lane's loads from it have returned: an instruction that reads all of their
    // results is issued (in order) before the barrier, so the slot takes the unit `depth` ahead BEFORE the products,
    // and a slot's period is the longer of the memory latency and the work on `depth` units, not their sum.
    asm volatile("" ::"r"(all) : "memory");
    __syncwarp();
    if (i + q.depth < n) feed(slot, bar);
    const uint32_t xo = (uint32_t)sc * 256, io = (uint32_t)sc * (2 * Mp * 4);
#pragma unroll
    for (int c = 0; c < 2; ++c) {
#pragma unroll
      for (int j = 0; j < NP; ++j) {
        const uint32_t xa = xlane + (uint32_t)(j * 8) * q.pstride + xo + c * 128;
        const uint4 p0 = lds128(xa), p1 = lds128(xa + 16);                  // low plane, items 2t and 2t + 1
        const uint4 h0 = lds128(xa + xhigh), h1 = lds128(xa + xhigh + 16);  // high plane
        const float2 up = lds64f(ilane + io + (uint32_t)(c * Mp + j * 8) * 4);
#pragma unroll
        for (int b = 0; b < RB; ++b) {
          const uint32_t lo[4] = {wl[b][c].x, wl[b][c].y, wl[b][c].z, wl[b][c].w};
          const uint32_t hi[4] = {wh[b][c].x, wh[b][c].y, wh[b][c].z, wh[b][c].w};
          uint32_t le[4], lq[4], he[4], hq[4];  // signed bytes 16 (q - 8) of the even and of the odd nibbles
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            le[k] = ((lo[k] << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
            lq[k] = (lo[k] & 0xF0F0F0F0u) ^ 0x80808080u;
            he[k] = ((hi[k] << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
            hq[k] = (hi[k] & 0xF0F0F0F0u) ^ 0x80808080u;
          }
          const float s_lo = c ? __uint_as_float(s2_lo[b] & 0xFFFF0000u) : __uint_as_float(s2_lo[b] << 16);
          const float s_hi = c ? __uint_as_float(s2_hi[b] & 0xFFFF0000u) : __uint_as_float(s2_hi[b] << 16);
          int al[4], ah[4];
          imma_first<false>(al, le[0], he[0], le[1], he[1], p0.x, p0.y);
          imma_first<true>(ah, le[0], he[0], le[1], he[1], h0.x, h0.y);
          imma_acc<false>(al, lq[0], hq[0], lq[1], hq[1], p0.z, p0.w);
          imma_acc<true>(ah, lq[0], hq[0], lq[1], hq[1], h0.z, h0.w);
          imma_acc<false>(al, le[2], he[2], le[3], he[3], p1.x, p1.y);
          imma_acc<true>(ah, le[2], he[2], le[3], he[3], h1.x, h1.y);
          imma_acc<false>(al, lq[2], hq[2], lq[3], hq[3], p1.z, p1.w);
          imma_acc<true>(ah, lq[2], hq[2], lq[3], hq[3], h1.z, h1.w);
          fin[b][j][0] = fmaf(s_lo * up.x, (float)(al[0] + (ah[0] << 8)), fin[b][j][0]);
          fin[b][j][1] = fmaf(s_lo * up.y, (float)(al[1] + (ah[1] << 8)), fin[b][j][1]);
          fin[b][j][2] = fmaf(s_hi * up.x, (float)(al[2] + (ah[2] << 8)), fin[b][j][2]);
          fin[b][j][3] = fmaf(s_hi * up.y, (float)(al[3] + (ah[3] << 8)), fin[b][j][3]);
        }
      }
    }
    slot += kSlotBytes;
    bar += 8;
    if (++d == q.depth) {
      d = 0;
      slot = ring0;
      bar = bar0;
      ph ^= 1;
    }
    if (++sc == nscl && i + 1 < n) {
      // the tile is finished and more follow.  Whole (begun at its first super-chunk): out from registers; begun by
      // the previous warp (only the first tile of a run can be): kept for the sums at the end.
      if (sc_start == 0) {
        store_tile(tile, fin);
      } else {
#pragma unroll
        for (int b = 0; b < RB; ++b)
#pragma unroll
          for (int j = 0; j < NP; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) first[b][j][e] = fin[b][j][e];
      }
#pragma unroll
      for (int b = 0; b < RB; ++b)
#pragma unroll
        for (int j = 0; j < NP; ++j)
#pragma unroll
          for (int e = 0; e < 4; ++e) fin[b][j][e] = 0.f;
      sc = 0;
      sc_start = 0;
      ++tile;
    }
  }
  // ---- the last tile of the run: whole -> out; else its part goes to shared memory (the warp's own ring, drained).
  // The part of a first tile begun by the previous warp goes there too.
  cp_async_wait_all();
  if (n > 0) {
    if (sc_start == 0 && sc == nscl)
      store_tile(tile, fin);
    else
      park(ring0 + kSegBytes, fin);
    if (first_tile != last_tile) park(ring0, first);
  }
  __syncthreads();
  // ---- tiles shared by several warps: their parts are added in warp order
  const int ring_bytes = q.depth * kSlotBytes;
  const uint32_t rings = smem_u32(smem + kHeader);
  constexpr int kGroups = kRows * Mp / 32;  // a warp takes 32 outputs of one tile at a time
  for (int it = warp; it < (T1 - T0) * kGroups; it += W) {
    const int tl = it / kGroups, rem = (it - tl * kGroups) * 32 + lane;
    const unsigned ua = (unsigned)tl * nscl, ub = ua + nscl - 1;  // (W * units of a CTA stays far below 2^32)
    // the warp that holds unit u: the last one whose run begins at or before u
    const int wa = min(W - 1, (int)((W * (ua + 1) - 1) / (unsigned)U)), wb = min(W - 1, (int)((W * (ub + 1) - 1) / (unsigned)U));
    if (wa == wb) continue;  // one warp had the whole tile
    const int tok = rem / kRows, row = rem - tok * kRows;
    const int r = (T0 + tl) * kRows + row;
    if (tok >= q.M || r >= q.N) continue;
    float sum = 0.f;
    for (int w = wa; w <= wb; ++w) {
      const unsigned w0 = (unsigned)(w * U) / W, w1 = (unsigned)((w + 1) * U) / W;
      if (w0 == w1) continue;  // (fewer units than warps: a warp without work)
      // the first tile of its run, when more tiles follow, is the part parked first; any other part second
      const int which = (w0 >= ua && w1 - 1 > ub) ? 0 : 1;
      sum += lds32f(rings + w * ring_bytes + which * kSegBytes + (tok * kRows + row) * 4);
    }
    out(tok, r, sum);
  }
  if (*abort_flag && tid == 0) atomicCAS(q.status, kStatusOk, kStatusGemvTimeout);
}

struct MidPlan {
  int NP, RB, W, depth, grid, ns;
  size_t smem;
  MidParams q;
};

// partial_cap: bytes of fp32 scratch for cutting K into slices across CTAs (0: K must fit whole)
bool make_mid_plan(int M, int N, int K, int flags, int sm_count, size_t partial_cap, MidPlan* out) {
  MidPlan pl{};
  pl.NP = (M + 7) / 8;
  const int Mp = pl.NP * 8, nsc = K / 256;
  const int forced_depth = (flags >> 4) & 0xF;  // bits 4-7: ring slots per warp (diagnostics)
  const int forced_rb = (flags >> 10) & 3;      // bits 10-11: 16-row blocks per tile (diagnostics)
  const int forced_ns = (flags >> 24) & 0xF;    // bits 24-27: K slices across CTAs (diagnostics)
  // 32-row tiles (twelve warps for sixteen tokens) measured slower (8 tokens: 14.9 against 13.5 us; 16: 22.6 against
  // 19.4) and run only when asked for
  struct Shape { int RB, W; };
  const Shape shapes[2] = {{2, pl.NP == 2 ? 12 : 16}, {1, 16}};
  // K whole where its X fits beside rings of two slots (28672 x 8192 at eight tokens: 31.5 us whole, 37.2 in two
  // slices); else K slices across CTAs (blockIdx.y), as few as let the slice's X fit beside rings of three slots (two
  // at worst): 3584 x 18944 takes 3 at eight tokens, 5 at sixteen.  The slices' fp32 partial sums are added by a
  // kernel behind.
  // Fewer row tiles than half the SMs: K slices also where X would fit whole, as many as fill the SMs (512 x 3584: 32
  // tiles, 4 slices)
  int ns_min = 1;
  {
    const int n16 = (N + 15) / 16;
    if (n16 * 2 <= sm_count && !forced_ns && !(flags & kFlagForceNoSplitK))
      for (int ns = std::min(std::min(nsc, 8), sm_count / n16); ns >= 2; --ns)
        if ((nsc + (nsc + ns - 1) / ns - 1) / ((nsc + ns - 1) / ns) == ns && (size_t)ns * M * N * sizeof(float) <= partial_cap) {
          ns_min = ns;
          break;
        }
  }
  bool found = false;
  for (int want_depth = 4; want_depth >= 2 && !found; --want_depth) {
    for (int ns = ns_min; ns <= std::min(nsc, 8) && !found; ++ns) {
      if (want_depth == 4 && ns > ns_min) break;  // first pass: K whole (or in its fewest slices), any depth
      if (forced_ns && ns != forced_ns) continue;
      if (ns > 1 && ((flags & kFlagForceNoSplitK) || (size_t)ns * M * N * sizeof(float) > partial_cap)) continue;
      const int scps = (nsc + ns - 1) / ns;
      if ((nsc + scps - 1) / scps != ns) continue;
      const int pstride = scps * 256 + 16;
      const size_t x_bytes = (size_t)2 * Mp * pstride, info_bytes = (size_t)2 * scps * Mp * 4;
      for (const Shape& sh : shapes) {
        if (forced_rb ? forced_rb != sh.RB : sh.RB == 2) continue;
        const int slot = sh.RB * kBlockBytes;
        int depth = kMaxDepth;
        if (forced_depth >= 2 && forced_depth <= kMaxDepth) depth = forced_depth;
        for (; depth >= 2; --depth)
          if (kHeader + (size_t)sh.W * depth * slot + x_bytes + info_bytes <= (size_t)kSmemMax) break;
        if (depth < std::min(want_depth, 3) && ns > ns_min && !(forced_depth && depth >= 2)) continue;
        if (depth < 2) continue;
        // the parts of the at most two partial tiles of a warp go into its drained ring
        if ((size_t)2 * Mp * sh.RB * 16 * 4 > (size_t)depth * slot) continue;
        pl.RB = sh.RB;
        pl.W = sh.W;
        pl.depth = depth;
        pl.ns = ns;
        pl.q.scps = scps;
        pl.q.pstride = pstride;
        pl.q.info_off = (int)x_bytes;
        pl.q.off_x = kHeader + sh.W * depth * slot;
        pl.smem = pl.q.off_x + x_bytes + info_bytes;
        found = true;
        break;
      }
    }
  }
  if (!found) return false;
  pl.q.depth = pl.depth;
  pl.q.M = M;
  pl.q.N = N;
  pl.q.K = K;
  pl.q.nsc = nsc;
  pl.q.n_tiles = (N + pl.RB * 16 - 1) / (pl.RB * 16);
  pl.grid = std::max(1, std::min(sm_count / pl.ns, pl.q.n_tiles));
  *out = pl;
  return true;
}

template <int NP, int RB, int W>
int launch_mid(const MidPlan& pl, bool pdl, cudaStream_t stream) {
  auto kernel = w4_gemv_mid_kernel<NP, RB, W>;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_done[dev]) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 0 && dev < 64) attr_done[dev] = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(pl.grid, pl.ns);
  cfg.blockDim = dim3(W * 32);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  int na = 0;
  if (pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, pl.q);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

}  // namespace

bool gemv_mid_applies(const void* X, const void* Wq, const void* S, int M, int N, int K, int G, int flags,
                      int sm_count, size_t partial_cap) {
  const bool forced = (flags & kFlagMidKernel) == kFlagMidKernel;
  if (flags & (kFlagFloatX | kFlagWideX | kFlagNoMidKernel)) return false;
  if (!forced && (flags & kFlagMidKernel)) return false;  // one of the other two kernels is asked for
  if (M < 2 || M > 16 || G != 128 || K % 256 || N < 1) return false;
  // Two to four tokens (padded to eight): only where K is long -- 3584 x 18944: 14.2-14.7 us against 17.4-21.5 with
  // the other kernels, 28672 x 8192: 31 against 32-34.5, 5120 x 13824: 15 against 20-26 -- not on the 7B-shaped tall
  // matrices, where the streaming kernel is 2.5-3.7 us shorter, nor at two tokens on 8192 x 28672 (39.0 against 37.2;
  // 28672 x 8192 at two tokens: 30.8 against 32.0).
  if (M < 5 && !forced && (K < 8192 || (M == 2 && K >= 16384 && (long)N * K > (192l << 20)))) return false;
  // Measured against the other two kernels (chained launches, weights from DRAM), five to sixteen tokens: shorter on
  // every shape tried, 7B-shaped and 70B class, from 3584 x 3584 (6.8 against 7.9 us at five tokens) to 152064 x 3584
  // (65 against 77 us); 18944 x 3584: 12.6 against 15.8 us at eight tokens, 17.4 against 25.4 at sixteen.  Matrices with
  // few rows too, their K in slices across CTAs (512 x 3584: 6.2 against 7.6 us at eight tokens, 7.0 against 9.1 at
  // sixteen; 64 x 3584: 5.5 against 9.1).
  if ((reinterpret_cast<uintptr_t>(Wq) & 15) || (reinterpret_cast<uintptr_t>(S) & 3) ||
      (reinterpret_cast<uintptr_t>(X) & 15))
    return false;
  MidPlan pl;
  return make_mid_plan(M, N, K, flags, sm_count, partial_cap, &pl);
}

size_t gemv_mid_scratch_bytes(int M, int N, int K, int flags, int sm_count, size_t partial_cap) {
  MidPlan pl;
  if (!make_mid_plan(M, N, K, flags, sm_count, partial_cap, &pl)) return 0;
  return pl.ns > 1 ? (size_t)pl.ns * M * N * sizeof(float) : 0;
}

int gemv_mid_describe(int M, int N, int K, int flags, int sm_count, size_t partial_cap, char* buf, int buflen) {
  MidPlan pl;
  if (!make_mid_plan(M, N, K, flags, sm_count, partial_cap, &pl)) return 0;
  return snprintf(buf, buflen,
                  "many-token kernel: %d CTAs of %d warps (1 per SM), %d tiles of %d rows x %d super-chunks cut into "
                  "equal runs per warp, %d token group(s) of 8, 2 planes (16-bit X), ring depth %d, K slices across "
                  "CTAs %d%s, %zu KB smem",
                  pl.grid * pl.ns, pl.W, pl.q.n_tiles, pl.RB * 16, pl.q.scps, pl.NP, pl.depth, pl.ns,
                  pl.ns > 1 ? " (sum kernel)" : "", pl.smem >> 10);
}

int gemv_mid_launch(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, const Workspace& ws,
                    int flags, int sm_count, cudaStream_t stream) {
  MidPlan pl;
  if (!make_mid_plan(M, N, K, flags, sm_count, ws.partial ? ws.partial_bytes : 0, &pl)) return kErrTooLarge;
  pl.q.X = static_cast<const __nv_bfloat16*>(X);
  pl.q.Wq = static_cast<const unsigned char*>(Wq);
  pl.q.S = static_cast<const __nv_bfloat16*>(S);
  pl.q.Y = static_cast<__nv_bfloat16*>(Y);
  pl.q.status = ws.status;
  pl.q.partial = pl.ns > 1 ? ws.partial : nullptr;
  const bool pdl = (flags & kFlagNoPdl) == 0;
  int rc;
  if (pl.RB == 1)
    rc = pl.NP == 1 ? launch_mid<1, 1, 16>(pl, pdl, stream) : launch_mid<2, 1, 16>(pl, pdl, stream);
  else
    rc = pl.NP == 1 ? launch_mid<1, 2, 16>(pl, pdl, stream) : launch_mid<2, 2, 12>(pl, pdl, stream);
  if (rc != 0 || pl.ns == 1) return rc;
  GemvParams p{};  // what the kernel that adds the slices reads
  p.Y = pl.q.Y;
  p.M = M;
  p.N = N;
  p.K = K;
  p.nslices = pl.ns;
  p.partial = ws.partial;
  p.status = ws.status;
  return launch_sum_slices(p, sm_count, pdl, stream);
}

}  // namespace b2
