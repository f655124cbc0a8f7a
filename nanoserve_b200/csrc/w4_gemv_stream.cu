// W4A16 decode GEMV for sm_100a, register-streaming kernel:  Y[M,N] (bf16) = X[M,K] (bf16) . dequant(Wq, S)^T.
//
// Replaces the reference's w4a16_gemv_kernel / w4a16_gemv (kernels/quant/w4a16.cuh:42-115) for G % 128 == 0 and
// K % 128 == 0 (every shape of the benchmark configurations); other shapes run the shared-memory ring kernel of
// w4_gemv.cu.  Same operands, same weight format.
//
// Why this shape of kernel.  The GEMV moves 0.52 bytes per weight and does almost no arithmetic, so what a launch
// costs beyond its bytes is start-up, hand-overs and tail.  Here there is no producer warp, no ring of barriers and
// no reducer warp: a CTA of eight warps owns up to 128 consecutive rows, a warp owns a 16-row block (or a K slice of
// one) for the whole launch and keeps its partial sums in registers.
//   * Weights go from global memory straight into registers, in the fragment layout of mma.sync.m16n8k32: lane
//     (g, t) loads 16 bytes (32 nibbles) of rows g and g + 8 per 128-wide chunk of K, and keeps kRing chunks in
//     flight (64 registers).  A warp has 6 to 8 KB outstanding, a CTA 48 to 64 KB, two CTAs per SM: enough to
//     cover the HBM latency at full bandwidth.  Every 64-byte piece a quad reads is followed by its other half one
//     chunk later; the loads ask L2 for the whole 128-byte line.
//   * The CTA is launched with programmatic stream serialization and uses half an SM (256 threads x 128
//     registers, well under half the shared memory), so the CTAs of the NEXT kernel of the stream become resident
//     while this one still computes and have their first chunks (constant data) in registers before their input
//     exists.  Scales of the CTA's rows are copied to shared memory with cp.async in the same prefetch phase.
//   * Unpack: (w & 0x0F0F0F0F) holds the four even-k nibbles of a word as bytes, (w & 0xF0F0F0F0) the four odd-k
//     nibbles times 16: ready-made unsigned A fragments, two LOP3 per eight weights, no shift, no conversion.
//   * X is staged once per CTA, after griddepcontrol.wait, as block fixed point: per (token, 128-chunk) every value
//     is scaled by a power of two so that the largest magnitude lands in [2^(8P-3), 2^(8P-2)), rounded to an
//     integer and split into P signed base-256 digits ("planes"; P = 4 for M <= 2, P = 2 above).  The planes of all
//     tokens are the COLUMNS of the mma's B operand (M x P columns, eight per mma), so one token costs the same
//     number of mma instructions with four planes as with one, and the 32-bit form makes the product exact to
//     fp32 rounding for M <= 2.  The zero-point is the initial value of an accumulator (-128 times the digit sum of
//     the chunk, exact in integers).  One int-to-float conversion per (row, chunk, column), times group scale and
//     the chunk's power of two, fp32 accumulation over the chunks.
//   * K reduction: inside the mma across a quad; across the K slices of a row block (when a CTA gives several
//     warps to one block) through shared memory at the very end, in slice order; across CTAs (only when the
//     staged X of a long K and many tokens does not fit) through fp32 partial sums and the sum kernel.
//   * Optional prologue (add + RMSNorm, SwiGLU) while X is staged; optional tensor-parallel epilogue (peer stores
//     into every rank's gathered row, one arrival signal per launch) and input wait.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "w4_gemv_shared.cuh"

namespace b2 {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kHeader = 3072;       // abort flag; mbarriers [warp][slot] at 64; RMSNorm partial sums [16][16] at 1024,
constexpr int kBarOffset = 64;      // factors [16] at 2048; the weight ring follows (1024-byte aligned)
constexpr int kMaxDepth = 8;
constexpr int kStagedBarOffset = 576;  // mbarrier of the bulk copies of a pre-staged X
constexpr int kLastOffset = 32;    // split K summed in the kernel: "this CTA is the last of its row group"
constexpr int kZeroOffset = 640;    // 64 bytes of zeros: what lanes without a real B column or info record read
constexpr int kNormSs = 1024;
constexpr int kNormInv = 2048;
constexpr int kSmemTwoPerSm = 112 * 1024;
constexpr int kSmemMax = 227 * 1024;

struct StreamParams {
  const uint32_t* Wq;
  int wrow;          // 32-bit words per row of Wq (K / 8)
  int ks;            // warps that share one 16-row block along K (1, 2, 4 or 8)
  int nsc;           // 256-wide super-chunks in K
  int scps;          // super-chunks per cross-CTA slice (blockIdx.y)
  int gs_pitch;      // scale columns per row held in shared memory
  int sc_contig;     // the CTA's scales are one contiguous 16-byte aligned region of S
  int off_info, off_sc, off_x, off_red;
  int pstride;       // bytes between planes of the staged X
  int depth;         // ring slots per warp
  int epi;           // kEpi*
  int n_tiles;       // row tiles of the matrix; > 0: the CTAs share them evenly (tile range from blockIdx.x), ks == 1
  int cluster;       // CTAs per cluster (1: no cluster launch); they share the conversion of X
};

// ---- thread-block clusters: the CTAs of a cluster split the conversion of X and write every piece into the shared
// memory of all of them (plain distributed-shared-memory stores), then meet at the cluster barrier
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 16 bytes into this CTA's shared memory and into the same place of every other CTA of the cluster
template <bool CL>
__device__ __forceinline__ void share128(uint32_t addr, const uint4& v, uint32_t crank, uint32_t csize) {
  sts128(addr, v);
  if constexpr (!CL) return;
  for (uint32_t r = 0; r < csize; ++r) {
    if (r == crank) continue;
    uint32_t ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(addr), "r"(r));
    asm volatile("st.shared::cluster.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(ra), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
  }
}

__device__ __forceinline__ uint32_t lds_u16s(uint32_t addr) {
  unsigned short v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void imma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1, int c0, int c1, int c2, int c3) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c0), "r"(c1), "r"(c2), "r"(c3));
}

// ---- staging of X --------------------------------------------------------------------------------------------
// A work item is 16 consecutive k of one token (two packed weight words of a lane).  Per (token, 128-chunk): e =
// biased exponent of the largest |x| (clamped); every x is multiplied by 2^(8P - 3 - (e - 127)) and rounded to an
// integer v, |v| < 2^(8P-2); v = sum_p 256^p d_p with signed digits d_p in [-128, 127] (add 0x80 to every byte below
// the top one, let the carries run, flip those bytes' top bits back).  Per plane p the item stores 16 bytes
// { d_p of k = 0,2,4,6 | 8,10,12,14 | 1,3,5,7 | 9,11,13,15 }: the B fragments of one even-nibble and one odd-nibble
// mma (the contraction index of an mma is a dummy, so the order the nibble masks produce is matched here and the
// weights are never shuffled).  Plane (m, p) is column m P + p; item i of a plane sits at byte 16 i.
// info[chunk][column pair] = { zc, zc', up, up' }: zc = -128 * (digit sum of the chunk) -- the zero-point 8 times
// the 16 the nibble products carry -- and up = 2^(e - 127 - (8P - 3)) * 256^p / 16 as a float.  A chunk that holds
// an inf or a nan gets nan factors, so the outputs become nan.
// NM: one token with the add + RMSNorm prologue whose whole row is one item per thread (K <= 4096, no K slices, no
// cluster): X, R and the norm weights are loaded ONCE, the sum of squares is reduced over the CTA in the middle of the
// item, and the conversion goes on from registers -- one L2 round trip and one barrier instead of two and two.  `ss`:
// eight floats of shared memory.
template <int P, bool CL, bool NM>
__device__ __forceinline__ void stage_x_planes(const GemvParams& p, uint32_t xs_base, int pstride, uint32_t info_base,
                                               const float* inv, int cb, int nch, int tid, uint32_t crank,
                                               uint32_t csize, float* ss) {
  constexpr int B = 8 * P;
  constexpr uint32_t kBias = P == 4 ? 0x00808080u : 0x00000080u;
  // items in flight per thread: a load from L2 takes a microsecond under the weight stream.  (Five -- all of a
  // thread's loads at K = 18944 -- was measured too: the 23 registers more cost more than the round trips saved.)
  constexpr int UN = 2;
  const int items_tok = nch * 8;
  const int items = p.M * items_tok;
  const int items_pad = (items + 31) & ~31;
  const int half_mp = (p.M * P) >> 1;
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  // the CTAs of a cluster take rounds of kThreads * UN items in turn; NM: exactly one trip for every thread
  for (int it0 = tid + (int)crank * kThreads * UN; it0 < (NM ? kThreads : items_pad);
       it0 += NM ? kThreads : kThreads * UN * (int)csize) {
    uint4 va[UN], vb[UN];
#pragma unroll
    for (int q = 0; q < UN; ++q) {
      va[q] = zero4;
      vb[q] = zero4;
    }
    if constexpr (NM) {
      const bool valid = it0 < items;
      const int k0 = it0 * 16;
      uint4 sv[2] = {zero4, zero4}, wv[2] = {zero4, zero4};
      float acc = 0.f;
      if (valid) {
        uint4 xv[2], rv[2] = {zero4, zero4};
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          xv[u] = ld_l2(reinterpret_cast<const uint4*>(p.X + k0 + 8 * u));
          if (p.R != nullptr) rv[u] = ld_l2(reinterpret_cast<const uint4*>(p.R + k0 + 8 * u));
          wv[u] = ld_l2(reinterpret_cast<const uint4*>(p.Wn + k0 + 8 * u));
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          float a[8], b[8];
          unpack8_bf16(xv[u], a);
          if (p.R != nullptr) {
            unpack8_bf16(rv[u], b);
#pragma unroll
            for (int e = 0; e < 8; ++e) a[e] = __bfloat162float(__float2bfloat16(a[e] + b[e]));
          }
          sv[u] = pack8_bf16(a);  // the (rounded) sum is a bf16 value: exact
          if (p.R != nullptr && blockIdx.x == 0 && p.Xout != nullptr)
            *reinterpret_cast<uint4*>(p.Xout + k0 + 8 * u) = sv[u];
#pragma unroll
          for (int e = 0; e < 8; ++e) acc += a[e] * a[e];
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if ((tid & 31) == 0) ss[tid >> 5] = acc;
      __syncthreads();
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) tot += ss[w];
      const float sc = rsqrtf(tot / p.K + p.eps);
      if (valid) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          float a[8], b[8];
          unpack8_bf16(sv[u], a);
          unpack8_bf16(wv[u], b);
#pragma unroll
          for (int e = 0; e < 8; ++e) a[e] = a[e] * sc * b[e];
          (u == 0 ? va[0] : vb[0]) = pack8_bf16(a);
        }
      }
    } else {
#pragma unroll
      for (int q = 0; q < UN; ++q) {
        const int it = it0 + q * kThreads;
        if (it < items) {
          const int m = it / items_tok;
          const int r = it - m * items_tok;
          const int k0 = cb * 128 + r * 16;
          va[q] = load_x_unit(p, m, k0, inv);
          vb[q] = load_x_unit(p, m, k0 + 8, inv);
        }
      }
    }
#pragma unroll
    for (int q = 0; q < UN; ++q) {
      const int it = it0 + q * kThreads;
      if (it >= items_pad) break;  // whole warps leave together: the shuffles below stay converged
      const bool valid = it < items;
      int m = 0, r = 0;
      if (valid) {
        m = it / items_tok;
        r = it - m * items_tok;
      }
      const uint32_t w[8] = {va[q].x, va[q].y, va[q].z, va[q].w, vb[q].x, vb[q].y, vb[q].z, vb[q].w};
      // largest magnitude of the chunk (8 items = 8 consecutive lanes): bf16 magnitudes order like their bit patterns
      uint32_t mx = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) mx = max(mx, max(w[i] & 0x7FFFu, (w[i] >> 16) & 0x7FFFu));
      mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      uint32_t eb = mx >> 7;
      const bool bad = eb == 255u;
      eb = min(254u, max(40u, eb));
      const float down = __uint_as_float((uint32_t)(B + 251 - (int)eb) << 23);
      uint32_t u[16];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if constexpr (P == 2) {
          // |v| < 2^14: the rounding is one fused multiply-add with 1.5 * 2^23, which leaves v in the low mantissa
          // bits (round to nearest even, like cvt.rni, at the rate of the fma pipe instead of the conversion unit's)
          constexpr uint32_t kMagicBits = 0x4B400000u;
          u[2 * i] = (__float_as_uint(fmaf(__uint_as_float(w[i] << 16), down, 12582912.f)) - kMagicBits + kBias) ^ kBias;
          u[2 * i + 1] =
              (__float_as_uint(fmaf(__uint_as_float(w[i] & 0xFFFF0000u), down, 12582912.f)) - kMagicBits + kBias) ^ kBias;
        } else {
          u[2 * i] = ((uint32_t)__float2int_rn(__uint_as_float(w[i] << 16) * down) + kBias) ^ kBias;
          u[2 * i + 1] = ((uint32_t)__float2int_rn(__uint_as_float(w[i] & 0xFFFF0000u) * down) + kBias) ^ kBias;
        }
      }
      // byte transposes: four values x P digits -> P words of four digits
      uint32_t pl[P][4];  // [plane][even lo, even hi, odd lo, odd hi]
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int b = (j & 1) * 8 + (j >> 1);  // first k of the word: 0, 8, 1, 9; then every second one
        const uint32_t t0 = __byte_perm(u[b], u[b + 2], 0x5140), t2 = __byte_perm(u[b + 4], u[b + 6], 0x5140);
        pl[0][j] = __byte_perm(t0, t2, 0x5410);
        pl[1][j] = __byte_perm(t0, t2, 0x7632);
        if constexpr (P == 4) {
          const uint32_t t1 = __byte_perm(u[b], u[b + 2], 0x7362), t3 = __byte_perm(u[b + 4], u[b + 6], 0x7362);
          pl[2][j] = __byte_perm(t1, t3, 0x5410);
          pl[3][j] = __byte_perm(t1, t3, 0x7632);
        }
      }
      int zc[P];
#pragma unroll
      for (int l = 0; l < P; ++l) {
        int c = __dp4a((int)pl[l][0], 0x01010101, 0);
        c = __dp4a((int)pl[l][1], 0x01010101, c);
        c = __dp4a((int)pl[l][2], 0x01010101, c);
        c = __dp4a((int)pl[l][3], 0x01010101, c);
        c += __shfl_xor_sync(0xffffffffu, c, 4);
        c += __shfl_xor_sync(0xffffffffu, c, 2);
        c += __shfl_xor_sync(0xffffffffu, c, 1);
        zc[l] = -128 * c;
        if (valid)
          share128<CL>(xs_base + (m * P + l) * pstride + r * 16, make_uint4(pl[l][0], pl[l][1], pl[l][2], pl[l][3]), crank,
                   csize);
      }
      if (valid && (r & 7) == 0) {
        const int ch = r >> 3;
#pragma unroll
        for (int j = 0; j < P / 2; ++j) {
          const uint32_t up0 = bad ? 0x7FC00000u : (uint32_t)((int)eb - B - 1 + 16 * j) << 23;
          const uint32_t up1 = bad ? 0x7FC00000u : (uint32_t)((int)eb - B + 7 + 16 * j) << 23;
          share128<CL>(info_base + (ch * half_mp + ((m * P) >> 1) + j) * 16,
                   make_uint4((uint32_t)zc[2 * j], (uint32_t)zc[2 * j + 1], up0, up1), crank, csize);
        }
      }
    }
  }
}

// Everything a lane carries through the main loop: running shared-memory addresses (incremented, never recomputed),
// the ring position, and the constants the unpack needs in registers.
template <int NT>
struct LoopState {
  uint32_t xaddr[NT], xstep[NT], iaddr[NT], istep[NT];
  int sel_a[NT];
  uint32_t sc_row;
  int sc_rstep, goff[2];
  uint32_t a_u0, a_u1, k_nib_lo, k_nib_hi;
  uint32_t ring0, bar0, slot, bar, ph;
  int d, depth;
  volatile int* abort_flag;
  // feed: this lane's share of a slot's copies (16 bytes of row r4 + 4 j, j = 0 .. 4 RB - 1)
  const unsigned char* src;       // row r4 of the warp's tile, this lane's 16-byte column, NEXT super-chunk to feed
  uint32_t row4;                  // bytes between rows r4 + 4 j and r4 + 4 (j + 1)
  uint32_t valid;                 // bit j: row r4 + 4 j exists (all ones except in the last tile of a ragged N)
  uint32_t dst_even, dst_odd;     // swizzled offset in the slot for even / odd j (without j * 512)
};

// Copies this lane's 16-byte pieces of the next super-chunk into the slot at `slot` and lets the slot's barrier count
// the lane in when they have landed.  A warp instruction covers four rows x 128 bytes: whole lines.  Rows beyond N
// are zero-filled (their source address is clamped to row r4).  The layout in the slot is that of a 128-byte-swizzled
// tile: 16-byte unit u of row r at u ^ (r & 7).
template <int RB, int NT>
__device__ __forceinline__ void feed_slot(LoopState<NT>& st, uint32_t slot, uint32_t bar) {
  const unsigned char* s = st.src;
  if (st.valid == (1u << (4 * RB)) - 1u) {
#pragma unroll
    for (int j = 0; j < 4 * RB; ++j) {
      asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16;" ::"r"(slot + ((j & 1) ? st.dst_odd : st.dst_even) +
                                                                            j * 512),
                   "l"(s)
                   : "memory");
      s += st.row4;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 4 * RB; ++j) {
      const bool ok = (st.valid >> j) & 1u;
      asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16, %2;" ::"r"(slot + ((j & 1) ? st.dst_odd
                                                                                                 : st.dst_even) + j * 512),
                   "l"(ok ? s + (size_t)j * st.row4 : s), "r"(ok ? 16u : 0u)
                   : "memory");
    }
  }
  cp_async_mbar_arrive_noinc(bar);
  st.src += 128;
}

// The A-side words of this lane for the slot st.slot: rows g and g + 8 of every 16-row block, 32 bytes each.
template <int RB, int NT>
__device__ __forceinline__ void load_fragments(const LoopState<NT>& st, uint32_t (&f)[2 * RB][8]) {
#pragma unroll
  for (int i = 0; i < 2 * RB; ++i) {
    const uint4 v0 = lds128(st.slot + i * 1024 + st.a_u0), v1 = lds128(st.slot + i * 1024 + st.a_u1);
    f[i][0] = v0.x; f[i][1] = v0.y; f[i][2] = v0.z; f[i][3] = v0.w;
    f[i][4] = v1.x; f[i][5] = v1.y; f[i][6] = v1.z; f[i][7] = v1.w;
  }
}

// One super-chunk of the warp: wait for its slot, pull the fragments out, products and scaling, then hand the slot the
// super-chunk `depth` ahead.  GD1: one quantization group per 128-chunk (G == 128), the scale offsets just advance.
template <int NT, int P, int RB, bool GD1>
__device__ __forceinline__ void gemv_step(LoopState<NT>& st, float (&fin)[RB][NT][4], int sc, bool refill, int gdiv,
                                          int gs0) {
  constexpr int kSlotBytes = RB * 16 * 128;
  // scales of this lane's rows (bf16 -> fp32 is a shift); they do not depend on the weights' arrival
  float s_lo[RB][2], s_hi[RB][2];
#pragma unroll
  for (int rb = 0; rb < RB; ++rb)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (NT == 1 && h != 0) continue;  // one tile: all of a lane's accumulators belong to one chunk, goff[0] tracks it
      s_lo[rb][h] = __uint_as_float(lds_u16s(st.sc_row + (2 * rb) * st.sc_rstep + st.goff[h]) << 16);
      s_hi[rb][h] = __uint_as_float(lds_u16s(st.sc_row + (2 * rb + 1) * st.sc_rstep + st.goff[h]) << 16);
    }
  uint32_t cur[2 * RB][8];
  mbar_wait(st.bar, st.ph, st.abort_flag);
  load_fragments<RB>(st, cur);
  {
    // The slot is free as soon as every lane's loads from it have returned: an instruction that reads all of their
    // results is issued (in order) before the barrier, so the slot takes the super-chunk `depth` ahead BEFORE the
    // products -- a slot's period is the longer of the memory latency and the work on `depth` super-chunks, not
    // their sum.
    uint32_t all = 0;
#pragma unroll
    for (int i = 0; i < 2 * RB; ++i)
      all ^= (cur[i][0] ^ cur[i][1] ^ cur[i][2]) ^ (cur[i][3] ^ cur[i][4] ^ cur[i][5]) ^ (cur[i][6] ^ cur[i][7]);
    asm volatile("" ::"r"(all) : "memory");
    __syncwarp();
    if (refill) feed_slot<RB>(st, st.slot, st.bar);
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    uint4 x[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) x[j] = lds128(st.xaddr[nt] + j * 16);
    const uint4 inf = lds128(st.iaddr[nt]);
    st.xaddr[nt] += st.xstep[nt];
    st.iaddr[nt] += st.istep[nt];
    const float up0 = __uint_as_float(inf.z), up1 = __uint_as_float(inf.w);
#pragma unroll
    for (int rb = 0; rb < RB; ++rb) {
      // unpack on the fly: (w & 0x0F0F0F0F) / (w & 0xF0F0F0F0) are the A fragments of the even- / odd-nibble mma
      int acc_e[4], acc_o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t a0 = cur[2 * rb][2 * j], a1 = cur[2 * rb + 1][2 * j];
        const uint32_t a2 = cur[2 * rb][2 * j + 1], a3 = cur[2 * rb + 1][2 * j + 1];
        if (j == 0) {
          imma_u8s8(acc_e, a0 & st.k_nib_lo, a1 & st.k_nib_lo, a2 & st.k_nib_lo, a3 & st.k_nib_lo, x[j].x, x[j].y, 0, 0,
                    0, 0);
          imma_u8s8(acc_o, a0 & st.k_nib_hi, a1 & st.k_nib_hi, a2 & st.k_nib_hi, a3 & st.k_nib_hi, x[j].z, x[j].w,
                    (int)inf.x, (int)inf.y, (int)inf.x, (int)inf.y);
        } else {
          imma_u8s8(acc_e, a0 & st.k_nib_lo, a1 & st.k_nib_lo, a2 & st.k_nib_lo, a3 & st.k_nib_lo, x[j].x, x[j].y,
                    acc_e[0], acc_e[1], acc_e[2], acc_e[3]);
          imma_u8s8(acc_o, a0 & st.k_nib_hi, a1 & st.k_nib_hi, a2 & st.k_nib_hi, a3 & st.k_nib_hi, x[j].z, x[j].w,
                    acc_o[0], acc_o[1], acc_o[2], acc_o[3]);
        }
      }
      const int sel = NT == 1 ? 0 : st.sel_a[nt];
      const float sl = sel ? s_lo[rb][1] : s_lo[rb][0], sh = sel ? s_hi[rb][1] : s_hi[rb][0];
      fin[rb][nt][0] = fmaf(sl * up0, (float)(acc_e[0] * 16 + acc_o[0]), fin[rb][nt][0]);
      fin[rb][nt][1] = fmaf(sl * up1, (float)(acc_e[1] * 16 + acc_o[1]), fin[rb][nt][1]);
      fin[rb][nt][2] = fmaf(sh * up0, (float)(acc_e[2] * 16 + acc_o[2]), fin[rb][nt][2]);
      fin[rb][nt][3] = fmaf(sh * up1, (float)(acc_e[3] * 16 + acc_o[3]), fin[rb][nt][3]);
    }
  }
  st.slot += kSlotBytes;
  st.bar += 8;
  if (++st.d == st.depth) {
    st.d = 0;
    st.slot = st.ring0;
    st.bar = st.bar0;
    st.ph ^= 1;
  }
  // scale offsets of the next super-chunk (one tile: goff[0] follows the lane's own chunk)
  if constexpr (GD1) {
    st.goff[0] += 4;
    st.goff[1] += 4;
  } else {
    st.goff[0] = ((2 * (sc + 1) + (NT == 1 ? st.sel_a[0] : 0)) / gdiv - gs0) * 2;
    st.goff[1] = ((2 * (sc + 1) + 1) / gdiv - gs0) * 2;
  }
}

// The same step for more than one token ("one-group" layout): the fragments come out of shared memory, so a lane is
// free to take 16 bytes of the even chunk and 16 bytes of the odd chunk of its row instead of 32 consecutive bytes;
// every mma then stays inside one quantization group, the B operand needs ONE column per (token, plane), and a
// super-chunk costs 2 x 4 mma per column tile instead of 8 per tile of twice as many columns.  mma row g reads slot
// row rho(g) = (g >> 1) | ((g & 1) << 2) so that the eight lanes of a shared-memory phase land in opposite halves
// of the swizzled 128-byte rows.  Columns: m P + p; B fragments: lane (g, t) holds column nt * 8 + g, items 2t and
// 2t + 1 of the chunk; accumulators: columns nt * 8 + 2t, + 1.
template <int NT, int P, bool GD1>
__device__ __forceinline__ void gemv_step_one(LoopState<NT>& st, float (&fin)[1][NT][4], int sc, bool refill, int gdiv,
                                              int gs0) {
  constexpr int kSlotBytes = 16 * 128;
  float s_lo[2], s_hi[2];
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    s_lo[c] = __uint_as_float(lds_u16s(st.sc_row + st.goff[c]) << 16);
    s_hi[c] = __uint_as_float(lds_u16s(st.sc_row + st.sc_rstep + st.goff[c]) << 16);
  }
  mbar_wait(st.bar, st.ph, st.abort_flag);
  uint4 wl[2], wh[2];
  wl[0] = lds128(st.slot + st.a_u0);
  wh[0] = lds128(st.slot + 1024 + st.a_u0);
  wl[1] = lds128(st.slot + st.a_u1);
  wh[1] = lds128(st.slot + 1024 + st.a_u1);
  {
    // (the slot is refilled before the products, as in gemv_step)
    uint32_t all = 0;
#pragma unroll
    for (int c = 0; c < 2; ++c)
      all ^= (wl[c].x ^ wl[c].y ^ wl[c].z) ^ (wl[c].w ^ wh[c].x ^ wh[c].y) ^ (wh[c].z ^ wh[c].w);
    asm volatile("" ::"r"(all) : "memory");
    __syncwarp();
    if (refill) feed_slot<1>(st, st.slot, st.bar);
  }
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const uint32_t lo[4] = {wl[c].x, wl[c].y, wl[c].z, wl[c].w};
    const uint32_t hi[4] = {wh[c].x, wh[c].y, wh[c].z, wh[c].w};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      // (steps are zero for lanes that read the block of zeros: their chunk offset is zero too)
      const uint32_t xa = st.xaddr[nt] + c * (st.xstep[nt] >> 1);
      const uint4 x0 = lds128(xa), x1 = lds128(xa + 16);
      const uint4 inf = lds128(st.iaddr[nt] + c * (st.istep[nt] >> 1));
      int acc_e[4], acc_o[4];
      imma_u8s8(acc_e, lo[0] & st.k_nib_lo, hi[0] & st.k_nib_lo, lo[1] & st.k_nib_lo, hi[1] & st.k_nib_lo, x0.x, x0.y, 0,
                0, 0, 0);
      imma_u8s8(acc_o, lo[0] & st.k_nib_hi, hi[0] & st.k_nib_hi, lo[1] & st.k_nib_hi, hi[1] & st.k_nib_hi, x0.z, x0.w,
                (int)inf.x, (int)inf.y, (int)inf.x, (int)inf.y);
      imma_u8s8(acc_e, lo[2] & st.k_nib_lo, hi[2] & st.k_nib_lo, lo[3] & st.k_nib_lo, hi[3] & st.k_nib_lo, x1.x, x1.y,
                acc_e[0], acc_e[1], acc_e[2], acc_e[3]);
      imma_u8s8(acc_o, lo[2] & st.k_nib_hi, hi[2] & st.k_nib_hi, lo[3] & st.k_nib_hi, hi[3] & st.k_nib_hi, x1.z, x1.w,
                acc_o[0], acc_o[1], acc_o[2], acc_o[3]);
      const float up0 = __uint_as_float(inf.z), up1 = __uint_as_float(inf.w);
      fin[0][nt][0] = fmaf(s_lo[c] * up0, (float)(acc_e[0] * 16 + acc_o[0]), fin[0][nt][0]);
      fin[0][nt][1] = fmaf(s_lo[c] * up1, (float)(acc_e[1] * 16 + acc_o[1]), fin[0][nt][1]);
      fin[0][nt][2] = fmaf(s_hi[c] * up0, (float)(acc_e[2] * 16 + acc_o[2]), fin[0][nt][2]);
      fin[0][nt][3] = fmaf(s_hi[c] * up1, (float)(acc_e[3] * 16 + acc_o[3]), fin[0][nt][3]);
    }
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    st.xaddr[nt] += st.xstep[nt];
    st.iaddr[nt] += st.istep[nt];
  }
  st.slot += kSlotBytes;
  st.bar += 8;
  if (++st.d == st.depth) {
    st.d = 0;
    st.slot = st.ring0;
    st.bar = st.bar0;
    st.ph ^= 1;
  }
  if constexpr (GD1) {
    st.goff[0] += 4;
    st.goff[1] += 4;
  } else {
    st.goff[0] = ((2 * (sc + 1)) / gdiv - gs0) * 2;
    st.goff[1] = ((2 * (sc + 1) + 1) / gdiv - gs0) * 2;
  }
}

// NT: tiles of eight B columns.  P: planes per token.  RB: 16-row blocks per warp.  GD1: G == 128.
//
// Every warp owns a private ring of q.depth shared-memory slots (RB * 16 rows x 128 bytes each: one 256-wide piece of K,
// a "super-chunk") and is its own producer: its lanes copy their 16-byte pieces with cp.async (four rows x 128 bytes per
// warp instruction: whole lines) onto the slot's mbarrier, and refill the slot as soon as the warp has pulled its
// fragments out of it.  No warp ever waits for another warp.  Measured on the way, same bytes, no arithmetic: loads
// straight into registers keep only four to six instructions per warp in flight whatever the code issues (8 warps:
// 3.0 TB/s, 32 warps: 6.1); per-warp tiled TMA boxes of 2 KB stay near 5 TB/s (the copy engine, not DRAM, sets the
// pace: prefetching the matrix into L2 first changed nothing); cp.async rings reach 6.4 TB/s with 64 KB in flight
// per SM.
//
// Lane (g, t) reads the 32 bytes [32t, 32t + 32) of row g (and g + 8, ...) of a slot: k in [64t, 64t + 64) of the
// super-chunk.  The k-slots of one mma then span two quantization groups (lanes 0-1 hold chunk 2j, lanes 2-3 chunk
// 2j + 1), which an accumulator must not mix: the B operand therefore has TWO columns per (token, plane), one whose
// digits are non-zero only in the k-slots of the even chunk and one for the odd chunk -- 2 M P columns, eight per
// mma.  For one token with four planes that is exactly one mma tile, and every accumulator of every lane is a real
// partial sum.
// CL: launched in clusters of q.cluster CTAs that share the conversion of X.  The plain variant holds no cluster
// instruction at all: with them in the code, a launch WITHOUT the cluster attribute was 0.7 us slower than before.
// NM: the add + RMSNorm prologue merged into the conversion of X (see stage_x_planes); an instantiation of its own, so
// that the plain kernel's code does not grow (with both forms inlined in one kernel the layer pass lost 2 us).
template <int NT, int P, int RB, bool GD1, bool ONE, bool CL, bool NM>
__global__ void __launch_bounds__(kThreads, 2) w4_gemv_stream_kernel(const GemvParams p, const StreamParams q) {
  extern __shared__ __align__(1024) unsigned char smem[];
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int MP = p.M * P;
  constexpr int kSlots = NT * 4;        // accumulator column pairs per warp and row block
  constexpr int kRows = RB * 16;        // rows per warp
  constexpr int kSlotBytes = kRows * 128;

  // ---- geometry: the CTA owns kWarps / ks row tiles of kRows rows; a warp one K slice of one of them
  const int tpc = kWarps / q.ks;
  const int tl = warp / q.ks, sl_in = warp - tl * q.ks;
  // balanced form: the grid is two CTAs per SM and every CTA takes its even share of the row tiles (6 or 7 of its 8
  // warps busy) -- for row counts that are neither one nor two full CTAs per SM
  int tile0 = blockIdx.x * tpc, ntile = tpc;
  if (q.n_tiles > 0) {
    tile0 = (int)(((long)blockIdx.x * q.n_tiles) / gridDim.x);
    ntile = (int)(((long)(blockIdx.x + 1) * q.n_tiles) / gridDim.x) - tile0;
  }
  const int row0 = tile0 * kRows;                          // first row of the CTA
  const int rows_cta = max(0, min(ntile * kRows, p.N - row0));  // 0: a CTA that only pads the grid to whole clusters
  const int wrow0 = row0 + tl * kRows;                     // first row of the warp
  const int scb = blockIdx.y * q.scps, sce = min(q.nsc, scb + q.scps);  // the CTA's super-chunks of K
  const int nscc = sce - scb;
  const int s0 = scb + (nscc * sl_in) / q.ks, s1 = scb + (nscc * (sl_in + 1)) / q.ks;  // the warp's
  const bool active = tl < ntile && wrow0 < p.N && s0 < s1;
  const uint32_t bar0 = smem_u32(smem + kBarOffset) + warp * (8 * kMaxDepth);
  const uint32_t ring0 = smem_u32(smem + kHeader) + warp * q.depth * kSlotBytes;
  if (tid < 4) sts128(smem_u32(smem + kZeroOffset) + tid * 16, make_uint4(0u, 0u, 0u, 0u));
  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < kWarps * kMaxDepth; ++i) mbar_init(smem_u32(smem + kBarOffset) + 8 * i, 32);
    mbar_init(smem_u32(smem + kStagedBarOffset), 1);
    fence_mbar_init();
  }
  __syncthreads();
  pdl_launch_dependents();  // the next kernel of the stream may become resident and start its own weight stream

  // ---- weight stream: constant data, needs nothing from the previous kernel.  Rows beyond N are zero-filled.
  LoopState<NT> st;
  {
    const int r4 = lane >> 3, c16 = lane & 7;
    const int last = p.N - 1 - wrow0;  // last valid row of the warp's tile, relative (negative: none)
    st.row4 = (uint32_t)q.wrow * 16u;
    st.src = reinterpret_cast<const unsigned char*>(q.Wq) + ((size_t)(active ? wrow0 : 0) + min(r4, max(last, 0))) * q.wrow * 4 +
             (size_t)s0 * 128 + c16 * 16;
    st.valid = 0;
#pragma unroll
    for (int j = 0; j < 4 * RB; ++j)
      if (r4 + 4 * j <= last) st.valid |= 1u << j;
    st.dst_even = r4 * 128 + ((uint32_t)(c16 ^ r4) << 4);
    st.dst_odd = r4 * 128 + ((uint32_t)(c16 ^ (r4 + 4)) << 4);
    st.depth = q.depth;
  }
  if (active)
    for (int d = 0; d < q.depth && s0 + d < s1; ++d) feed_slot<RB>(st, ring0 + d * kSlotBytes, bar0 + 8 * d);

  // ---- scales of the CTA's rows and chunks -> shared memory [rows_cta][gs_pitch] bf16
  const int cb = 2 * scb, ncc = 2 * nscc;  // in 128-chunks
  const int gs0 = cb / p.gdiv;
  const uint32_t sc_base = smem_u32(smem + q.off_sc);
  {
    const __nv_bfloat16* src = p.S + (size_t)row0 * p.KG + gs0;
    if (q.sc_contig) {
      const int bytes = rows_cta * p.KG * 2;
      const int units = bytes >> 4;
      for (int i = tid; i < units; i += kThreads)
        cp_async<16>(sc_base + i * 16, reinterpret_cast<const unsigned char*>(src) + i * 16, 16u);
      const int tail = (bytes & 15) >> 1;
      if (tid < tail)
        reinterpret_cast<unsigned short*>(smem + q.off_sc)[units * 8 + tid] =
            __ldg(reinterpret_cast<const unsigned short*>(src) + units * 8 + tid);
    } else {
      const int total = rows_cta * q.gs_pitch;
      for (int e = tid; e < total; e += kThreads) {
        const int r = e / q.gs_pitch, j = e - r * q.gs_pitch;
        reinterpret_cast<unsigned short*>(smem + q.off_sc)[e] =
            __ldg(reinterpret_cast<const unsigned short*>(src) + (size_t)r * p.KG + min(j, p.KG - 1 - gs0));
      }
    }
  }

  // ---- everything below depends on the previous kernel of the stream
  pdl_wait_prior_grid();
  if (p.tp.announce_world && blockIdx.x == 0 && blockIdx.y == 0 && warp == 0) tp_announce(p.tp, lane);
  if (p.tp.wait_sig != nullptr) {
    if (tid == 0) tp_wait(p.tp, abort_flag);
    __syncthreads();
  }
  const uint32_t info_base = smem_u32(smem + q.off_info);
  const uint32_t xs_base = smem_u32(smem + q.off_x);
  {
    float* inv = reinterpret_cast<float*>(smem + kNormInv);
    float* ss = reinterpret_cast<float*>(smem + kNormSs);
    uint32_t crank = 0;
    if constexpr (CL) crank = cluster_ctarank();
    if (P == 4 && !ONE && p.pro == kProStaged) {
      // X arrives converted (the producing GEMV's epilogue did it, one 128-chunk per CTA): four digit planes of K
      // bytes and 32 bytes of info per chunk, in the layout of this kernel's shared memory -- five bulk copies
      const uint32_t xbar = smem_u32(smem + kStagedBarOffset);
      const unsigned char* xb = reinterpret_cast<const unsigned char*>(p.X);
      const uint32_t plane_bytes = (uint32_t)ncc * 128u, info_bytes = (uint32_t)ncc * 32u;
      if (tid == 0) {
        mbar_arrive_expect_tx(xbar, 4u * plane_bytes + info_bytes);
#pragma unroll
        for (int l = 0; l < 4; ++l)
          bulk_g2s(xs_base + l * q.pstride, xb + (size_t)l * p.K + (size_t)cb * 128, plane_bytes, xbar);
        bulk_g2s(info_base, xb + (size_t)4 * p.K + (size_t)cb * 32, info_bytes, xbar);
      }
      mbar_wait(xbar, 0, abort_flag);
    } else if constexpr (NM) {
      stage_x_planes<P, false, true>(p, xs_base, q.pstride, info_base, inv, cb, ncc, tid, 0u, 1u, ss);
    } else {
      if (p.pro == kProAddRmsNorm) rmsnorm_factors<kThreads>(p, ss, inv, tid);
      stage_x_planes<P, CL, false>(p, xs_base, q.pstride, info_base, inv, cb, ncc, tid, crank,
                                   CL ? (uint32_t)q.cluster : 1u, ss);
    }
  }
  // The scales were copied with cp.async.wait_all semantics per thread; the weight copies of the ring are tracked by
  // their mbarriers, but wait_all waits for them as well, so only the scale copies' own group is waited for here.
  cp_async_wait_all();
  if constexpr (CL)
    cluster_sync_all();  // every CTA's share of X has landed in every CTA; nobody writes remote memory after this
  else
    __syncthreads();

  // ---- main loop
  float fin[RB][NT][4];
#pragma unroll
  for (int rb = 0; rb < RB; ++rb)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) fin[rb][nt][i] = 0.f;

  // mma row g of this lane <-> row `grow` of a 16-row block (two-chunk layout: g; one-group layout: rho(g))
  const int grow = ONE ? ((g >> 1) | ((g & 1) << 2)) : g;
  if (active) {
    const uint32_t zero_base = smem_u32(smem + kZeroOffset);
    st.sc_row = sc_base + ((tl * kRows + grow) * q.gs_pitch) * 2;
    st.sc_rstep = 8 * q.gs_pitch * 2;
    st.k_nib_lo = 0x0F0F0F0Fu;
    st.k_nib_hi = 0xF0F0F0F0u;
    asm volatile("" : "+r"(st.k_nib_lo), "+r"(st.k_nib_hi));
    st.ring0 = ring0;
    st.bar0 = bar0;
    st.slot = ring0;
    st.bar = bar0;
    st.d = 0;
    st.ph = 0;
    st.abort_flag = abort_flag;
    const int s_refill_end = s1 - q.depth;  // super-chunks before this one refill their slot
    if constexpr (ONE) {
      // Column c = m P + p.  Lanes without a real column read a block of zeros (stride zero): no predicates in the loop.
      const int chunk_info = (MP >> 1) * 16;  // bytes of info per chunk
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int colb = nt * 8 + g, cola = nt * 8 + 2 * t;
        const bool bval = colb < MP, aval = cola < MP;
        st.sel_a[nt] = 0;
        st.xaddr[nt] = bval ? xs_base + colb * q.pstride + t * 32 + (s0 - scb) * 256 : zero_base;
        st.xstep[nt] = bval ? 256 : 0;
        st.iaddr[nt] = aval ? info_base + (cola >> 1) * 16 + (s0 - scb) * 2 * chunk_info : zero_base;
        st.istep[nt] = aval ? 2 * chunk_info : 0;
      }
      st.goff[0] = (((2 * s0) / p.gdiv) - gs0) * 2;
      st.goff[1] = (((2 * s0 + 1) / p.gdiv) - gs0) * 2;
      // fragment source: slot row rho(g), 16-byte unit t of the even chunk / 4 + t of the odd chunk, swizzled by the row
      st.a_u0 = grow * 128 + ((uint32_t)(t ^ grow) << 4);
      st.a_u1 = grow * 128 + ((uint32_t)((4 + t) ^ grow) << 4);
      for (int sc = s0; sc < s1; ++sc)
        gemv_step_one<NT, P, GD1>(st, fin, sc, sc < s_refill_end, p.gdiv, gs0);
    } else {
      // Column c = h M P + (m P + p): h = which chunk of the super-chunk.  B fragments: lane (g, t) holds column
      // nt * 8 + g, and only the lanes whose k-slots lie in that column's chunk (t >> 1 == h) hold digits;
      // accumulators: columns nt * 8 + 2t, + 1.  Lanes without a real column read a block of zeros (stride zero).
      const int istep = MP * 16;  // bytes of info per super-chunk (two chunks of M P / 2 column pairs)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int colb = nt * 8 + g, cola = nt * 8 + 2 * t;
        const int hb = colb / MP, cb_ = colb - hb * MP;
        const int ha = cola / MP, ca_ = cola - ha * MP;
        const bool bval = colb < 2 * MP && hb == (t >> 1);
        const bool aval = cola < 2 * MP;
        st.sel_a[nt] = aval ? ha : 0;
        st.xaddr[nt] = bval ? xs_base + cb_ * q.pstride + t * 64 + (s0 - scb) * 256 : zero_base;
        st.xstep[nt] = bval ? 256 : 0;
        st.iaddr[nt] = aval ? info_base + ((ha * MP + ca_) >> 1) * 16 + (s0 - scb) * istep : zero_base;
        st.istep[nt] = aval ? istep : 0;
      }
      st.goff[0] = (((2 * s0 + (NT == 1 ? st.sel_a[0] : 0)) / p.gdiv) - gs0) * 2;  // one tile: the lane's own chunk
      st.goff[1] = (((2 * s0 + 1) / p.gdiv) - gs0) * 2;
      // fragment source: row g (+ 8 i) of the slot, 16-byte units 2t and 2t + 1, swizzled by the row
      st.a_u0 = g * 128 + ((uint32_t)((2 * t) ^ g) << 4);
      st.a_u1 = g * 128 + ((uint32_t)((2 * t + 1) ^ g) << 4);
      for (int sc = s0; sc < s1; ++sc) gemv_step<NT, P, RB, GD1>(st, fin, sc, sc < s_refill_end, p.gdiv, gs0);
    }
  }

  if (NT == 1 && q.ks == 1 && p.nslices == 1 &&
      (p.tp.world == 0 || (RB == 2 && q.epi == kEpiSwigluPairs && p.tp.defer))) {
    // ---- one tile, no K slices: the lanes of a quad hold the chunks and planes of the same rows; a shuffle or two,
    // and the outputs go straight from registers to Y
    float v_lo[RB], v_hi[RB];
    int m = 0;
    bool writer = false;
#pragma unroll
    for (int rb = 0; rb < RB; ++rb) {
      v_lo[rb] = fin[rb][0][0] + fin[rb][0][1];
      v_hi[rb] = fin[rb][0][2] + fin[rb][0][3];
      if constexpr (ONE) {
        // columns 2t, 2t + 1 = planes of token (2t) / P
        if (P == 4) {
          v_lo[rb] += __shfl_xor_sync(0xffffffffu, v_lo[rb], 1);
          v_hi[rb] += __shfl_xor_sync(0xffffffffu, v_hi[rb], 1);
        }
        m = P == 4 ? (t >> 1) : t;
        writer = (P == 4 ? (t & 1) == 0 : true) && m < p.M;
      } else {
        v_lo[rb] += __shfl_xor_sync(0xffffffffu, v_lo[rb], 2);
        v_hi[rb] += __shfl_xor_sync(0xffffffffu, v_hi[rb], 2);
        if (P == 4) {
          v_lo[rb] += __shfl_xor_sync(0xffffffffu, v_lo[rb], 1);
          v_hi[rb] += __shfl_xor_sync(0xffffffffu, v_hi[rb], 1);
        }
        m = P == 4 ? 0 : t;  // two planes: lanes t = 0, 1 of a quad hold tokens 0, 1
        writer = P == 4 ? t == 0 : (t < 2 && t < p.M);
      }
    }
    if (RB == 2 && P == 4 && !ONE && q.epi == kEpiSwigluStaged) {
      // silu(gate) * up as above, then straight into the converted form the next GEMV (kProStaged) copies into its
      // shared memory: this CTA's 128 activations are one 128-chunk of that GEMV's K, a warp's 16 are one item.
      // Same arithmetic as stage_x_planes on the bf16 activations, so that GEMV's outputs are bit-identical.
      auto act = [](float gv, float uv) {
        const float a = __bfloat162float(__float2bfloat16(gv)), b = __bfloat162float(__float2bfloat16(uv));
        return __float2bfloat16(a / (1.f + __expf(-a)) * b);
      };
      const uint32_t blo = t == 0 ? (uint32_t)__bfloat16_as_ushort(act(v_lo[0], v_lo[RB - 1])) : 0u;
      const uint32_t bhi = t == 0 ? (uint32_t)__bfloat16_as_ushort(act(v_hi[0], v_hi[RB - 1])) : 0u;
      uint32_t mx = max(blo & 0x7FFFu, bhi & 0x7FFFu);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      uint32_t* s_mx = reinterpret_cast<uint32_t*>(smem + kNormSs);   // [8] warp maxima
      int* s_zc = reinterpret_cast<int*>(smem + kNormSs + 64);        // [8][4] digit sums of the warps' items
      if (lane == 0) s_mx[warp] = mx;
      __syncthreads();
      uint32_t cm = 0;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) cm = max(cm, s_mx[w]);
      uint32_t eb = cm >> 7;
      const bool bad = eb == 255u;
      eb = min(254u, max(40u, eb));
      constexpr int B = 32;
      constexpr uint32_t kBias = 0x00808080u;
      const float down = __uint_as_float((uint32_t)(B + 251 - (int)eb) << 23);
      const uint32_t u_lo = ((uint32_t)__float2int_rn(__uint_as_float(blo << 16) * down) + kBias) ^ kBias;
      const uint32_t u_hi = ((uint32_t)__float2int_rn(__uint_as_float(bhi << 16) * down) + kBias) ^ kBias;
      uint32_t u[16];  // digit sets of the item's 16 values: lane 4 g holds k = g and k = g + 8
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        u[i] = __shfl_sync(0xffffffffu, u_lo, 4 * i);
        u[i + 8] = __shfl_sync(0xffffffffu, u_hi, 4 * i);
      }
      const int k_act = p.N >> 1;
      unsigned char* yb = reinterpret_cast<unsigned char*>(p.Y);
      if (lane == 0) {
        uint32_t pl[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int b = (j & 1) * 8 + (j >> 1);
          const uint32_t t0 = __byte_perm(u[b], u[b + 2], 0x5140), t2 = __byte_perm(u[b + 4], u[b + 6], 0x5140);
          const uint32_t t1 = __byte_perm(u[b], u[b + 2], 0x7362), t3 = __byte_perm(u[b + 4], u[b + 6], 0x7362);
          pl[0][j] = __byte_perm(t0, t2, 0x5410);
          pl[1][j] = __byte_perm(t0, t2, 0x7632);
          pl[2][j] = __byte_perm(t1, t3, 0x5410);
          pl[3][j] = __byte_perm(t1, t3, 0x7632);
        }
        const size_t item = (size_t)(wrow0 >> 5);  // 16 activations per warp
#pragma unroll
        for (int l = 0; l < 4; ++l) {
          int c = __dp4a((int)pl[l][0], 0x01010101, 0);
          c = __dp4a((int)pl[l][1], 0x01010101, c);
          c = __dp4a((int)pl[l][2], 0x01010101, c);
          c = __dp4a((int)pl[l][3], 0x01010101, c);
          s_zc[warp * 4 + l] = c;
          if (active)
            *reinterpret_cast<uint4*>(yb + (size_t)l * k_act + item * 16) =
                make_uint4(pl[l][0], pl[l][1], pl[l][2], pl[l][3]);
        }
      }
      __syncthreads();
      if (tid < 2 && row0 < p.N) {  // the chunk's two info records (column pairs of planes 0,1 and 2,3)
        int z0 = 0, z1 = 0;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
          z0 += s_zc[w * 4 + 2 * tid];
          z1 += s_zc[w * 4 + 2 * tid + 1];
        }
        const uint32_t up0 = bad ? 0x7FC00000u : (uint32_t)((int)eb - B - 1 + 16 * tid) << 23;
        const uint32_t up1 = bad ? 0x7FC00000u : (uint32_t)((int)eb - B + 7 + 16 * tid) << 23;
        *reinterpret_cast<uint4*>(yb + (size_t)4 * k_act + ((size_t)blockIdx.x * 2 + tid) * 16) =
            make_uint4((uint32_t)(-128 * z0), (uint32_t)(-128 * z1), up0, up1);
      }
    } else if (RB == 1 && q.epi == kEpiSwigluPairs8 && p.tp.world == 0) {
      // blocks of 8 gate rows and their 8 up rows: the lane's row g is a gate row, its row g + 8 the matching up row
      const float a = __bfloat162float(__float2bfloat16(v_lo[0])), b = __bfloat162float(__float2bfloat16(v_hi[0]));
      const int n = (wrow0 >> 1) + grow, n_act = p.N >> 1;
      if (writer && active && n < n_act) p.Y[(size_t)m * n_act + n] = __float2bfloat16(a / (1.f + __expf(-a)) * b);
    } else if (RB == 2 && q.epi == kEpiSwigluPairs) {
      // rows come as 16 gate rows followed by their 16 up rows: the warp's first block is gate, its second up, and a
      // lane holds both halves of its rows.  Each half is rounded to bf16 first (what a plain launch would have
      // stored), then silu(gate) * up in fp32 as ns_swiglu computes it, one rounding at the store.
      auto act = [](float gv, float uv) {
        const float a = __bfloat162float(__float2bfloat16(gv)), b = __bfloat162float(__float2bfloat16(uv));
        return __float2bfloat16(a / (1.f + __expf(-a)) * b);
      };
      const int n = (wrow0 >> 1) + grow, n_act = p.N >> 1;
      const __nv_bfloat16 a_lo = act(v_lo[0], v_lo[RB - 1]), a_hi = act(v_hi[0], v_hi[RB - 1]);
      if (p.tp.world) {
        // Tensor parallel (one token, deferred signal: nothing but the stores): the lanes t = 0 of four neighbouring
        // quads hold four consecutive rows; one of them collects the four and stores 8 bytes into the gathered
        // activation row of every rank (two-byte stores over NVLink are dear).
        const uint32_t lo = __bfloat16_as_ushort(a_lo), hi = __bfloat16_as_ushort(a_hi);
        uint32_t l[4] = {lo, 0, 0, 0}, h[4] = {hi, 0, 0, 0};
#pragma unroll
        for (int i = 1; i < 4; ++i) {
          l[i] = __shfl_down_sync(0xffffffffu, lo, 4 * i);
          h[i] = __shfl_down_sync(0xffffffffu, hi, 4 * i);
        }
        if ((lane & 15) == 0 && active) {  // rows n .. n + 3 and n + 8 .. n + 11 (n a multiple of 4)
          const uint2 pl = make_uint2(l[0] | (l[1] << 16), l[2] | (l[3] << 16));
          const uint2 ph = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
          const size_t at = (size_t)p.tp.seg_dst[0] + n;
          for (int r = 0; r < p.tp.world; ++r) {
            __nv_bfloat16* y = static_cast<__nv_bfloat16*>(p.tp.y_peer[r]) + at;
            if ((reinterpret_cast<uintptr_t>(y) & 7) == 0) {
              *reinterpret_cast<uint2*>(y) = pl;
              *reinterpret_cast<uint2*>(y + 8) = ph;
            } else {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                y[i] = __ushort_as_bfloat16((unsigned short)l[i]);
                y[8 + i] = __ushort_as_bfloat16((unsigned short)h[i]);
              }
            }
          }
        }
      } else if (writer && active) {
        if (n < n_act) p.Y[(size_t)m * n_act + n] = a_lo;
        if (n + 8 < n_act) p.Y[(size_t)m * n_act + n + 8] = a_hi;
      }
    } else {
#pragma unroll
      for (int rb = 0; rb < RB; ++rb) {
        const int n = wrow0 + rb * 16 + grow;
        if (writer && active) {
          if (n < p.N) p.Y[(size_t)m * p.N + n] = __float2bfloat16(v_lo[rb]);
          if (n + 8 < p.N) p.Y[(size_t)m * p.N + n + 8] = __float2bfloat16(v_hi[rb]);
        }
      }
    }
  } else {
    // ---- every accumulator column pair of the warp goes to shared memory; the sums over the chunks of a super-chunk
    // (two-chunk layout), the planes of a token and the K slices of a row tile are taken after the barrier, in fixed
    // order
    float* red = reinterpret_cast<float*>(smem + q.off_red);  // [warp][column pair][kRows]
#pragma unroll
    for (int rb = 0; rb < RB; ++rb)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int slot = nt * 4 + t;
        red[(warp * kSlots + slot) * kRows + rb * 16 + grow] = fin[rb][nt][0] + fin[rb][nt][1];
        red[(warp * kSlots + slot) * kRows + rb * 16 + grow + 8] = fin[rb][nt][2] + fin[rb][nt][3];
      }
    __syncthreads();
    const int slice = blockIdx.y;
    const int half_mp = MP >> 1;
    // a thread sums four consecutive rows of one token: 16-byte partial-sum stores, 8-byte output stores (also into
    // the peers' gathered rows, where two-byte stores over NVLink are dear)
    const int quads = (rows_cta + 3) >> 2;
    // a work item is (token, four rows, warp of the row tile along K): the ks items of an output sit in adjacent
    // lanes and meet in a butterfly of shuffles (a fixed tree: deterministic).  One thread per output used to walk
    // all ks warps' sums alone -- with four warps per tile eight threads of the CTA did all the adding.
    const int items = p.M * quads * q.ks;
    for (int it = tid; it < ((items + 31) & ~31); it += kThreads) {
      const int s = it % q.ks, idx = it / q.ks;
      const bool valid = it < items;
      const int m = valid ? idx / quads : 0, r0 = valid ? (idx - m * quads) * 4 : 0;
      float f[4] = {0.f, 0.f, 0.f, 0.f};
      if (valid) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = min(r0 + i, rows_cta - 1);
          const int tile = r / kRows, rr = r - tile * kRows;
          const float* src = red + ((tile * q.ks + s) * kSlots) * kRows + rr;
#pragma unroll
          for (int h = 0; h < (ONE ? 1 : 2); ++h)
#pragma unroll
            for (int j = 0; j < P / 2; ++j) f[i] += src[(h * half_mp + ((m * P) >> 1) + j) * kRows];
        }
      }
      for (int o = 1; o < q.ks; o <<= 1)
#pragma unroll
        for (int i = 0; i < 4; ++i) f[i] += __shfl_xor_sync(0xffffffffu, f[i], o);
      if (!valid || s != 0) continue;
      const int n0 = row0 + r0;
      if (p.nslices > 1) {
        float* d = p.partial + ((size_t)slice * p.M + m) * p.N + n0;
        if ((p.N & 3) == 0 && n0 + 3 < p.N) {
          __stcg(reinterpret_cast<float4*>(d), make_float4(f[0], f[1], f[2], f[3]));
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (n0 + i < p.N) __stcg(d + i, f[i]);
        }
      } else {
        store_out4(p, m, n0, make_float4(f[0], f[1], f[2], f[3]));
      }
    }
    if (p.nslices > 1 && !p.sum_kernel) {
      // K slices added up in the kernel: the CTAs of a row group count themselves in; the last one to arrive -- which
      // has thereby seen the partial sums of the others -- adds the slices in slice order (the same sums, the same
      // bits, as the kernel behind would produce) and resets the counter for the next launch.
      volatile int* s_last = reinterpret_cast<volatile int*>(smem + kLastOffset);
      __threadfence();
      __syncthreads();
      if (tid == 0) {
        const int old = atomicAdd(p.counters + blockIdx.x, 1);
        const int last = old == p.nslices - 1;
        if (last) p.counters[blockIdx.x] = 0;
        *s_last = last;
      }
      __syncthreads();
      if (*s_last) {
        __threadfence();
        for (int idx = tid; idx < p.M * quads; idx += kThreads) {
          const int m = idx / quads, n0 = row0 + (idx - m * quads) * 4;
          store_out4(p, m, n0, sum_slices4(p, m, n0));
        }
      }
    }
    if (p.tp.world && !p.tp.defer) {
      __syncthreads();
      if (warp == 0) tp_signal(p.tp, lane);
    }
  }
  if (*abort_flag) {
    if (tid == 0) atomicCAS(p.status, kStatusOk, kStatusGemvTimeout);
    // give copies that may still be in flight time to land before the shared memory is released
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
}

struct StreamPlan {
  bool one;
  int P, NT, RB, ks, nslices, scps, grid_x;
  size_t smem;
  StreamParams q;
};

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Shared memory of a CTA whose warps own RB * 16 rows each, `scps` super-chunks of K and `depth` ring slots.
size_t stream_smem(int M, int P, int NT, int RB, int tpc, int scps, int gs_pitch, int depth, StreamParams* q) {
  const int MP = M * P, rows = RB * 16;
  size_t off = kHeader + (size_t)kWarps * depth * rows * 128;
  q->off_info = (int)off;
  off += (size_t)scps * MP * 16;
  q->off_sc = (int)off;
  off = align_up(off + (size_t)tpc * rows * gs_pitch * 2 + 16, 128);
  q->off_x = (int)off;
  q->pstride = scps * 256 + 16;
  off = align_up(off + (size_t)MP * q->pstride, 128);
  q->off_red = (int)off;
  off += (size_t)kWarps * NT * 4 * rows * 4;
  q->depth = depth;
  return off;
}

// plain: no prologue.  Launches with one sit in fused decode steps and keep K whole where it fits: with the slices
// the step was slower, whoever adds them (3584 x 18944 with a pre-converted X: 633 -> 617 tok/s with the sum kernel
// behind, 601 with the last CTA adding)
bool make_stream_plan(int M, int N, int K, int G, const void* S, int flags, int sm_count, size_t partial_cap,
                      StreamPlan* out, int epilogue = kEpiNone, bool plain = true) {
  StreamPlan pl{};
  // One token: the two-chunk layout, four planes (32-bit block fixed point): its 2 x 4 columns fill exactly one mma
  // tile.  More tokens: the one-group layout, M P columns; four planes while they fit one tile (M <= 2), two above.
  pl.one = M > 1;
  pl.P = M <= 2 ? 4 : 2;
  pl.NT = pl.one ? (M * pl.P + 7) / 8 : 1;
  // 32 rows per warp where 16 would make more than 1.25 CTAs per SM (fewer, longer CTAs stream better than an
  // uneven second wave); bits 10-11 of the flags force 16 (1) or 32 (2) rows (diagnostics)
  {
    const long c1 = ((N + 15) / 16 + kWarps - 1) / kWarps;  // CTAs with 16 rows per warp
    pl.RB = c1 * 4 > (long)sm_count * 5 ? 2 : 1;
    // ... except where they fill both CTA slots of every SM almost exactly (37888 rows on 148 SMs: 296 CTAs): sixteen
    // warps per SM with five ring slots each then stream better than eight with two (13.1 against 14.1 us)
    if (c1 * 100 > (long)sm_count * 185 && c1 <= 2l * sm_count) pl.RB = 1;
  }
  if (((flags >> 10) & 3) == 1) pl.RB = 1;
  if (((flags >> 10) & 3) == 2) pl.RB = 2;
  if (pl.one) pl.RB = 1;
  if (epilogue != kEpiNone) pl.RB = epilogue == kEpiSwigluPairs8 ? 1 : 2;  // a warp owns a gate block and its up block
  const int rows = pl.RB * 16;
  const int nsc = K / 256, gdiv = G / 128, KG = K / G;
  const int n_tiles = (N + rows - 1) / rows;
  // warps per row tile: as few as keep every SM busy with one CTA (each warp then has a long run of K to stream),
  // more for matrices with few rows.  Bits 20-23 of the flags force a value (diagnostics).
  int ks = 1;
  while (ks < 8 && (long)n_tiles * ks < (long)sm_count * kWarps * 3 / 4 && nsc / (ks * 2) >= 2) ks *= 2;
  const int forced_ks = (flags >> 20) & 0xF;
  if (forced_ks == 1 || forced_ks == 2 || forced_ks == 4 || forced_ks == 8) ks = forced_ks;
  if (epilogue != kEpiNone) ks = 1;  // the register epilogue: a warp holds whole dot products
  // K slices across CTAs: only when the staged X of one CTA does not fit otherwise
  const int forced_ns = (flags >> 24) & 0x1F;
  const int forced_depth = (flags >> 4) & 0xF;  // bits 4-7: ring slots per warp (diagnostics)
  // the shared-memory plan for `k` warps per row tile; passes: 1 = only plans that fit two CTAs per SM
  auto search = [&](int k, int passes, int only_ns = 0) {
    const int tpc_k = kWarps / k;
    for (int pass = 0; pass < passes; ++pass) {
      const size_t cap = pass == 0 ? kSmemTwoPerSm : kSmemMax;
      for (int ns = 1; ns <= std::min(nsc, 16); ++ns) {
        if (forced_ns && ns != forced_ns) continue;
        if (only_ns && ns != only_ns) continue;
        if (pass == 0 && ns > 1 && !forced_ns && !only_ns) break;  // first choice: no split, two CTAs per SM
        const int scps = (nsc + ns - 1) / ns;
        if ((nsc + scps - 1) / scps != ns) continue;
        if (ns > 1 && ((flags & kFlagForceNoSplitK) || (size_t)ns * M * N * sizeof(float) > partial_cap)) continue;
        const int gs_pitch = ns == 1 ? KG : (2 * scps + gdiv - 1) / gdiv + 1;
        // as many ring slots as fit (a warp never needs more than its own super-chunks), at least two
        const int longest = (scps + k - 1) / k;
        for (int depth = std::min(kMaxDepth, std::max(2, longest)); depth >= 2; --depth) {
          if (forced_depth >= 2 && forced_depth <= kMaxDepth && depth != forced_depth && depth > 2) continue;
          StreamParams q{};
          const size_t smem = stream_smem(M, pl.P, pl.NT, pl.RB, tpc_k, scps, gs_pitch, depth, &q);
          if (smem > cap) continue;
          pl.nslices = ns;
          pl.scps = scps;
          pl.smem = smem;
          pl.q = q;
          pl.q.gs_pitch = gs_pitch;
          return true;
        }
      }
    }
    return false;
  };
  // Fewer CTAs than SMs (SMs idle, the second CTA slot of the others empty): twice the warps per tile double the CTAs,
  // if those still fit two per SM and all at once.  One token: 16384 x 4096 11.3 -> 9.4 us, 14336 x 4096 11.1 -> 8.6,
  // 28672 x 4096 (32 rows per warp) 16.4 -> 12.3, 16384 x 8192 23.0 -> 16.0.  Not at 148 or 296 CTAs (18944 x 3584:
  // 8.2 against 9.4 us), nor where a CTA needs an SM of its own (28672 x 8192 with 32 rows per warp: 23.0 against 30.3).
  bool found = false;
  {
    const long ctas = (n_tiles + kWarps / ks - 1) / (kWarps / ks);
    if (!pl.one && epilogue == kEpiNone && !forced_ks && ks < 8 && nsc / (ks * 2) >= 2 && ctas * 100 < sm_count * 97l &&
        (n_tiles + kWarps / (2 * ks) - 1) / (kWarps / (2 * ks)) <= 2l * sm_count && search(2 * ks, 1)) {
      ks *= 2;
      found = true;
    }
  }
  if (!found) found = search(ks, 2);
  if (!found) return false;
  // A long K with few rows, one token: the converted X of the whole K takes an SM per CTA (3584 x 18944: 112 CTAs of
  // 214 KB, every one converting 18944 values).  K slices across CTAs instead -- as many as still give at most two
  // CTAs per SM, one warp per row tile, every CTA converting its slice only -- and the sum kernel behind:
  // 3584 x 18944 13.4 -> 11.0 us (10 slices), 8192 x 28672 29.5 -> 27.7 (4 slices).
  if (plain && !pl.one && epilogue == kEpiNone && pl.RB == 1 && pl.smem > kSmemTwoPerSm && pl.nslices == 1 && !forced_ns &&
      !forced_ks && !(flags & kFlagForceNoSplitK)) {
    const long ctas_x = (n_tiles + kWarps - 1) / kWarps;
    for (int ns = (int)std::min<long>(16, 2l * sm_count / ctas_x); ns >= 2; --ns) {
      const StreamPlan keep = pl;
      if (search(1, 1, ns)) {
        ks = 1;
        break;
      }
      pl = keep;
    }
  }
  pl.ks = ks;
  const int tpc = kWarps / ks;
  pl.grid_x = (n_tiles + tpc - 1) / tpc;
  // Uneven waves.  (a) 16 rows per warp and a few CTAs more than SMs (1.05 to 1.25 per SM): the SMs that hold two are
  // the critical path (20000 x 4096: 12.4 us); instead two CTAs on EVERY SM, each with its even share of the row tiles
  // and some of its warps idle (10.4 us).  (b) CTAs that fit one per SM only, below.
  // Row counts that leave some CTA slots empty otherwise (28672 or 65536 rows) gain nothing from the even shares
  // (24.6 against 24.2 us, 23.0 against 22.5): bandwidth is a shared resource, a lighter SM just finishes early.
  // Not with forced rows per warp / K warps (diagnostics), an epilogue, or several tokens.
  int balanced_tiles = 0;
  const bool may_balance = !pl.one && epilogue == kEpiNone && ks == 1 && ((flags >> 10) & 3) == 0 && !forced_ks;
  if (may_balance && pl.RB == 1 && pl.smem <= kSmemTwoPerSm && pl.grid_x * 100l > sm_count * 105l &&
      pl.grid_x * 4l <= sm_count * 5l) {
    balanced_tiles = n_tiles;
    pl.grid_x = 2 * sm_count;
  }
  // (b) CTAs that fit one per SM only (32 rows per warp at K = 8192) and do not fill their last wave: whole waves of
  // CTAs with even shares of the tiles, at least four warps busy (57344 x 8192: 224 CTAs 50.7 us, 296 CTAs 47.5 us)
  if (may_balance && !balanced_tiles && pl.smem > kSmemTwoPerSm && pl.nslices == 1 && pl.grid_x > sm_count &&
      pl.grid_x % sm_count != 0) {
    const int waves = (pl.grid_x + sm_count - 1) / sm_count;
    if ((long)n_tiles >= (long)waves * sm_count * 4) {
      balanced_tiles = n_tiles;
      pl.grid_x = waves * sm_count;
    }
  }
  pl.q.ks = ks;
  pl.q.nsc = nsc;
  pl.q.scps = pl.scps;
  pl.q.wrow = K / 8;
  pl.q.sc_contig = pl.nslices == 1 && (reinterpret_cast<uintptr_t>(S) & 15) == 0;
  pl.q.epi = epilogue;
  pl.q.n_tiles = balanced_tiles;
  // CTAs per cluster.  The conversion of X (M * K / 16 items; every CTA needs all of them) can go round by round of
  // 512 items over the CTAs of a cluster, which write every piece into the shared memory of all of them.  Measured,
  // it does not pay: a cluster launch costs more than the rounds it saves (3584 x 18944 at one token, three rounds:
  // 13.3 us plain, 14.2 us in clusters of four; 18944 x 3584 at eight tokens, four rounds: level with the ring
  // kernel at best), a grid that fills every SM loses 4 us with clusters of four and 7 us with eight (the CTAs of a
  // cluster must sit in one GPC, so some SMs get two CTAs while others idle), and the mere presence of cluster
  // instructions in a kernel made its plain launches 0.7 us slower (hence the separate instantiation).  So it is
  // off unless B2_GEMV_CLUSTER=2|4|8 asks for it (diagnostics, and the test that keeps the path correct).
  {
    static const int forced = [] {
      const char* e = std::getenv("B2_GEMV_CLUSTER");
      const int v = e ? std::atoi(e) : 0;
      return (v == 1 || v == 2 || v == 4 || v == 8) ? v : 0;
    }();
    int c = 1;
    if (forced) c = forced;
    while (c > 1 && pl.grid_x < c) c /= 2;
    pl.q.cluster = c;
    pl.grid_x = (pl.grid_x + c - 1) / c * c;
  }
  *out = pl;
  return true;
}

template <int NT, int P, int RB, bool GD1, bool ONE, bool CL, bool NM = false>
int launch_stream_g(const GemvParams& p, const StreamPlan& pl, bool pdl, cudaStream_t stream) {
  auto kernel = w4_gemv_stream_kernel<NT, P, RB, GD1, ONE, CL, NM>;
  // Raising the dynamic shared-memory limit and the carve-out is remembered per device: done once.
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 0 && dev < 64) attr_done[dev] = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(pl.grid_x, pl.nslices);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (pl.q.cluster > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = pl.q.cluster;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, p, pl.q);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

template <int NT, int P, int RB, bool ONE>
int launch_stream(const GemvParams& p, const StreamPlan& pl, bool pdl, cudaStream_t stream) {
  if (pl.q.cluster > 1)
    return p.gdiv == 1 ? launch_stream_g<NT, P, RB, true, ONE, true>(p, pl, pdl, stream)
                       : launch_stream_g<NT, P, RB, false, ONE, true>(p, pl, pdl, stream);
  if constexpr (!ONE && NT == 1) {
    // one token, add + RMSNorm over a row of at most 4096 values: the merged prologue
    if (p.pro == kProAddRmsNorm && p.M == 1 && p.nslices == 1 && p.K <= 16 * kThreads)
      return p.gdiv == 1 ? launch_stream_g<NT, P, RB, true, ONE, false, true>(p, pl, pdl, stream)
                         : launch_stream_g<NT, P, RB, false, ONE, false, true>(p, pl, pdl, stream);
  }
  return p.gdiv == 1 ? launch_stream_g<NT, P, RB, true, ONE, false>(p, pl, pdl, stream)
                     : launch_stream_g<NT, P, RB, false, ONE, false>(p, pl, pdl, stream);
}

}  // namespace

bool gemv_stream_applies(const void* Wq, int M, int N, int K, int G, int flags) {
  if ((flags & (kFlagRingKernel | kFlagFloatX)) || M < 1 || M > 16 || N < 1 || G % 128 || K % 256 || K % G ||
      (reinterpret_cast<uintptr_t>(Wq) & 15))
    return false;
  if (flags & kFlagStreamKernel) return true;
  // Which kernel is faster, from measurements on the 7B-shaped and 70B-class linears (chained launches, weights from
  // DRAM): one token always streams; two tokens on the large 7B-shaped matrices (gate/up, down) but not on the small
  // ones (q, k, v, o: the ring kernel is 0.7 us shorter there) nor on the 70B class; three to eight tokens only on
  // tall matrices with a short K (gate/up), where the staging of M x K activations per CTA stays small.
  const long weights = (long)N * K;
  if (M == 1) return true;
  if (weights > 160l << 20) return false;
  if (M == 2) return N >= 8192 || K >= 8192;
  if (M <= 4) return K <= 4096 && N >= 8192;
  if (M <= 8) return K <= 4096 && N >= 32768;
  return false;
}

size_t gemv_stream_grid(int M, int N, int K, int G, int flags, int sm_count, size_t partial_cap) {
  StreamPlan pl;
  if (!make_stream_plan(M, N, K, G, nullptr, flags, sm_count, partial_cap, &pl)) return 0;
  return (size_t)pl.grid_x * pl.nslices;
}

int gemv_stream_describe(int M, int N, int K, int G, int flags, int sm_count, size_t partial_cap, int counters_cap,
                         char* buf, int buflen) {
  StreamPlan pl;
  if (!make_stream_plan(M, N, K, G, nullptr, flags, sm_count, partial_cap, &pl)) return 0;
  const char* sums = pl.nslices == 1 ? ""
                     : ((flags & kFlagNoSplitSumKernel) && !(flags & kFlagSplitSumKernel) && pl.grid_x <= counters_cap)
                         ? " (last CTA sums)"
                         : " (sum kernel)";
  return snprintf(buf, buflen,
                  "streaming kernel: %d CTAs of 8 warps, %d rows per warp, %d warp(s) per row tile along K, %s layout, "
                  "%d planes (%d-bit X), ring depth %d, K slices across CTAs %d%s, cluster %d, %zu KB smem",
                  pl.grid_x * pl.nslices, pl.RB * 16, pl.ks, pl.one ? "one-group" : "two-chunk", pl.P, pl.P * 8, pl.q.depth,
                  pl.nslices, sums, pl.q.cluster, pl.smem >> 10) +
         (pl.q.n_tiles ? snprintf(buf + strlen(buf), buflen - strlen(buf), ", %d row tiles shared evenly", pl.q.n_tiles) : 0);
}

size_t gemv_stream_scratch_bytes(int M, int N, int K, int G, int flags, int sm_count, size_t partial_cap) {
  StreamPlan pl;
  if (!make_stream_plan(M, N, K, G, nullptr, flags, sm_count, partial_cap, &pl)) return 0;
  return pl.nslices > 1 ? (size_t)pl.nslices * M * N * sizeof(float) : 0;
}

// Returns kStreamNotApplicable when the shape has to go to the ring kernel (no plan fits).
int gemv_stream_launch(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int G,
                       const GemvPrologue& pro, const Workspace& ws, int flags, int sm_count, cudaStream_t stream,
                       const GemvTp* tp) {
  StreamPlan pl;
  const bool have_scratch = ws.partial != nullptr;
  // a tensor-parallel producer signals its peers after its stores: no sum kernel behind it, so no split across CTAs
  bool no_split = !have_scratch || (tp != nullptr && tp->world > 0);
  if (pro.kind == kProStaged && (M != 1 || (reinterpret_cast<uintptr_t>(X) & 15) || (K & 127))) return kErrNotImplemented;
  if (pro.epilogue == kEpiSwigluStaged) {
    // a CTA must own exactly one 128-chunk of the consumer's K: 256 rows; no tensor-parallel form
    if (M != 1 || (N & 255) || (tp != nullptr && tp->world > 0) || (reinterpret_cast<uintptr_t>(Y) & 15))
      return kErrNotImplemented;
    no_split = true;
  } else if (pro.epilogue == kEpiSwigluPairs8) {
    if (M != 1 || (N & 15) || (tp != nullptr && tp->world > 0)) return kErrNotImplemented;
    no_split = true;
  } else if (pro.epilogue == kEpiSwigluPairs) {
    // served by the register epilogue of the one-token kernel only: a caller that gets this code runs the plain
    // launch followed by the SwiGLU prologue of the next one
    // (tensor parallel: a producer with a deferred signal only -- the register epilogue has no CTA-wide tail)
    if (M != 1 || (N & 31) || (tp != nullptr && tp->world > 0 && !tp->defer)) return kErrNotImplemented;
    no_split = true;
  } else if (pro.epilogue != kEpiNone) {
    return kErrBadShape;
  }
  if (!make_stream_plan(M, N, K, G, S, no_split ? (flags | kFlagForceNoSplitK) : flags, sm_count, ws.partial_bytes, &pl,
                        pro.epilogue, pro.kind == kProNone))
    return pro.epilogue != kEpiNone ? kErrNotImplemented : kStreamNotApplicable;
  if (pro.epilogue != kEpiNone &&
      (pl.nslices != 1 || pl.one || pl.RB != (pro.epilogue == kEpiSwigluPairs8 ? 1 : 2) || pl.ks != 1))
    return kErrNotImplemented;
  GemvParams p{};
  p.X = static_cast<const __nv_bfloat16*>(X);
  p.S = static_cast<const __nv_bfloat16*>(S);
  p.Y = static_cast<__nv_bfloat16*>(Y);
  p.M = M; p.N = N; p.K = K; p.G = G;
  p.KG = K / G;
  p.gdiv = G / 128;
  p.nchunks = K / 128;
  p.nslices = pl.nslices;
  p.cps = 2 * pl.scps;
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
      p.tp.local_count = ws.counters + ws.n_counters - 1;
    }
  }
  // K slices: added up by the last CTA of a row group to arrive (the default where the counters suffice; no launch
  // behind), or by the sum kernel (kFlagSplitSumKernel)
  // K slices: added up by the sum kernel behind (the default: 3584 x 18944 11.0 us against 11.7), or by the last CTA
  // of a row group to arrive (kFlagNoSplitSumKernel)
  p.sum_kernel = pl.nslices > 1 ? 1 : 0;
  if (pl.nslices > 1 && (flags & kFlagNoSplitSumKernel) && !(flags & kFlagSplitSumKernel) &&
      ws.counters && pl.grid_x <= ws.n_counters - 1 && !(tp != nullptr && tp->world > 0))
    p.sum_kernel = 0;
  pl.q.Wq = static_cast<const uint32_t*>(Wq);
  const bool pdl = (flags & kFlagNoPdl) == 0;
  int rc;
  if (!pl.one) {
    rc = pl.RB == 2 ? launch_stream<1, 4, 2, false>(p, pl, pdl, stream) : launch_stream<1, 4, 1, false>(p, pl, pdl, stream);
  } else if (pl.P == 4) {
    rc = launch_stream<1, 4, 1, true>(p, pl, pdl, stream);
  } else {
    switch (pl.NT) {
      case 1: rc = launch_stream<1, 2, 1, true>(p, pl, pdl, stream); break;
      case 2: rc = launch_stream<2, 2, 1, true>(p, pl, pdl, stream); break;
      case 3: rc = launch_stream<3, 2, 1, true>(p, pl, pdl, stream); break;
      default: rc = launch_stream<4, 2, 1, true>(p, pl, pdl, stream); break;
    }
  }
  if (rc != 0 || !p.sum_kernel) return rc;
  return launch_sum_slices(p, sm_count, pdl, stream);
}

}  // namespace b2
