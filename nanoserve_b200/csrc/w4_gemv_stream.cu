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

#include "w4_gemv_shared.cuh"

namespace b2 {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kHeader = 2048;       // abort flag, RMSNorm partial sums [16][16] at 256, factors [16] at 1280
constexpr int kNormSs = 256;
constexpr int kNormInv = 1280;
constexpr int kSmemTwoPerSm = 112 * 1024;
constexpr int kSmemMax = 227 * 1024;

struct StreamParams {
  const uint32_t* Wq;
  int wrow;          // 32-bit words per row of Wq (K / 8)
  int ks;            // warps that share one 16-row block along K (1, 2, 4 or 8)
  int nch;           // 128-chunks in K
  int cps;           // chunks per cross-CTA slice (blockIdx.y)
  int gs_pitch;      // scale columns per row held in shared memory
  int sc_contig;     // the CTA's scales are one contiguous 16-byte aligned region of S
  int off_info, off_sc, off_x, off_red;
  int pstride;       // bytes between planes of the staged X
};

__device__ __forceinline__ uint4 ldg_stream(const uint32_t* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
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
template <int P>
__device__ __forceinline__ void stage_x_planes(const GemvParams& p, uint32_t xs_base, int pstride, uint32_t info_base,
                                               const float* inv, int cb, int nch, int tid) {
  constexpr int B = 8 * P;
  constexpr uint32_t kBias = P == 4 ? 0x00808080u : 0x00000080u;
  constexpr int UN = 2;  // items in flight per thread: a load from L2 takes a microsecond under the weight stream
  const int items_tok = nch * 8;
  const int items = p.M * items_tok;
  const int items_pad = (items + 31) & ~31;
  const int half_mp = (p.M * P) >> 1;
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  for (int it0 = tid; it0 < items_pad; it0 += kThreads * UN) {
    uint4 va[UN], vb[UN];
#pragma unroll
    for (int q = 0; q < UN; ++q) {
      va[q] = zero4;
      vb[q] = zero4;
      const int it = it0 + q * kThreads;
      if (it < items) {
        const int m = it / items_tok;
        const int r = it - m * items_tok;
        const int k0 = cb * 128 + r * 16;
        va[q] = load_x_unit(p, m, k0, inv);
        vb[q] = load_x_unit(p, m, k0 + 8, inv);
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
        u[2 * i] = ((uint32_t)__float2int_rn(__uint_as_float(w[i] << 16) * down) + kBias) ^ kBias;
        u[2 * i + 1] = ((uint32_t)__float2int_rn(__uint_as_float(w[i] & 0xFFFF0000u) * down) + kBias) ^ kBias;
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
        if (valid) sts128(xs_base + (m * P + l) * pstride + r * 16, make_uint4(pl[l][0], pl[l][1], pl[l][2], pl[l][3]));
      }
      if (valid && (r & 7) == 0) {
        const int ch = r >> 3;
#pragma unroll
        for (int j = 0; j < P / 2; ++j) {
          const uint32_t up0 = bad ? 0x7FC00000u : (uint32_t)((int)eb - B - 1 + 16 * j) << 23;
          const uint32_t up1 = bad ? 0x7FC00000u : (uint32_t)((int)eb - B + 7 + 16 * j) << 23;
          sts128(info_base + (ch * half_mp + ((m * P) >> 1) + j) * 16,
                 make_uint4((uint32_t)zc[2 * j], (uint32_t)zc[2 * j + 1], up0, up1));
        }
      }
    }
  }
}

// NT: tiles of eight B columns (M x P columns in all).  P: planes per token.  RING: chunks a lane keeps in flight.
template <int NT, int P, int RING>
__global__ void __launch_bounds__(kThreads, 2) w4_gemv_stream_kernel(const GemvParams p, const StreamParams q) {
  extern __shared__ __align__(128) unsigned char smem[];
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int MP = p.M * P;

  // ---- geometry: the CTA owns kWarps / ks row blocks of 16 rows; a warp one K slice of one of them
  const int rbpc = kWarps / q.ks;
  const int rbl = warp / q.ks, sl_in = warp - rbl * q.ks;
  const int row0 = blockIdx.x * rbpc * 16;                 // first row of the CTA
  const int rows_cta = min(rbpc * 16, p.N - row0);
  const int cb = blockIdx.y * q.cps, ce = min(q.nch, cb + q.cps);  // the CTA's chunks of K
  const int ncc = ce - cb;
  const int c0 = cb + (ncc * sl_in) / q.ks, c1 = cb + (ncc * (sl_in + 1)) / q.ks;  // the warp's chunks
  const bool active = row0 + rbl * 16 < p.N;
  if (tid == 0) *abort_flag = 0;

  pdl_launch_dependents();  // the next kernel of the stream may become resident and start its own prefetch

  // ---- weight prefetch: constant data, needs nothing from the previous kernel
  const int row_lo = min(row0 + rbl * 16 + g, p.N - 1), row_hi = min(row0 + rbl * 16 + g + 8, p.N - 1);
  const uint32_t* wlo = q.Wq + (size_t)row_lo * q.wrow + t * 4;
  const uint32_t* whi = q.Wq + (size_t)row_hi * q.wrow + t * 4;
  uint4 wb[RING][2];
#pragma unroll
  for (int d = 0; d < RING; ++d) {
    wb[d][0] = make_uint4(0u, 0u, 0u, 0u);
    wb[d][1] = make_uint4(0u, 0u, 0u, 0u);
    if (active && c0 + d < c1) {
      wb[d][0] = ldg_stream(wlo + (c0 + d) * 16);
      wb[d][1] = ldg_stream(whi + (c0 + d) * 16);
    }
  }
  // ---- scales of the CTA's rows and chunks -> shared memory [rows_cta][gs_pitch] bf16
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
  if (p.tp.wait_sig != nullptr) {
    if (tid == 0) tp_wait(p.tp, abort_flag);
    __syncthreads();
  }
  const uint32_t info_base = smem_u32(smem + q.off_info);
  const uint32_t xs_base = smem_u32(smem + q.off_x);
  {
    float* inv = reinterpret_cast<float*>(smem + kNormInv);
    if (p.pro == kProAddRmsNorm) rmsnorm_factors<kThreads>(p, reinterpret_cast<float*>(smem + kNormSs), inv, tid);
    stage_x_planes<P>(p, xs_base, q.pstride, info_base, inv, cb, ncc, tid);
  }
  cp_async_wait_all();
  __syncthreads();

  // ---- main loop
  float fin[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) fin[nt][i] = 0.f;

  if (active && c0 < c1) {
    // B fragments: lane (g, t) holds column nt * 8 + g, items 2t and 2t + 1 of the chunk
    uint32_t xaddr[NT], iaddr[NT];
    bool bval[NT], aval[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int colb = nt * 8 + g, cola = nt * 8 + 2 * t;
      bval[nt] = colb < MP;
      aval[nt] = cola < MP;
      xaddr[nt] = xs_base + (bval[nt] ? colb : 0) * q.pstride + t * 32;
      iaddr[nt] = info_base + ((aval[nt] ? cola : 0) >> 1) * 16;
    }
    const int istep = (MP >> 1) * 16;  // bytes of info per chunk
    // this lane's scales: rows g and g + 8 of the warp's block
    const uint32_t sc_lo = sc_base + ((rbl * 16 + g) * q.gs_pitch) * 2;
    const uint32_t sc_hi = sc_base + ((min(rbl * 16 + g + 8, rows_cta - 1)) * q.gs_pitch) * 2;
    uint32_t k_nib_lo = 0x0F0F0F0Fu, k_nib_hi = 0xF0F0F0F0u;
    asm volatile("" : "+r"(k_nib_lo), "+r"(k_nib_hi));
    const int gdiv = p.gdiv;

    for (int cc = c0; cc < c1; cc += RING) {
#pragma unroll
      for (int d = 0; d < RING; ++d) {
        const int c = cc + d;
        if (c < c1) {
          // unpack: A fragments of the two even-nibble and the two odd-nibble products
          const uint32_t lo[4] = {wb[d][0].x, wb[d][0].y, wb[d][0].z, wb[d][0].w};
          const uint32_t hi[4] = {wb[d][1].x, wb[d][1].y, wb[d][1].z, wb[d][1].w};
          uint32_t ae[2][4], ao[2][4];
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            ae[j][0] = lo[2 * j] & k_nib_lo;
            ae[j][1] = hi[2 * j] & k_nib_lo;
            ae[j][2] = lo[2 * j + 1] & k_nib_lo;
            ae[j][3] = hi[2 * j + 1] & k_nib_lo;
            ao[j][0] = lo[2 * j] & k_nib_hi;
            ao[j][1] = hi[2 * j] & k_nib_hi;
            ao[j][2] = lo[2 * j + 1] & k_nib_hi;
            ao[j][3] = hi[2 * j + 1] & k_nib_hi;
          }
          // the registers are free again: fetch the chunk RING ahead
          if (c + RING < c1) {
            wb[d][0] = ldg_stream(wlo + (c + RING) * 16);
            wb[d][1] = ldg_stream(whi + (c + RING) * 16);
          }
          const int crel = c - cb;
          const int gi = (gdiv == 1 ? c : c / gdiv) - gs0;
          const float s_lo = __uint_as_float(lds_u16s(sc_lo + gi * 2) << 16);
          const float s_hi = __uint_as_float(lds_u16s(sc_hi + gi * 2) << 16);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            uint4 x0 = make_uint4(0u, 0u, 0u, 0u), x1 = make_uint4(0u, 0u, 0u, 0u);
            if (bval[nt]) {
              x0 = lds128(xaddr[nt] + crel * 128);
              x1 = lds128(xaddr[nt] + crel * 128 + 16);
            }
            uint4 inf = make_uint4(0u, 0u, 0u, 0u);
            if (aval[nt]) inf = lds128(iaddr[nt] + crel * istep);
            int acc_e[4], acc_o[4];
            imma_u8s8(acc_e, ae[0][0], ae[0][1], ae[0][2], ae[0][3], x0.x, x0.y, 0, 0, 0, 0);
            imma_u8s8(acc_o, ao[0][0], ao[0][1], ao[0][2], ao[0][3], x0.z, x0.w, (int)inf.x, (int)inf.y, (int)inf.x,
                      (int)inf.y);
            imma_u8s8(acc_e, ae[1][0], ae[1][1], ae[1][2], ae[1][3], x1.x, x1.y, acc_e[0], acc_e[1], acc_e[2],
                      acc_e[3]);
            imma_u8s8(acc_o, ao[1][0], ao[1][1], ao[1][2], ao[1][3], x1.z, x1.w, acc_o[0], acc_o[1], acc_o[2],
                      acc_o[3]);
            const float up0 = __uint_as_float(inf.z), up1 = __uint_as_float(inf.w);
            fin[nt][0] = fmaf(s_lo * up0, (float)(acc_e[0] * 16 + acc_o[0]), fin[nt][0]);
            fin[nt][1] = fmaf(s_lo * up1, (float)(acc_e[1] * 16 + acc_o[1]), fin[nt][1]);
            fin[nt][2] = fmaf(s_hi * up0, (float)(acc_e[2] * 16 + acc_o[2]), fin[nt][2]);
            fin[nt][3] = fmaf(s_hi * up1, (float)(acc_e[3] * 16 + acc_o[3]), fin[nt][3]);
          }
        }
      }
    }
  }

  // ---- the warp's sums per (token, row): digits of one token are added here, K slices after the barrier
  float* red = reinterpret_cast<float*>(smem + q.off_red);  // [warp][token][16 rows]
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int cola = nt * 8 + 2 * t;
    float v_lo = fin[nt][0] + fin[nt][1], v_hi = fin[nt][2] + fin[nt][3];
    if constexpr (P == 4) {
      v_lo += __shfl_xor_sync(0xffffffffu, v_lo, 1);
      v_hi += __shfl_xor_sync(0xffffffffu, v_hi, 1);
    }
    const bool writer = cola < MP && (P == 2 || (t & 1) == 0);
    if (writer) {
      const int m = cola / P;
      red[(warp * p.M + m) * 16 + g] = v_lo;
      red[(warp * p.M + m) * 16 + g + 8] = v_hi;
    }
  }
  __syncthreads();
  const int slice = blockIdx.y;
  for (int idx = tid; idx < p.M * rows_cta; idx += kThreads) {
    const int m = idx / rows_cta, r = idx - m * rows_cta;
    const float* src = red + (((r >> 4) * q.ks) * p.M + m) * 16 + (r & 15);
    float sum = 0.f;
    for (int s = 0; s < q.ks; ++s) sum += src[s * p.M * 16];
    const int n = row0 + r;
    if (p.nslices > 1)
      __stcg(p.partial + ((size_t)slice * p.M + m) * p.N + n, sum);
    else if (p.tp.world)
      tp_store(p.tp, m, n, __float2bfloat16(sum));
    else
      p.Y[(size_t)m * p.N + n] = __float2bfloat16(sum);
  }
  if (p.tp.world) {
    __syncthreads();
    if (warp == 0) tp_signal(p.tp, lane);
  }
  if (*abort_flag && tid == 0) atomicCAS(p.status, kStatusOk, kStatusGemvTimeout);
}

struct StreamPlan {
  int P, NT, ks, nslices, cps, grid_x;
  size_t smem;
  StreamParams q;
};

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Shared memory of a CTA that owns `rbpc` row blocks and `cps` chunks of K.
size_t stream_smem(int M, int P, int rbpc, int cps, int gs_pitch, StreamParams* q) {
  const int MP = M * P;
  size_t off = kHeader;
  q->off_info = (int)off;
  off += (size_t)cps * (MP / 2) * 16;
  q->off_sc = (int)off;
  off = align_up(off + (size_t)rbpc * 16 * gs_pitch * 2 + 16, 128);
  q->off_x = (int)off;
  q->pstride = cps * 128 + 16;
  off = align_up(off + (size_t)MP * q->pstride, 128);
  q->off_red = (int)off;
  off += (size_t)kWarps * M * 16 * 4;
  return off;
}

bool make_stream_plan(int M, int N, int K, int G, const void* S, int flags, int sm_count, size_t partial_cap,
                      StreamPlan* out) {
  StreamPlan pl{};
  pl.P = M <= 2 ? 4 : 2;
  pl.NT = (M * pl.P + 7) / 8;
  const int nch = K / 128, gdiv = G / 128, KG = K / G;
  const int n_rb = (N + 15) / 16;
  // warps per row block: as few as keep every SM busy with one CTA (each warp then has a long run of chunks to
  // stream), more for matrices with few rows.  Bits 20-23 of the flags force a value (diagnostics).
  int ks = 1;
  while (ks < 8 && (long)n_rb * ks < (long)sm_count * kWarps * 3 / 4 && nch / (ks * 2) >= 2) ks *= 2;
  const int forced_ks = (flags >> 20) & 0xF;
  if (forced_ks == 1 || forced_ks == 2 || forced_ks == 4 || forced_ks == 8) ks = forced_ks;
  pl.ks = ks;
  const int rbpc = kWarps / ks;
  pl.grid_x = (n_rb + rbpc - 1) / rbpc;
  // K slices across CTAs: only when the staged X of one CTA does not fit otherwise
  const int forced_ns = (flags >> 24) & 0x3F;
  bool found = false;
  for (int pass = 0; pass < 2 && !found; ++pass) {
    const size_t cap = pass == 0 ? kSmemTwoPerSm : kSmemMax;
    for (int ns = 1; ns <= std::min(nch, 16); ++ns) {
      if (forced_ns && ns != forced_ns) continue;
      if (pass == 0 && ns > 1 && !forced_ns) break;  // first choice: no split, two CTAs per SM
      const int cps = (nch + ns - 1) / ns;
      if ((nch + cps - 1) / cps != ns) continue;
      if (ns > 1 && ((flags & kFlagForceNoSplitK) || (size_t)ns * M * N * sizeof(float) > partial_cap)) continue;
      const int gs_pitch = ns == 1 ? KG : (cps + gdiv - 1) / gdiv + 1;
      StreamParams q{};
      const size_t smem = stream_smem(M, pl.P, rbpc, cps, gs_pitch, &q);
      if (smem > cap) continue;
      pl.nslices = ns;
      pl.cps = cps;
      pl.smem = smem;
      pl.q = q;
      pl.q.gs_pitch = gs_pitch;
      found = true;
      break;
    }
  }
  if (!found) return false;
  pl.q.ks = ks;
  pl.q.nch = nch;
  pl.q.cps = pl.cps;
  pl.q.wrow = K / 8;
  pl.q.sc_contig = pl.nslices == 1 && (reinterpret_cast<uintptr_t>(S) & 15) == 0;
  *out = pl;
  return true;
}

template <int NT, int P, int RING>
int launch_stream(const GemvParams& p, const StreamPlan& pl, bool pdl, cudaStream_t stream) {
  auto kernel = w4_gemv_stream_kernel<NT, P, RING>;
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
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, p, pl.q);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

}  // namespace

bool gemv_stream_applies(const void* Wq, int M, int N, int K, int G, int flags) {
  return !(flags & (kFlagRingKernel | kFlagFloatX)) && M >= 1 && M <= 16 && N >= 1 && G % 128 == 0 && K % 128 == 0 &&
         K % G == 0 && (reinterpret_cast<uintptr_t>(Wq) & 15) == 0;
}

size_t gemv_stream_grid(int M, int N, int K, int G, int flags, int sm_count, size_t partial_cap) {
  StreamPlan pl;
  if (!make_stream_plan(M, N, K, G, nullptr, flags, sm_count, partial_cap, &pl)) return 0;
  return (size_t)pl.grid_x * pl.nslices;
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
  const bool no_split = !have_scratch || (tp != nullptr && tp->world > 0);
  if (!make_stream_plan(M, N, K, G, S, no_split ? (flags | kFlagForceNoSplitK) : flags, sm_count, ws.partial_bytes, &pl))
    return kStreamNotApplicable;
  GemvParams p{};
  p.X = static_cast<const __nv_bfloat16*>(X);
  p.S = static_cast<const __nv_bfloat16*>(S);
  p.Y = static_cast<__nv_bfloat16*>(Y);
  p.M = M; p.N = N; p.K = K; p.G = G;
  p.KG = K / G;
  p.gdiv = G / 128;
  p.nchunks = K / 128;
  p.nslices = pl.nslices;
  p.cps = pl.cps;
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
    if (tp->world > 0) {
      if (!ws.counters || ws.n_counters < 2) return kErrWorkspace;
      p.tp.local_count = ws.counters + ws.n_counters - 1;
    }
  }
  p.sum_kernel = pl.nslices > 1 ? 1 : 0;
  pl.q.Wq = static_cast<const uint32_t*>(Wq);
  const bool pdl = (flags & kFlagNoPdl) == 0;
  int rc;
  if (pl.P == 4) {
    rc = launch_stream<1, 4, 8>(p, pl, pdl, stream);
  } else {
    switch (pl.NT) {
      case 1: rc = launch_stream<1, 2, 8>(p, pl, pdl, stream); break;
      case 2: rc = launch_stream<2, 2, 6>(p, pl, pdl, stream); break;
      case 3: rc = launch_stream<3, 2, 4>(p, pl, pdl, stream); break;
      default: rc = launch_stream<4, 2, 4>(p, pl, pdl, stream); break;
    }
  }
  if (rc != 0 || !p.sum_kernel) return rc;
  return launch_sum_slices(p, sm_count, pdl, stream);
}

}  // namespace b2
