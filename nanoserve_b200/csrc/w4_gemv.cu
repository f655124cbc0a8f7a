// W4A16 decode GEMV for sm_100a:  Y[M,N] (bf16) = X[M,K] (bf16) . dequant(Wq, S)^T,  1 <= M <= 16.
//
// Replaces the reference's w4a16_gemv_kernel / w4a16_gemv (kernels/quant/w4a16.cuh:42-115), which
// serves M in {1,2,4,8} only on CUDA cores.  Same operands, same weight format, fp32 accumulation.
//
// Design (HBM-bound: every weight byte is read exactly once, X is tiny and lives in shared memory):
//   * One persistent CTA per SM.  A producer lane streams the packed weights of a 32-row group into a
//     shared-memory ring with tiled TMA loads through a tensor map over Wq: boxes of 32 rows x 128 bytes
//     (two K chunks) with the 128-byte swizzle, up to NCW/2 boxes per stage, completion counted on an
//     mbarrier; several stages are in flight from the first instruction.  (Per-row untiled bulk copies
//     were measured first: the TMA unit retires about one copy per 70 cycles whatever its size, so 1 KB
//     row segments cap at ~4 TB/s; tiled boxes reach the copy-kernel bandwidth.)
//   * NCW consumer warps each take one 128-wide K chunk of the stage for both 16-row blocks.  A lane
//     reads 16 bytes (32 nibbles) per row with one 128-bit shared load; the swizzle plus a fixed
//     permutation of which tile row feeds which mma row makes those loads bank-conflict free.
//   * Unpack: three shifts + four LOP3 per word give bf16 pairs {128+q[p], 128+q[p+4]}; these feed the
//     A operand of mma.sync.m16n8k16 directly.  The contraction index of an mma is a dummy, so the
//     pairing is matched by permuting X once, when it is staged into shared memory -- the weights are
//     never shuffled.  Tokens sit on the n-side of the mma (8 per tile, two tiles for M > 8).
//   * Zero-point and scale: for G % 128 == 0 a chunk lies in one group, so the integer partial sum of
//     the chunk is scaled once in fp32 (more exact than scaling each weight).  The -8 is applied either
//     exactly per weight pair (bf16x2 subtract) or folded as -136 * sum(x) per chunk.  For smaller G
//     each lane scales its own words in bf16 (the rounding the reference's tensor-core path applies).
//   * K reduction: inside the mma across the four lanes of a quad, then across warps through shared
//     memory (one named barrier per row group), then -- only when K is split across CTAs to fill the
//     machine -- through fp32 partials in scratch memory, summed in fixed order by the last CTA to arrive
//     (an atomic counter per row group; nobody waits on anybody, the result is deterministic).
#include <algorithm>
#include <cstdio>

#include "ptx.cuh"
#include "tensor_map.h"
#include "w4_common.cuh"
#include "w4_internal.h"

namespace b2 {

namespace {

constexpr int kRowsPerGroup = 32;      // rows of W per stage / tile
constexpr int kChunkK = 128;           // K elements per consumer-warp work item
constexpr int kChunkBytes = 64;        // packed bytes of one row in one chunk
constexpr int kRedPitch = 36;          // floats per (warp, token) row of the reduction buffer: 32 + 4 pad
constexpr int kMaxStages = 8;
constexpr int kSmemLimit = 232448;     // 227 KB opt-in maximum per CTA on sm_100
constexpr int kHeaderBytes = 512;      // flags + barriers (first 256 B), a 256-byte block of zeros

struct GemvParams {
  const __nv_bfloat16* X;
  const uint32_t* Wq;
  const __nv_bfloat16* S;
  __nv_bfloat16* Y;
  int M, N, K, G;
  int KG;           // K / G
  int nchunks;      // ceil(K / 128)
  int nrg;          // ceil(N / 32)
  int nslices;      // CTAs sharing one row group along K
  int cps;          // chunks per slice
  int ntiles;       // nrg * nslices
  int nstages;
  int xs_m_stride;  // bytes between tokens of the staged X
  float* partial;   // [nslices][M][N]
  int* counters;    // [nrg]
  int* status;
  int dbg;  // diagnostics: bit 0 = take every scale as 1 (no scale loads), bit 1 = skip the math
};

template <int NCW>
struct Geo {
  static constexpr int kBoxBytes = kRowsPerGroup * 128;           // 32 rows x 128 B (two chunks), swizzled
  static constexpr int kStageBytes = (NCW / 2) * kBoxBytes;
  static constexpr int kThreads = (NCW + 1) * 32;
  static constexpr int kConsumerThreads = NCW * 32;
};

__host__ __device__ constexpr int red_bytes(int ncw, int mt) { return 2 * ncw * mt * 8 * kRedPitch * 4; }

__device__ __forceinline__ void consumer_sync(int nthreads) {
  asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
}

// Stages X[0..M) x [k-range of the slice] into shared memory, permuted so that the 16 bytes a lane
// needs for word j of its chunk are contiguous: for the 8 values x[b..b+8) the four registers are
// {x[b+p], x[b+p+4]}, p = 0..3 -- the pairing unpack_w4_biased produces.  Unit (j, t) of a chunk sits at
// byte (j*4 + t) * 16.  Also writes the per-(token, chunk) sums of x used by the folded zero-point.
template <int NCW>
__device__ __forceinline__ void stage_x(const GemvParams& p, uint32_t xs_base, float* xsum, int cb, int ce,
                                        int ctid) {
  const int nch = ce - cb;
  const int units = p.M * nch * 16;
  const int units_pad = (units + 31) & ~31;
  for (int u = ctid; u < units_pad; u += Geo<NCW>::kConsumerThreads) {
    float part = 0.f;
    if (u < units) {
      const int m = u / (nch * 16);
      const int r = u - m * nch * 16;
      const int ch = r >> 4, jt = r & 15;
      const int j = jt >> 2, t = jt & 3;
      const int k0 = (cb + ch) * kChunkK + 32 * t + 8 * j;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (k0 < p.K) v = __ldg(reinterpret_cast<const uint4*>(p.X + (size_t)m * p.K + k0));
      uint4 o;
      o.x = __byte_perm(v.x, v.z, 0x5410);  // {x0, x4}
      o.y = __byte_perm(v.x, v.z, 0x7632);  // {x1, x5}
      o.z = __byte_perm(v.y, v.w, 0x5410);  // {x2, x6}
      o.w = __byte_perm(v.y, v.w, 0x7632);  // {x3, x7}
      sts128(xs_base + m * p.xs_m_stride + ch * 256 + jt * 16, o);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        part += f.x + f.y;
      }
    }
    // 16 consecutive units (one half-warp) make up one (token, chunk)
    part += __shfl_xor_sync(0xffffffffu, part, 8);
    part += __shfl_xor_sync(0xffffffffu, part, 4);
    part += __shfl_xor_sync(0xffffffffu, part, 2);
    part += __shfl_xor_sync(0xffffffffu, part, 1);
    if (u < units && (u & 15) == 0) xsum[u >> 4] = part;  // index m * nch + ch
  }
}

// MT: token tiles of 8 (1 or 2).  NCW: consumer warps (= chunks per stage).  G128: G % 128 == 0.
// FOLD: zero-point folded into a per-chunk correction (only with G128).
template <int MT, int NCW, bool G128, bool FOLD>
__global__ void __launch_bounds__((NCW + 1) * 32, 1)
    w4_gemv_kernel(const __grid_constant__ CUtensorMap tmap_w, const GemvParams p) {
  using geo = Geo<NCW>;
  extern __shared__ __align__(1024) unsigned char smem[];
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem);
  int* last_flag = reinterpret_cast<int*>(smem + 8);
  const uint32_t bar_full = smem_u32(smem + 64);
  const uint32_t bar_empty = bar_full + 8 * kMaxStages;
  const uint32_t zero_base = smem_u32(smem + 256);
  float* red = reinterpret_cast<float*>(smem + kHeaderBytes);
  float* xsum = reinterpret_cast<float*>(smem + kHeaderBytes + red_bytes(NCW, MT));
  // xsum holds M * cps floats (<= 16 * 148 * 4 B is too much in general; the host caps cps so that
  // xsum + xs fit); it is placed before xs and sized M * cps * 4 rounded to 128.
  const int xsum_bytes = (p.M * p.cps * 4 + 127) & ~127;
  const uint32_t xs_base = smem_u32(smem + kHeaderBytes + red_bytes(NCW, MT) + xsum_bytes);
  const int xs_bytes = (p.M * p.xs_m_stride + 127) & ~127;
  const uint32_t ring_base = (xs_base + xs_bytes + 1023) & ~1023u;  // swizzled boxes: 1024-byte aligned

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    *abort_flag = 0;
    *last_flag = 0;
    for (int s = 0; s < p.nstages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, NCW);
    }
    fence_mbar_init();
  }
  __syncthreads();
  {
    if (warp == NCW) {
      // ------------------------------------------------------------ producer warp
      if (lane == 0) {
        tma_prefetch_desc(&tmap_w);
        int s = 0;
        uint32_t ph = 0;
        for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x) {
          const int sl = tile / p.nrg, rg = tile - sl * p.nrg;
          const int cb = sl * p.cps, ce = min(p.nchunks, cb + p.cps);
          const int row0 = rg * kRowsPerGroup;
          for (int c0 = cb; c0 < ce; c0 += NCW) {
            const int nbox = (min(NCW, ce - c0) + 1) >> 1;
            mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag);
            // out-of-range rows and K columns are zero-filled and still counted in the transaction bytes
            mbar_arrive_expect_tx(bar_full + 8 * s, (uint32_t)(nbox * geo::kBoxBytes));
            for (int b = 0; b < nbox; ++b)
              tma_load_2d(ring_base + s * geo::kStageBytes + b * geo::kBoxBytes, &tmap_w, (c0 + 2 * b) * 16, row0,
                          bar_full + 8 * s);
            if (++s == p.nstages) {
              s = 0;
              ph ^= 1;
            }
          }
        }
      }
      __syncwarp();
    } else {
      // ------------------------------------------------------------ consumer warps
      const int g = lane >> 2, t = lane & 3;
      // tile row fed to mma row g: neighbouring g get rows 4 apart, so that the eight lanes of one shared-
      // memory access phase land in opposite halves of the swizzled 128-byte rows (no bank conflicts)
      const int gr = (g >> 1) | ((g & 1) << 2);
      const int ctid = tid;  // consumer warps are warps 0..NCW-1
      // chunk `warp` of a stage sits in box warp/2, 64-byte half warp%2; 16-byte unit index XOR (row % 8 = gr)
      const uint32_t w_lane_off = (warp >> 1) * geo::kBoxBytes + gr * 128 +
                                  ((uint32_t(((warp & 1) << 2) | t) ^ uint32_t(gr)) << 4);
      const int gdiv = G128 ? p.G / kChunkK : 1;  // chunks per quantization group
      // the stage ring is walked with counters: no division in the loop
      int s = 0;
      uint32_t ph = 0;
      int staged_slice = -1, tcount = 0;
      for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x, ++tcount) {
        const int sl = tile / p.nrg, rg = tile - sl * p.nrg;
        const int cb = sl * p.cps, ce = min(p.nchunks, cb + p.cps);
        const int nch = ce - cb;
        const int row0 = rg * kRowsPerGroup;
        if (sl != staged_slice) {
          if (staged_slice >= 0) consumer_sync(geo::kConsumerThreads);  // all done with the old slice
          stage_x<NCW>(p, xs_base, xsum, cb, ce, ctid);
          if (ctid < 16) sts128(zero_base + ctid * 16, make_uint4(0u, 0u, 0u, 0u));
          consumer_sync(geo::kConsumerThreads);
          staged_slice = sl;
        }
        // B-fragment source of this lane: its token's staged X, or a block of zeros for padding tokens
        uint32_t xaddr[MT], xstep[MT];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const int m = mt * 8 + g;
          const bool real = m < p.M;
          xaddr[mt] = real ? xs_base + m * p.xs_m_stride + warp * 256 + t * 16 : zero_base + t * 16;
          xstep[mt] = real ? NCW * 256 : 0;
        }
        // G128: lane i fetches the scale of row row0 + i; the quad layout is rebuilt with shuffles
        const int n_lane = row0 + lane;
        const __nv_bfloat16* s_lane = p.S + (size_t)(n_lane < p.N ? n_lane : 0) * p.KG;
        const bool s_valid = n_lane < p.N && !(p.dbg & 1);

        float fin[2][MT][4];
#pragma unroll
        for (int rb = 0; rb < 2; ++rb)
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int i = 0; i < 4; ++i) fin[rb][mt][i] = 0.f;

        for (int c = cb + warp, c0 = cb; c0 < ce; c0 += NCW, c += NCW) {
          const bool active = c < ce;

          // scales first: their latency overlaps the wait for the stage
          float sc[2][2] = {{1.f, 1.f}, {1.f, 1.f}};
          uint32_t sc2[2][2] = {{0x3F803F80u, 0x3F803F80u}, {0x3F803F80u, 0x3F803F80u}};
          uint32_t srow = p.dbg & 1 ? 0x3F80u : 0u;
          if (active) {
            if constexpr (G128) {
              if (s_valid) srow = __bfloat16_as_ushort(__ldg(s_lane + (gdiv == 1 ? c : c / gdiv)));
            } else if (!(p.dbg & 1)) {
              const int k_lane = c * kChunkK + 32 * t;
              const int grp = k_lane < p.K ? k_lane / p.G : -1;
#pragma unroll
              for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                  const int n = row0 + rb * 16 + gr + 8 * hh;
                  __nv_bfloat16 sv = __float2bfloat16(0.f);
                  if (n < p.N && grp >= 0) sv = __ldg(p.S + (size_t)n * p.KG + grp);
                  sc2[rb][hh] = bf16_dup(sv);
                }
            }
          }

          if (lane == 0) mbar_wait(bar_full + 8 * s, ph, abort_flag);
          __syncwarp();

          if (active && !(p.dbg & 2)) {
            if constexpr (G128) {
#pragma unroll
              for (int rb = 0; rb < 2; ++rb)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh)
                  sc[rb][hh] = __uint_as_float(__shfl_sync(0xffffffffu, srow, rb * 16 + gr + 8 * hh) << 16);
            }
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
            const uint32_t wa = ring_base + s * geo::kStageBytes + w_lane_off;
#pragma unroll
            for (int rb = 0; rb < 2; ++rb) {
              const uint4 wl4 = lds128(wa + rb * 2048);
              const uint4 wh4 = lds128(wa + rb * 2048 + 1024);
              const uint32_t wl[4] = {wl4.x, wl4.y, wl4.z, wl4.w};
              const uint32_t wh[4] = {wh4.x, wh4.y, wh4.z, wh4.w};
              if constexpr (G128) {
                float acc[MT][2][4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  uint32_t rl[4], rh[4];
                  unpack_w4_biased(wl[j], rl);
                  unpack_w4_biased(wh[j], rh);
                  if constexpr (!FOLD) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                      rl[q] = sub136_bf16x2(rl[q]);
                      rh[q] = sub136_bf16x2(rh[q]);
                    }
                  }
#pragma unroll
                  for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                      if (j == 0)
                        mma_16816_bf16_zero(acc[mt][h], rl[2 * h], rh[2 * h], rl[2 * h + 1], rh[2 * h + 1],
                                            xf[mt][4 * j + 2 * h], xf[mt][4 * j + 2 * h + 1]);
                      else
                        mma_16816_bf16(acc[mt][h], rl[2 * h], rh[2 * h], rl[2 * h + 1], rh[2 * h + 1],
                                       xf[mt][4 * j + 2 * h], xf[mt][4 * j + 2 * h + 1]);
                    }
                }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                  float v0 = acc[mt][0][0] + acc[mt][1][0], v1 = acc[mt][0][1] + acc[mt][1][1];
                  float v2 = acc[mt][0][2] + acc[mt][1][2], v3 = acc[mt][0][3] + acc[mt][1][3];
                  if constexpr (FOLD) {
                    // columns 2t, 2t+1 of this tile are tokens mt*8 + 2t (+1)
                    const int m0 = mt * 8 + 2 * t;
                    const float xs0 = m0 < p.M ? xsum[m0 * nch + (c - cb)] : 0.f;
                    const float xs1 = m0 + 1 < p.M ? xsum[(m0 + 1) * nch + (c - cb)] : 0.f;
                    v0 = fmaf(-136.f, xs0, v0);
                    v1 = fmaf(-136.f, xs1, v1);
                    v2 = fmaf(-136.f, xs0, v2);
                    v3 = fmaf(-136.f, xs1, v3);
                  }
                  fin[rb][mt][0] = fmaf(sc[rb][0], v0, fin[rb][mt][0]);
                  fin[rb][mt][1] = fmaf(sc[rb][0], v1, fin[rb][mt][1]);
                  fin[rb][mt][2] = fmaf(sc[rb][1], v2, fin[rb][mt][2]);
                  fin[rb][mt][3] = fmaf(sc[rb][1], v3, fin[rb][mt][3]);
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
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_empty + 8 * s);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) xaddr[mt] += xstep[mt];
          if (++s == p.nstages) {
            s = 0;
            ph ^= 1;
          }
        }

        if (p.dbg & 4) continue;  // diagnostics: no reduction, no output
        // ---- K reduction across the consumer warps of this CTA
        float* rbuf = red + (tcount & 1) * (NCW * MT * 8 * kRedPitch);
#pragma unroll
        for (int rb = 0; rb < 2; ++rb)
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            float* r0 = rbuf + (warp * MT * 8 + mt * 8 + 2 * t) * kRedPitch + rb * 16 + gr;
            r0[0] = fin[rb][mt][0];
            r0[kRedPitch] = fin[rb][mt][1];
            r0[8] = fin[rb][mt][2];
            r0[kRedPitch + 8] = fin[rb][mt][3];
          }
        consumer_sync(geo::kConsumerThreads);
        const int nout = p.M * kRowsPerGroup;  // tokens beyond M are padding
        for (int o = ctid; o < nout; o += geo::kConsumerThreads) {
          const int tok = o >> 5, row = o & 31;
          float sum = 0.f;
#pragma unroll
          for (int w = 0; w < NCW; ++w) sum += rbuf[(w * MT * 8 + tok) * kRedPitch + row];
          const int n = row0 + row;
          if (n < p.N) {
            if (p.nslices == 1)
              p.Y[(size_t)tok * p.N + n] = __float2bfloat16(sum);
            else
              __stcg(p.partial + ((size_t)sl * p.M + tok) * p.N + n, sum);
          }
        }
        if (p.nslices > 1) {
          // ---- K reduction across CTAs: the last slice to arrive sums all partials in slice order
          __threadfence();
          consumer_sync(geo::kConsumerThreads);
          if (ctid == 0) {
            const int old = atomicAdd(p.counters + rg, 1);
            const int last = old == p.nslices - 1;
            if (last) p.counters[rg] = 0;  // ready for the next launch
            *last_flag = last;
          }
          consumer_sync(geo::kConsumerThreads);
          if (*last_flag) {
            __threadfence();
            for (int o = ctid; o < nout; o += geo::kConsumerThreads) {
              const int tok = o >> 5, row = o & 31;
              const int n = row0 + row;
              if (n < p.N) {
                float sum = 0.f;
                for (int q = 0; q < p.nslices; ++q) sum += __ldcg(p.partial + ((size_t)q * p.M + tok) * p.N + n);
                p.Y[(size_t)tok * p.N + n] = __float2bfloat16(sum);
              }
            }
          }
          consumer_sync(geo::kConsumerThreads);  // last_flag may be rewritten by the next tile
        }
      }
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
  int mt, ncw, nslices, cps, nstages, grid;
  bool g128, fold;
  size_t smem;
  int xs_m_stride;
};

size_t smem_without_ring(int M, int mt, int ncw, int cps) {
  const int xs_m_stride = cps * 256 + 64;
  const size_t xsum_bytes = ((size_t)M * cps * 4 + 127) & ~(size_t)127;
  const size_t xs_bytes = ((size_t)M * xs_m_stride + 127) & ~(size_t)127;
  return kHeaderBytes + red_bytes(ncw, mt) + xsum_bytes + xs_bytes + 1024;
}

bool make_plan(int M, int N, int K, int G, int flags, int sm_count, size_t partial_cap, int counters_cap,
               GemvPlan* out) {
  GemvPlan pl{};
  pl.mt = M > 8 ? 2 : 1;
  pl.ncw = (pl.mt == 1 && !(flags & kFlagNarrowCta)) ? 16 : 8;
  pl.g128 = (G % 128) == 0;
  pl.fold = pl.g128 && (flags & kFlagFoldZeroPoint);
  const int nchunks = (K + kChunkK - 1) / kChunkK;
  const int nrg = (N + kRowsPerGroup - 1) / kRowsPerGroup;
  const int stage_bytes = (pl.ncw / 2) * kRowsPerGroup * 128;
  pl.grid = std::max(1, sm_count);

  // Cost model in units of "one chunk of one row group" (2 KB of weights): a tile costs its chunk
  // count rounded up to whole stages, plus a fixed reduction overhead; split-K tiles pay the scratch
  // round trip as well.  Pick the slice count with the smallest makespan over the persistent CTAs.
  double best = 1e30;
  int best_ns = 0, best_cps = 0;
  const int max_ns = (flags & kFlagForceNoSplitK) ? 1 : std::min(nchunks, 64);
  for (int ns = 1; ns <= max_ns; ++ns) {
    const int cps = (nchunks + ns - 1) / ns;
    const int real_ns = (nchunks + cps - 1) / cps;
    if (real_ns != ns) continue;
    if (smem_without_ring(M, pl.mt, pl.ncw, cps) + 3 * (size_t)stage_bytes > (size_t)kSmemLimit) continue;
    if (ns > 1) {
      if ((size_t)ns * M * N * sizeof(float) > partial_cap) continue;
      if (nrg > counters_cap) continue;
    }
    const long tiles = (long)nrg * ns;
    const long per_cta = (tiles + pl.grid - 1) / pl.grid;
    const int stage_chunks = ((cps + pl.ncw - 1) / pl.ncw) * pl.ncw;
    // a stage with idle warps still moves only its real bytes; weigh real and padded equally
    const double tile_cost = 0.5 * (cps + stage_chunks) + 4.0 + (ns > 1 ? 12.0 : 0.0);
    const double cost = per_cta * tile_cost;
    if (cost < best) {
      best = cost;
      best_ns = ns;
      best_cps = cps;
    }
  }
  if (best_ns == 0) {
    // the staged X of the wide CTA does not fit: the narrow one leaves more shared memory for it
    if (pl.ncw == 16) return make_plan(M, N, K, G, flags | kFlagNarrowCta, sm_count, partial_cap, counters_cap, out);
    return false;
  }
  pl.nslices = best_ns;
  pl.cps = best_cps;
  pl.xs_m_stride = pl.cps * 256 + 64;
  const size_t fixed = smem_without_ring(M, pl.mt, pl.ncw, pl.cps);
  int stages = (int)(((size_t)kSmemLimit - fixed) / stage_bytes);
  stages = std::min(stages, pl.ncw == 16 ? 5 : kMaxStages);
  if (stages < 2) return false;
  pl.nstages = stages;
  pl.smem = fixed + (size_t)stages * stage_bytes;
  pl.grid = (int)std::min<long>(pl.grid, (long)nrg * pl.nslices);
  *out = pl;
  return true;
}

template <int MT, int NCW, bool G128, bool FOLD>
int launch_variant(const CUtensorMap& tmap, const GemvParams& p, const GemvPlan& pl, cudaStream_t stream) {
  auto kernel = w4_gemv_kernel<MT, NCW, G128, FOLD>;
  // Raising the dynamic shared-memory limit is idempotent and cheap; doing it on every launch keeps
  // the call correct on every device of a multi-GPU process without per-device bookkeeping.
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem);
  if (e != cudaSuccess) return (int)e;
  kernel<<<pl.grid, Geo<NCW>::kThreads, pl.smem, stream>>>(tmap, p);
  return (int)cudaGetLastError();
}

}  // namespace

size_t gemv_scratch_bytes(int M, int N, int K, int G, int flags, int sm_count, size_t partial_cap) {
  GemvPlan pl;
  if (!make_plan(M, N, K, G, flags, sm_count, partial_cap, 1 << 30, &pl)) return 0;
  return pl.nslices > 1 ? (size_t)pl.nslices * M * N * sizeof(float) : 0;
}

int gemv_launch(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int G,
                const Workspace& ws, int flags, int sm_count, cudaStream_t stream) {
  if (M < 1 || M > 16) return kErrUnsupportedM;
  if (N < 1 || K < 32 || G < 32 || K % 32 || G % 32 || K % G) return kErrBadShape;
  if (!X || !Wq || !S || !Y) return kErrBadPointer;
  if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(Wq) & 15) ||
      (reinterpret_cast<uintptr_t>(S) & 1) || (reinterpret_cast<uintptr_t>(Y) & 1))
    return kErrBadPointer;
  if (!ws.status) return kErrWorkspace;
  const bool have_scratch = ws.partial && ws.counters;
  GemvPlan pl;
  if (!make_plan(M, N, K, G, have_scratch ? flags : (flags | kFlagForceNoSplitK), sm_count,
                 ws.partial_bytes, ws.n_counters, &pl))
    return kErrTooLarge;

  // Wq as a 2-D tensor of 32-bit words [N rows, K/8 columns]; boxes of 32 words (two chunks) x 32 rows
  CUtensorMap tmap;
  if (!make_tensor_map_2d(&tmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, Wq, (uint64_t)N, (uint64_t)K / 8, kRowsPerGroup,
                          32, CU_TENSOR_MAP_SWIZZLE_128B))
    return kErrDevice;

  GemvParams p{};
  p.X = static_cast<const __nv_bfloat16*>(X);
  p.Wq = static_cast<const uint32_t*>(Wq);
  p.S = static_cast<const __nv_bfloat16*>(S);
  p.Y = static_cast<__nv_bfloat16*>(Y);
  p.M = M; p.N = N; p.K = K; p.G = G;
  p.KG = K / G;
  p.nchunks = (K + kChunkK - 1) / kChunkK;
  p.nrg = (N + kRowsPerGroup - 1) / kRowsPerGroup;
  p.nslices = pl.nslices;
  p.cps = pl.cps;
  p.ntiles = p.nrg * p.nslices;
  p.nstages = pl.nstages;
  p.xs_m_stride = pl.xs_m_stride;
  p.partial = ws.partial;
  p.counters = ws.counters;
  p.status = ws.status;
  p.dbg = (flags >> 8) & 15;

  if (pl.mt == 1) {
    if (pl.ncw == 16) {
      if (!pl.g128) return launch_variant<1, 16, false, false>(tmap, p, pl, stream);
      return pl.fold ? launch_variant<1, 16, true, true>(tmap, p, pl, stream)
                     : launch_variant<1, 16, true, false>(tmap, p, pl, stream);
    }
    if (!pl.g128) return launch_variant<1, 8, false, false>(tmap, p, pl, stream);
    return pl.fold ? launch_variant<1, 8, true, true>(tmap, p, pl, stream)
                   : launch_variant<1, 8, true, false>(tmap, p, pl, stream);
  }
  if (!pl.g128) return launch_variant<2, 8, false, false>(tmap, p, pl, stream);
  return pl.fold ? launch_variant<2, 8, true, true>(tmap, p, pl, stream)
                 : launch_variant<2, 8, true, false>(tmap, p, pl, stream);
}

}  // namespace b2
