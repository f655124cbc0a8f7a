// W4A16 prefill GEMM for sm_100a:  Y[M,N] (bf16) = X[M,K] (bf16) . dequant(Wq, S)^T  for M > 16.
//
// Replaces the reference's w4a16_gemm_kernel / w4a16_gemm_cfg (kernels/quant/w4a16.cuh:124-270): cp.async
// staging, a dequant pass into shared memory and mma.sync.m16n8k16 with 128x128x32 tiles, M and N
// multiples of 128 only.  Same numerics: each weight is dequantised to RN_bf16((q - 8) * s)
// (w4a16.cuh:196-197), the contraction accumulates in fp32, one rounding to bf16 at the store.
//
// Design (tensor-bound; one CTA per SM, one work item per CTA):
//   work     the output tiles in row-major order with the token tile fastest.  As many whole waves of tiles as
//            there are (tile count rounded down to a multiple of the SM count) are one item each; the tiles of the
//            last, partial wave may be split along K into several items each, which run as SMs come free, so the
//            tail of a launch is a fraction of a tile's time instead of a whole one (3584 x 18944 at M = 8192 has
//            448 tiles on 148 SMs: 3.03 waves).  The last item of a split tile to arrive adds the fp32 part-tiles
//            in split order (deterministic, nobody waits for anybody).
//   tile     MI x 128 tokens by 256 output features, K walked in blocks of 64
//   warp 0   TMA producer: per K block, the X tile(s) (128 rows x 128 B, 128-byte swizzle) and the packed
//            weight tile (256 rows x 32 B) land in a ring stage; completion counted on an mbarrier
//   warp 1   MMA issuer: one elected lane issues tcgen05.mma (cta_group::1, kind::f16, M=128, N=256, K=16)
//            from shared-memory descriptors into fp32 accumulators in TMEM (MI x 256 columns); the weight
//            operand is shared by the MI token tiles, so every weight is dequantised once per 128*MI tokens
//   warps 2-17 dequant: two threads per weight row of the tile, each owning a 32-wide half of the K block:
//            one 16-byte shared load of packed nibbles, LOP3 unpack to bf16 pairs, exact -8 (bf16x2
//            subtract), one bf16x2 multiply by the group scale, and four 16-byte stores into a K-major,
//            128-byte-swizzled bf16 tile (three buffers in rotation) that the MMA reads through the async
//            proxy (fence.proxy.async before the arrive)
//   epilogue the same sixteen warps read the accumulators with tcgen05.ld (32 lanes x 32 columns), convert to
//            bf16 and store rows of Y
// Ragged M, N and a K tail of 32 need no special path: TMA zero-fills out-of-range rows and columns, the
// scale of an out-of-range row or group is taken as 0, and the epilogue masks its stores.
// Every mbarrier wait is bounded; on a time-out the CTA records a status, still frees its TMEM and returns.
#include <cuda.h>

#include <algorithm>
#include <cstdio>
#include <mutex>

#include "ptx.cuh"
#include "tensor_map.h"
#include "w4_common.cuh"
#include "w4_internal.h"

namespace b2 {
namespace {

constexpr int kBN = 256;            // output features per tile (UMMA N)
constexpr int kBK = 64;             // K per block: one 128-byte swizzled row of bf16
constexpr int kATileBytes = 128 * 128;        // 128 tokens x 64 bf16
constexpr int kWpTileBytes = kBN * 32;        // 256 rows x 8 packed words
constexpr int kBdTileBytes = kBN * 128;       // 256 rows x 64 bf16
constexpr int kBdBuffers = 3;                 // dequantised tiles in rotation
constexpr int kDequantThreads = 512;        // two threads per weight row of the tile
constexpr int kGemmThreads = 32 * 2 + kDequantThreads;
constexpr int kGemmSmemLimit = 232448;

struct GemmParams {
  const __nv_bfloat16* S;
  __nv_bfloat16* Y;
  int M, N, K, G, KG;
  int nkb;  // K blocks of 64
  int tiles_x;      // token tiles (fastest in the tile order)
  int n_whole;      // the first n_whole tiles are one work item each
  int n_tail;       // the remaining tiles are tail_ks items each: item n_whole + z * n_tail + t = split z of tile t
  int tail_ks;
  float* partial;   // [tail_ks][n_tail][MI*256 columns][128 rows] fp32, split tiles only
  int* counters;    // one arrival counter per output tile, zero between launches
  int* status;
};

template <int MI>
struct GemmGeo {
  static constexpr int kStageBytes = MI * kATileBytes + kWpTileBytes;
  static constexpr int kStages = MI == 2 ? 3 : 5;
  static constexpr int kRingBytes = kStages * kStageBytes;
  static constexpr int kBdOffset = kRingBytes;
  static constexpr int kBarOffset = kBdOffset + kBdBuffers * kBdTileBytes;
  static constexpr int kSmemBytes = kBarOffset + 256 + 1024;  // barriers + slack for 1024-byte alignment
  static constexpr int kTmemCols = MI * kBN;                  // 256 or 512: powers of two
};

template <int MI>
__global__ void __launch_bounds__(kGemmThreads, 1)
    w4_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                   const GemmParams p) {
  using geo = GemmGeo<MI>;
  extern __shared__ unsigned char smem_raw[];
  // 128-byte-swizzled tiles need a 1024-byte aligned base
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* gen_base = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar_base = base + geo::kBarOffset;
  const uint32_t bar_full = bar_base;                        // [kStages]
  const uint32_t bar_empty = bar_base + 8 * 8;               // [kStages]
  const uint32_t bar_bd_full = bar_base + 16 * 8;            // [kBdBuffers]
  const uint32_t bar_bd_empty = bar_base + 20 * 8;           // [kBdBuffers]
  const uint32_t bar_acc = bar_base + 24 * 8;                // [1]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + geo::kBarOffset + 26 * 8);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + geo::kBarOffset + 27 * 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // token tiles vary fastest over the CTAs that run together: they then read many different X tiles and few
  // weight tiles at a time, which spreads the L2 traffic (74 CTAs pulling the same X tile at once made a few L2
  // slices the bottleneck)
  // (the hardware starts CTAs in index order, so the split tiles of the tail run last)
  const int item = blockIdx.x;
  const bool split = item >= p.n_whole;
  const int tail_t = split ? (item - p.n_whole) % p.n_tail : 0;   // tile of the tail
  const int tail_z = split ? (item - p.n_whole) / p.n_tail : 0;   // which K range of it
  const int tile = split ? p.n_whole + tail_t : item;
  const int ksplit = split ? p.tail_ks : 1;
  const int m0 = (tile % p.tiles_x) * (128 * MI);
  const int n0 = (tile / p.tiles_x) * kBN;
  // this CTA's share of the K blocks
  const int kb_per = (p.nkb + ksplit - 1) / ksplit;
  const int kb0 = tail_z * kb_per;
  const int nkb = max(0, min(p.nkb, kb0 + kb_per) - kb0);

  if (tid == 0) {
    *abort_flag = 0;
    for (int s = 0; s < geo::kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, kDequantThreads + 1);
    }
    for (int b = 0; b < kBdBuffers; ++b) {
      mbar_init(bar_bd_full + 8 * b, kDequantThreads);
      mbar_init(bar_bd_empty + 8 * b, 1);
    }
    mbar_init(bar_acc, 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_w);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), geo::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const bool poisoned = *reinterpret_cast<volatile int*>(p.status) != 0;

  if (!poisoned) {
    if (warp == 0) {
      // ------------------------------------------------------------ TMA producer
      if (lane == 0) {
        int s = 0;
        uint32_t ph = 0;
        for (int i = 0; i < nkb; ++i) {
          const int kb = kb0 + i;
          mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag);
          const uint32_t stage = base + s * geo::kStageBytes;
          mbar_arrive_expect_tx(bar_full + 8 * s, geo::kStageBytes);
#pragma unroll
          for (int mi = 0; mi < MI; ++mi)
            tma_load_2d(stage + mi * kATileBytes, &tmap_x, kb * kBK, m0 + mi * 128, bar_full + 8 * s);
          tma_load_2d(stage + MI * kATileBytes, &tmap_w, kb * (kBK / 8), n0, bar_full + 8 * s);
          if (++s == geo::kStages) { s = 0; ph ^= 1; }
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      // ------------------------------------------------------------ MMA issuer
      if (lane == 0) {
        constexpr uint32_t idesc = umma_idesc_bf16(128, kBN);
        int s = 0, b = 0;
        uint32_t ph = 0, bph = 0;
        for (int kb = 0; kb < nkb; ++kb) {
          mbar_wait(bar_full + 8 * s, ph, abort_flag);
          mbar_wait(bar_bd_full + 8 * b, bph, abort_flag);
          tc_fence_after_sync();
          const uint32_t a_addr = base + s * geo::kStageBytes;
          const uint32_t b_addr = base + geo::kBdOffset + b * kBdTileBytes;
#pragma unroll
          for (int kk = 0; kk < kBK / 16; ++kk) {
            const uint64_t db = umma_desc_k128(b_addr + kk * 32);
#pragma unroll
            for (int mi = 0; mi < MI; ++mi) {
              const uint64_t da = umma_desc_k128(a_addr + mi * kATileBytes + kk * 32);
              umma_f16_ss(tmem_base + mi * kBN, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            }
          }
          umma_commit(bar_empty + 8 * s);      // the X tile and the packed tile of this stage are consumed
          umma_commit(bar_bd_empty + 8 * b);   // the dequantised tile may be overwritten
          if (++s == geo::kStages) { s = 0; ph ^= 1; }
          if (++b == kBdBuffers) { b = 0; bph ^= 1; }
        }
        umma_commit(bar_acc);
      }
      __syncwarp();
    } else {
      // ------------------------------------------------------------ dequant warps, then epilogue
      const int dt = tid - 64;          // 0..511
      const int r = dt >> 1;            // weight row of the tile
      const int hf = dt & 1;            // which 32-wide half of the 64-wide K block (one scale each)
      const int n = n0 + r;
      const uint32_t bd_row = base + geo::kBdOffset + r * 128;
      const uint32_t sw = (uint32_t)(r & 7);
      // unpack constants pinned in registers: each (x & mask) | magic is then a single LOP3
      uint32_t k_mask = kNibblePairMask, k_magic = kMagic128x2;
      asm volatile("" : "+r"(k_mask), "+r"(k_magic));
      const __nv_bfloat16* s_row = p.S + (size_t)(n < p.N ? n : 0) * p.KG;
      int s = 0, b = 0;
      uint32_t ph = 0, bph = 0;
      // the scale of K block kb + 1 is fetched while block kb is unpacked: the L2 round trip stays off the
      // critical path of the hand-off to the MMA
      auto load_scale = [&](int kb) {
        const int k0 = kb * kBK + hf * 32;
        __nv_bfloat16 sv = __float2bfloat16(0.f);
        if (n < p.N && k0 < p.K) sv = __ldg(s_row + k0 / p.G);
        return bf16_dup(sv);
      };
      uint32_t s2_next = load_scale(kb0);
      for (int i = 0; i < nkb; ++i) {
        const uint32_t s2 = s2_next;
        if (i + 1 < nkb) s2_next = load_scale(kb0 + i + 1);

        // one lane per warp polls: many threads spinning on a shared-memory barrier slow the copies down
        if (lane == 0) mbar_wait(bar_full + 8 * s, ph, abort_flag);
        __syncwarp();
        const uint4 w4 = lds128(base + s * geo::kStageBytes + MI * kATileBytes + r * 32 + hf * 16);
        mbar_arrive(bar_empty + 8 * s);  // packed words are in registers
        const uint32_t words[4] = {w4.x, w4.y, w4.z, w4.w};

        if (lane == 0) mbar_wait(bar_bd_empty + 8 * b, bph ^ 1, abort_flag);
        __syncwarp();
        const uint32_t dst = bd_row + b * kBdTileBytes;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[4];
          v[0] = lop3_and_or(words[c], k_mask, k_magic);
          v[1] = lop3_and_or(words[c] >> 4, k_mask, k_magic);
          v[2] = lop3_and_or(words[c] >> 8, k_mask, k_magic);
          v[3] = lop3_and_or(words[c] >> 12, k_mask, k_magic);
#pragma unroll
          for (int q = 0; q < 4; ++q) v[q] = mul_bf16x2(sub136_bf16x2(v[q]), s2);
          // v[q] = {w[q], w[q+4]}  ->  natural order pairs {w0,w1} {w2,w3} {w4,w5} {w6,w7}
          uint4 o;
          o.x = __byte_perm(v[0], v[1], 0x5410);
          o.y = __byte_perm(v[2], v[3], 0x5410);
          o.z = __byte_perm(v[0], v[1], 0x7632);
          o.w = __byte_perm(v[2], v[3], 0x7632);
          sts128(dst + ((uint32_t(hf * 4 + c) ^ sw) << 4), o);
        }
        fence_proxy_async_smem();
        mbar_arrive(bar_bd_full + 8 * b);
        if (++s == geo::kStages) { s = 0; ph ^= 1; }
        if (++b == kBdBuffers) { b = 0; bph ^= 1; }
      }

      // ---- epilogue: TMEM -> registers -> bf16 -> global
      if (lane == 0) mbar_wait(bar_acc, 0, abort_flag);
      __syncwarp();
      tc_fence_after_sync();
      const int ew = warp - 2;           // 0..15
      const int quad = warp & 3;         // TMEM lane quadrant this warp may read
      const int grp = ew >> 2;           // 0..3: four warps share a quadrant and split the columns
      const int mi = MI == 2 ? grp >> 1 : 0;
      const int col_begin = MI == 2 ? (grp & 1) * (kBN / 2) : grp * (kBN / 4);
      const int col_end = col_begin + (MI == 2 ? kBN / 2 : kBN / 4);
      const int m = m0 + mi * 128 + quad * 32 + lane;
      const bool vec_ok = (p.N % 8) == 0;
      const bool parts = ksplit > 1;
      const int ntiles = p.n_tail, tile_id = tail_t;
      for (int c0 = col_begin; c0 < col_end; c0 += 32) {
        uint32_t v[32];
        if (nkb > 0) {
          tmem_ld_32x32(tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(mi * kBN + c0), v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = 0u;  // a split with no K blocks contributes zeros
        }
        if (parts) {
          // fp32 partial of this (split, tile), stored column-major inside the tile (row fastest): for a given
          // column the 32 lanes of a warp write 32 consecutive floats
          float* pt = p.partial + ((size_t)tail_z * ntiles + tile_id) * (size_t)(MI * 128 * kBN) +
                      (size_t)(mi * kBN + c0) * 128 + quad * 32 + lane;
#pragma unroll
          for (int e = 0; e < 32; ++e) __stcg(pt + e * 128, __uint_as_float(v[e]));
          continue;
        }
        if (m < p.M) {
          __nv_bfloat16* yrow = p.Y + (size_t)m * p.N + n0 + c0;
          if (vec_ok && n0 + c0 + 32 <= p.N) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 o;
              uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[8 * q + 2 * e]),
                                                               __uint_as_float(v[8 * q + 2 * e + 1]));
                ow[e] = *reinterpret_cast<const uint32_t*>(&h);
              }
              *reinterpret_cast<uint4*>(yrow + 8 * q) = o;
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (n0 + c0 + e < p.N) yrow[e] = __float2bfloat16(__uint_as_float(v[e]));
          }
        }
      }
      if (parts) {
        // the last of the ksplit CTAs of this tile to arrive sums the partials in split order (deterministic;
        // nobody waits for anybody) and stores bf16
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"r"(kDequantThreads) : "memory");
        int* flag = reinterpret_cast<int*>(gen_base + geo::kBarOffset + 28 * 8);
        if (tid == 64) {
          int* ctr = p.counters + tile_id;
          const int old = atomicAdd(ctr, 1);
          const int last = old == ksplit - 1;
          if (last) *ctr = 0;
          *flag = last;
        }
        asm volatile("bar.sync 1, %0;" ::"r"(kDequantThreads) : "memory");
        if (*flag) {
          __threadfence();
          for (int c0 = col_begin; c0 < col_end; c0 += 32) {
            float sum[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) sum[e] = 0.f;
            for (int z = 0; z < ksplit; ++z) {
              const float* pt = p.partial + ((size_t)z * ntiles + tile_id) * (size_t)(MI * 128 * kBN) +
                                (size_t)(mi * kBN + c0) * 128 + quad * 32 + lane;
#pragma unroll
              for (int e = 0; e < 32; ++e) sum[e] += __ldcg(pt + e * 128);
            }
            if (m < p.M) {
              __nv_bfloat16* yrow = p.Y + (size_t)m * p.N + n0 + c0;
              if (vec_ok && n0 + c0 + 32 <= p.N) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  uint4 o;
                  uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const __nv_bfloat162 h = __floats2bfloat162_rn(sum[8 * q + 2 * e], sum[8 * q + 2 * e + 1]);
                    ow[e] = *reinterpret_cast<const uint32_t*>(&h);
                  }
                  *reinterpret_cast<uint4*>(yrow + 8 * q) = o;
                }
              } else {
#pragma unroll
                for (int e = 0; e < 32; ++e)
                  if (n0 + c0 + e < p.N) yrow[e] = __float2bfloat16(sum[e]);
              }
            }
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (tid == 0) atomicCAS(p.status, kStatusOk, kStatusGemmTimeout);
    for (int i = 0; i < 64; ++i) __nanosleep(2000);  // let copies in flight land before the smem is released
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, geo::kTmemCols);
  }
}

// ------------------------------------------------------------------ host side
template <int MI>
int launch_gemm(const CUtensorMap& tx, const CUtensorMap& tw, const GemmParams& p, cudaStream_t stream) {
  auto kernel = w4_gemm_kernel<MI>;
  cudaError_t e =
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmGeo<MI>::kSmemBytes);
  if (e != cudaSuccess) return (int)e;
  const dim3 grid(p.n_whole + p.n_tail * p.tail_ks);
  kernel<<<grid, kGemmThreads, GemmGeo<MI>::kSmemBytes, stream>>>(tx, tw, p);
  return (int)cudaGetLastError();
}

}  // namespace

int gemm_launch(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int G,
                const Workspace& ws, int flags, int sm_count, cudaStream_t stream) {
  static_assert(GemmGeo<2>::kSmemBytes <= kGemmSmemLimit && GemmGeo<1>::kSmemBytes <= kGemmSmemLimit, "smem");
  if (M < 1) return kErrUnsupportedM;
  if (N < 1 || K < 32 || G < 32 || K % 32 || G % 32 || K % G) return kErrBadShape;
  if (!X || !Wq || !S || !Y) return kErrBadPointer;
  if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(Wq) & 15) ||
      (reinterpret_cast<uintptr_t>(S) & 1) || (reinterpret_cast<uintptr_t>(Y) & 15))
    return kErrBadPointer;
  if (!ws.status) return kErrWorkspace;

  CUtensorMap tx, tw;
  if (!make_tensor_map_2d(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, X, (uint64_t)M, (uint64_t)K, 128, kBK,
                 CU_TENSOR_MAP_SWIZZLE_128B))
    return kErrDevice;
  if (!make_tensor_map_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, Wq, (uint64_t)N, (uint64_t)K / 8, kBN, kBK / 8,
                 CU_TENSOR_MAP_SWIZZLE_NONE))
    return kErrDevice;

  GemmParams p{};
  p.S = static_cast<const __nv_bfloat16*>(S);
  p.Y = static_cast<__nv_bfloat16*>(Y);
  p.M = M; p.N = N; p.K = K; p.G = G;
  p.KG = K / G;
  p.nkb = (K + kBK - 1) / kBK;
  p.status = ws.status;
  // Whole waves of tiles run one tile per CTA.  The tiles of the last, partial wave are split along K when that
  // shortens it: pick the split whose makespan in K blocks is smallest, charging a split its fp32 round trip
  // (e.g. the 3584 x 18944 projection: 28 tiles at M = 512 run as 5 splits each; at M = 8192 the 4 tiles that
  // 3 waves of 148 leave over run as 8 splits each instead of a fourth wave).
  {
    const int mi = M <= 128 ? 1 : 2;
    p.tiles_x = (M + 128 * mi - 1) / (128 * mi);
    const long tiles = (long)p.tiles_x * ((N + kBN - 1) / kBN);
    if (tiles > 0x3fffffff) return kErrBadShape;
    const int sms = std::max(1, sm_count);
    const long n_tail = tiles % sms ? tiles % sms : std::min<long>(tiles, sms);
    long best_cost = -1;
    int best = 1;
    for (int ks = 1; ks <= 8; ++ks) {
      if (ks > 1 && ((flags & kFlagGemmWholeTiles) || !ws.partial || !ws.counters ||
                     (size_t)ks * n_tail * (size_t)(mi * 128 * kBN) * sizeof(float) > ws.partial_bytes ||
                     n_tail > ws.n_counters || p.nkb / ks < 8))
        break;
      const long waves = (n_tail * ks + sms - 1) / sms;
      const long cost = waves * ((p.nkb + ks - 1) / ks + (ks > 1 ? 6 + 2 * ks : 4));
      // a split must win by a margin: its fp32 partials cost memory traffic the model only roughly accounts for
      // (measured: 3584 x 18944 at M = 512 goes from 267 to 747 TFLOP/s with 5 splits)
      if (best_cost < 0 || cost * 100 < best_cost * (best == 1 ? 95 : 100)) {
        best_cost = cost;
        best = ks;
      }
    }
    p.n_tail = (int)n_tail;
    p.n_whole = (int)(tiles - n_tail);
    p.tail_ks = best;
    p.partial = ws.partial;
    p.counters = ws.counters;
  }
  return M <= 128 ? launch_gemm<1>(tx, tw, p, stream) : launch_gemm<2>(tx, tw, p, stream);
}

}  // namespace b2
