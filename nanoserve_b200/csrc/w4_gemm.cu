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
//   warp 1   MMA issuer: one elected lane issues tcgen05.mma (kind::f16, N=256, K=16) from shared-memory
//            descriptors into fp32 accumulators in TMEM (MI x 256 columns); the weight operand is shared by the MI
//            token tiles.  One CTA per tile: cta_group::1, M=128.  CTA pairs (the default where token tiles pair
//            up; see the block comment further down): cta_group::2, M=256 across the two CTAs, issued by the
//            rank-0 CTA, each CTA holding and unpacking half of the weight tile
//   warps 2-17 dequant: two threads per weight row of the tile, each owning a 32-wide half of the K block (pairs:
//            four threads per row of the CTA's 128 rows, a 16-wide quarter each):
//            one 16-byte (8-byte) shared load of packed nibbles, LOP3 unpack to bf16 pairs, exact -8 (bf16x2
//            subtract), one bf16x2 multiply by the group scale, and four 16-byte stores into a K-major,
//            128-byte-swizzled bf16 tile (three buffers in rotation, four for pairs) that the MMA reads through the async
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
  int tiles_x;      // token tiles (fastest in the tile order; padded to an even number for CTA pairs)
  int n_whole;      // the first n_whole tiles are one work item each
  int n_tail;       // the remaining tiles are tail_ks items each: item n_whole + z * n_tail + t = split z of tile t
  int tail_ks;
  float* partial;   // [tail_ks][n_tail][MI*256 columns][128 rows] fp32, split tiles only
  int* counters;    // one arrival counter per output tile, zero between launches
  int* status;
};

// ---- CTA pairs (clusters of two) on one tcgen05.mma.cta_group::2: the two CTAs work on neighbouring token tiles of
// the same weight tile.  Each loads and unpacks HALF of the weight tile (128 rows) into its own shared memory; the
// MMA, issued by the CTA of rank 0 for both, has M = 256 (128 token rows from each CTA's X tile, accumulators in each
// CTA's own TMEM) and reads the two halves of the N = 256 weight operand from the two CTAs.  Per CTA and K block the
// shared memory then serves 32 KB of weight-operand reads instead of 64, takes 16 KB of dequantised stores instead
// of 32, and every weight is unpacked once per 2 * 128 * MI tokens.  (Measured on the way: with one CTA per tile the
// operand reads of the MMAs alone take three quarters of the shared-memory bandwidth; a pair that only SHARED the
// unpacking -- each CTA copying its half into the peer's tile -- was slower than single CTAs, 0.57 against 0.68 of the
// dense peak, since it adds shared-memory traffic instead of removing it.)
__device__ __forceinline__ uint32_t cluster_ctarank_u32() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// tcgen05 in its two-CTA form.  Allocation, release of the permit and deallocation are executed by the same warp of
// BOTH CTAs; the MMA and its commits by one thread of the rank-0 CTA for both.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives once on the mbarrier (any CTA of the cluster) when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster)
               : "memory");
}
// Tiled load whose completion is counted on a barrier of the rank-0 CTA (the form that permits that).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const void* tmap, int x, int y, uint32_t bar_cluster) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
      "[%2];" ::"r"(dst_smem),
      "l"(tmap), "r"(bar_cluster), "r"(x), "r"(y)
      : "memory");
}
// Arrival on a barrier of the other CTA.  Default semantics, as for a barrier of the own CTA: the data the arrival
// vouches for is shared memory of THIS CTA, read by the tensor core through the async proxy (fence.proxy.async before
// the arrival); nothing of it is read by another CTA's threads.  (With .release.cluster the arriving warps spent two
// issue slots in three stalled on the memory barrier it implies.)
__device__ __forceinline__ void mbar_arrive_remote(uint32_t rbar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(rbar) : "memory");
}
// PAIR: the CTA holds HALF of the weight tile (128 rows): packed and dequantised tiles are half as large, which buys
// a fourth ring stage and a fourth dequantised buffer.
template <int MI, bool PAIR = false>
struct GemmGeo {
  static constexpr int kWRows = PAIR ? kBN / 2 : kBN;             // weight rows this CTA loads and unpacks
  static constexpr int kStageBytes = MI * kATileBytes + kWRows * 32;
  static constexpr int kStages = PAIR ? 4 : (MI == 2 ? 3 : 5);
  static constexpr int kRingBytes = kStages * kStageBytes;
  static constexpr int kBdOffset = kRingBytes;
  static constexpr int kBdBytes = kWRows * 128;                    // one dequantised buffer
  static constexpr int kBdCount = PAIR ? 4 : kBdBuffers;
  static constexpr int kBarOffset = kBdOffset + kBdCount * kBdBytes;
  static constexpr int kSmemBytes = kBarOffset + 512 + 1024;  // barriers + slack for 1024-byte alignment
  static constexpr int kTmemCols = MI * kBN;                  // 256 or 512: powers of two
};

template <int MI, bool PAIR>
__global__ void __launch_bounds__(kGemmThreads, 1)
    w4_gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                   const GemmParams p) {
  using geo = GemmGeo<MI, PAIR>;
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
  const uint32_t bar_full_w = bar_base + 32 * 8;             // [kStages], pairs only: this CTA's packed half
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + geo::kBarOffset + 26 * 8);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + geo::kBarOffset + 27 * 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // CTA pair: this CTA loads and unpacks rows [wr0, wr0 + kWRows) of the weight tile; the peer the other half
  uint32_t crank = 0;
  if constexpr (PAIR) crank = cluster_ctarank_u32();
  constexpr int kWRows = geo::kWRows;
  constexpr uint32_t kStageTx = MI * kATileBytes + kWRows * 32;  // bytes the copies of one stage deliver (one CTA)
  const int wr0 = PAIR ? (int)crank * kWRows : 0;
  const bool leader = crank == 0;
  // the same offsets in the shared memory of the peer and of the rank-0 CTA
  uint32_t peer_base = 0, lead_base = base;
  if constexpr (PAIR) {
    peer_base = mapa_u32(base, crank ^ 1u);
    lead_base = mapa_u32(base, 0u);
  }
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
      mbar_init(bar_full + 8 * s, 1);   // pairs: the X tiles of BOTH CTAs, counted on the rank-0 CTA's barrier
      mbar_init(bar_full_w + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, kDequantThreads + 1);
    }
    for (int b = 0; b < geo::kBdCount; ++b) {
      // this CTA's dequant threads and, on the rank-0 CTA of a pair, one arrival per dequant warp of the peer
      mbar_init(bar_bd_full + 8 * b, PAIR ? kDequantThreads + kDequantThreads / 32 : kDequantThreads);
      mbar_init(bar_bd_empty + 8 * b, 1);
    }
    mbar_init(bar_acc, 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_w);
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      tmem_alloc_pair(smem_u32(tmem_slot), geo::kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_slot), geo::kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();  // the peer's barriers are initialised before anybody arrives on them
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
          if constexpr (PAIR) {
            // X tiles of both CTAs complete on the rank-0 CTA's barrier (its producer expects the bytes of both);
            // the packed half on this CTA's own
            if (leader) mbar_arrive_expect_tx(bar_full + 8 * s, 2 * MI * kATileBytes);
#pragma unroll
            for (int mi = 0; mi < MI; ++mi)
              tma_load_2d_pair(stage + mi * kATileBytes, &tmap_x, kb * kBK, m0 + mi * 128,
                               lead_base + (bar_full - base) + 8 * s);
            mbar_arrive_expect_tx(bar_full_w + 8 * s, kWRows * 32);
            tma_load_2d(stage + MI * kATileBytes, &tmap_w, kb * (kBK / 8), n0 + wr0, bar_full_w + 8 * s);
          } else {
            mbar_arrive_expect_tx(bar_full + 8 * s, kStageTx);
#pragma unroll
            for (int mi = 0; mi < MI; ++mi)
              tma_load_2d(stage + mi * kATileBytes, &tmap_x, kb * kBK, m0 + mi * 128, bar_full + 8 * s);
            tma_load_2d(stage + MI * kATileBytes, &tmap_w, kb * (kBK / 8), n0 + wr0, bar_full + 8 * s);
          }
          if (++s == geo::kStages) { s = 0; ph ^= 1; }
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      // ------------------------------------------------------------ MMA issuer (pairs: the rank-0 CTA's, for both)
      if (lane == 0 && (!PAIR || leader)) {
        constexpr uint32_t idesc = umma_idesc_bf16(PAIR ? 256 : 128, kBN);
        int s = 0, b = 0;
        uint32_t ph = 0, bph = 0;
        for (int kb = 0; kb < nkb; ++kb) {
          if constexpr (PAIR) {
            // X tiles of both CTAs (counted here), dequantised halves of both CTAs (the peer's warps arrive here)
            mbar_wait(bar_full + 8 * s, ph, abort_flag);
            mbar_wait(bar_bd_full + 8 * b, bph, abort_flag);
          } else {
            mbar_wait(bar_full + 8 * s, ph, abort_flag);
            mbar_wait(bar_bd_full + 8 * b, bph, abort_flag);
          }
          tc_fence_after_sync();
          const uint32_t a_addr = base + s * geo::kStageBytes;
          const uint32_t b_addr = base + geo::kBdOffset + b * geo::kBdBytes;
#pragma unroll
          for (int kk = 0; kk < kBK / 16; ++kk) {
            const uint64_t db = umma_desc_k128(b_addr + kk * 32);
#pragma unroll
            for (int mi = 0; mi < MI; ++mi) {
              const uint64_t da = umma_desc_k128(a_addr + mi * kATileBytes + kk * 32);
              if constexpr (PAIR)
                umma_f16_ss_pair(tmem_base + mi * kBN, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
              else
                umma_f16_ss(tmem_base + mi * kBN, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            }
          }
          if constexpr (PAIR) {
            // the stage and the dequantised buffer are free in BOTH CTAs
            umma_commit_pair(bar_empty + 8 * s);
            umma_commit_pair(peer_base + (bar_empty - base) + 8 * s);
            umma_commit_pair(bar_bd_empty + 8 * b);
            umma_commit_pair(peer_base + (bar_bd_empty - base) + 8 * b);
          } else {
            umma_commit(bar_empty + 8 * s);      // the X tile and the packed tile of this stage are consumed
            umma_commit(bar_bd_empty + 8 * b);   // the dequantised tile may be overwritten
          }
          if (++s == geo::kStages) { s = 0; ph ^= 1; }
          if (++b == geo::kBdCount) { b = 0; bph ^= 1; }
        }
        if constexpr (PAIR) {
          umma_commit_pair(bar_acc);
          umma_commit_pair(peer_base + (bar_acc - base));
        } else {
          umma_commit(bar_acc);
        }
      }
      __syncwarp();
    } else {
      // ------------------------------------------------------------ dequant warps, then epilogue
      const int dt = tid - 64;          // 0..511
      // a thread owns kWords packed words of one row: a 32-wide half of the K block (one CTA per tile), or a
      // 16-wide quarter of it (CTA pair: this CTA unpacks 128 of the 256 rows)
      constexpr int kWords = PAIR ? 2 : 4;
      const int r = PAIR ? dt >> 2 : dt >> 1;   // row among the rows this CTA unpacks
      const int part = PAIR ? dt & 3 : dt & 1;  // which run of kWords words of the row
      const int hf = PAIR ? part >> 1 : part;   // which 32-wide half of the 64-wide K block (one scale each)
      const int n = n0 + wr0 + r;               // the weight row
      const uint32_t bd_off = geo::kBdOffset + r * 128;  // its place in this CTA's dequantised buffer
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
        if (lane == 0) mbar_wait((PAIR ? bar_full_w : bar_full) + 8 * s, ph, abort_flag);
        __syncwarp();
        uint32_t words[kWords];
        {
          const uint32_t src = base + s * geo::kStageBytes + MI * kATileBytes + r * 32 + part * (4 * kWords);
          if constexpr (PAIR) {
            const uint2 w2 = lds64(src);
            words[0] = w2.x; words[1] = w2.y;
          } else {
            const uint4 w4 = lds128(src);
            words[0] = w4.x; words[1] = w4.y; words[2] = w4.z; words[3] = w4.w;
          }
        }
        mbar_arrive(bar_empty + 8 * s);  // packed words are in registers

        if (lane == 0) mbar_wait(bar_bd_empty + 8 * b, bph ^ 1, abort_flag);
        __syncwarp();
        const uint32_t dst = bd_off + b * geo::kBdBytes;
#pragma unroll
        for (int c = 0; c < kWords; ++c) {
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
          const uint32_t at = dst + ((uint32_t(part * kWords + c) ^ sw) << 4);
          sts128(base + at, o);
        }
        if constexpr (PAIR) {
          // the MMA issuer sits in the rank-0 CTA: its own threads arrive one by one, the peer's once per warp (an
          // arrival on another CTA's barrier is a transaction of its own)
          fence_proxy_async_smem();
          if (leader) {
            mbar_arrive(bar_bd_full + 8 * b);
          } else {
            __syncwarp();  // the lanes' stores and fences are ordered before lane 0's release
            if (lane == 0) mbar_arrive_remote(lead_base + (bar_bd_full - base) + 8 * b);
          }
        } else {
          fence_proxy_async_smem();
          mbar_arrive(bar_bd_full + 8 * b);
        }
        if (++s == geo::kStages) { s = 0; ph ^= 1; }
        if (++b == geo::kBdCount) { b = 0; bph ^= 1; }
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
  // a CTA of a pair stays until its peer is done with it: the peer writes into this CTA's shared memory and arrives
  // on its barriers
  if constexpr (PAIR) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    if constexpr (PAIR)
      tmem_dealloc_pair(tmem_base, geo::kTmemCols);
    else
      tmem_dealloc(tmem_base, geo::kTmemCols);
  }
}

// ------------------------------------------------------------------ host side
template <int MI, bool PAIR>
int launch_gemm(const CUtensorMap& tx, const CUtensorMap& tw, const GemmParams& p, cudaStream_t stream) {
  auto kernel = w4_gemm_kernel<MI, PAIR>;
  cudaError_t e =
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmGeo<MI, PAIR>::kSmemBytes);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.n_whole + p.n_tail * p.tail_ks);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = GemmGeo<MI, PAIR>::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = PAIR ? 1 : 0;
  e = cudaLaunchKernelEx(&cfg, kernel, tx, tw, p);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

}  // namespace

int gemm_launch(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int G,
                const Workspace& ws, int flags, int sm_count, cudaStream_t stream) {
  static_assert(GemmGeo<2>::kSmemBytes <= kGemmSmemLimit && GemmGeo<1>::kSmemBytes <= kGemmSmemLimit &&
                    GemmGeo<2, true>::kSmemBytes <= kGemmSmemLimit,
                "smem");
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
  // CTA pairs (each unpacks half of the weight tile for both): where the token tiles pair up without much padding.
  // A lone token tile (M <= 256) would be paired with an empty one and do the whole unpack for half the product.
  const int mi_ = M <= 128 ? 1 : 2;
  const int tiles_m = (M + 128 * mi_ - 1) / (128 * mi_);
  const bool pair = !(flags & kFlagGemmNoPairs) && mi_ == 2 && (tiles_m % 2 == 0 || tiles_m >= 7);
  if (!make_tensor_map_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, Wq, (uint64_t)N, (uint64_t)K / 8, pair ? kBN / 2 : kBN,
                 kBK / 8, CU_TENSOR_MAP_SWIZZLE_NONE))
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
    const int mi = mi_;
    p.tiles_x = pair ? (tiles_m + 1) / 2 * 2 : tiles_m;  // pairs never straddle a row of tiles
    const long tiles = (long)p.tiles_x * ((N + kBN - 1) / kBN);
    if (tiles > 0x3fffffff) return kErrBadShape;
    const int sms = std::max(1, sm_count);
    const int sms_even = pair ? sms / 2 * 2 : sms;  // whole waves of pairs
    const long n_tail = tiles % sms_even ? tiles % sms_even : std::min<long>(tiles, sms_even);
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
  if (pair) return launch_gemm<2, true>(tx, tw, p, stream);
  return M <= 128 ? launch_gemm<1, false>(tx, tw, p, stream) : launch_gemm<2, false>(tx, tw, p, stream);
}

}  // namespace b2
