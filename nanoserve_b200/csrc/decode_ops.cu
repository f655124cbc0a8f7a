// Small kernels that sit between the quantized linears of a batch-1 decode step and read the current
// position from device memory, so that one captured CUDA graph serves every step:
//   b2_rope_kv_store     bias add + rotary embedding on q and k of the new token, k/v appended to the cache
//   b2_decode_attention  one query token against the cached keys/values (grouped-query attention)
//   b2_greedy_next       argmax over the logits, position += 1, embedding row of the chosen token
// The reference does these steps with PyTorch ops and a Python-side position (python/nanoserve/qwen.py:119-133,
// 147-151, 174-177: bias add, rope, _store_kv, SDPA over the cache, argmax); a host-side position would force one
// graph per step.  Arithmetic follows the reference's conventions: bf16 storage, fp32 math, rotate-half RoPE with
// angle = pos * inv_freq[i] (kernels/fused/rope.cuh:14-43), softmax scale 1/sqrt(D).
#include <cfloat>
#include <cstdint>
#include <cuda_bf16.h>

#include "../../include/nanoserve_b200.h"
#include "w4_internal.h"

namespace {

using bf16 = __nv_bfloat16;

// The small kernels of a decode step are launched with programmatic stream serialization, like the GEMVs around them:
// they become resident while the previous kernel drains and start the moment it has completed, which takes the
// launch latency off the step's critical path.  Under such a launch the SM's L1 is not invalidated between the
// producer of the inputs and the loads, so everything a previous kernel may have written is read with
// ld.global.cg (L2), never through the non-coherent path.
__device__ __forceinline__ void pdl_begin() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ float ld_bf16(const bf16* p) {
  return __bfloat162float(__ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(p))));
}
// E (2 or 4) consecutive bf16 as floats with one L2 load.
template <int E>
__device__ __forceinline__ void ld_row(const bf16* p, float (&f)[E]) {
  static_assert(E == 2 || E == 4, "head dimension 64 or 128");
  if constexpr (E == 4) {
    const uint2 v = __ldcg(reinterpret_cast<const uint2*>(p));
    f[0] = __uint_as_float(v.x << 16);
    f[1] = __uint_as_float(v.x & 0xFFFF0000u);
    f[2] = __uint_as_float(v.y << 16);
    f[3] = __uint_as_float(v.y & 0xFFFF0000u);
  } else {
    const unsigned v = __ldcg(reinterpret_cast<const unsigned*>(p));
    f[0] = __uint_as_float(v << 16);
    f[1] = __uint_as_float(v & 0xFFFF0000u);
  }
}
template <typename... Args>
cudaError_t launch_pdl(void (*kernel)(Args...), dim3 grid, dim3 block, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// grid: Hq + 2*Hk blocks (one per head of the fused qkv row), block: D/2 threads.
// With wait_sig set, qkv is the gathered output of a tensor-parallel GEMV (b2_w4_linear_tp): every block first waits
// (bounded) until all producing CTAs of all ranks have counted themselves in, then reads qkv from L2.
__global__ void rope_kv_store_kernel(bf16* qkv, const bf16* __restrict__ bias,
                                     const float* __restrict__ inv_freq, const int* __restrict__ pos_ptr,
                                     bf16* __restrict__ cache_k, bf16* __restrict__ cache_v, int Hq, int Hk, int D,
                                     int max_len, const unsigned* wait_sig, const int* epoch, unsigned wait_per_epoch,
                                     int* status) {
  const int h = blockIdx.x, i = threadIdx.x, half = D / 2;
  pdl_begin();
  if (wait_sig != nullptr) {
    if (i == 0) {
      const unsigned target = ((unsigned)*reinterpret_cast<const volatile int*>(epoch) + 1u) * wait_per_epoch;
      const long long t0 = clock64();
      for (;;) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(wait_sig) : "memory");
        if ((int)(v - target) >= 0) break;
        if (clock64() - t0 > 1000000000LL) {  // about half a second: report and go on with what is there
          if (status != nullptr) atomicCAS(status, 0, b2::kStatusGemvTimeout);
          break;
        }
        __nanosleep(40);
      }
    }
    __syncthreads();
  }
  const int pos = __ldcg(pos_ptr);
  bf16* x = qkv + (size_t)h * D;
  float a = __bfloat162float(__ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(x) + i)));
  float b = __bfloat162float(__ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(x) + i + half)));
  if (bias != nullptr) {  // the projection output is stored in bf16, then the bias is added in bf16 (q += bq)
    a = __bfloat162float(__float2bfloat16(a + __bfloat162float(bias[(size_t)h * D + i])));
    b = __bfloat162float(__float2bfloat16(b + __bfloat162float(bias[(size_t)h * D + i + half])));
  }
  if (h < Hq + Hk) {  // q and k heads rotate, v heads do not
    float sn, cs;
    sincosf((float)pos * inv_freq[i], &sn, &cs);
    const float ra = a * cs - b * sn, rb = b * cs + a * sn;
    a = ra;
    b = rb;
  }
  const bf16 oa = __float2bfloat16(a), ob = __float2bfloat16(b);
  x[i] = oa;
  x[i + half] = ob;
  if (h >= Hq && pos < max_len) {
    const int kh = h - Hq;
    bf16* dst = (kh < Hk ? cache_k + ((size_t)kh * max_len + pos) * D
                         : cache_v + ((size_t)(kh - Hk) * max_len + pos) * D);
    dst[i] = oa;
    dst[i + half] = ob;
  }
}

// Decode attention in two launches.  Pass 1, grid (Hk, kSplits): a CTA takes one KV head and one slice of the
// cached positions; it first copies the slice's K and V rows into shared memory with 16-byte loads that are all in
// flight together (one L2 round trip for the whole slice; a loop of dependent-looking 8-byte loads per position
// cost a round trip per position: 16 us per layer at 600 positions), then warp w serves query head w of the group
// (Hq / Hk <= 8 heads share a KV head); lanes split the head dimension; online softmax per warp.  It writes
// un-normalised partials (max, sum, acc[D]) per (query head, split).  Pass 2, grid Hq: merges the splits, all of
// its loads issued before the first use.  With 4 KV heads x 32 splits the first pass fills 128 SMs however long
// the cache is.
constexpr int kSplits = 32;
constexpr int kTileRows = 32;  // positions staged in shared memory at a time

template <int D>
__global__ void __launch_bounds__(256) decode_attention_partial_kernel(
    const bf16* q, const bf16* cache_k, const bf16* cache_v, const int* pos_ptr, float* part, int Hq, int Hk,
    int max_len, float scale) {
  constexpr int E = D / 32;        // elements per lane
  constexpr int kRowU4 = D / 8;    // 16-byte units per row
  __shared__ __align__(16) bf16 s_k[kTileRows * D];
  __shared__ __align__(16) bf16 s_v[kTileRows * D];
  const int kh = blockIdx.x, sp = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rep = Hq / Hk;
  pdl_begin();
  const int h = kh * rep + min(warp, rep - 1);
  const int n = min(__ldcg(pos_ptr) + 1, max_len);
  const int per = (n + kSplits - 1) / kSplits;
  const int j0 = sp * per, j1 = min(n, j0 + per);
  const uint4* kbase = reinterpret_cast<const uint4*>(cache_k + (size_t)kh * max_len * D);
  const uint4* vbase = reinterpret_cast<const uint4*>(cache_v + (size_t)kh * max_len * D);
  float qf[E];
  ld_row<E>(q + (size_t)h * D + lane * E, qf);
#pragma unroll
  for (int e = 0; e < E; ++e) qf[e] *= scale;
  float m = -FLT_MAX, l = 0.f, acc[E];
#pragma unroll
  for (int e = 0; e < E; ++e) acc[e] = 0.f;
  for (int t0 = j0; t0 < j1; t0 += kTileRows) {
    const int rows = min(kTileRows, j1 - t0);
    const int units = rows * kRowU4;
    if (t0 > j0) __syncthreads();  // everybody is done with the previous tile
    // all loads first, then all stores: one round trip for the tile
    constexpr int kPerThread = (kTileRows * kRowU4 + 255) / 256;
    uint4 kv[kPerThread], vv[kPerThread];
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
      const int u = threadIdx.x + i * 256;
      if (u < units) {
        kv[i] = __ldcg(kbase + (size_t)t0 * kRowU4 + u);
        vv[i] = __ldcg(vbase + (size_t)t0 * kRowU4 + u);
      }
    }
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
      const int u = threadIdx.x + i * 256;
      if (u < units) {
        reinterpret_cast<uint4*>(s_k)[u] = kv[i];
        reinterpret_cast<uint4*>(s_v)[u] = vv[i];
      }
    }
    __syncthreads();
    if (warp < rep) {
      for (int r = 0; r < rows; ++r) {
        float s = 0.f, kf[E], vf[E];
#pragma unroll
        for (int e = 0; e < E; ++e) {
          kf[e] = __bfloat162float(s_k[r * D + lane * E + e]);
          vf[e] = __bfloat162float(s_v[r * D + lane * E + e]);
        }
#pragma unroll
        for (int e = 0; e < E; ++e) s += qf[e] * kf[e];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        const float mn = fmaxf(m, s);
        const float corr = __expf(m - mn), pj = __expf(s - mn);
        l = l * corr + pj;
#pragma unroll
        for (int e = 0; e < E; ++e) acc[e] = acc[e] * corr + pj * vf[e];
        m = mn;
      }
    }
  }
  if (warp >= rep) return;
  float* out = part + ((size_t)h * kSplits + sp) * (D + 2);
  if (lane == 0) {
    out[0] = m;
    out[1] = l;
  }
#pragma unroll
  for (int e = 0; e < E; ++e) out[2 + lane * E + e] = acc[e];
}

template <int D>
__global__ void decode_attention_merge_kernel(const float* part, bf16* out) {
  const int h = blockIdx.x, d = threadIdx.x;  // block: D threads
  pdl_begin();
  const float* p = part + (size_t)h * kSplits * (D + 2);
  // every load of the merge is issued before the first use: one L2 round trip, not one per split
  float ms[kSplits], ls[kSplits], as[kSplits];
#pragma unroll
  for (int s = 0; s < kSplits; ++s) {
    ms[s] = __ldcg(p + s * (D + 2));
    ls[s] = __ldcg(p + s * (D + 2) + 1);
    as[s] = __ldcg(p + s * (D + 2) + 2 + d);
  }
  float mm = -FLT_MAX;
#pragma unroll
  for (int s = 0; s < kSplits; ++s) mm = fmaxf(mm, ms[s]);
  float num = 0.f, den = 0.f;
#pragma unroll
  for (int s = 0; s < kSplits; ++s) {
    const float f = ms[s] == -FLT_MAX ? 0.f : __expf(ms[s] - mm);
    num += f * as[s];
    den += f * ls[s];
  }
  out[(size_t)h * D + d] = __float2bfloat16(den > 0.f ? num / den : 0.f);
}

// The attention of one decode step in ONE launch: bias add + RoPE on q and k of the new token, the new k/v row
// appended to the cache, the partial pass over the cache, and the merge.  Same grid and tile loop as the two-launch
// form above.  Every warp prepares its own query head in registers (bias, rotation, rounding to bf16 as
// b2_rope_kv_store stores it).  The CTA whose slice holds the new position computes the new k and v rows, stores them
// to the cache and serves them to its own tile loop from shared memory.  The last CTA of a KV head to have written
// its partials (an arrival counter per KV head; nobody waits) merges the splits of that head's query heads.
// Launches per layer of a decode step: 5 instead of 7.
template <int D>
__global__ void __launch_bounds__(256) decode_attention_fused_kernel(
    const bf16* qkv, const bf16* __restrict__ bias, const float* __restrict__ inv_freq, const int* pos_ptr,
    bf16* cache_k, bf16* cache_v, float* part, int* counters, bf16* out, int Hq, int Hk, int max_len, float scale,
    const unsigned* wait_sig, const int* epoch, unsigned wait_per_epoch, int* status, const b2::GemvTp ann,
    int early) {
  constexpr int E = D / 32;        // elements per lane
  constexpr int kRowU4 = D / 8;    // 16-byte units per row
  constexpr int half = D / 2;
  __shared__ __align__(16) bf16 s_k[kTileRows * D];
  __shared__ __align__(16) bf16 s_v[kTileRows * D];
  __shared__ __align__(16) bf16 s_newk[D];
  __shared__ __align__(16) bf16 s_newv[D];
  __shared__ float s_f[8 * kSplits];   // merge: weight of every (query head of the group, split)
  __shared__ float s_den[8];
  __shared__ int s_last;
  const int kh = blockIdx.x, sp = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rep = Hq / Hk;
  const uint4* kbase = reinterpret_cast<const uint4*>(cache_k + (size_t)kh * max_len * D);
  const uint4* vbase = reinterpret_cast<const uint4*>(cache_v + (size_t)kh * max_len * D);
  constexpr int kPerThread = (kTileRows * kRowU4 + 255) / 256;
  uint4 kv[kPerThread], vv[kPerThread];
  int pos = 0, n = 0, per = 0, j0 = 0, j1 = 0;
  auto slice = [&]() {
    pos = __ldcg(pos_ptr);
    n = min(pos + 1, max_len);
    per = (n + kSplits - 1) / kSplits;
    j0 = sp * per;
    j1 = min(n, j0 + per);
  };
  auto request = [&](int t0) {
    const int units = min(kTileRows, j1 - t0) * kRowU4;
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
      const int u = tid + i * 256;
      if (u < units && t0 + u / kRowU4 != pos) {  // the row this launch appends is not in the cache yet
        kv[i] = __ldcg(kbase + (size_t)t0 * kRowU4 + u);
        vv[i] = __ldcg(vbase + (size_t)t0 * kRowU4 + u);
      }
    }
  };
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // `early`: the position and the cached rows below it were written by earlier steps, not by the kernel in front of
  // this one (which produces qkv): the first tile's rows are requested while that kernel still runs
  if (early) {
    slice();
    if (j0 < j1) request(j0);
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // deferred signal of the tensor-parallel GEMV in front of this kernel (it has completed)
  if (ann.announce_world && blockIdx.x == 0 && blockIdx.y == 0 && tid < ann.announce_world)
    asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(ann.announce_peer[tid]) : "memory");
  if (wait_sig != nullptr) {
    if (tid == 0) {
      const unsigned target = ((unsigned)*reinterpret_cast<const volatile int*>(epoch) + 1u) * wait_per_epoch;
      const long long t0 = clock64();
      for (;;) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(wait_sig) : "memory");
        if ((int)(v - target) >= 0) break;
        if (clock64() - t0 > 1000000000LL) {  // about half a second: report and go on with what is there
          if (status != nullptr) atomicCAS(status, 0, b2::kStatusGemvTimeout);
          break;
        }
        __nanosleep(40);
      }
    }
    __syncthreads();
  }
  if (!early) {
    slice();
    if (j0 < j1) request(j0);
  }
  const bool owner = pos < max_len && pos >= j0 && pos < j1;  // this CTA's slice holds the new position

  // ---- the new k and v rows (owner only): thread i < D/2 rotates the pair (i, i + D/2) of k, the next D/2 threads
  // add the bias to a pair of v
  if (owner && tid < D) {
    const bool is_v = tid >= half;
    const int i = is_v ? tid - half : tid;
    const int hh = Hq + (is_v ? Hk : 0) + kh;
    const bf16* x = qkv + (size_t)hh * D;
    float a = ld_bf16(x + i), b = ld_bf16(x + i + half);
    if (bias != nullptr) {
      a = __bfloat162float(__float2bfloat16(a + __bfloat162float(bias[(size_t)hh * D + i])));
      b = __bfloat162float(__float2bfloat16(b + __bfloat162float(bias[(size_t)hh * D + i + half])));
    }
    if (!is_v) {
      float sn, cs;
      sincosf((float)pos * inv_freq[i], &sn, &cs);
      const float ra = a * cs - b * sn, rb = b * cs + a * sn;
      a = ra;
      b = rb;
    }
    const bf16 oa = __float2bfloat16(a), ob = __float2bfloat16(b);
    bf16* sm = is_v ? s_newv : s_newk;
    sm[i] = oa;
    sm[i + half] = ob;
    bf16* dst = (is_v ? cache_v : cache_k) + ((size_t)kh * max_len + pos) * D;
    dst[i] = oa;
    dst[i + half] = ob;
  }

  // ---- this warp's query head: bias, rotation, bf16 rounding, softmax scale
  const int h = kh * rep + min(warp, rep - 1);
  float qf[E];
  {
    ld_row<E>(qkv + (size_t)h * D + lane * E, qf);
    if (bias != nullptr) {
#pragma unroll
      for (int e = 0; e < E; ++e)
        qf[e] = __bfloat162float(__float2bfloat16(qf[e] + __bfloat162float(bias[(size_t)h * D + lane * E + e])));
    }
#pragma unroll
    for (int e = 0; e < E; ++e) {
      const float other = __shfl_xor_sync(0xffffffffu, qf[e], 16);  // the element D/2 away
      float sn, cs;
      sincosf((float)pos * inv_freq[(lane * E + e) % half], &sn, &cs);
      const float r = lane < 16 ? qf[e] * cs - other * sn : qf[e] * cs + other * sn;
      qf[e] = __bfloat162float(__float2bfloat16(r)) * scale;
    }
  }

  float m = -FLT_MAX, l = 0.f, acc[E];
#pragma unroll
  for (int e = 0; e < E; ++e) acc[e] = 0.f;
  for (int t0 = j0; t0 < j1; t0 += kTileRows) {
    const int rows = min(kTileRows, j1 - t0);
    const int units = rows * kRowU4;
    if (t0 > j0) request(t0);
    __syncthreads();  // everybody is done with the previous tile; the new rows are in shared memory
#pragma unroll
    for (int i = 0; i < kPerThread; ++i) {
      const int u = tid + i * 256;
      if (u < units) {
        const bool fresh = t0 + u / kRowU4 == pos;
        reinterpret_cast<uint4*>(s_k)[u] = fresh ? reinterpret_cast<const uint4*>(s_newk)[u % kRowU4] : kv[i];
        reinterpret_cast<uint4*>(s_v)[u] = fresh ? reinterpret_cast<const uint4*>(s_newv)[u % kRowU4] : vv[i];
      }
    }
    __syncthreads();
    if (warp < rep) {
      for (int r = 0; r < rows; ++r) {
        float s = 0.f, kf[E], vf[E];
#pragma unroll
        for (int e = 0; e < E; ++e) {
          kf[e] = __bfloat162float(s_k[r * D + lane * E + e]);
          vf[e] = __bfloat162float(s_v[r * D + lane * E + e]);
        }
#pragma unroll
        for (int e = 0; e < E; ++e) s += qf[e] * kf[e];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        const float mn = fmaxf(m, s);
        const float corr = __expf(m - mn), pj = __expf(s - mn);
        l = l * corr + pj;
#pragma unroll
        for (int e = 0; e < E; ++e) acc[e] = acc[e] * corr + pj * vf[e];
        m = mn;
      }
    }
  }
  if (warp < rep) {
    float* o = part + ((size_t)h * kSplits + sp) * (D + 2);
    if (lane == 0) {
      __stcg(o, m);
      __stcg(o + 1, l);
    }
#pragma unroll
    for (int e = 0; e < E; ++e) __stcg(o + 2 + lane * E + e, acc[e]);
  }

  if (counters == nullptr) return;  // a merge launch follows
  // ---- the last CTA of this KV head to arrive merges the splits
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(counters + kh, 1);
    const int last = old == kSplits - 1;
    if (last) counters[kh] = 0;  // ready for the next launch (launches that share the counters are stream-ordered)
    s_last = last;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // weight of every (query head, split): exp(m - max m), and the denominator of every head
  if (warp < rep) {
    const int hq = kh * rep + warp;
    const float* pp = part + ((size_t)hq * kSplits + lane) * (D + 2);  // kSplits == 32: one split per lane
    const float ms = __ldcg(pp), ls = __ldcg(pp + 1);
    float mm = ms;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o));
    const float f = ms == -FLT_MAX ? 0.f : __expf(ms - mm);
    float den = f * ls;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
    s_f[warp * kSplits + lane] = f;
    if (lane == 0) s_den[warp] = den;
  }
  __syncthreads();
  for (int item = tid; item < rep * D; item += 256) {
    const int w = item / D, d = item - w * D;
    const int hq = kh * rep + w;
    const float* pp = part + (size_t)hq * kSplits * (D + 2) + 2 + d;
    float as[kSplits];
#pragma unroll
    for (int sidx = 0; sidx < kSplits; ++sidx) as[sidx] = __ldcg(pp + sidx * (D + 2));
    float num = 0.f;
#pragma unroll
    for (int sidx = 0; sidx < kSplits; ++sidx) num += s_f[w * kSplits + sidx] * as[sidx];
    const float den = s_den[w];
    out[(size_t)hq * D + d] = __float2bfloat16(den > 0.f ? num / den : 0.f);
  }
}

// Greedy choice in two launches.  Pass 1, kArgBlocks CTAs: each scans a slice of the logits and writes its best
// (value, index).  Pass 2, one CTA: picks the best of those (lowest index on ties, as torch.argmax returns the
// first occurrence), records the token, advances step and position, and copies the token's embedding row.
constexpr int kArgBlocks = 148;

__device__ __forceinline__ void argmax_merge(float& best, int& bi, float ov, int oi) {
  if (ov > best || (ov == best && oi < bi)) {
    best = ov;
    bi = oi;
  }
}

__global__ void __launch_bounds__(256) argmax_partial_kernel(const bf16* __restrict__ logits, int V,
                                                             float* __restrict__ pv, int* __restrict__ pi) {
  __shared__ float s_v[8];
  __shared__ int s_i[8];
  float best = -FLT_MAX;
  int bi = 0x7fffffff;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < V; i += gridDim.x * blockDim.x) {
    const float v = __bfloat162float(logits[i]);
    if (v > best) {  // indices ascend within a thread, so the first occurrence is kept
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    argmax_merge(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  if ((threadIdx.x & 31) == 0) {
    s_v[threadIdx.x >> 5] = best;
    s_i[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) argmax_merge(best, bi, s_v[w], s_i[w]);
    pv[blockIdx.x] = best;
    pi[blockIdx.x] = bi;
  }
}

__global__ void __launch_bounds__(256) greedy_finish_kernel(const float* __restrict__ pv, const int* __restrict__ pi,
                                                            int nparts, int V, const bf16* __restrict__ embed, int H,
                                                            int* __restrict__ pos_ptr, long long* __restrict__ out_tokens,
                                                            int* __restrict__ step_ptr, bf16* __restrict__ x_next) {
  __shared__ float s_v[8];
  __shared__ int s_i[8];
  __shared__ int s_tok;
  float best = -FLT_MAX;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) argmax_merge(best, bi, pv[i], pi[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    argmax_merge(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  if ((threadIdx.x & 31) == 0) {
    s_v[threadIdx.x >> 5] = best;
    s_i[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) argmax_merge(best, bi, s_v[w], s_i[w]);
    if (bi < 0 || bi >= V) bi = 0;
    s_tok = bi;
    out_tokens[*step_ptr] = bi;
    *step_ptr += 1;
    *pos_ptr += 1;
  }
  __syncthreads();
  const bf16* row = embed + (size_t)s_tok * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) x_next[i] = row[i];
}

}  // namespace

// One thread waits (bounded) for an arrival counter of a fused all-gather: kernels that follow on the stream may then
// read the gathered rows without a wait of their own.
__global__ void tp_wait_kernel(const unsigned* wait_sig, int* epoch, unsigned wait_per_epoch, int* status,
                               const b2::GemvTp ann, int advance_epoch) {
  // deferred signal of the kernel in front of this one (complete: plain stream order), one thread per rank
  if (threadIdx.x < ann.announce_world)
    asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(ann.announce_peer[threadIdx.x]) : "memory");
  if (threadIdx.x != 0) return;
  const unsigned target = ((unsigned)*reinterpret_cast<const volatile int*>(epoch) + 1u) * wait_per_epoch;
  const long long t0 = clock64();
  for (;;) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(wait_sig) : "memory");
    if ((int)(v - target) >= 0) break;
    if (clock64() - t0 > 1000000000LL) {
      if (status != nullptr) atomicCAS(status, 0, b2::kStatusGemvTimeout);
      break;
    }
    __nanosleep(40);
  }
  if (advance_epoch) *epoch += 1;  // the use of the counters that this wait closes is over
}

namespace b2 {
int tp_wait_launch(const void* wait_sig, const void* epoch, unsigned wait_per_epoch, int* status, cudaStream_t stream,
                   const GemvTp* announce, int advance_epoch) {
  if (!wait_sig || !epoch) return kErrBadPointer;
  GemvTp ann;
  if (announce != nullptr) ann = *announce;
  tp_wait_kernel<<<1, 32, 0, stream>>>(static_cast<const unsigned*>(wait_sig),
                                       static_cast<int*>(const_cast<void*>(epoch)), wait_per_epoch, status, ann,
                                       advance_epoch);
  return (int)cudaGetLastError();
}
int rope_kv_store_launch(void* qkv, const void* bias, const void* inv_freq, const void* pos, void* cache_k,
                         void* cache_v, int Hq, int Hk, int D, int max_len, const void* wait_sig, const void* epoch,
                         unsigned wait_per_epoch, int* status, cudaStream_t stream) {
  if (Hq < 1 || Hk < 1 || D < 2 || D % 2 || D / 2 > 1024 || max_len < 1) return kErrBadShape;
  if (!qkv || !inv_freq || !pos || !cache_k || !cache_v) return kErrBadPointer;
  if (wait_sig != nullptr && !epoch) return kErrBadPointer;
  // the kernel moves bf16 pairs: 4-byte alignment of the activations, the bias and the caches
  if ((reinterpret_cast<uintptr_t>(qkv) & 3) || (reinterpret_cast<uintptr_t>(bias) & 3) ||
      (reinterpret_cast<uintptr_t>(cache_k) & 3) || (reinterpret_cast<uintptr_t>(cache_v) & 3) ||
      (reinterpret_cast<uintptr_t>(inv_freq) & 3) || (reinterpret_cast<uintptr_t>(pos) & 3))
    return kErrBadPointer;
  const cudaError_t e = launch_pdl(rope_kv_store_kernel, dim3(Hq + 2 * Hk), dim3(D / 2), stream,
                                   static_cast<bf16*>(qkv), static_cast<const bf16*>(bias),
                                   static_cast<const float*>(inv_freq), static_cast<const int*>(pos),
                                   static_cast<bf16*>(cache_k), static_cast<bf16*>(cache_v), Hq, Hk, D, max_len,
                                   static_cast<const unsigned*>(wait_sig), static_cast<const int*>(epoch),
                                   wait_per_epoch, status);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}
}  // namespace b2

namespace b2 {
int decode_attention_fused_launch(const void* qkv, const void* bias, const void* inv_freq, const void* pos,
                                  void* cache_k, void* cache_v, void* out, void* workspace, int Hq, int Hk, int D,
                                  int max_len, const GemvTp* tp, int flags, int* status, cudaStream_t stream) {
  static_assert(kSplits == 32, "the merge takes one split per lane");
  if (Hq < 1 || Hk < 1 || Hq % Hk || Hq / Hk > 8 || max_len < 1) return b2::kErrBadShape;
  if (D != 128 && D != 64) return b2::kErrNotImplemented;
  if (!qkv || !inv_freq || !cache_k || !cache_v || !pos || !out || !workspace) return b2::kErrBadPointer;
  GemvTp ann;
  if (tp != nullptr) ann = *tp;
  const void* wait_sig = ann.wait_sig;
  const void* epoch = ann.epoch;
  const unsigned wait_per_epoch = ann.wait_per_epoch;
  if (wait_sig != nullptr && !epoch) return b2::kErrBadPointer;
  // 8-byte loads of q, 16-byte loads and stores of cache rows, float partials and counters in the workspace
  if ((reinterpret_cast<uintptr_t>(qkv) & 7) || (reinterpret_cast<uintptr_t>(bias) & 3) ||
      (reinterpret_cast<uintptr_t>(cache_k) & 15) || (reinterpret_cast<uintptr_t>(cache_v) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 1) || (reinterpret_cast<uintptr_t>(workspace) & 3) ||
      (reinterpret_cast<uintptr_t>(pos) & 3) || (reinterpret_cast<uintptr_t>(inv_freq) & 3))
    return b2::kErrBadPointer;
  const float scale = 1.f / sqrtf((float)D);
  float* part = static_cast<float*>(workspace);
  const bool one_launch = (flags & 1) != 0;
  int* counters = one_launch ? reinterpret_cast<int*>(part + (size_t)Hq * kSplits * (D + 2)) : nullptr;
  const dim3 grid(Hk, kSplits);
  auto go = [&](auto kernel) {
    return launch_pdl(kernel, grid, dim3(256), stream, static_cast<const bf16*>(qkv),
                      static_cast<const bf16*>(bias), static_cast<const float*>(inv_freq),
                      static_cast<const int*>(pos), static_cast<bf16*>(cache_k), static_cast<bf16*>(cache_v), part,
                      counters, static_cast<bf16*>(out), Hq, Hk, max_len, scale,
                      static_cast<const unsigned*>(wait_sig), static_cast<const int*>(epoch), wait_per_epoch, status,
                      ann, (flags & 2) ? 1 : 0);
  };
  cudaError_t e = D == 128 ? go(decode_attention_fused_kernel<128>) : go(decode_attention_fused_kernel<64>);
  if (e == cudaSuccess && !one_launch) {
    e = D == 128 ? launch_pdl(decode_attention_merge_kernel<128>, dim3(Hq), dim3(128), stream,
                              static_cast<const float*>(part), static_cast<bf16*>(out))
                 : launch_pdl(decode_attention_merge_kernel<64>, dim3(Hq), dim3(64), stream,
                              static_cast<const float*>(part), static_cast<bf16*>(out));
  }
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}
}  // namespace b2

extern "C" {

int b2_rope_kv_store(void* qkv, const void* bias, const void* inv_freq, const void* pos, void* cache_k, void* cache_v,
                     int Hq, int Hk, int D, int max_len, void* stream) {
  return b2::rope_kv_store_launch(qkv, bias, inv_freq, pos, cache_k, cache_v, Hq, Hk, D, max_len, nullptr, nullptr, 0,
                                  nullptr, static_cast<cudaStream_t>(stream));
}

size_t b2_decode_workspace_bytes(int Hq, int D) {
  const size_t attn = (size_t)Hq * kSplits * (D + 2) * sizeof(float);
  const size_t arg = (size_t)kArgBlocks * (sizeof(float) + sizeof(int));
  return attn > arg ? attn : arg;
}

int b2_decode_attention(const void* q, const void* cache_k, const void* cache_v, const void* pos, void* out,
                        void* workspace, int Hq, int Hk, int D, int max_len, void* stream) {
  if (Hq < 1 || Hk < 1 || Hq % Hk || Hq / Hk > 8 || max_len < 1) return b2::kErrBadShape;
  if (D != 128 && D != 64) return b2::kErrNotImplemented;
  if (!q || !cache_k || !cache_v || !pos || !out || !workspace) return b2::kErrBadPointer;
  // 8-byte loads of q, 16-byte loads of the cache rows, float partials in the workspace
  if ((reinterpret_cast<uintptr_t>(q) & 7) || (reinterpret_cast<uintptr_t>(cache_k) & 15) ||
      (reinterpret_cast<uintptr_t>(cache_v) & 15) || (reinterpret_cast<uintptr_t>(out) & 1) ||
      (reinterpret_cast<uintptr_t>(workspace) & 3) || (reinterpret_cast<uintptr_t>(pos) & 3))
    return b2::kErrBadPointer;
  const float scale = 1.f / sqrtf((float)D);
  const auto st = static_cast<cudaStream_t>(stream);
  float* part = static_cast<float*>(workspace);
  const dim3 grid(Hk, kSplits);
  if (D == 128) {
    launch_pdl(decode_attention_partial_kernel<128>, grid, dim3(256), st, static_cast<const bf16*>(q),
               static_cast<const bf16*>(cache_k), static_cast<const bf16*>(cache_v), static_cast<const int*>(pos), part,
               Hq, Hk, max_len, scale);
    launch_pdl(decode_attention_merge_kernel<128>, dim3(Hq), dim3(128), st, static_cast<const float*>(part),
               static_cast<bf16*>(out));
  } else {
    launch_pdl(decode_attention_partial_kernel<64>, grid, dim3(256), st, static_cast<const bf16*>(q),
               static_cast<const bf16*>(cache_k), static_cast<const bf16*>(cache_v), static_cast<const int*>(pos), part,
               Hq, Hk, max_len, scale);
    launch_pdl(decode_attention_merge_kernel<64>, dim3(Hq), dim3(64), st, static_cast<const float*>(part),
               static_cast<bf16*>(out));
  }
  return (int)cudaGetLastError();
}

size_t b2_decode_attention_fused_workspace_bytes(int Hq, int Hk, int D) {
  return (size_t)Hq * kSplits * (D + 2) * sizeof(float) + (size_t)Hk * sizeof(int);
}

int b2_greedy_next(const void* logits, int V, const void* embed, int H, void* pos, void* out_tokens, void* step,
                   void* x_next, void* workspace, void* stream) {
  if (V < 1 || H < 1) return b2::kErrBadShape;
  if (!logits || !embed || !pos || !out_tokens || !step || !x_next || !workspace) return b2::kErrBadPointer;
  const auto st = static_cast<cudaStream_t>(stream);
  float* pv = static_cast<float*>(workspace);
  int* pi = reinterpret_cast<int*>(pv + kArgBlocks);
  argmax_partial_kernel<<<kArgBlocks, 256, 0, st>>>(static_cast<const bf16*>(logits), V, pv, pi);
  greedy_finish_kernel<<<1, 256, 0, st>>>(pv, pi, kArgBlocks, V, static_cast<const bf16*>(embed), H,
                                          static_cast<int*>(pos), static_cast<long long*>(out_tokens),
                                          static_cast<int*>(step), static_cast<bf16*>(x_next));
  return (int)cudaGetLastError();
}

// Second half of b2_greedy_next for callers whose logits kernel already reduced blocks of the vocabulary
// (b2_lm_head): picks the largest of `nparts` (value, index) pairs, lowest index on ties, then does what
// b2_greedy_next does with the token.
int b2_greedy_pick(const void* part_max, const void* part_idx, int nparts, int V, const void* embed, int H, void* pos,
                   void* out_tokens, void* step, void* x_next, void* stream) {
  if (V < 1 || H < 1 || nparts < 1) return b2::kErrBadShape;
  if (!part_max || !part_idx || !embed || !pos || !out_tokens || !step || !x_next) return b2::kErrBadPointer;
  greedy_finish_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(part_max), static_cast<const int*>(part_idx), nparts, V,
      static_cast<const bf16*>(embed), H, static_cast<int*>(pos), static_cast<long long*>(out_tokens),
      static_cast<int*>(step), static_cast<bf16*>(x_next));
  return (int)cudaGetLastError();
}

}  // extern "C"
