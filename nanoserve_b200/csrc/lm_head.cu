// bf16 vocabulary projection of the decode step with the greedy argmax in its epilogue:
//   logits[M, V] (bf16) = X[M, K] (bf16) . W[V, K]^T (bf16), fp32 accumulation, 1 <= M <= 8;
//   per 128-row block the largest logit of token 0 and its index (lowest index on ties).
//
// The reference keeps the lm_head in bf16 and runs it through F.linear, then argmax on the host side of the step
// (python/nanoserve/qwen.py:164,174-177).  At batch 1 this is a 1.09 GB stream for the 152064 x 3584 Qwen2.5-7B
// head -- a quarter of the bytes of a W4 decode step -- so it gets the same treatment as the quantized GEMV:
// weights go from global memory straight into registers in mma fragment layout (lane (g, t) loads 16 bytes of rows
// g and g + 8 per 32-wide chunk of K, eight chunks in flight), mma.sync.m16n8k16 bf16 with the tokens in the
// columns, no shared-memory staging of W, CTAs of half an SM launched with programmatic stream serialization so
// that the weight stream starts while the previous kernel drains.  The 16 bytes a lane loads are eight
// consecutive k; the contraction index of an mma is a dummy, so the B fragment is simply the same 16 bytes of X.
// The final residual add + RMSNorm of the model can be folded into the staging of X (same prologue as the GEMV).
#include <cfloat>

#include "../../include/nanoserve_b200.h"
#include "w4_gemv_shared.cuh"

namespace b2 {

namespace {

constexpr int kThreads = 256;
constexpr int kRowsPerCta = 128;
constexpr int kRing = 8;

__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__global__ void __launch_bounds__(kThreads, 2)
    lm_head_kernel(const GemvParams p, const __nv_bfloat16* __restrict__ W, float* __restrict__ part_v,
                   int* __restrict__ part_i, int idx_offset) {
  extern __shared__ __align__(128) unsigned char smem[];
  float* ss = reinterpret_cast<float*>(smem);              // [16][16] RMSNorm partial sums
  float* inv = reinterpret_cast<float*>(smem + 1024);      // [16]
  float* s_v = reinterpret_cast<float*>(smem + 1088);      // [8] per-warp maxima
  int* s_i = reinterpret_cast<int*>(smem + 1120);          // [8]
  const uint32_t xs = smem_u32(smem + 1280);               // X as bf16 [M][K]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int V = p.N, K = p.K;
  const int row0 = blockIdx.x * kRowsPerCta + warp * 16;
  const bool active = row0 < V;
  const int nch = K / 32;

  pdl_launch_dependents();
  const int row_lo = min(row0 + g, V - 1), row_hi = min(row0 + g + 8, V - 1);
  const unsigned char* wlo = reinterpret_cast<const unsigned char*>(W + (size_t)row_lo * K) + t * 16;
  const unsigned char* whi = reinterpret_cast<const unsigned char*>(W + (size_t)row_hi * K) + t * 16;
  uint4 wb[kRing][2];
#pragma unroll
  for (int d = 0; d < kRing; ++d) {
    wb[d][0] = make_uint4(0u, 0u, 0u, 0u);
    wb[d][1] = make_uint4(0u, 0u, 0u, 0u);
    if (active && d < nch) {
      wb[d][0] = ldg_stream16(wlo + d * 64);
      wb[d][1] = ldg_stream16(whi + d * 64);
    }
  }

  pdl_wait_prior_grid();
  // X (after the optional add + RMSNorm) as bf16 in shared memory
  if (p.pro == kProAddRmsNorm) rmsnorm_factors<kThreads>(p, ss, inv, tid);
  for (int u = tid; u < p.M * (K / 8); u += kThreads) {
    const int m = u / (K / 8), k0 = (u - m * (K / 8)) * 8;
    sts128(xs + (m * K + k0) * 2, load_x_unit(p, m, k0, inv));
  }
  __syncthreads();

  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  if (active) {
    const bool bval = g < p.M;
    const uint32_t xaddr = xs + ((bval ? g : 0) * K + t * 8) * 2;
    for (int cc = 0; cc < nch; cc += kRing) {
#pragma unroll
      for (int d = 0; d < kRing; ++d) {
        const int c = cc + d;
        if (c < nch) {
          const uint4 lo = wb[d][0], hi = wb[d][1];
          if (c + kRing < nch) {
            wb[d][0] = ldg_stream16(wlo + (c + kRing) * 64);
            wb[d][1] = ldg_stream16(whi + (c + kRing) * 64);
          }
          uint4 x = make_uint4(0u, 0u, 0u, 0u);
          if (bval) x = lds128(xaddr + c * 64);
          mma_16816_bf16(acc, lo.x, hi.x, lo.y, hi.y, x.x, x.y);
          mma_16816_bf16(acc, lo.z, hi.z, lo.w, hi.w, x.z, x.w);
        }
      }
    }
  }

  // ---- epilogue: bf16 logits of every token; argmax of token 0 over the CTA's rows
  float best = -FLT_MAX;
  int bi = 0x7fffffff;
  if (active) {
    const int m0 = 2 * t;
    __nv_bfloat16* Y = p.Y;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int n = row0 + g + 8 * h;
      if (n < V) {
        const __nv_bfloat16 v0 = __float2bfloat16(acc[2 * h]), v1 = __float2bfloat16(acc[2 * h + 1]);
        if (Y != nullptr) {
          if (m0 < p.M) Y[(size_t)m0 * V + n] = v0;
          if (m0 + 1 < p.M) Y[(size_t)(m0 + 1) * V + n] = v1;
        }
        if (t == 0) {
          const float f = __bfloat162float(v0);
          if (f > best || (f == best && n < bi)) {
            best = f;
            bi = n;
          }
        }
      }
    }
  }
  if (part_v != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      s_v[warp] = best;
      s_i[warp] = bi;
    }
    __syncthreads();
    if (tid == 0) {
      for (int w = 1; w < 8; ++w)
        if (s_v[w] > best || (s_v[w] == best && s_i[w] < bi)) {
          best = s_v[w];
          bi = s_i[w];
        }
      part_v[blockIdx.x] = best;
      part_i[blockIdx.x] = bi == 0x7fffffff ? bi : bi + idx_offset;
    }
  }
}

}  // namespace

int lm_head_launch(const void* X, const void* W, void* logits, int M, int V, int K, const GemvPrologue& pro,
                   float* part_v, int* part_i, int idx_offset, cudaStream_t stream) {
  if (M < 1 || M > 8) return kErrUnsupportedM;
  if (V < 1 || K < 32 || K % 32) return kErrBadShape;
  if (!X || !W) return kErrBadPointer;
  if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 15) ||
      (reinterpret_cast<uintptr_t>(logits) & 1))
    return kErrBadPointer;
  if ((part_v == nullptr) != (part_i == nullptr)) return kErrBadPointer;
  if (pro.kind != kProNone && pro.kind != kProAddRmsNorm) return kErrBadShape;
  if (pro.kind == kProAddRmsNorm &&
      (!pro.Wn || (reinterpret_cast<uintptr_t>(pro.Wn) & 15) || (reinterpret_cast<uintptr_t>(pro.R) & 15) ||
       (reinterpret_cast<uintptr_t>(pro.Xout) & 15)))
    return kErrBadPointer;
  const size_t smem = 1280 + (size_t)M * K * 2;
  if (smem > 100 * 1024) return kErrTooLarge;
  GemvParams p{};
  p.X = static_cast<const __nv_bfloat16*>(X);
  p.Y = static_cast<__nv_bfloat16*>(logits);
  p.M = M; p.N = V; p.K = K;
  p.pro = pro.kind;
  p.R = static_cast<const __nv_bfloat16*>(pro.R);
  p.Wn = static_cast<const __nv_bfloat16*>(pro.Wn);
  p.Xout = static_cast<__nv_bfloat16*>(pro.Xout);
  p.eps = pro.eps;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(lm_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(lm_head_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return (int)e;
    if (dev >= 0 && dev < 64) attr_done[dev] = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((V + kRowsPerCta - 1) / kRowsPerCta);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, lm_head_kernel, p, static_cast<const __nv_bfloat16*>(W), part_v,
                                           part_i, idx_offset);
  return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

}  // namespace b2

extern "C" {

int b2_lm_head_blocks(int V) { return V < 1 ? 0 : (V + b2::kRowsPerCta - 1) / b2::kRowsPerCta; }

int b2_lm_head(const void* X, const void* W, void* logits, int M, int V, int K, int prologue, const void* R,
               const void* Wn, float eps, void* Xout, void* part_max, void* part_idx, int idx_offset, void* stream) {
  b2::GemvPrologue pro;
  pro.kind = prologue;
  pro.R = R;
  pro.Wn = Wn;
  pro.Xout = Xout;
  pro.eps = eps;
  return b2::lm_head_launch(X, W, logits, M, V, K, pro, static_cast<float*>(part_max), static_cast<int*>(part_idx),
                            idx_offset, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
