// bf16 vocabulary projection of the decode step with the greedy argmax in its epilogue:
//   logits[M, V] (bf16) = X[M, K] (bf16) . W[V, K]^T (bf16), fp32 accumulation, 1 <= M <= 8, K % 64 == 0;
//   per 128-row block the largest logit of token 0 and its index (lowest index on ties).
//
// The reference keeps the lm_head in bf16 and runs it through F.linear, then argmax on the host side of the step
// (python/nanoserve/qwen.py:164,174-177).  At batch 1 this is a 1.09 GB stream for the 152064 x 3584 Qwen2.5-7B
// head -- a quarter of the bytes of a W4 decode step -- so it gets the same treatment as the quantized GEMV:
// every warp owns 16 rows of W and a private ring of shared-memory slots (16 rows x 128 bytes: 64 values of K) that
// its own lanes fill with 16-byte cp.async copies, four rows x 128 bytes per warp instruction (whole lines), each
// slot completing on its own mbarrier; nobody waits for another warp.  (Loads straight into registers, 16 bytes of
// rows g and g + 8 per lane, moved half lines and kept few loads in flight: 3.0 TB/s on this matrix.)  The
// fragments of mma.sync.m16n8k16 (bf16, tokens in the columns) come out of the slot with 16-byte shared loads: the
// 16 bytes a lane reads are eight consecutive k; the contraction index of an mma is a dummy, so the B fragment is
// simply the same 16 bytes of X.  16-byte unit u of slot row r sits at u ^ ((r & 1) << 2), which keeps the eight
// lanes of a shared-memory phase (rows g, g + 1; units t) on different banks.  Two CTAs per SM, launched with
// programmatic stream serialization: the weight stream starts while the previous kernel drains, and a CTA's X
// staging hides behind the other CTA's stream.  The final residual add + RMSNorm of the model can be folded into
// the staging of X (same prologue as the GEMV).
#include <algorithm>
#include <cfloat>

#include "../../include/nanoserve_b200.h"
#include "w4_gemv_shared.cuh"

namespace b2 {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int kRowsPerCta = 128;
constexpr int kSlotBytes = 16 * 128;
constexpr int kMaxDepth = 6;
constexpr int kBarOffset = 1152;   // [kWarps][8] mbarriers
constexpr int kAbortOffset = 1664;
constexpr int kXOffset = 1792;     // X as bf16 [M][K], then the rings (128-byte aligned)
constexpr int kSmemTwoPerSm = 112 * 1024;

__global__ void __launch_bounds__(kThreads, 2)
    lm_head_kernel(const GemvParams p, const __nv_bfloat16* __restrict__ W, float* __restrict__ part_v,
                   int* __restrict__ part_i, int idx_offset, int depth) {
  extern __shared__ __align__(128) unsigned char smem[];
  float* ss = reinterpret_cast<float*>(smem);              // [16][16] RMSNorm partial sums
  float* inv = reinterpret_cast<float*>(smem + 1024);      // [16]
  float* s_v = reinterpret_cast<float*>(smem + 1088);      // [8] per-warp maxima
  int* s_i = reinterpret_cast<int*>(smem + 1120);          // [8]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kAbortOffset);
  const uint32_t xs = smem_u32(smem + kXOffset);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int V = p.N, K = p.K;
  const int row0 = blockIdx.x * kRowsPerCta + warp * 16;
  const bool active = row0 < V;
  const int nslots = K / 64;
  const uint32_t ring0 = xs + (((uint32_t)p.M * K * 2 + 127u) & ~127u) + warp * depth * kSlotBytes;
  const uint32_t bar0 = smem_u32(smem + kBarOffset) + warp * 64;

  pdl_launch_dependents();
  if (tid == 0) *abort_flag = 0;
  if (lane < depth) mbar_init(bar0 + 8 * lane, 32);
  fence_mbar_init();
  __syncwarp();

  // this lane's share of a slot: rows 4 j + (lane >> 3), j = 0..3, 16-byte unit lane & 7
  const int frow = lane >> 3, funit = lane & 7;
  const unsigned char* src = reinterpret_cast<const unsigned char*>(W) + funit * 16;
  const size_t row_bytes = (size_t)K * 2;
  const uint32_t fdst = frow * 128 + ((funit ^ ((frow & 1) << 2)) << 4);
  const bool whole = row0 + 16 <= V;
  auto feed = [&](int ks, int d) {
    const uint32_t slot = ring0 + d * kSlotBytes + fdst;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int row = row0 + 4 * j + frow;
      const bool ok = whole || row < V;
      const unsigned char* sp = src + (size_t)(ok ? row : row0) * row_bytes + (size_t)ks * 128;
      asm volatile("cp.async.cg.shared.global.L2::128B [%0], [%1], 16, %2;" ::"r"(slot + j * 512), "l"(sp),
                   "r"(ok ? 16u : 0u)
                   : "memory");
    }
    cp_async_mbar_arrive_noinc(bar0 + 8 * d);
  };
  if (active) {
    for (int d = 0; d < depth; ++d)
      if (d < nslots) feed(d, d);
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
    const uint32_t pg = (uint32_t)(g & 1) << 2;
    const uint32_t a_u0 = g * 128 + (((uint32_t)t ^ pg) << 4), a_u1 = g * 128 + (((uint32_t)(t + 4) ^ pg) << 4);
    int d = 0;
    uint32_t ph = 0;
    for (int ks = 0; ks < nslots; ++ks) {
      const uint32_t slot = ring0 + d * kSlotBytes;
      mbar_wait(bar0 + 8 * d, ph, abort_flag);
      const uint4 lo0 = lds128(slot + a_u0), hi0 = lds128(slot + 1024 + a_u0);
      const uint4 lo1 = lds128(slot + a_u1), hi1 = lds128(slot + 1024 + a_u1);
      __syncwarp();
      if (ks + depth < nslots) feed(ks + depth, d);
      uint4 x0 = make_uint4(0u, 0u, 0u, 0u), x1 = x0;
      if (bval) {
        x0 = lds128(xaddr + ks * 128);
        x1 = lds128(xaddr + ks * 128 + 64);
      }
      mma_16816_bf16(acc, lo0.x, hi0.x, lo0.y, hi0.y, x0.x, x0.y);
      mma_16816_bf16(acc, lo0.z, hi0.z, lo0.w, hi0.w, x0.z, x0.w);
      mma_16816_bf16(acc, lo1.x, hi1.x, lo1.y, hi1.y, x1.x, x1.y);
      mma_16816_bf16(acc, lo1.z, hi1.z, lo1.w, hi1.w, x1.z, x1.w);
      if (++d == depth) {
        d = 0;
        ph ^= 1;
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
  }
  __syncthreads();
  if (part_v != nullptr && tid == 0) {
    for (int w = 1; w < 8; ++w)
      if (s_v[w] > best || (s_v[w] == best && s_i[w] < bi)) {
        best = s_v[w];
        bi = s_i[w];
      }
    part_v[blockIdx.x] = best;
    part_i[blockIdx.x] = bi == 0x7fffffff ? bi : bi + idx_offset;
  }
  if (*abort_flag) {
    // a copy never completed: record it, and let what is in flight land before the shared memory is released
    if (tid == 0 && p.status != nullptr) atomicCAS(p.status, kStatusOk, kStatusGemvTimeout);
    cp_async_wait_all();
    __syncthreads();
  }
}

}  // namespace

int lm_head_launch(const void* X, const void* W, void* logits, int M, int V, int K, const GemvPrologue& pro,
                   float* part_v, int* part_i, int idx_offset, int* status, cudaStream_t stream) {
  if (M < 1 || M > 8) return kErrUnsupportedM;
  if (V < 1 || K < 64 || K % 64) return kErrBadShape;
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
  // as many slots per warp as fit beside X with two CTAs on an SM
  const size_t fixed = kXOffset + (((size_t)M * K * 2 + 127) & ~(size_t)127);
  if (fixed + (size_t)kWarps * 2 * kSlotBytes > (size_t)kSmemTwoPerSm) return kErrTooLarge;
  const int depth = (int)std::min<size_t>(kMaxDepth, (kSmemTwoPerSm - fixed) / ((size_t)kWarps * kSlotBytes));
  const size_t smem = fixed + (size_t)kWarps * depth * kSlotBytes;
  GemvParams p{};
  p.X = static_cast<const __nv_bfloat16*>(X);
  p.Y = static_cast<__nv_bfloat16*>(logits);
  p.M = M; p.N = V; p.K = K;
  p.pro = pro.kind;
  p.R = static_cast<const __nv_bfloat16*>(pro.R);
  p.Wn = static_cast<const __nv_bfloat16*>(pro.Wn);
  p.Xout = static_cast<__nv_bfloat16*>(pro.Xout);
  p.eps = pro.eps;
  p.status = status;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(lm_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTwoPerSm);
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
                                           part_i, idx_offset, depth);
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
  int rc = 0;
  int* status = b2::device_status_word(&rc);  // a copy that never completes is reported there (b2_device_status)
  if (!status) return rc;
  return b2::lm_head_launch(X, W, logits, M, V, K, pro, static_cast<float*>(part_max), static_cast<int*>(part_idx),
                            idx_offset, status, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
