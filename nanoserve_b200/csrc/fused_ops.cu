// Element-wise neighbours of the quantized linears: residual add + RMSNorm, rotary position embedding
// and SwiGLU, with the semantics of the reference's ns_rmsnorm / ns_rope / ns_swiglu
// (csrc/nanoserve_ops.cu:21-45; kernels/fused/rmsnorm.cuh:11-52, rope.cuh:14-43, swiglu.cuh:35-52):
// bf16 in and out, fp32 arithmetic, the residual stream rounded to bf16 before it is normalised.
// All three are bandwidth-trivial at decode sizes; they exist so a decoder step needs no other library.
#include <cstdint>
#include <cuda_bf16.h>

#include "fused_ops.h"
#include "w4_internal.h"

namespace b2 {
namespace {

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

// One CTA per token row.  Pass 1 forms x + r (rounded to bf16, written back) and the sum of squares;
// pass 2 re-reads the row (the CTA's own writes, still in L1/L2) and scales it.
__global__ void __launch_bounds__(512) rmsnorm_kernel(__nv_bfloat16* __restrict__ x,
                                                      const __nv_bfloat16* __restrict__ r,
                                                      const __nv_bfloat16* __restrict__ w,
                                                      __nv_bfloat16* __restrict__ y, int H, float eps) {
  __shared__ float warp_part[16];
  __shared__ float total;
  const size_t row = blockIdx.x;
  __nv_bfloat16* xr = x + row * H;
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float a[8];
    load8(xr + i, a);
    if (r != nullptr) {
      float b[8];
      load8(r + row * H + i, b);
#pragma unroll
      for (int e = 0; e < 8; ++e) a[e] = __bfloat162float(__float2bfloat16(a[e] + b[e]));
      store8(xr + i, a);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += a[e] * a[e];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? warp_part[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (threadIdx.x == 0) total = v;
  }
  __syncthreads();
  const float inv = rsqrtf(total / H + eps);
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float a[8], g[8];
    load8(xr + i, a);
    load8(w + i, g);
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = a[e] * inv * g[e];
    store8(y + row * H + i, a);
  }
}

// One thread rotates eight (i, i + D/2) pairs of one head of one token, angle = (pos0 + t) * inv_freq[i].
__global__ void __launch_bounds__(256) rope_kernel(__nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k,
                                                   const float* __restrict__ inv_freq, int T, int Hq, int Hk,
                                                   int D, int pos0, long long q_stride, long long k_stride) {
  const int per_head = D / 16;
  const long long total = (long long)T * (Hq + Hk) * per_head;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(idx % per_head);
    const long long ht = idx / per_head;
    const int h = (int)(ht % (Hq + Hk));
    const int t = (int)(ht / (Hq + Hk));
    __nv_bfloat16* head = h < Hq ? q + t * q_stride + (long long)h * D : k + t * k_stride + (long long)(h - Hq) * D;
    float lo[8], hi[8];
    load8(head + c * 8, lo);
    load8(head + D / 2 + c * 8, hi);
    const float pos = (float)(pos0 + t);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float sn, cs;
      sincosf(pos * inv_freq[c * 8 + e], &sn, &cs);
      const float a = lo[e], b = hi[e];
      lo[e] = a * cs - b * sn;
      hi[e] = b * cs + a * sn;
    }
    store8(head + c * 8, lo);
    store8(head + D / 2 + c * 8, hi);
  }
}

__global__ void __launch_bounds__(256) swiglu_kernel(const __nv_bfloat16* __restrict__ gate,
                                                     const __nv_bfloat16* __restrict__ up,
                                                     __nv_bfloat16* __restrict__ out, size_t n8) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float g[8], u[8];
    load8(gate + i * 8, g);
    load8(up + i * 8, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) g[e] = g[e] / (1.f + __expf(-g[e])) * u[e];
    store8(out + i * 8, g);
  }
}

// The kernels above load and store 16 bytes at a time: a pointer that is not 16-byte aligned (a view into the middle
// of a row) would fault on the device, so it is refused on the host instead.
bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

unsigned blocks_for(size_t n, int block) {
  const size_t b = (n + block - 1) / block;
  return (unsigned)(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

}  // namespace

int rmsnorm_launch(void* x, const void* r, const void* w, void* y, int T, int H, float eps, cudaStream_t s) {
  if (T < 1 || H < 8 || H % 8) return kErrBadShape;
  if (!x || !w || !y) return kErrBadPointer;
  if (!aligned16(x) || !aligned16(r) || !aligned16(w) || !aligned16(y)) return kErrBadPointer;
  const int threads = H >= 4096 ? 512 : 256;
  rmsnorm_kernel<<<T, threads, 0, s>>>(static_cast<__nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(r),
                                       static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), H,
                                       eps);
  return (int)cudaGetLastError();
}

int rope_launch(void* q, void* k, const void* inv_freq, int T, int Hq, int Hk, int D, int pos0,
                long long q_stride, long long k_stride, cudaStream_t s) {
  if (T < 1 || D < 16 || D % 16 || Hq < 0 || Hk < 0 || q_stride % 8 || k_stride % 8) return kErrBadShape;
  if (!q || !k || !inv_freq) return kErrBadPointer;
  if (!aligned16(q) || !aligned16(k) || (reinterpret_cast<uintptr_t>(inv_freq) & 3)) return kErrBadPointer;
  const size_t total = (size_t)T * (Hq + Hk) * (D / 16);
  rope_kernel<<<blocks_for(total, 256), 256, 0, s>>>(static_cast<__nv_bfloat16*>(q),
                                                     static_cast<__nv_bfloat16*>(k),
                                                     static_cast<const float*>(inv_freq), T, Hq, Hk, D, pos0,
                                                     q_stride, k_stride);
  return (int)cudaGetLastError();
}

int swiglu_launch(const void* gate, const void* up, void* out, int T, int I, cudaStream_t s) {
  if (T < 1 || I < 1 || ((long long)T * I) % 8) return kErrBadShape;  // reference: -1 (nanoserve_ops.cu:39)
  if (!gate || !up || !out) return kErrBadPointer;
  if (!aligned16(gate) || !aligned16(up) || !aligned16(out)) return kErrBadPointer;
  const size_t n8 = (size_t)T * I / 8;
  swiglu_kernel<<<blocks_for(n8, 256), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(gate),
                                                    static_cast<const __nv_bfloat16*>(up),
                                                    static_cast<__nv_bfloat16*>(out), n8);
  return (int)cudaGetLastError();
}

}  // namespace b2
