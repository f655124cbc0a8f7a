// Round-to-nearest symmetric 4-bit group quantizer (cold path: runs once per weight matrix).
//
// Same arithmetic, bit for bit, as the reference's quantize_w4_kernel (kernels/quant/w4a16.cuh:274-297):
//   per (row, group): mx = max|w|;  s = bf16_rn(mx > 0 ? mx / 7 : 1);  q = clamp(rint_even(w / float(s)) + 8, 0, 15)
// with IEEE fp32 division.  The reference walks a group with one thread; here one warp owns a group,
// each lane converts whole 8-element words from 16-byte loads, and the maximum is a shuffle reduction
// (max is order-independent, so the result is identical).
#include <algorithm>

#include "ptx.cuh"
#include "w4_internal.h"

namespace b2 {
namespace {

__global__ void __launch_bounds__(256) w4_quantize_kernel(const __nv_bfloat16* __restrict__ W,
                                                          uint32_t* __restrict__ Wq,
                                                          __nv_bfloat16* __restrict__ S, int N, int K, int G) {
  const int KG = K / G;
  const int lane = threadIdx.x & 31;
  const size_t total = (size_t)N * KG;
  const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
  for (size_t idx = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; idx < total; idx += warps) {
    const size_t n = idx / KG;
    const int g = (int)(idx - n * KG);
    const __nv_bfloat16* w = W + n * K + (size_t)g * G;
    const int words = G / 8;
    float mx = 0.f;
    for (int j = lane; j < words; j += 32) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(w) + j);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        mx = fmaxf(mx, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const __nv_bfloat16 sb = __float2bfloat16(mx > 0.f ? __fdiv_rn(mx, 7.f) : 1.f);
    const float sf = __bfloat162float(sb);
    if (lane == 0) S[idx] = sb;
    for (int j = lane; j < words; j += 32) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(w) + j);
      const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v);
      uint32_t word = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int q = min(15, max(0, __float2int_rn(__fdiv_rn(__bfloat162float(e[i]), sf)) + 8));
        word |= static_cast<uint32_t>(q) << (4 * i);
      }
      Wq[n * (K / 8) + (size_t)g * words + j] = word;
    }
  }
}

}  // namespace

int quantize_launch(const void* W, void* Wq, void* S, int N, int K, int G, cudaStream_t stream) {
  if (G <= 0 || K <= 0 || N <= 0 || K % G || G % 32) return kErrBadShape;
  if (!W || !Wq || !S) return kErrBadPointer;
  // 16-byte loads of W need 16-byte aligned rows and groups: K % 8 == 0 follows from G % 32 == 0
  if (reinterpret_cast<uintptr_t>(W) & 15) return kErrBadPointer;
  const size_t groups = (size_t)N * (K / G);
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1)
    return kErrDevice;
  const size_t blocks = std::min<size_t>((groups + 7) / 8, (size_t)sms * 32);  // grid-stride: 32 CTAs per SM at most
  w4_quantize_kernel<<<(unsigned)blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(W),
                                                          static_cast<uint32_t*>(Wq),
                                                          static_cast<__nv_bfloat16*>(S), N, K, G);
  return (int)cudaGetLastError();
}

}  // namespace b2
