// Device helpers shared by the W4A16 kernels: the packed-int4 format and its unpack.
//
// Format (fixed by the operator boundary; reference kernels/quant/w4a16.cuh:5-9):
//   Wq [N, K/8] uint32, word j of row n packs k = 8j..8j+7, value 8j+i in bits 4i..4i+3
//   S  [N, K/G] bf16,   w[n,k] = (q - 8) * S[n, k/G]
#pragma once
#include <cstdint>
#include <cuda_bf16.h>

namespace b2 {

// bf16 bit patterns used by the unpack: 0x4300 = 128.0 (exponent 2^7, so the 7 mantissa bits count
// in units of 1), 0x4308 = 136.0 = 128 + the zero-point 8.
constexpr uint32_t kMagic128x2 = 0x43004300u;
constexpr uint32_t kMagic136x2 = 0x43084308u;
constexpr uint32_t kNibblePairMask = 0x000F000Fu;

// One packed word -> four bf16x2 registers holding 128 + q, with the pairing the bit layout gives for
// free: r[p] = { 128 + q[p] (low half), 128 + q[p + 4] (high half) }, p = 0..3.  Three shifts and four
// three-input logic ops per eight weights; the integers 128..143 are exact in bf16.
__device__ __forceinline__ void unpack_w4_biased(uint32_t w, uint32_t (&r)[4]) {
  r[0] = (w & kNibblePairMask) | kMagic128x2;
  r[1] = ((w >> 4) & kNibblePairMask) | kMagic128x2;
  r[2] = ((w >> 8) & kNibblePairMask) | kMagic128x2;
  r[3] = ((w >> 12) & kNibblePairMask) | kMagic128x2;
}

// (a & b) | c as one LOP3; pass the constants in registers (two immediates would cost two instructions).
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// bf16x2 subtract of 136: (128 + q) - 136 = q - 8, exact.
__device__ __forceinline__ uint32_t sub136_bf16x2(uint32_t v) {
  __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&v);
  const uint32_t c = kMagic136x2;
  a = __hsub2(a, *reinterpret_cast<const __nv_bfloat162*>(&c));
  return *reinterpret_cast<uint32_t*>(&a);
}
// bf16x2 multiply (round-to-nearest-even per half).
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t v, uint32_t s2) {
  __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&v);
  a = __hmul2(a, *reinterpret_cast<const __nv_bfloat162*>(&s2));
  return *reinterpret_cast<uint32_t*>(&a);
}
__device__ __forceinline__ uint32_t bf16_dup(__nv_bfloat16 s) {
  const uint32_t b = __bfloat16_as_ushort(s);
  return b | (b << 16);
}

// 16-byte shared-memory accesses by 32-bit shared address.
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

}  // namespace b2
