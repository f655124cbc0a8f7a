// Host launchers of the small element-wise operators that sit either side of every quantized linear in
// a decoder layer (residual add + RMSNorm, rotary embedding, SwiGLU).
#pragma once
#include <cuda_runtime.h>

namespace b2 {
int rmsnorm_launch(void* x, const void* r, const void* w, void* y, int T, int H, float eps, cudaStream_t s);
int rope_launch(void* q, void* k, const void* inv_freq, int T, int Hq, int Hk, int D, int pos0,
                long long q_stride, long long k_stride, cudaStream_t s);
int swiglu_launch(const void* gate, const void* up, void* out, int T, int I, cudaStream_t s);
}  // namespace b2
