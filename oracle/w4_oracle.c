/*
 * CPU oracle for the W4A16 quantized-linear path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the host-side check the reference project runs
 * before it times its W4A16 kernels, plus the arithmetic of its quantizer and of
 * its deterministic test-input generator.  Nothing here is shipped or measured as
 * the product: only the test suite, the smoke check and the CPU-baseline leg of
 * the benchmark may call it.
 *
 * Parity status: PINNED.  tests/test_oracle.py checks this file against
 *   - the reference's recorded known answer for the RTN quantizer on its own
 *     seeded inputs (7.05 % relative Frobenius error; results/ncu/w4_gemv_m8.txt:11,
 *     produced by bench/bench_w4a16.cu:138-196), and
 *   - outputs of the reference's own kernels (ns_w4_quantize / ns_w4_linear built
 *     unchanged from csrc/nanoserve_ops.cu) captured on a B200 and committed under
 *     tests/golden/.
 *
 * Each function cites the reference lines it follows (paths inside the reference
 * project).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

/* ---- a minimal parallel-for over [0, n) with POSIX threads (no OpenMP dependency) ---- */
typedef void (*orc_body_fn)(int begin, int end, void* ctx);
typedef struct { orc_body_fn fn; void* ctx; int begin, end; } orc_task;
static void* orc_task_run(void* p) {
  orc_task* t = (orc_task*)p;
  t->fn(t->begin, t->end, t->ctx);
  return NULL;
}
static void orc_parallel_for(int n, int threads, orc_body_fn fn, void* ctx) {
  if (threads <= 1 || n <= 1) { fn(0, n, ctx); return; }
  if (threads > n) threads = n;
  if (threads > 256) threads = 256;
  pthread_t tid[256];
  orc_task task[256];
  for (int t = 0; t < threads; ++t) {
    task[t].fn = fn; task[t].ctx = ctx;
    task[t].begin = (int)((long long)n * t / threads);
    task[t].end = (int)((long long)n * (t + 1) / threads);
    if (pthread_create(&tid[t], NULL, orc_task_run, &task[t]) != 0) { /* run inline on failure */
      fn(task[t].begin, task[t].end, ctx);
      tid[t] = (pthread_t)0; task[t].fn = NULL;
    }
  }
  for (int t = 0; t < threads; ++t)
    if (task[t].fn) pthread_join(tid[t], NULL);
}

/* ---- bf16 <-> fp32, round-to-nearest-even (what __float2bfloat16 does) ---- */
static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff; /* NaN */
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

uint16_t orc_f32_to_bf16(float f) { return f32_to_bf16(f); }
float orc_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }

/*
 * Deterministic hash fill of a bf16 array: bench/bench_w4a16.cu:32-40 (fill_kernel).
 * Element i gets bf16( u * 1.732f * scale ), u uniform in [-1, 1) from a 32-bit mix of i.
 */
void orc_fill_bf16(uint16_t* p, size_t n, uint32_t seed, float scale) {
  for (size_t i = 0; i < n; ++i) {
    uint32_t h = (uint32_t)i * 2654435761u ^ seed;
    h ^= h >> 15; h *= 2246822519u; h ^= h >> 13; h *= 3266489917u; h ^= h >> 16;
    const float u = (float)(h & 0xFFFFFF) / 16777216.f * 2.f - 1.f;
    volatile float t = u * 1.732f; /* two separately rounded products, as on the device */
    p[i] = f32_to_bf16(t * scale);
  }
}

/*
 * RTN symmetric group quantizer: kernels/quant/w4a16.cuh:274-297 (quantize_w4_kernel).
 * Per (row, group): mx = max|w|; s = bf16(mx > 0 ? mx / 7 : 1); q = clamp(rint(w / s) + 8, 0, 15),
 * rint = round-half-even (__float2int_rn).  Word j of a row packs k = 8j..8j+7, value 8j+i in
 * bits 4i..4i+3 (w4a16.cuh:6).  Returns -1 for the shapes ns_w4_quantize rejects
 * (csrc/nanoserve_ops.cu:67).
 */
int orc_w4_quantize(const uint16_t* W, uint32_t* Wq, uint16_t* S, int N, int K, int G) {
  if (G <= 0 || K % G || G % 32) return -1;
  const int KG = K / G;
  for (int n = 0; n < N; ++n)
    for (int g = 0; g < KG; ++g) {
      const uint16_t* w = W + (size_t)n * K + (size_t)g * G;
      float mx = 0.f;
      for (int i = 0; i < G; ++i) mx = fmaxf(mx, fabsf(bf16_to_f32(w[i])));
      const uint16_t sb = f32_to_bf16(mx > 0.f ? mx / 7.f : 1.f);
      const float sf = bf16_to_f32(sb);
      S[(size_t)n * KG + g] = sb;
      for (int j = 0; j < G / 8; ++j) {
        uint32_t word = 0;
        for (int i = 0; i < 8; ++i) {
          const float r = bf16_to_f32(w[j * 8 + i]) / sf;
          int q = (int)lrintf(r) + 8; /* default rounding mode: nearest-even */
          q = q < 0 ? 0 : (q > 15 ? 15 : q);
          word |= (uint32_t)q << (4 * i);
        }
        Wq[(size_t)n * (K / 8) + (size_t)g * (G / 8) + j] = word;
      }
    }
  return 0;
}

/*
 * Host dequantisation "exactly as the kernels see" the packed bits:
 * bench/bench_w4a16.cu:156-162.  Wd[n,k] = (q - 8) * float(S[n, k/G]) in fp32 (exact product).
 */
void orc_w4_dequant(const uint32_t* Wq, const uint16_t* S, int N, int K, int G, float* Wd) {
  const int KG = K / G;
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) {
      const uint32_t word = Wq[(size_t)n * (K / 8) + k / 8];
      const int q = (word >> (4 * (k % 8))) & 0xF;
      Wd[(size_t)n * K + k] = (float)(q - 8) * bf16_to_f32(S[(size_t)n * KG + k / G]);
    }
}

/* The integer the format stores at (n, k), minus the fixed zero-point 8 (w4a16.cuh:6-8). */
void orc_w4_unpack(const uint32_t* Wq, int N, int K, int8_t* Q) {
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) {
      const uint32_t word = Wq[(size_t)n * (K / 8) + k / 8];
      Q[(size_t)n * K + k] = (int8_t)(((word >> (4 * (k % 8))) & 0xF) - 8);
    }
}

/*
 * Dequant-then-matmul check: bench/bench_w4a16.cu:156-173 (dequantise, then cpu_ref).  Y[m,n] =
 * float( sum_k double(float(X[m,k])) * Wd[n,k] ), double accumulation in ascending k.
 * threads <= 1 runs the loops exactly as the reference does (single thread); threads > 1
 * splits the n loop over POSIX threads (same per-element arithmetic, so the same result).
 * Returns the thread count used, or -1 when out of memory.
 */
typedef struct {
  const uint32_t* Wq; const uint16_t* S; const float* Xf; float* Wd; float* Y;
  int M, N, K, G;
} orc_lin_ctx;
static void orc_lin_body(int n0, int n1, void* p) {
  const orc_lin_ctx* c = (const orc_lin_ctx*)p;
  const int K = c->K, KG = c->K / c->G;
  for (int n = n0; n < n1; ++n)
    for (int k = 0; k < K; ++k) {
      const uint32_t word = c->Wq[(size_t)n * (K / 8) + k / 8];
      const int q = (word >> (4 * (k % 8))) & 0xF;
      c->Wd[(size_t)n * K + k] = (float)(q - 8) * bf16_to_f32(c->S[(size_t)n * KG + k / c->G]);
    }
  for (int n = n0; n < n1; ++n)
    for (int m = 0; m < c->M; ++m) {
      double acc = 0;
      const float* x = c->Xf + (size_t)m * K;
      const float* w = c->Wd + (size_t)n * K;
      for (int k = 0; k < K; ++k) acc += (double)x[k] * w[k];
      c->Y[(size_t)m * c->N + n] = (float)acc;
    }
}
int orc_w4_linear_f32(const uint16_t* X, const uint32_t* Wq, const uint16_t* S, float* Y, int M,
                      int N, int K, int G, int threads) {
  float* Wd = (float*)malloc((size_t)N * K * sizeof(float));
  float* Xf = (float*)malloc((size_t)M * K * sizeof(float));
  if (!Wd || !Xf) { free(Wd); free(Xf); return -1; }
  for (size_t i = 0; i < (size_t)M * K; ++i) Xf[i] = bf16_to_f32(X[i]);
  orc_lin_ctx c = {Wq, S, Xf, Wd, Y, M, N, K, G};
  const int used = threads > 1 ? (threads > N ? N : threads) : 1;
  orc_parallel_for(N, used, orc_lin_body, &c);
  free(Wd);
  free(Xf);
  return used;
}

/* Same, rounded once to bf16: what ns_w4_linear stores (csrc/nanoserve_ops.cu:75-90, w4a16.cuh:26). */
int orc_w4_linear_bf16(const uint16_t* X, const uint32_t* Wq, const uint16_t* S, uint16_t* Y, int M,
                       int N, int K, int G, int threads) {
  float* Yf = (float*)malloc((size_t)M * N * sizeof(float));
  if (!Yf) return -1;
  const int used = orc_w4_linear_f32(X, Wq, S, Yf, M, N, K, G, threads);
  for (size_t i = 0; i < (size_t)M * N; ++i) Y[i] = f32_to_bf16(Yf[i]);
  free(Yf);
  return used;
}

/*
 * The tensor-core path rounds each dequantised weight to bf16 before the multiply
 * (w4a16.cuh:196-197 with kernels/fused/vec.cuh:14-19); this is that tile value.
 */
void orc_w4_dequant_bf16(const uint32_t* Wq, const uint16_t* S, int N, int K, int G, uint16_t* Wd) {
  const int KG = K / G;
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) {
      const uint32_t word = Wq[(size_t)n * (K / 8) + k / 8];
      const int q = (word >> (4 * (k % 8))) & 0xF;
      Wd[(size_t)n * K + k] = f32_to_bf16((float)(q - 8) * bf16_to_f32(S[(size_t)n * KG + k / G]));
    }
}

/* Dense bf16-weight linear in double: the un-quantised comparison of bench_w4a16.cu:192-196. */
typedef struct { const uint16_t* X; const uint16_t* W; float* Y; int M, N, K; } orc_dense_ctx;
static void orc_dense_body(int n0, int n1, void* p) {
  const orc_dense_ctx* c = (const orc_dense_ctx*)p;
  for (int n = n0; n < n1; ++n)
    for (int m = 0; m < c->M; ++m) {
      double acc = 0;
      for (int k = 0; k < c->K; ++k)
        acc += (double)bf16_to_f32(c->X[(size_t)m * c->K + k]) * bf16_to_f32(c->W[(size_t)n * c->K + k]);
      c->Y[(size_t)m * c->N + n] = (float)acc;
    }
}
int orc_max_threads(void);
void orc_dense_linear_f32(const uint16_t* X, const uint16_t* W, float* Y, int M, int N, int K) {
  orc_dense_ctx c = {X, W, Y, M, N, K};
  orc_parallel_for(N, orc_max_threads(), orc_dense_body, &c);
}

/* Largest |a - ref| relative to the largest |ref|: bench/bench_w4a16.cu:94-103. */
float orc_max_rel_err(const float* a, const float* ref, size_t n) {
  float scale = 0.f;
  for (size_t i = 0; i < n; ++i) scale = fmaxf(scale, fabsf(ref[i]));
  float w = 0.f;
  for (size_t i = 0; i < n; ++i) {
    if (!isfinite(a[i])) return INFINITY;
    w = fmaxf(w, fabsf(a[i] - ref[i]) / (scale + 1e-6f));
  }
  return w;
}

/* Relative Frobenius error: bench/bench_w4a16.cu:104-111. */
float orc_rel_fro(const float* a, const float* ref, size_t n) {
  double num = 0, den = 0;
  for (size_t i = 0; i < n; ++i) {
    num += (double)(a[i] - ref[i]) * (a[i] - ref[i]);
    den += (double)ref[i] * ref[i];
  }
  return (float)sqrt(num / den);
}

int orc_max_threads(void) {
  const long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n > 0 ? (int)n : 1;
}
