// extern "C" entry points of libnanoserve.so (declared in include/nanoserve_b200.h).
//
// Plain pointers and sizes only; no PyTorch types.  Per-device state (SM count, scratch memory, status
// word) is created lazily under a mutex, once per device, with that device current.
#include <atomic>
#include <cstdio>
#include <mutex>

#include "../../include/nanoserve_b200.h"
#include "fused_ops.h"
#include "w4_internal.h"

namespace {

constexpr int kMaxDevices = 64;
constexpr size_t kPartialBytes = 96ull << 20;  // split-K partial sums (GEMM: two 256 KB part-tiles per SM)
constexpr int kCounters = 1 << 16;             // one per 32-row group: N up to 2 M rows
constexpr size_t kXStageBytes = 4ull << 20;    // X of a GEMV launch in its staged form: M * K up to 1.8 M values

struct DeviceState {
  std::atomic<bool> ready{false};  // release-stored once the fields below are final, acquire-loaded outside the mutex
  int sm_count = 0;
  b2::Workspace ws;
};
DeviceState g_dev[kMaxDevices];
std::mutex g_mu;

// Returns the state of the current device, creating it on first use.  rc receives 0 or an error code.
DeviceState* device_state(int* rc) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { *rc = (int)e; return nullptr; }
  if (dev < 0 || dev >= kMaxDevices) { *rc = b2::kErrTooLarge; return nullptr; }
  DeviceState& st = g_dev[dev];
  if (st.ready.load(std::memory_order_acquire)) { *rc = 0; return &st; }
  std::lock_guard<std::mutex> lock(g_mu);
  if (st.ready.load(std::memory_order_relaxed)) { *rc = 0; return &st; }
  e = cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) { *rc = (int)e; return nullptr; }
  void *partial = nullptr, *small = nullptr;
  e = cudaMalloc(&partial, kPartialBytes + kXStageBytes);
  if (e != cudaSuccess) { *rc = b2::kErrWorkspace; return nullptr; }
  e = cudaMalloc(&small, (kCounters + 64) * sizeof(int));
  if (e != cudaSuccess) { cudaFree(partial); *rc = b2::kErrWorkspace; return nullptr; }
  e = cudaMemset(small, 0, (kCounters + 64) * sizeof(int));
  if (e == cudaSuccess) e = cudaDeviceSynchronize();  // the memset is not ordered with non-blocking streams
  if (e != cudaSuccess) { cudaFree(partial); cudaFree(small); *rc = (int)e; return nullptr; }
  st.ws.partial = static_cast<float*>(partial);
  st.ws.partial_bytes = kPartialBytes;
  st.ws.xstage = static_cast<unsigned char*>(partial) + kPartialBytes;
  st.ws.xstage_bytes = kXStageBytes;
  st.ws.status = static_cast<int*>(small);          // word 0
  st.ws.counters = static_cast<int*>(small) + 64;   // 256-byte offset
  st.ws.n_counters = kCounters;
  st.ready.store(true, std::memory_order_release);
  *rc = 0;
  return &st;
}

// The state of the current device if it exists already; never creates it (the status calls must not allocate).
DeviceState* device_state_if_ready(int* dev_out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  *dev_out = dev;
  return g_dev[dev].ready.load(std::memory_order_acquire) ? &g_dev[dev] : nullptr;
}

}  // namespace

namespace b2 {
int* device_status_word(int* rc) {
  DeviceState* st = device_state(rc);
  return st ? st->ws.status : nullptr;
}
}  // namespace b2

namespace {

int linear_dispatch(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int G,
                    int flags, void* stream) {
  if (M < 1) return b2::kErrUnsupportedM;
  int rc = 0;
  DeviceState* st = device_state(&rc);
  if (!st) return rc;
  const auto s = static_cast<cudaStream_t>(stream);
  if (M <= 16) return b2::gemv_launch(X, Wq, S, Y, M, N, K, G, st->ws, flags, st->sm_count, s);
  return b2::gemm_launch(X, Wq, S, Y, M, N, K, G, st->ws, flags, st->sm_count, s);
}

// The public descriptor as the kernels take it.
int to_gemv_tp(const b2_tp_desc* tp, b2::GemvTp* out) {
  b2::GemvTp t;
  if (tp->world < 0 || tp->world > b2::kMaxTpRanks || tp->announce_world < 0 || tp->announce_world > b2::kMaxTpRanks)
    return b2::kErrBadShape;
  t.world = tp->world;
  for (int r = 0; r < tp->world; ++r) {
    t.y_peer[r] = tp->y_peer[r];
    t.sig_peer[r] = static_cast<unsigned*>(tp->sig_peer[r]);
  }
  t.ld = tp->ld;
  t.seg_end[0] = tp->seg_end[0];
  t.seg_end[1] = tp->seg_end[1];
  for (int i = 0; i < 3; ++i) t.seg_dst[i] = tp->seg_dst[i];
  t.wait_sig = static_cast<const unsigned*>(tp->wait_sig);
  t.epoch = static_cast<const int*>(tp->epoch);
  t.wait_per_epoch = tp->wait_per_epoch;
  t.defer = tp->defer_signal;
  t.announce_world = tp->announce_world;
  for (int r = 0; r < tp->announce_world; ++r) {
    if (!tp->announce_peer[r] || (reinterpret_cast<uintptr_t>(tp->announce_peer[r]) & 3)) return b2::kErrBadPointer;
    t.announce_peer[r] = static_cast<unsigned*>(tp->announce_peer[r]);
  }
  *out = t;
  return 0;
}

}  // namespace

extern "C" {

int ns_w4_linear(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int G,
                 void* stream) {
  return linear_dispatch(X, Wq, S, Y, M, N, K, G, 0, stream);
}

int b2_w4_linear(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int G,
                 int flags, void* stream) {
  return linear_dispatch(X, Wq, S, Y, M, N, K, G, flags, stream);
}

int b2_w4_linear_fused(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int G, int prologue,
                       const void* R, const void* Wn, float eps, void* Xout, int flags, void* stream) {
  if (M < 1 || M > 16) return b2::kErrUnsupportedM;
  int rc = 0;
  DeviceState* st = device_state(&rc);
  if (!st) return rc;
  b2::GemvPrologue pro;
  pro.kind = prologue & 0xFF;
  pro.epilogue = (prologue >> 8) & 0xFF;
  pro.R = R;
  pro.Wn = Wn;
  pro.Xout = Xout;
  pro.eps = eps;
  return b2::gemv_launch_ex(X, Wq, S, Y, M, N, K, G, pro, st->ws, flags, st->sm_count,
                            static_cast<cudaStream_t>(stream));
}

int b2_w4_linear_tp(const void* X, const void* Wq, const void* S, int M, int N, int K, int G, int prologue,
                    const void* R, const void* Wn, float eps, void* Xout, const b2_tp_desc* tp, int flags,
                    void* stream) {
  if (M < 1 || M > 16) return b2::kErrUnsupportedM;
  if (!tp) return b2::kErrBadPointer;
  int rc = 0;
  DeviceState* st = device_state(&rc);
  if (!st) return rc;
  b2::GemvPrologue pro;
  pro.kind = prologue & 0xFF;
  pro.epilogue = (prologue >> 8) & 0xFF;
  pro.R = R;
  pro.Wn = Wn;
  pro.Xout = Xout;
  pro.eps = eps;
  b2::GemvTp t;
  if (const int bad = to_gemv_tp(tp, &t)) return bad;
  if (tp->world == 0 && !tp->wait_sig) return b2::kErrBadShape;  // nothing tensor-parallel about this call
  void* y = tp->world > 0 ? tp->y_peer[0] : tp->y_local;
  return b2::gemv_launch_ex(X, Wq, S, y, M, N, K, G, pro, st->ws, flags, st->sm_count,
                            static_cast<cudaStream_t>(stream), &t);
}

size_t b2_w4_gemv_grid(int M, int N, int K, int G, int flags) {
  int rc = 0;
  DeviceState* st = device_state(&rc);
  if (!st) return 0;
  return b2::gemv_grid(M, N, K, G, flags, st->sm_count, st->ws.partial_bytes, st->ws.n_counters - 1);
}

int b2_w4_gemv_describe(int M, int N, int K, int G, int flags, char* buf, int buflen) {
  int rc = 0;
  DeviceState* st = device_state(&rc);
  if (!st) return rc;
  return b2::gemv_describe(M, N, K, G, flags, st->sm_count, st->ws.partial_bytes, st->ws.n_counters - 1, buf, buflen);
}

int b2_tp_wait(const void* wait_sig, const void* epoch, unsigned wait_per_epoch, void* stream) {
  int rc = 0;
  DeviceState* st = device_state(&rc);
  if (!st) return rc;
  return b2::tp_wait_launch(wait_sig, epoch, wait_per_epoch, st->ws.status, static_cast<cudaStream_t>(stream));
}

int b2_tp_wait_desc(const b2_tp_desc* tp, int advance_epoch, void* stream) {
  if (!tp) return b2::kErrBadPointer;
  int rc = 0;
  DeviceState* st = device_state(&rc);
  if (!st) return rc;
  b2::GemvTp t;
  if (const int bad = to_gemv_tp(tp, &t)) return bad;
  return b2::tp_wait_launch(tp->wait_sig, tp->epoch, tp->wait_per_epoch, st->ws.status,
                            static_cast<cudaStream_t>(stream), &t, advance_epoch);
}

int b2_rope_kv_store_tp(void* qkv, const void* bias, const void* inv_freq, const void* pos, void* cache_k,
                        void* cache_v, int Hq, int Hk, int D, int max_len, const void* wait_sig, const void* epoch,
                        unsigned wait_per_epoch, void* stream) {
  int rc = 0;
  DeviceState* st = device_state(&rc);
  if (!st) return rc;
  return b2::rope_kv_store_launch(qkv, bias, inv_freq, pos, cache_k, cache_v, Hq, Hk, D, max_len, wait_sig, epoch,
                                  wait_per_epoch, st->ws.status, static_cast<cudaStream_t>(stream));
}

int b2_decode_attention_fused(const void* qkv, const void* bias, const void* inv_freq, const void* pos, void* cache_k,
                              void* cache_v, void* out, void* workspace, int Hq, int Hk, int D, int max_len,
                              const b2_tp_desc* tp, int flags, void* stream) {
  int* status = nullptr;
  b2::GemvTp t;
  if (tp != nullptr) {  // only a wait can time out
    int rc = 0;
    DeviceState* st = device_state(&rc);
    if (!st) return rc;
    status = st->ws.status;
    if (const int bad = to_gemv_tp(tp, &t)) return bad;
  }
  return b2::decode_attention_fused_launch(qkv, bias, inv_freq, pos, cache_k, cache_v, out, workspace, Hq, Hk, D,
                                           max_len, tp != nullptr ? &t : nullptr, flags, status,
                                           static_cast<cudaStream_t>(stream));
}

int ns_w4_quantize(const void* W, void* Wq, void* S, int N, int K, int G, void* stream) {
  return b2::quantize_launch(W, Wq, S, N, K, G, static_cast<cudaStream_t>(stream));
}

int ns_rmsnorm(void* x, const void* r, const void* w, void* y, int T, int H, float eps, void* stream) {
  return b2::rmsnorm_launch(x, r, w, y, T, H, eps, static_cast<cudaStream_t>(stream));
}

int ns_rope(void* q, void* k, const void* inv_freq, int T, int Hq, int Hk, int D, int pos0,
            long long q_stride, long long k_stride, void* stream) {
  return b2::rope_launch(q, k, inv_freq, T, Hq, Hk, D, pos0, q_stride, k_stride,
                         static_cast<cudaStream_t>(stream));
}

int ns_swiglu(const void* gate, const void* up, void* out, int T, int I, void* stream) {
  return b2::swiglu_launch(gate, up, out, T, I, static_cast<cudaStream_t>(stream));
}

int ns_flash_fwd(const void*, const void*, const void*, void*, int, int, int, int, long long, long long,
                 long long, int, int, void*) {
  return b2::kErrNotImplemented;
}

int b2_init(void) {
  int rc = 0;
  device_state(&rc);
  return rc;
}

int b2_device_status(void) {
  int dev = -1;
  DeviceState* st = device_state_if_ready(&dev);
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return (int)e;
  int word = 0, word2 = 0;
  if (st) {
    e = cudaMemcpy(&word, st->ws.status, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return (int)e;
  }
  b2::noalloc_status_word(dev, &word2);  // the fixed array of b2_w4_gemv_noalloc, if that entry point has run
  return (word | word2) == 0 ? 0 : b2::kErrDevice;
}

int b2_clear_status(void) {
  int dev = -1;
  DeviceState* st = device_state_if_ready(&dev);
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return (int)e;
  // a time-out may have left arrival counters half counted: clear them with the status word
  if (st) e = cudaMemset(st->ws.status, 0, (kCounters + 64) * sizeof(int));
  b2::noalloc_clear(dev);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  return (int)e;
}

size_t b2_w4_gemv_scratch_bytes(int M, int N, int K, int G, int flags) {
  int rc = 0;
  DeviceState* st = device_state(&rc);
  if (!st) return 0;
  return b2::gemv_scratch_bytes(M, N, K, G, flags, st->sm_count, st->ws.partial_bytes);
}

const char* b2_version(void) { return "nanoserve-b200 0.1 sm_100a"; }

}  // extern "C"
