// b2_w4_gemv_noalloc: the decode GEMV for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc where they call the GEMV: a serving process that
// hands its whole device-memory budget to a pool at start-up and forbids later driver allocations, a
// plugin running inside another runtime's stream callback or capture region, a real-time loop that must
// not take the allocator's lock.  For them the scratch memory the split-K path needs (fp32 partial sums,
// one arrival counter per 32-row group, a status word) lives in a fixed array in the library's own
// device image instead of in memory obtained at run time.  Every GPU that loads the library carries the
// array (8 MiB + 16 KiB + 256 B) until the process exits, whether or not this entry point is used.
//
// Rules that follow from sharing one array:
//   * Calls on one device share it.  Two calls whose kernels overlap in time (different streams, or
//     graph branches) race on the partial sums and counters; serialise them on one stream.
//   * The array keeps what the previous call left.  The counters must be zero when a launch starts; a
//     launch leaves them zero, and each call clears them again on its stream before the launch in case an
//     earlier launch was cut short.  Partial sums are always written before they are read.
//   * The first call on a device looks up the array's device address (once per device, with that device
//     current).  It allocates nothing, but it is set-up work: make that first call before any stream
//     capture.
#include <atomic>
#include <mutex>

#include "../../include/nanoserve_b200.h"
#include "w4_internal.h"

namespace {

constexpr size_t kPartialBytes = 8ull << 20;  // 2 Mi floats of split-K partial sums
constexpr int kCounters = 4096;               // row groups of 32: N up to 131072
constexpr size_t kCountersOffset = kPartialBytes;
constexpr size_t kStatusOffset = kCountersOffset + kCounters * sizeof(int);
constexpr size_t kScratchBytes = kStatusOffset + 256;
constexpr long long kMaxOutputs = 1 << 20;    // M * N: two K slices of fp32 partial sums fit in the 8 MiB
constexpr int kMaxDevices = 64;

// In host code this name is only a handle for the runtime (cudaGetSymbolAddress); it is not a device
// address and must never be passed to a kernel.
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

struct DeviceSlot {
  std::atomic<bool> ready{false};  // release-stored after base and sm_count, acquire-loaded outside the mutex
  unsigned char* base = nullptr;  // device address of g_scratch on this device
  int sm_count = 0;
};
DeviceSlot g_slot[kMaxDevices];
std::mutex g_mu;

}  // namespace

namespace b2 {

// The status word of the fixed scratch array of device `dev`, for b2_device_status / b2_clear_status: they must not
// allocate either, so they read this word directly instead of creating the library's malloc'ed per-device state.
// Returns false when b2_w4_gemv_noalloc has not run on the device (nothing to report).  The caller has synchronised.
bool noalloc_status_word(int dev, int* word) {
  if (dev < 0 || dev >= kMaxDevices || !g_slot[dev].ready.load(std::memory_order_acquire)) return false;
  return cudaMemcpy(word, g_slot[dev].base + kStatusOffset, sizeof(int), cudaMemcpyDeviceToHost) == cudaSuccess;
}
// Clears that word and the arrival counters (a time-out may have left them half counted).
bool noalloc_clear(int dev) {
  if (dev < 0 || dev >= kMaxDevices || !g_slot[dev].ready.load(std::memory_order_acquire)) return false;
  return cudaMemset(g_slot[dev].base + kCountersOffset, 0, kCounters * sizeof(int) + 256) == cudaSuccess;
}

}  // namespace b2

extern "C" int b2_w4_gemv_noalloc(const void* X, const void* Wq, const void* S, void* Y, int M, int N, int K, int G,
                                  void* stream) {
  if (M < 1 || M > 16) return b2::kErrUnsupportedM;
  if (N < 1 || K < 32 || G < 32 || K % 32 || G % 32 || K % G) return b2::kErrBadShape;
  if ((long long)M * N > kMaxOutputs || (N + 31) / 32 > kCounters) return b2::kErrTooLarge;

  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return b2::kErrTooLarge;
  DeviceSlot& slot = g_slot[dev];
  if (!slot.ready.load(std::memory_order_acquire)) {
    std::lock_guard<std::mutex> lock(g_mu);
    if (!slot.ready.load(std::memory_order_relaxed)) {
      void* ptr = nullptr;
      e = cudaGetSymbolAddress(&ptr, g_scratch);  // device `dev` is current: this is its copy of the array
      if (e != cudaSuccess) return (int)e;
      e = cudaDeviceGetAttribute(&slot.sm_count, cudaDevAttrMultiProcessorCount, dev);
      if (e != cudaSuccess) return (int)e;
      slot.base = static_cast<unsigned char*>(ptr);
      // the status word starts at zero with the image; clear it anyway, on the caller's stream, before first use
      e = cudaMemsetAsync(slot.base + kStatusOffset, 0, sizeof(int), static_cast<cudaStream_t>(stream));
      if (e != cudaSuccess) return (int)e;
      slot.ready.store(true, std::memory_order_release);
    }
  }

  const auto st = static_cast<cudaStream_t>(stream);
  b2::Workspace ws;
  ws.partial = reinterpret_cast<float*>(slot.base);
  ws.partial_bytes = kPartialBytes;
  ws.counters = reinterpret_cast<int*>(slot.base + kCountersOffset);
  ws.n_counters = kCounters;
  ws.status = reinterpret_cast<int*>(slot.base + kStatusOffset);
  e = cudaMemsetAsync(ws.counters, 0, kCounters * sizeof(int), st);
  if (e != cudaSuccess) return (int)e;
  return b2::gemv_launch(X, Wq, S, Y, M, N, K, G, ws, b2::kFlagNoAutotune, slot.sm_count, st);  // no events, no sync
}
