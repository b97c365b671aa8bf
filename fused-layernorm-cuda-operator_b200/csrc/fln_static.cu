// LayerNorm backward for callers that are not allowed to allocate device memory.
//
// Who that is: a host that runs inside a fixed memory plan -- an inference server or a
// plugin runtime that hands out all device memory at start-up and forbids cudaMalloc
// afterwards, a control loop that cannot afford the device-wide synchronization cudaMalloc
// and cudaFree imply, or plain C code that has no caching allocator to lean on.  The regular
// backward needs a scratch buffer for the per-CTA partial sums of dgamma / dbeta and leaves
// providing it to the caller; this entry point brings its own.
//
// The scratch is one file-scope __device__ array of FLN_STATIC_SCRATCH_BYTES.  It is part of
// the library image: every GPU on which the library gets loaded carries it until the
// process exits, whether or not this function is ever called.
//
// In host code the name of a __device__ array is only a host-side handle, not an address the
// GPU can use, so the device address is looked up with cudaGetSymbolAddress -- once per
// device, with that device current, on the first call made for it.
#include <atomic>
#include <mutex>

#include "fln_common.cuh"

namespace {

static __device__ __align__(256) unsigned char g_static_scratch[FLN_STATIC_SCRATCH_BYTES];

// what the entry point accepts; tests lower it to see the refusal (fln_set_static_scratch_limit)
std::atomic<size_t> g_scratch_limit{FLN_STATIC_SCRATCH_BYTES};

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_addr[kMaxDevices] = {};

// Device address of the scratch array on the current device; nullptr if it cannot be had.
void* scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    cudaGetLastError();
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();
      return nullptr;
    }
    g_scratch_addr[dev] = ptr;
  }
  return g_scratch_addr[dev];
}

}  // namespace

extern "C" int fln_layernorm_backward_static(const void* dy, const void* x, const float* mean,
                                             const float* rstd, const void* gamma, void* dx,
                                             void* dgamma, void* dbeta, int64_t rows, int64_t cols,
                                             int dtype, void* stream) {
  if (rows < 0 || cols <= 0 || cols > 0x7fffffff || rows > 0x7fffffff) return FLN_ERR_SHAPE;
  if (dtype != FLN_F32 && dtype != FLN_BF16 && dtype != FLN_F16) return FLN_ERR_DTYPE;
  // the same sizing rule as the regular entry point, checked against the fixed capacity
  const size_t need = fln_backward_workspace_bytes(rows, cols, dtype);
  if (need > g_scratch_limit.load(std::memory_order_relaxed)) return FLN_ERR_STATIC_SCRATCH;
  void* scratch = scratch_for_current_device();
  if (scratch == nullptr) return FLN_ERR_LAUNCH;
  // Nothing in the scratch has to start at zero: stage 1 overwrites every partial row that
  // stage 2 reads, so whatever the previous call left behind is never observed.
  return fln_norm_backward(FLN_LAYERNORM, dy, x, mean, rstd, gamma, nullptr, dx, dgamma, dbeta,
                           nullptr, scratch, (size_t)FLN_STATIC_SCRATCH_BYTES, rows, cols, dtype,
                           stream);
}

extern "C" void fln_set_static_scratch_limit(size_t bytes) {
  // never beyond the array itself; 0 restores the full capacity
  if (bytes == 0 || bytes > (size_t)FLN_STATIC_SCRATCH_BYTES) bytes = FLN_STATIC_SCRATCH_BYTES;
  g_scratch_limit.store(bytes, std::memory_order_relaxed);
}
