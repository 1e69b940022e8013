// Per-device one-time set-up for host launch code. Function attributes such as the dynamic
// shared-memory limit (cudaFuncSetAttribute) and properties such as the SM count belong to a
// device, not to the process: a program that drives several GPUs from one process has to apply
// them once on each. `run(f)` calls `f` the first time it is reached with a given device current
// (f must be idempotent: two threads may both run it) and remembers success per device.
#pragma once
#include <atomic>
#include <cuda_runtime.h>

namespace bdh {

struct PerDeviceOnce {
  static constexpr int MAX_DEVICES = 64;
  std::atomic<unsigned long long> done{0};
  template <class F>
  int run(F&& f) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return f();
    const unsigned long long bit = 1ull << dev;
    if (done.load(std::memory_order_acquire) & bit) return 0;
    const int rc = f();
    if (rc == 0) done.fetch_or(bit, std::memory_order_release);
    return rc;
  }
};

// cuTensorMapEncodeTiled is a driver call and needs the device's primary context to be current on the
// calling thread. The runtime binds it lazily, on a thread's first runtime call that needs it - and a
// worker thread (an autograd engine thread, say) may reach a tensor-map encode before it has made one:
// the encode then fails with CUDA_ERROR_INVALID_CONTEXT. cudaFree(nullptr) is the documented no-op that
// forces the binding; it is done once per thread and device.
inline void bind_primary_context() {
  static thread_local unsigned long long bound = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= PerDeviceOnce::MAX_DEVICES) return;
  if (bound & (1ull << dev)) return;
  cudaFree(nullptr);
  bound |= 1ull << dev;
}

// SM count of the current device (cached per device).
inline int current_device_sms() {
  static std::atomic<int> cache[PerDeviceOnce::MAX_DEVICES];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= PerDeviceOnce::MAX_DEVICES) dev = 0;
  int n = cache[dev].load(std::memory_order_relaxed);
  if (!n) {
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cache[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

}  // namespace bdh
