// Once-per-device set-up of a kernel's function attributes.
//
// cudaFuncSetAttribute (opt-in dynamic shared memory above 48 KB, the shared-memory
// carve-out) changes per-device state: a kernel configured while device 0 was current
// is still unconfigured on device 1 of the same process.  A process-wide "configured"
// flag therefore makes the first launch on a second device fail.  DeviceOnce keeps one
// bit per device ordinal.  Two host threads may both see "needed" and both run the
// set-up; that is harmless (the attribute calls are idempotent).
#pragma once

#include <atomic>
#include <cuda_runtime.h>

namespace b200 {

struct DeviceOnce {
  std::atomic<unsigned long long> done{0};

  // True when the set-up has not been recorded for the current device; *dev receives its ordinal.
  bool needed(int* dev) {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess) d = 0;
    *dev = d;
    if (d < 0 || d >= 64) return true;
    return ((done.load(std::memory_order_acquire) >> d) & 1ull) == 0ull;
  }
  void mark(int dev) {
    if (dev >= 0 && dev < 64) done.fetch_or(1ull << dev, std::memory_order_release);
  }
};

}  // namespace b200
