// One-time, per-device set-up of kernel attributes.
//
// cudaFuncSetAttribute (dynamic shared-memory limit, carveout preference) applies to the CURRENT device only, so a
// process that drives several GPUs must repeat it on each of them, and two host threads may reach the same launcher
// at once.  PerDeviceOnce runs a set-up function once per device ordinal, under std::call_once, and remembers the
// code it returned; later calls on that device only read the stored code.
#pragma once
#include <cuda_runtime.h>

#include <mutex>

namespace lmoe {

constexpr int kMaxDevices = 64;

inline int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) dev = 0;
  return dev % kMaxDevices;
}

class PerDeviceOnce {
 public:
  // `fn` returns 0 or an error code; it runs with the calling thread's current device.
  template <typename F>
  int run(F&& fn) {
    const int dev = current_device();
    std::call_once(flags_[dev], [&] { rc_[dev] = fn(); });
    return rc_[dev];
  }

 private:
  std::once_flag flags_[kMaxDevices];
  int rc_[kMaxDevices] = {};
};

}  // namespace lmoe
