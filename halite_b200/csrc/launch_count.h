// Process-wide count of kernel launches issued through this extension (each launcher call
// that returned cudaSuccess counts once). Read by benchmarks to report how many of this
// library's kernels ran inside a timed region.
#pragma once

#include <atomic>

namespace hb {
inline std::atomic<long>& launch_counter() {
  static std::atomic<long> c{0};
  return c;
}
}  // namespace hb
