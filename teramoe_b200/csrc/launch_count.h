// Process-wide count of kernel launches issued through the Python bindings (one per launcher call).
// Benchmarks read it around their timed region to report how many of this library's kernels ran.
#pragma once
#include <atomic>
#include <cstdint>

namespace tmoe {
inline std::atomic<int64_t>& launch_counter() {
    static std::atomic<int64_t> c{0};
    return c;
}
inline void count_launch() { launch_counter().fetch_add(1, std::memory_order_relaxed); }
}  // namespace tmoe
