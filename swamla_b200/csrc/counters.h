// Process-wide count of kernel launches issued by the library (read through lmoe_launch_count).
#pragma once
#include <atomic>
namespace lmoe {
extern std::atomic<long long> g_launch_count;
inline void count_launch(int n = 1) { g_launch_count.fetch_add(n, std::memory_order_relaxed); }
}  // namespace lmoe
