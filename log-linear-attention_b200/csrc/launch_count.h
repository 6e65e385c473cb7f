// Process-wide count of kernel launches issued by this library (read with llattn_kernel_launches()).
// Every launch site is followed by LLATTN_LAUNCHED(); the counter is one relaxed atomic add on the host.
#pragma once
#include <atomic>

namespace llattn {
extern std::atomic<unsigned long long> g_kernel_launches;
}
#define LLATTN_LAUNCHED() ((void)llattn::g_kernel_launches.fetch_add(1ull, std::memory_order_relaxed))
