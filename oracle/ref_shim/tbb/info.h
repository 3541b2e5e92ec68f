// Minimal stand-in for <tbb/info.h>: test infrastructure only.
//
// The reference's emitted CPU drivers ask oneTBB for exactly one thing from this header,
// tbb::info::default_concurrency() (emitter: src/backend/stitch_and_generate_cpu.cpp:26-31).
// oneTBB is not installed here, so this reports the size of the std::thread pool that
// tbb/parallel_for.h (same folder) runs on. NACHO_REF_THREADS overrides the count.
#pragma once
#include <cstdlib>
#include <thread>

namespace tbb {
namespace info {
inline int default_concurrency() {
    if (const char *env = std::getenv("NACHO_REF_THREADS")) {
        int n = std::atoi(env);
        if (n > 0) return n;
    }
    unsigned hw = std::thread::hardware_concurrency();
    return hw ? static_cast<int>(hw) : 1;
}
}  // namespace info
}  // namespace tbb
