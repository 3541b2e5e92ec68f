// Minimal stand-in for <tbb/parallel_for.h>: test infrastructure only.
//
// The reference's emitted CPU drivers use one overload, tbb::parallel_for(first, last, body)
// over a range of thread ids (emitter: src/backend/stitch_and_generate_cpu.cpp:138-154).
// This runs that overload on a persistent std::thread pool so that the per-call cost is a
// wake-up rather than thread creation, which is what a real oneTBB arena would give.
#pragma once
#include <atomic>
#include <condition_variable>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

#include "tbb/info.h"

namespace tbb {
namespace detail_shim {

class Pool {
public:
    static Pool &instance() {
        static Pool pool;
        return pool;
    }

    // Runs body(i) for i in [first, last); returns when all are done.
    void run(int first, int last, const std::function<void(int)> &body) {
        if (last <= first) return;
        std::unique_lock<std::mutex> call_lock(call_mutex_);  // one parallel_for at a time
        ensure_workers(tbb::info::default_concurrency() - 1);
        {
            std::lock_guard<std::mutex> g(m_);
            body_ = &body;
            next_.store(first, std::memory_order_relaxed);
            last_ = last;
            pending_ = static_cast<int>(workers_.size());
            ++epoch_;
        }
        cv_.notify_all();
        drain();
        std::unique_lock<std::mutex> g(m_);
        done_cv_.wait(g, [&] { return pending_ == 0; });
        body_ = nullptr;
    }

private:
    Pool() = default;
    ~Pool() {
        {
            std::lock_guard<std::mutex> g(m_);
            stop_ = true;
            ++epoch_;
        }
        cv_.notify_all();
        for (auto &w : workers_) w.join();
    }

    void ensure_workers(int n) {
        while (static_cast<int>(workers_.size()) < n) {
            unsigned long seen;
            {
                std::lock_guard<std::mutex> g(m_);
                seen = epoch_;
            }
            workers_.emplace_back([this, seen] { worker(seen); });
        }
    }

    void drain() {
        for (;;) {
            int i = next_.fetch_add(1, std::memory_order_relaxed);
            if (i >= last_) break;
            (*body_)(i);
        }
    }

    void worker(unsigned long seen) {
        for (;;) {
            {
                std::unique_lock<std::mutex> g(m_);
                cv_.wait(g, [&] { return epoch_ != seen; });
                seen = epoch_;
                if (stop_) return;
            }
            drain();
            {
                std::lock_guard<std::mutex> g(m_);
                if (--pending_ == 0) done_cv_.notify_one();
            }
        }
    }

    std::mutex call_mutex_;
    std::mutex m_;
    std::condition_variable cv_, done_cv_;
    std::vector<std::thread> workers_;
    const std::function<void(int)> *body_ = nullptr;
    std::atomic<int> next_{0};
    int last_ = 0;
    int pending_ = 0;
    unsigned long epoch_ = 0;
    bool stop_ = false;
};

}  // namespace detail_shim

template <typename Index, typename Body>
void parallel_for(Index first, Index last, const Body &body) {
    std::function<void(int)> f = [&](int i) { body(static_cast<Index>(i)); };
    detail_shim::Pool::instance().run(static_cast<int>(first), static_cast<int>(last), f);
}

}  // namespace tbb
