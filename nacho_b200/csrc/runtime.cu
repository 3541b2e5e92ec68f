// Library runtime: status text, scratch pool, launch counter, per-kernel event timing and the
// free wrapper. Host code only.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

#include "common.cuh"

namespace nb200 {

namespace {

thread_local char g_cuda_error[256] = "";
std::atomic<uint64_t> g_launches{0};
std::atomic<int> g_profile_on{0};

std::mutex g_ws_mutex;
std::atomic<uint64_t> g_ws_epoch{0};
std::map<std::pair<std::pair<int, int>, cudaStream_t>, Workspace> g_workspaces;

struct TimedLaunch {
    cudaEvent_t start, stop;
};
struct KernelTimes {
    std::vector<TimedLaunch> pending;
    int64_t launches = 0;
    double total_ms = 0.0;
};
std::mutex g_prof_mutex;
std::map<std::string, KernelTimes> g_prof;
std::vector<cudaEvent_t> g_event_pool;

cudaEvent_t get_event() {
    if (!g_event_pool.empty()) {
        cudaEvent_t e = g_event_pool.back();
        g_event_pool.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
}

// Folds finished event pairs into the totals. Caller holds g_prof_mutex.
void settle(KernelTimes &k) {
    for (auto &t : k.pending) {
        float ms = 0.f;
        if (cudaEventSynchronize(t.stop) == cudaSuccess &&
            cudaEventElapsedTime(&ms, t.start, t.stop) == cudaSuccess) {
            k.total_ms += ms;
            k.launches += 1;
        }
        g_event_pool.push_back(t.start);
        g_event_pool.push_back(t.stop);
    }
    k.pending.clear();
}

}  // namespace

int note_cuda_error(cudaError_t e, const char *what) {
    std::snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s", what, cudaGetErrorString(e));
    cudaGetLastError();  // clear the sticky-free error state
    return e == cudaErrorMemoryAllocation ? NB200_E_NOMEM : NB200_E_CUDA;
}

int note_timeout(int site, int tile, const char *where) {
    static const char *const names[] = {"?", "look-back over earlier tiles", "bulk copy into shared memory", "tile wider than its key"};
    std::snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s gave up at tile %d", where, names[site >= 1 && site <= 3 ? site : 0], tile);
    return NB200_E_TIMEOUT;
}

int acquire_workspace(cudaStream_t stream, size_t bytes, Workspace **out, int slot) {
    int dev = 0;
    NB200_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> g(g_ws_mutex);
    Workspace &ws = g_workspaces[{{dev, slot}, stream}];
    if (!ws.host) NB200_CUDA(cudaHostAlloc(reinterpret_cast<void **>(&ws.host), 64 * sizeof(int64_t), cudaHostAllocDefault));
    if (bytes > ws.dev_bytes) {
        if (ws.dev) {
            NB200_CUDA(cudaStreamSynchronize(stream));
            NB200_CUDA(cudaFree(ws.dev));
            ws.dev = nullptr;
            ws.dev_bytes = 0;
        }
        size_t want = bytes + bytes / 4 + 4096;
        NB200_CUDA(cudaMalloc(&ws.dev, want));
        ws.dev_bytes = want;
    }
    ++ws.generation;
    *out = &ws;
    return NB200_OK;
}

uint64_t workspace_epoch() { return g_ws_epoch.load(std::memory_order_acquire); }

LaunchScope::LaunchScope(const char *name, cudaStream_t stream)
    : name_(name), stream_(stream), start_(nullptr), timed_(g_profile_on.load(std::memory_order_relaxed) != 0) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (timed_) {
        std::lock_guard<std::mutex> g(g_prof_mutex);
        start_ = get_event();
        cudaEventRecord(start_, stream_);
    }
}

LaunchScope::~LaunchScope() {
    if (!timed_) return;
    std::lock_guard<std::mutex> g(g_prof_mutex);
    cudaEvent_t stop = get_event();
    cudaEventRecord(stop, stream_);
    g_prof[name_].pending.push_back({start_, stop});
}

}  // namespace nb200

using namespace nb200;

extern "C" {

int nb200_version(void) { return NB200_VERSION; }

const char *nb200_strerror(int status) {
    switch (status) {
        case NB200_OK: return "ok";
        case NB200_E_BADARG: return "bad argument";
        case NB200_E_CUDA: return "CUDA runtime error";
        case NB200_E_OVERFLOW: return "result length or work count exceeds int32";
        case NB200_E_CAPACITY: return "result arrays too small";
        case NB200_E_TIMEOUT: return "bounded device-side wait gave up";
        case NB200_E_NOMEM: return "device allocation failed";
        case NB200_E_UNSUPPORTED: return "size beyond the limit of this entry point";
        default: return "unknown status";
    }
}

const char *nb200_last_cuda_error(void) { return g_cuda_error; }

int nb200_free_async(void *p, void *stream) {
    if (!p) return NB200_OK;
    NB200_CUDA(cudaFreeAsync(p, static_cast<cudaStream_t>(stream)));
    return NB200_OK;
}

int nb200_release_workspaces(void) {
    std::lock_guard<std::mutex> g(g_ws_mutex);
    int prev = 0;
    cudaGetDevice(&prev);
    for (auto &kv : g_workspaces) {
        cudaSetDevice(kv.first.first.first);
        if (kv.second.dev) {
            cudaDeviceSynchronize();
            cudaFree(kv.second.dev);
        }
        if (kv.second.host) cudaFreeHost(kv.second.host);
    }
    g_workspaces.clear();
    g_ws_epoch.fetch_add(1, std::memory_order_release);
    cudaSetDevice(prev);
    return NB200_OK;
}

uint64_t nb200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int nb200_profile_enable(int on) {
    g_profile_on.store(on ? 1 : 0, std::memory_order_relaxed);
    return NB200_OK;
}

int nb200_profile_reset(void) {
    std::lock_guard<std::mutex> g(g_prof_mutex);
    for (auto &kv : g_prof) {
        settle(kv.second);
        kv.second.launches = 0;
        kv.second.total_ms = 0.0;
    }
    return NB200_OK;
}

int nb200_profile_read(const char *name, int64_t *launches, double *total_ms) {
    if (!name) return NB200_E_BADARG;
    std::lock_guard<std::mutex> g(g_prof_mutex);
    auto it = g_prof.find(name);
    if (it == g_prof.end()) {
        if (launches) *launches = 0;
        if (total_ms) *total_ms = 0.0;
        return NB200_OK;
    }
    settle(it->second);
    if (launches) *launches = it->second.launches;
    if (total_ms) *total_ms = it->second.total_ms;
    return NB200_OK;
}

int nb200_profile_names(char *buf, size_t buf_len) {
    if (!buf || buf_len == 0) return NB200_E_BADARG;
    std::lock_guard<std::mutex> g(g_prof_mutex);
    std::string s;
    for (auto &kv : g_prof) {
        if (!s.empty()) s += ",";
        s += kv.first;
    }
    std::snprintf(buf, buf_len, "%s", s.c_str());
    return NB200_OK;
}

}  // extern "C"
