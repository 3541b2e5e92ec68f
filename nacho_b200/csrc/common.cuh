// Shared host/device plumbing of the nacho_b200 library: status handling, the per-stream
// scratch pool, the launch counter and the optional per-kernel event timing.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "nacho_b200.h"

namespace nb200 {

// ---- status ---------------------------------------------------------------------------

// Records a failing CUDA call for nb200_last_cuda_error() and returns NB200_E_CUDA
// (NB200_E_NOMEM for allocation failures). Replaces the throwing CHECK_CUDA of
// runtime/cuda_utils/cuda_utils.h:13-20 with a status code.
int note_cuda_error(cudaError_t e, const char *what);
// Records which bounded device-side wait gave up (site code and tile of a DeviceStatus) in the
// message nb200_last_cuda_error returns; the value is NB200_E_TIMEOUT.
int note_timeout(int site, int tile, const char *where);

#define NB200_CUDA(call)                                               \
    do {                                                               \
        cudaError_t nb200_e_ = (call);                                 \
        if (nb200_e_ != cudaSuccess) return ::nb200::note_cuda_error(nb200_e_, #call); \
    } while (0)

// ---- scratch pool ---------------------------------------------------------------------

// Grow-only device scratch keyed by (device, stream). The returned block stays valid until
// the next acquire with the same key or nb200_release_workspaces(); calls on one stream are
// ordered by the stream, so reuse across calls is safe. Also carries a small pinned host
// block for result-length read-backs.
struct Workspace {
    void *dev = nullptr;
    size_t dev_bytes = 0;
    int64_t *host = nullptr;  // pinned, 64 int64 slots
    uint64_t generation = 0;  // bumped by every acquire: a holder can tell whether the block was handed out again
};

// `slot` selects one of several independent blocks per (device, stream): a driver that keeps an
// intermediate alive across calls into other drivers takes slot 1 for it.
int acquire_workspace(cudaStream_t stream, size_t bytes, Workspace **out, int slot = 0);

// Counts the calls of nb200_release_workspaces(): a Workspace pointer obtained under an earlier
// value is dangling.
uint64_t workspace_epoch();

// Carves 256-byte-aligned sub-blocks out of a Workspace.
class Carver {
public:
    explicit Carver(void *base) : p_(reinterpret_cast<uintptr_t>(base)), used_(0) {}
    Carver() : p_(0), used_(0) {}
    template <typename T>
    T *take(size_t count) {
        size_t bytes = (count * sizeof(T) + 255) & ~size_t(255);
        T *r = p_ ? reinterpret_cast<T *>(p_ + used_) : nullptr;
        used_ += bytes;
        return r;
    }
    size_t used() const { return used_; }

private:
    uintptr_t p_;
    size_t used_;
};

// ---- launches and timing --------------------------------------------------------------

// Brackets one kernel launch: counts it and, while profiling is on, records a start/stop
// event pair on `stream` under `name`.
class LaunchScope {
public:
    LaunchScope(const char *name, cudaStream_t stream);
    ~LaunchScope();

private:
    const char *name_;
    cudaStream_t stream_;
    cudaEvent_t start_;
    bool timed_;
};

// Error word shared by kernels with bounded waits: 0 = fine, otherwise a site code.
struct DeviceStatus {
    int error;
    int detail;
};

// ---- device helpers -------------------------------------------------------------------

#ifdef __CUDACC__
__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }
__device__ __forceinline__ int warp_id() { return threadIdx.x >> 5; }

template <typename T>
__device__ __forceinline__ T ld_nc(const T *p) {
    return __ldg(p);
}
#endif

}  // namespace nb200
