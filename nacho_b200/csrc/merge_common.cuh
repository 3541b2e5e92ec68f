// Definitions shared by the merge kernels (CSR element-wise, COO3 / CSF3 tensor add): the set
// operation and launch-mode enums, the control block of single-pass launches, and the small
// scan kernel that sits between the two passes of the count -> scan -> fill route.
#pragma once

#include "block_utils.cuh"
#include "common.cuh"

namespace nb200 {

enum SetOp { OP_UNION = 0, OP_INTERSECT = 1 };

// What one launch of the tile kernel does.
//   MODE_COUNT  count the tile's result entries (first pass of the two-pass scheme)
//   MODE_FILL   write the result; the tile's output base comes from the scanned counts
//   MODE_FUSED  single pass: count, obtain the base by look-back over earlier tiles, write
enum Mode { MODE_COUNT = 0, MODE_FILL = 1, MODE_FUSED = 2 };

// Device-side control block of a fused launch.
struct FusedCtl {
    int ticket;           // next tile number to hand out
    DeviceStatus status;  // bounded-wait failures
    long long total;      // result entries, written by the last tile
};

// Exclusive prefix of the per-tile counts, in place, by one CTA; the grand total goes to
// *total_out (64-bit so that the host can detect int32 overflow).
static __global__ void __launch_bounds__(1024) k_scan_tiles(int32_t *counts, int32_t n, int64_t *total_out) {
    __shared__ long long warp_sums[33];
    __shared__ long long carry_s;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    for (int base = 0; base < n; base += 1024) {
        const int i = base + threadIdx.x;
        const long long v = i < n ? counts[i] : 0;
        long long incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            long long nb = __shfl_up_sync(FULL_MASK, incl, o);
            if (lane_id() >= o) incl += nb;
        }
        if (lane_id() == 31) warp_sums[warp_id()] = incl;
        __syncthreads();
        if (warp_id() == 0) {
            long long w = warp_sums[lane_id()];
            long long wi = w;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                long long nb = __shfl_up_sync(FULL_MASK, wi, o);
                if (lane_id() >= o) wi += nb;
            }
            warp_sums[lane_id()] = wi - w;
            if (lane_id() == 31) warp_sums[32] = wi;
        }
        __syncthreads();
        const long long carry = carry_s;
        const long long excl = carry + warp_sums[warp_id()] + incl - v;
        if (i < n) counts[i] = (int32_t)min(excl, (long long)INT32_MAX);
        __syncthreads();
        if (threadIdx.x == 0) carry_s = carry + warp_sums[32];
        __syncthreads();
    }
    if (threadIdx.x == 0) *total_out = carry_s;
}

}  // namespace nb200
