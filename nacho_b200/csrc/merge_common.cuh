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
//   MODE_REDUCE no result tensor: the products of the entries both operands hold are summed
//               (inner product); the tile's partial sum is added to a double in the control block
enum Mode { MODE_COUNT = 0, MODE_FILL = 1, MODE_FUSED = 2, MODE_REDUCE = 3 };

// Device-side control block of a fused launch.
struct FusedCtl {
    int ticket;           // next tile number to hand out
    DeviceStatus status;  // bounded-wait failures
    long long total;      // result entries, written by the last tile (MODE_REDUCE: the bits of a double, the running sum)
};

// Optional second result form of the coordinate merge: the CSF3 levels above k. When a fused
// launch of the COO3 tile kernel is given one of these, it does not write the merged i and j
// columns; instead every tile flags the result entries that open a new i slice or a new (i, j)
// fibre, obtains the number of slices / fibres of all earlier tiles by a second bounded look-back
// (packed as slices << 31 | fibres in `tile_state`, one zeroed word per tile), and writes
// i_idx / j_ptr / j_idx / k_ptr directly. The last tile leaves the totals in `totals`.
struct CsfTotals {
    int n_i, n_j;
};
struct CsfLevelsOut {
    int32_t *i_idx, *j_ptr, *j_idx, *k_ptr;
    int32_t cap_i, cap_j;  // entries the arrays can hold (offset arrays: one more)
    uint64_t *tile_state;
    CsfTotals *totals;
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

// Device-wide exclusive prefix of n int32 counts, in place, in one pass: 2048 counts per CTA,
// CTA totals chained by bounded look-back. `state` holds one zeroed 8-byte word per CTA and
// `ctl` is zeroed; the grand total lands in ctl->total. A give-up of a bounded wait is
// recorded in ctl->status and leaves the tail of the array unscanned.
constexpr int SCAN_NT = 256, SCAN_VT = 8;

static __global__ void __launch_bounds__(SCAN_NT) k_scan_lookback(int32_t *data, int32_t n, uint64_t *state_raw, FusedCtl *ctl) {
    __shared__ int scan_tmp[40];
    __shared__ long long s_base;
    volatile uint64_t *state = state_raw;
    const int tid = threadIdx.x;
    const int t = blockIdx.x;  // CTAs are dispatched in index order; waits on earlier tiles are bounded
    const int64_t p0 = ((int64_t)t * SCAN_NT + tid) * SCAN_VT;
    int v[SCAN_VT];
    int mine = 0;
#pragma unroll
    for (int q = 0; q < SCAN_VT; ++q) {
        v[q] = p0 + q < n ? data[p0 + q] : 0;
        mine += v[q];
    }
    int total;
    int run = block_excl_sum<SCAN_NT>(mine, scan_tmp, total);
    if (warp_id() == 0) {
        const int64_t b = lookback_exclusive(state, t, total, &ctl->status);
        if (lane_id() == 0) s_base = b;
    }
    __syncthreads();
    const long long base = s_base;
    if (base < 0) return;
    long long acc = base + run;
#pragma unroll
    for (int q = 0; q < SCAN_VT; ++q) {
        if (p0 + q < n) data[p0 + q] = (int32_t)min(acc, (long long)INT32_MAX);
        acc += v[q];
    }
    if (t == (int)gridDim.x - 1 && tid == SCAN_NT - 1) ctl->total = acc;
}

}  // namespace nb200
