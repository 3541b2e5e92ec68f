// Register and warp building blocks of the merge kernels: the bitonic merge network a thread runs
// over the keys it holds, and the merge-path cut of one diagonal found by the 32 lanes of a warp
// together (32-ary search: three rounds for a tile of a few thousand entries).
#pragma once

#include "block_utils.cuh"

namespace nb200 {

// Sorts N keys held in registers that form a bitonic sequence (ascending run, then descending
// run). For N that is not a power of two the keys are treated as the top N slots of the next
// power-of-two network whose lower slots hold zeros; compare-exchanges that would touch
// those virtual slots leave them unchanged and are dropped at compile time.
template <int N>
__device__ __forceinline__ void bitonic_merge(uint32_t (&r)[N]) {
    constexpr int NET = N <= 8 ? 8 : (N <= 16 ? 16 : 32);
    constexpr int PAD = NET - N;
#pragma unroll
    for (int d = NET / 2; d > 0; d >>= 1) {
#pragma unroll
        for (int i = PAD; i < NET; ++i) {
            if ((i & d) == 0) {
                const uint32_t lo = min(r[i - PAD], r[i + d - PAD]), hi = max(r[i - PAD], r[i + d - PAD]);
                r[i - PAD] = lo;
                r[i + d - PAD] = hi;
            }
        }
    }
}

// Merge-path cut of diagonal d (0 <= d) between the sorted lists kx[0, na) and ky[0, nb): the
// x entries of kx and y = d - x entries of ky that come first in merged order. Keys carry the
// operand in their last bit (kx even, ky odd), so the kx entry of a position orders before the ky
// entry of the same position. All 32 lanes call this together and get the same answer, x.
__device__ __forceinline__ int warp_count_cut(const uint32_t *kx, const int na, const uint32_t *ky, const int nb, const int d) {
    if (d >= na + nb) return na;
    int lo = max(0, d - nb), hi = min(d, na);
    while (lo < hi) {  // number of leading m in [lo, hi) with kx[m] < ky[d - 1 - m]
        const int step = (hi - lo + 31) >> 5;
        const int p = lo + (lane_id() + 1) * step - 1;
        const bool ok = p < hi && kx[p] < ky[d - 1 - p];
        const int c = __popc(__ballot_sync(FULL_MASK, ok));
        lo += c * step;
        hi = min(lo + step - 1, hi);
    }
    return lo;
}

}  // namespace nb200
