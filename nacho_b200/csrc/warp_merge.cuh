// Warp-wide merging of two sorted key lists held in shared memory, with the merged keys left
// "striped" over the warp's registers: slot e of the warp's 32 * V slots lives in register
// r[e / 32] of lane e % 32. Striped slots are what a coalesced store wants (the 32 lanes of one
// register are 32 consecutive result entries), so a warp that merges this way needs no staging
// array for its output, no CTA-wide barrier between its phases and no per-thread binary search:
//
//   warp_merge_cut      the merge-path cut of one diagonal, found by the 32 lanes together
//                       (32-ary search, three rounds for a tile of a few thousand entries);
//   warp_load_bitonic   the warp's A entries ascending, all-ones padding, its B entries descending:
//                       conflict-free shared-memory loads (consecutive lanes, consecutive words);
//   warp_bitonic_merge  a bitonic merge network over the 32 * V slots: the strides of 32 slots and
//                       more are compare-exchanges between registers of one lane, the strides below
//                       32 are butterfly shuffles.
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

// Sorts the 32 * V striped keys of a warp that form a bitonic sequence in slot order. On return
// slot e holds the e-th smallest key.
template <int V>
__device__ __forceinline__ void warp_bitonic_merge(uint32_t (&r)[V]) {
    bitonic_merge<V>(r);  // strides of 32 slots and more: same lane, different registers
    const int lane = lane_id();
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        const bool upper = (lane & d) != 0;  // the upper lane of a pair keeps the larger key
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const uint32_t o = __shfl_xor_sync(FULL_MASK, r[j], d);
            r[j] = ((r[j] < o) != upper) ? r[j] : o;
        }
    }
}

// Merge-path cut of diagonal d (0 <= d) between the sorted lists kx[0, na) and ky[0, nb): the
// x entries of kx and y = d - x entries of ky that come first in merged order. Keys carry the
// operand in their last bit (kx even, ky odd), so the kx entry of a position orders before the ky
// entry of the same position. All 32 lanes call these together and get the same answer.
// warp_count_cut returns x; warp_merge_cut also returns y, one larger where the cut would
// otherwise separate the two entries of one position.
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

__device__ __forceinline__ void warp_merge_cut(const uint32_t *kx, const int na, const uint32_t *ky, const int nb, const int d,
                                               int &x, int &y) {
    x = warp_count_cut(kx, na, ky, nb, d);
    y = min(d, na + nb) - x;
    if (x > 0 && y < nb && (kx[x - 1] ^ ky[y]) == 1u) ++y;
}

// Loads a warp's share of two sorted lists as one bitonic sequence: slots [0, ca) take
// kx[0, ca) ascending, slots [32 V - cb, 32 V) take ky[0, cb) descending, the slots between are
// all-ones. ca + cb <= 32 V.
template <int V>
__device__ __forceinline__ void warp_load_bitonic(uint32_t (&r)[V], const uint32_t *kx, const int ca, const uint32_t *ky, const int cb) {
    const int lane = lane_id();
#pragma unroll
    for (int j = 0; j < V; ++j) {
        const int e = 32 * j + lane;
        const bool is_a = e < ca, is_b = e >= 32 * V - cb;
        const uint32_t *p = is_a ? kx + e : (is_b ? ky + (32 * V - 1 - e) : kx);  // always a staged word
        const uint32_t v = *p;
        r[j] = (is_a || is_b) ? v : 0xffffffffu;
    }
}

// For sorted striped keys: bit j of the result says that slot 32 j + lane and the slot after it
// hold the two operands' entries of one position (keys that differ in the last bit only). The
// slot after the warp's last one counts as all-ones.
template <int V>
__device__ __forceinline__ unsigned warp_pair_mask(const uint32_t (&r)[V]) {
    const int lane = lane_id();
    unsigned same = 0;
#pragma unroll
    for (int j = 0; j < V; ++j) {
        // lane 31's successor is lane 0's next register
        const uint32_t after = j + 1 < V ? r[j + 1 < V ? j + 1 : j] : 0xffffffffu;
        const uint32_t src = lane == 0 ? after : r[j];
        const uint32_t nxt = __shfl_sync(FULL_MASK, src, (lane + 1) & 31);
        same |= (unsigned)((r[j] ^ nxt) == 1u) << j;
    }
    return same;
}

// The mask of the slot before: bit j of the result is bit j of lane - 1's mask, and for lane 0
// bit j - 1 of lane 31's (slot 0 has no predecessor).
__device__ __forceinline__ unsigned warp_shift_mask_up(const unsigned mask) {
    const int lane = lane_id();
    const unsigned up = __shfl_sync(FULL_MASK, mask, (lane + 31) & 31);
    return lane == 0 ? (up << 1) : up;
}

}  // namespace nb200
