// CTA-level building blocks shared by the merge kernels: warp/CTA scans, the k-ary warp
// searches used for partitioning, and the bounded look-back used by single-pass kernels.
#pragma once

#include "common.cuh"

namespace nb200 {

constexpr unsigned FULL_MASK = 0xffffffffu;

// ---- warp scans -----------------------------------------------------------------------

__device__ __forceinline__ int warp_incl_sum(int v) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int n = __shfl_up_sync(FULL_MASK, v, o);
        if (lane_id() >= o) v += n;
    }
    return v;
}

__device__ __forceinline__ unsigned warp_incl_max(unsigned v) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        unsigned n = __shfl_up_sync(FULL_MASK, v, o);
        if (lane_id() >= o) v = max(v, n);
    }
    return v;
}

// Exclusive sum over the CTA; `total` receives the CTA-wide sum. `tmp` is >= 33 ints of
// shared memory; the function syncs before reusing it, so calls may follow one another.
template <int NT>
__device__ __forceinline__ int block_excl_sum(int v, int *tmp, int &total) {
    constexpr int NW = NT / 32;
    int incl = warp_incl_sum(v);
    __syncthreads();
    if (lane_id() == 31) tmp[warp_id()] = incl;
    __syncthreads();
    if (warp_id() == 0) {
        int w = lane_id() < NW ? tmp[lane_id()] : 0;
        int wi = warp_incl_sum(w);
        if (lane_id() < NW) tmp[lane_id()] = wi - w;
        if (lane_id() == NW - 1) tmp[32] = wi;
    }
    __syncthreads();
    total = tmp[32];
    return tmp[warp_id()] + incl - v;
}

// Exclusive running maximum over the CTA for two independent sequences at once (va, vb).
// `tmp` is >= 64 unsigned of shared memory.
template <int NT>
__device__ __forceinline__ void block_excl_max2(unsigned va, unsigned vb, unsigned *tmp,
                                                unsigned &ea, unsigned &eb) {
    constexpr int NW = NT / 32;
    unsigned ia = warp_incl_max(va), ib = warp_incl_max(vb);
    __syncthreads();
    if (lane_id() == 31) {
        tmp[warp_id()] = ia;
        tmp[32 + warp_id()] = ib;
    }
    __syncthreads();
    if (warp_id() == 0) {
        unsigned wa = lane_id() < NW ? tmp[lane_id()] : 0u;
        unsigned wb = lane_id() < NW ? tmp[32 + lane_id()] : 0u;
        unsigned sa = warp_incl_max(wa), sb = warp_incl_max(wb);
        // exclusive across warps: shift by one
        unsigned pa = __shfl_up_sync(FULL_MASK, sa, 1), pb = __shfl_up_sync(FULL_MASK, sb, 1);
        if (lane_id() == 0) pa = pb = 0u;
        if (lane_id() < NW) {
            tmp[lane_id()] = pa;
            tmp[32 + lane_id()] = pb;
        }
    }
    __syncthreads();
    unsigned pa = __shfl_up_sync(FULL_MASK, ia, 1), pb = __shfl_up_sync(FULL_MASK, ib, 1);
    if (lane_id() == 0) pa = pb = 0u;
    ea = max(tmp[warp_id()], pa);
    eb = max(tmp[32 + warp_id()], pb);
}

// ---- warp k-ary searches ----------------------------------------------------------------

// Largest i in [lo, hi] with pred(i) true, given pred(lo) is true and pred is monotone
// (true ... true false ... false). All 32 lanes call this together; each step probes 32
// candidates at once, so the depth is ceil(log32(range)) dependent loads instead of log2.
template <typename Pred>
__device__ __forceinline__ int64_t warp_last_true(int64_t lo, int64_t hi, Pred pred) {
    while (lo < hi) {
        int64_t span = hi - lo;
        int64_t step = (span + 31) >> 5;
        int64_t idx = lo + (int64_t)(lane_id() + 1) * step;
        bool ok = idx <= hi && pred(idx);
        int c = __popc(__ballot_sync(FULL_MASK, ok));
        int64_t nlo = lo + (int64_t)c * step;
        int64_t nhi = nlo + step - 1;
        lo = nlo;
        hi = nhi < hi ? nhi : hi;
    }
    return lo;
}

// Number of leading true values of a monotone pred over [lo, hi), returned as lo + count.
template <typename Pred>
__device__ __forceinline__ int64_t warp_count_true(int64_t lo, int64_t hi, Pred pred) {
    while (lo < hi) {
        int64_t span = hi - lo;
        int64_t step = (span + 31) >> 5;
        int64_t p = lo + (int64_t)(lane_id() + 1) * step - 1;
        bool ok = p < hi && pred(p);
        int c = __popc(__ballot_sync(FULL_MASK, ok));
        int64_t nlo = lo + (int64_t)c * step;
        int64_t nhi = nlo + step - 1;
        lo = nlo;
        hi = nhi < hi ? nhi : hi;
    }
    return lo;
}

}  // namespace nb200
