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

// Barrier policies for the CTA-level scans below: the whole CTA, or the first COUNT threads
// of it on hardware barrier ID (used when one extra warp of the CTA has another job).
struct WholeCta {
    __device__ static __forceinline__ void sync() { __syncthreads(); }
};
template <int ID, int COUNT>
struct NamedBarrier {
    __device__ static __forceinline__ void sync() { asm volatile("bar.sync %0, %1;" ::"n"(ID), "n"(COUNT) : "memory"); }
    __device__ static __forceinline__ void arrive() { asm volatile("bar.arrive %0, %1;" ::"n"(ID), "n"(COUNT) : "memory"); }
};

// Exclusive sum over the first NT threads of the CTA; `total` receives their sum. `tmp` is >= 33
// ints of shared memory; the function syncs before reusing it, so calls may follow one another.
template <int NT, typename Bar = WholeCta>
__device__ __forceinline__ int block_excl_sum(int v, int *tmp, int &total) {
    constexpr int NW = NT / 32;
    int incl = warp_incl_sum(v);
    Bar::sync();
    if (lane_id() == 31) tmp[warp_id()] = incl;
    Bar::sync();
    if (warp_id() == 0) {
        int w = lane_id() < NW ? tmp[lane_id()] : 0;
        int wi = warp_incl_sum(w);
        if (lane_id() < NW) tmp[lane_id()] = wi - w;
        if (lane_id() == NW - 1) tmp[32] = wi;
    }
    Bar::sync();
    total = tmp[32];
    return tmp[warp_id()] + incl - v;
}

// Two exclusive sums at once (va, vb) over the first NT threads; `ta` / `tb` receive the totals.
// `tmp` is >= 66 ints of shared memory.
template <int NT, typename Bar = WholeCta>
__device__ __forceinline__ void block_excl_sum2(int va, int vb, int *tmp, int &ea, int &eb, int &ta, int &tb) {
    constexpr int NW = NT / 32;
    const int ia = warp_incl_sum(va), ib = warp_incl_sum(vb);
    Bar::sync();
    if (lane_id() == 31) {
        tmp[warp_id()] = ia;
        tmp[33 + warp_id()] = ib;
    }
    Bar::sync();
    if (warp_id() == 0) {
        const int wa = lane_id() < NW ? tmp[lane_id()] : 0, wb = lane_id() < NW ? tmp[33 + lane_id()] : 0;
        const int sa = warp_incl_sum(wa), sb = warp_incl_sum(wb);
        if (lane_id() < NW) {
            tmp[lane_id()] = sa - wa;
            tmp[33 + lane_id()] = sb - wb;
        }
        if (lane_id() == NW - 1) {
            tmp[32] = sa;
            tmp[65] = sb;
        }
    }
    Bar::sync();
    ta = tmp[32];
    tb = tmp[65];
    ea = tmp[warp_id()] + ia - va;
    eb = tmp[33 + warp_id()] + ib - vb;
}

// Exclusive running maximum over the CTA for two independent sequences at once (va, vb).
// `tmp` is >= 64 unsigned of shared memory.
template <int NT, typename Bar = WholeCta>
__device__ __forceinline__ void block_excl_max2(unsigned va, unsigned vb, unsigned *tmp,
                                                unsigned &ea, unsigned &eb) {
    constexpr int NW = NT / 32;
    unsigned ia = warp_incl_max(va), ib = warp_incl_max(vb);
    Bar::sync();
    if (lane_id() == 31) {
        tmp[warp_id()] = ia;
        tmp[32 + warp_id()] = ib;
    }
    Bar::sync();
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
    Bar::sync();
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

// ---- bounded decoupled look-back ----------------------------------------------------------

// Chained scan across CTAs in one pass: every tile publishes its own count ("aggregate") as
// soon as it knows it, then walks back over its predecessors' words, 32 at a time, adding
// aggregates until it meets a tile that already knows its inclusive prefix. A word carries a
// 2-bit state and a 62-bit value and is written with one 8-byte store, so no fence is needed
// between the two. A tile waits only on tiles with lower numbers, so tiles must be numbered in
// an order in which their CTAs start: the CTA index (the hardware hands CTAs out in index
// order, the numbering the kernels here use) or an atomic ticket taken at CTA start.
//
// Every wait is bounded: after LOOKBACK_POLL_LIMIT polls of one word the walk gives up,
// records the tile in `status` and returns -1; the caller then skips its writes. The tile
// still publishes a prefix so that its successors do not wait on it in turn.
constexpr uint64_t LB_AGGREGATE = 1ull << 62;
constexpr uint64_t LB_PREFIX = 2ull << 62;
constexpr uint64_t LB_VALUE_MASK = (1ull << 62) - 1;
constexpr int LOOKBACK_POLL_LIMIT = 1 << 22;
constexpr int ERR_LOOKBACK_TIMEOUT = 1;

__device__ __forceinline__ uint64_t ld_relaxed_gpu(const volatile uint64_t *p) {
    uint64_t v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_relaxed_gpu(volatile uint64_t *p, uint64_t v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ int ld_relaxed_gpu_i32(const int *p) {
    int v;
    asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_relaxed_gpu_i32(int *p, int v) {
    asm volatile("st.relaxed.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Sum of the counts of tiles [0, t), read off the tile words of the predecessors, 32 at a time
// from the nearest one backwards; publishes nothing. A round is complete once every word up to
// the nearest tile that already knows its prefix is published (the words beyond it are not
// needed); until then the warp polls, sleeping `sleep_ns` between polls -- or `hurry_ns` once
// `*hurry` is non-zero (the caller's own tile is waiting for the result by then, so the poll
// traffic no longer competes with useful work). Returns -1 (and records the tile in `status`) if
// a bounded wait gives up after `poll_limit` polls of one round. Called by all 32 lanes of one
// warp, t > 0.
template <int DEPTH = 1>
__device__ __forceinline__ int64_t lookback_predecessors(volatile uint64_t *state, int t, DeviceStatus *status,
                                                         unsigned sleep_ns, const volatile int *hurry = nullptr,
                                                         unsigned hurry_ns = 64, const int poll_limit = LOOKBACK_POLL_LIMIT) {
    // One round covers DEPTH * 32 predecessors, nearest first (word j of a lane is tile
    // pos - 32 j - lane), with all of a lane's loads in flight together.
    int64_t exclusive = 0;
    for (int pos = t - 1;; pos -= 32 * DEPTH) {
        uint64_t s[DEPTH];
        unsigned need[DEPTH];
        bool found = false;
        for (int polls = 0;; ++polls) {
#pragma unroll
            for (int j = 0; j < DEPTH; ++j) {
                const int idx = pos - 32 * j - lane_id();
                s[j] = idx >= 0 ? ld_relaxed_gpu(state + idx) : LB_PREFIX;  // before tile 0: an empty prefix
            }
            bool ready = true;
            found = false;
#pragma unroll
            for (int j = 0; j < DEPTH; ++j) {
                const unsigned prefix_lanes = __ballot_sync(FULL_MASK, (s[j] >> 62) == 2);
                const unsigned published = __ballot_sync(FULL_MASK, (s[j] >> 62) != 0);
                if (found) {
                    need[j] = 0u;  // beyond the nearest prefix: not needed
                } else {
                    const int first = prefix_lanes ? __ffs(prefix_lanes) - 1 : 31;
                    need[j] = first == 31 ? FULL_MASK : (1u << (first + 1)) - 1u;
                    ready = ready && (published & need[j]) == need[j];
                    found = prefix_lanes != 0u;
                }
            }
            if (ready) break;
            if (polls >= poll_limit) {
                if (lane_id() == 0 && atomicCAS(&status->error, 0, ERR_LOOKBACK_TIMEOUT) == 0) status->detail = t;
                return -1;
            }
            __nanosleep(hurry && *hurry ? hurry_ns : sleep_ns);
        }
        long long v = 0;
#pragma unroll
        for (int j = 0; j < DEPTH; ++j) v += (need[j] >> lane_id()) & 1u ? (long long)(s[j] & LB_VALUE_MASK) : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL_MASK, v, o);
        exclusive += v;
        if (found) return exclusive;
    }
}

// Publishes the tile's count, walks back, publishes the inclusive prefix. Returns the sum of the
// counts of tiles [0, t), or -1 after a give-up (the tile then still publishes a prefix so that
// its successors do not wait on it). Called by all 32 lanes of one warp.
__device__ __forceinline__ int64_t lookback_exclusive(volatile uint64_t *state, int t, int64_t aggregate,
                                                      DeviceStatus *status) {
    if (lane_id() == 0) st_relaxed_gpu(state + t, (t == 0 ? LB_PREFIX : LB_AGGREGATE) | (uint64_t)aggregate);
    if (t == 0) return 0;
    const int64_t exclusive = lookback_predecessors(state, t, status, 32);
    if (lane_id() == 0) st_relaxed_gpu(state + t, LB_PREFIX | (uint64_t)(exclusive < 0 ? 0 : exclusive + aggregate));
    return exclusive;
}

}  // namespace nb200
