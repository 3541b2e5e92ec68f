// SpGEMM C = A * B by expand - sort - compress, row by row.
//
// What the reference does (GPU only, compiler.cpp:145-148): expand every product
// a.values[p] * b.values[q] with key k = b.cols[q] in (i, j ascending, k ascending) order
// (src/backend/compute.cpp:526-611), sort each row's products by k with a global segmented sort
// (src/backend/stitch_and_generate_gpu.cpp:79-94), flag run heads, scan, and sum runs with
// warp shuffles plus atomics (:96-124, :257-363). All its counters are int32 and it
// materialises every product in HBM.
//
// Here rows are binned by their product count P_i (64-bit counters throughout) and no product
// ever reaches HBM:
//   small   P_i <= 32      one warp per row: products in registers, bitonic sort by shuffles
//   medium  P_i <= 256     one CTA per row: products in shared memory, bitonic sort there
//   ranked  P_i <= 65535   one CTA per row: a bitmap of the produced columns in shared memory is
//   heavy   P_i  > 65535   turned into the rank of every column within the result row, then every
//                          product is added straight into its final position of C (float32
//                          reductions in L2 on the row's own compact output range). Heavy rows
//                          keep 32-bit ranks, take larger CTAs and start in order of weight.
// Matrices wider than the bitmap (262144 columns) are walked in column windows of that width.
// Two passes: symbolic (unique columns per row -> row offsets by a scan) and numeric (fill).
// Small and medium rows sum equal-column products in expansion order (ascending j), a fixed
// order; ranked and heavy rows sum with float32 atomics, like the reference does for every row.
#include <algorithm>
#include <climits>
#include <cstring>
#include <mutex>

#include "merge_common.cuh"

namespace nb200 {

namespace {

constexpr int SMALL_P = 32;
#ifndef ESC_MEDIUM_P
#define ESC_MEDIUM_P 256
#endif
constexpr int MEDIUM_P = ESC_MEDIUM_P;
constexpr int MED_NT = 128;
constexpr unsigned long long RANKED_P = 65535;   // 16-bit ranks up to here
constexpr unsigned long long GIANT_P = 1ull << 20;

struct CsrView {
    const int32_t *rp;
    const int32_t *col;
    const float *val;
};

// Device-side counters of one call.
struct EscCtl {
    unsigned long long products;
    int n_small, n_medium, n_ranked;
    int n_giant, n_heavy;  // heavy rows with more / at most GIANT_P products
    int pad;
};

// heavy_rows holds the giant rows from its front and the other heavy rows from its back, so
// that the heaviest rows are handed out first.
struct RowLists {
    int32_t *small_rows, *medium_rows, *ranked_rows, *heavy_rows;
};

// P[p] = products of the first p stored entries of A (p = 0 .. nnz(A), counted from A's first row
// offset, which need not be 0): B's row lengths summed
// in one pass, 2048 entries per CTA, CTA totals chained by bounded look-back.
__global__ void __launch_bounds__(256) k_esc_product_prefix(CsrView A, CsrView B, int32_t nnz_a, unsigned long long *__restrict__ P,
                                                             uint64_t *state_raw, FusedCtl *ctl) {
    constexpr int VT = 8;
    __shared__ unsigned long long warp_sums[9];
    __shared__ long long s_base;
    volatile uint64_t *state = state_raw;
    const int tid = threadIdx.x, t = blockIdx.x;  // CTAs are dispatched in index order; waits on earlier tiles are bounded
    const int64_t p0 = ((int64_t)t * 256 + tid) * VT;
    const int32_t *a_col = A.col + ld_nc(A.rp);
    unsigned len[VT];
    unsigned long long mine = 0;
#pragma unroll
    for (int q = 0; q < VT; ++q) {
        len[q] = 0;
        if (p0 + q < nnz_a) {
            const int32_t j = ld_nc(a_col + p0 + q);
            len[q] = (unsigned)(ld_nc(B.rp + j + 1) - ld_nc(B.rp + j));
        }
        mine += len[q];
    }
    unsigned long long incl = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const unsigned long long up = __shfl_up_sync(FULL_MASK, incl, d);
        if (lane_id() >= d) incl += up;
    }
    if (lane_id() == 31) warp_sums[warp_id()] = incl;
    __syncthreads();
    if (tid == 0) {
        unsigned long long run = 0;
        for (int w = 0; w < 8; ++w) {
            const unsigned long long c = warp_sums[w];
            warp_sums[w] = run;
            run += c;
        }
        warp_sums[8] = run;
    }
    __syncthreads();
    if (warp_id() == 0) {
        const int64_t b = lookback_exclusive(state, t, (int64_t)warp_sums[8], &ctl->status);
        if (lane_id() == 0) s_base = b;
    }
    __syncthreads();
    if (s_base < 0) return;
    unsigned long long run = (unsigned long long)s_base + warp_sums[warp_id()] + incl - mine;
#pragma unroll
    for (int q = 0; q < VT; ++q) {
        if (p0 + q <= nnz_a) P[p0 + q] = run;
        run += len[q];
    }
}

// Expand phase 1 (src/backend/compute.cpp:541-611): per-row product counts, and the bins.
// Rows without products get their count (0) written here. The counts come from the prefix P of
// B's row lengths over A's entries (k_esc_product_prefix): a hub row costs one subtraction.
__global__ void __launch_bounds__(256) k_esc_rowwork(CsrView A, const unsigned long long *__restrict__ P, int32_t rows,
                                                     int32_t *__restrict__ row_count, RowLists lists, EscCtl *ctl) {
    __shared__ unsigned long long warp_p[8];
    const int i = blockIdx.x * 256 + threadIdx.x;  // one lane per row: its products are a difference of the prefix
    unsigned long long p = 0;
    if (i < rows) {
        const int32_t base = ld_nc(A.rp);
        p = ld_nc(P + (ld_nc(A.rp + i + 1) - base)) - ld_nc(P + (ld_nc(A.rp + i) - base));
    }
    if (i < rows) {  // lanes of a warp that take the same branch share one atomic
        if (p == 0) {
            if (row_count) row_count[i] = 0;
        } else if (p <= SMALL_P) {
            lists.small_rows[atomicAdd(&ctl->n_small, 1)] = i;
        } else if (p <= MEDIUM_P) {
            lists.medium_rows[atomicAdd(&ctl->n_medium, 1)] = i;
        } else if (p <= RANKED_P) {
            lists.ranked_rows[atomicAdd(&ctl->n_ranked, 1)] = i;
        } else if (p > GIANT_P) {
            lists.heavy_rows[atomicAdd(&ctl->n_giant, 1)] = i;
        } else {
            lists.heavy_rows[rows - 1 - atomicAdd(&ctl->n_heavy, 1)] = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) p += __shfl_xor_sync(FULL_MASK, p, o);
    // one atomic per CTA for the product total
    if (lane_id() == 0) warp_p[warp_id()] = p;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long sum = 0;
        for (int v = 0; v < 8; ++v) sum += warp_p[v];
        if (sum) atomicAdd(&ctl->products, sum);
    }
}

// The same with the product counts taken row by row: one lane per row walks its entries (the warp
// shares the work of its longer rows). For matrices of short rows, where a prefix pass over A's
// entries costs more than it saves.
__global__ void __launch_bounds__(256) k_esc_rowwork_walk(CsrView A, CsrView B, int32_t rows, int32_t *__restrict__ row_count,
                                                     RowLists lists, EscCtl *ctl) {
    __shared__ unsigned long long warp_p[8];
    const int i = blockIdx.x * 256 + threadIdx.x;  // one lane per row; the warp shares the work of its longer rows
    int32_t lo = 0, hi = 0;
    if (i < rows) {
        lo = ld_nc(A.rp + i);
        hi = ld_nc(A.rp + i + 1);
    }
    unsigned long long p = 0;
    const bool together = hi - lo > 32;
    if (!together) {
        for (int32_t e = lo; e < hi; ++e) {
            const int32_t j = ld_nc(A.col + e);
            p += (unsigned long long)(ld_nc(B.rp + j + 1) - ld_nc(B.rp + j));
        }
    }
    for (unsigned todo = __ballot_sync(FULL_MASK, together); todo; todo &= todo - 1) {
        const int r = __ffs(todo) - 1;
        const int32_t l = __shfl_sync(FULL_MASK, lo, r), h = __shfl_sync(FULL_MASK, hi, r);
        unsigned long long q = 0;
        for (int32_t e = l + lane_id(); e < h; e += 32) {
            const int32_t j = ld_nc(A.col + e);
            q += (unsigned long long)(ld_nc(B.rp + j + 1) - ld_nc(B.rp + j));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(FULL_MASK, q, o);
        if (lane_id() == r) p = q;
    }
    if (i < rows) {  // lanes of a warp that take the same branch share one atomic
        if (p == 0) {
            if (row_count) row_count[i] = 0;
        } else if (p <= SMALL_P) {
            lists.small_rows[atomicAdd(&ctl->n_small, 1)] = i;
        } else if (p <= MEDIUM_P) {
            lists.medium_rows[atomicAdd(&ctl->n_medium, 1)] = i;
        } else if (p <= RANKED_P) {
            lists.ranked_rows[atomicAdd(&ctl->n_ranked, 1)] = i;
        } else if (p > GIANT_P) {
            lists.heavy_rows[atomicAdd(&ctl->n_giant, 1)] = i;
        } else {
            lists.heavy_rows[rows - 1 - atomicAdd(&ctl->n_heavy, 1)] = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) p += __shfl_xor_sync(FULL_MASK, p, o);
    // one atomic per CTA for the product total
    if (lane_id() == 0) warp_p[warp_id()] = p;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long sum = 0;
        for (int v = 0; v < 8; ++v) sum += warp_p[v];
        if (sum) atomicAdd(&ctl->products, sum);
    }
}

// ------------------------------------------------------------------------- small rows ----

// Compare-exchange step of a 32-wide bitonic sort held one key per lane.
__device__ __forceinline__ uint64_t warp_bitonic_sort(uint64_t key) {
#pragma unroll
    for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
        for (int j = k >> 1; j > 0; j >>= 1) {
            const uint64_t other = __shfl_xor_sync(FULL_MASK, key, j);
            const bool up = (lane_id() & k) == 0;        // ascending block?
            const bool lower = (lane_id() & j) == 0;     // lower lane of the pair?
            const bool take_min = up == lower;
            key = take_min ? min(key, other) : max(key, other);
        }
    }
    return key;
}

__device__ __forceinline__ uint32_t warp_bitonic_sort32(uint32_t key) {
#pragma unroll
    for (int k = 2; k <= 32; k <<= 1) {
#pragma unroll
        for (int j = k >> 1; j > 0; j >>= 1) {
            const uint32_t other = __shfl_xor_sync(FULL_MASK, key, j);
            const bool take_min = ((lane_id() & k) == 0) == ((lane_id() & j) == 0);
            key = take_min ? min(key, other) : max(key, other);
        }
    }
    return key;
}

#ifndef ESC_SMALL_ROWS
#define ESC_SMALL_ROWS 4
#endif

// Rows with at most 32 products, ESC_SMALL_ROWS of them per warp. Lane l holds product l of a row's
// expansion order; the sort key is (column << 32 | l), so equal columns stay in expansion order.
// NARROW: B has fewer than 2^27 columns, so (column << 5 | lane) fits 32 bits and the sort
// moves half as much through the shuffles.
//
// A row's work is a chain of five dependent loads (row number, A's offsets, A's columns, B's
// offsets, B's columns) and little else, so a warp walks the chain for its rows side by side: the
// loads of one link are issued for all of them before any is used.
template <bool NUMERIC, bool NARROW>
__global__ void __launch_bounds__(256) k_esc_small(CsrView A, CsrView B, const int32_t *__restrict__ row_list, int n_rows,
                                                   int32_t *__restrict__ row_count, const int32_t *__restrict__ c_rp,
                                                   int32_t *__restrict__ c_col, float *__restrict__ c_val) {
    constexpr int R = ESC_SMALL_ROWS;
    const int w = ((blockIdx.x * 256 + threadIdx.x) >> 5) * R;
    if (w >= n_rows) return;
    const int lane = lane_id();
    int32_t i[R], lo[R], hi[R], out[R];
    uint32_t my_col[R];
    float my_val[R];
    bool have[R];
#pragma unroll
    for (int r = 0; r < R; ++r) i[r] = w + r < n_rows ? ld_nc(row_list + w + r) : -1;
    bool one_round = true;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        lo[r] = hi[r] = out[r] = 0;
        if (i[r] >= 0) {
            lo[r] = ld_nc(A.rp + i[r]);
            hi[r] = ld_nc(A.rp + i[r] + 1);
            if (NUMERIC) out[r] = ld_nc(c_rp + i[r]);
        }
        one_round &= hi[r] - lo[r] <= 32;
        my_col[r] = 0;
        my_val[r] = 0.f;
        have[r] = false;
    }
    // Expansion, 32 entries of a row at a time (one round unless the row holds entries whose rows of B
    // are empty): lane l reads entry l and its row of B; the products of the round take the lanes
    // [base, base + total) in expansion order, each finding its entry among the round's non-empty
    // ones from the mask of slice starts.
    auto place = [&](int r, int base, int32_t b_lo, int len, float a) -> int {
        const int incl = warp_incl_sum(len);
        const int start = base + incl - len;                       // first lane of this entry's products
        const unsigned nonempty = __ballot_sync(FULL_MASK, len > 0);
        const unsigned starts = __reduce_or_sync(FULL_MASK, len > 0 ? 1u << start : 0u);  // the row has at most 32 products
        const int total = __shfl_sync(FULL_MASK, incl, 31);
        // the entry of lane `lane`'s product: the n-th non-empty one, n = slice starts at or before the lane
        const int nth = __popc(starts & (0xffffffffu >> (31 - lane)));
        const int owner = nth > 0 ? (int)__fns(nonempty, 0, nth) : 0;
        const int32_t o_lo = __shfl_sync(FULL_MASK, b_lo, owner);
        const int o_start = __shfl_sync(FULL_MASK, start, owner);
        const float o_a = __shfl_sync(FULL_MASK, a, owner);
        if (lane >= base && lane < base + total) {
            my_col[r] = (uint32_t)ld_nc(B.col + o_lo + (lane - o_start));
            if (NUMERIC) my_val[r] = o_a * ld_nc(B.val + o_lo + (lane - o_start));
            have[r] = true;
        }
        return total;
    };
    if (one_round) {  // uniform: every link of the chain for all rows at once
        int32_t j[R], b_lo[R], len[R];
        float a[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            j[r] = lo[r] + lane < hi[r] ? ld_nc(A.col + lo[r] + lane) : -1;
            a[r] = NUMERIC && j[r] >= 0 ? ld_nc(A.val + lo[r] + lane) : 0.f;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            b_lo[r] = len[r] = 0;
            if (j[r] >= 0) {
                b_lo[r] = ld_nc(B.rp + j[r]);
                len[r] = ld_nc(B.rp + j[r] + 1) - b_lo[r];
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) place(r, 0, b_lo[r], len[r], a[r]);
    } else {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            int base = 0;
            for (int32_t chunk = lo[r]; chunk < hi[r]; chunk += 32) {  // uniform across the warp
                int32_t b_lo = 0, len = 0;
                float a = 0.f;
                if (chunk + lane < hi[r]) {
                    const int32_t j = ld_nc(A.col + chunk + lane);
                    b_lo = ld_nc(B.rp + j);
                    len = ld_nc(B.rp + j + 1) - b_lo;
                    if (NUMERIC) a = ld_nc(A.val + chunk + lane);
                }
                base += place(r, base, b_lo, len, a);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        if (i[r] < 0) continue;  // uniform
        if (!NUMERIC) {
            // distinct columns: a lane counts if it is the first of the lanes that hold its column
            const unsigned peers = __match_any_sync(FULL_MASK, have[r] ? my_col[r] : 0x80000000u | (uint32_t)lane);
            const unsigned firsts = __ballot_sync(FULL_MASK, have[r] && lane == __ffs(peers) - 1);
            if (lane == 0) row_count[i[r]] = __popc(firsts);
            continue;
        }
        uint32_t col;
        int src;
        bool valid;
        if (NARROW) {
            uint32_t key = have[r] ? ((my_col[r] << 5) | (uint32_t)lane) : ~0u;
            key = warp_bitonic_sort32(key);
            col = key >> 5;
            src = (int)(key & 31u);
            valid = key != ~0u;
        } else {
            uint64_t key = have[r] ? (((uint64_t)my_col[r] << 32) | (uint32_t)lane) : ~0ull;
            key = warp_bitonic_sort(key);
            col = (uint32_t)(key >> 32);
            src = (int)(key & 31u);
            valid = key != ~0ull;
        }
        const uint32_t prev_col = __shfl_up_sync(FULL_MASK, col, 1);
        const bool head = valid && (lane == 0 || prev_col != col);
        const unsigned heads = __ballot_sync(FULL_MASK, head);
        float v = __shfl_sync(FULL_MASK, my_val[r], src);  // value of the product now at this lane
        float acc = v;
        // longest run of equal columns in this row (distance from a head to the next head or to
        // the end of the valid lanes): the summation loop needs no more steps than that
        const unsigned later = lane < 31 ? (heads >> (lane + 1)) : 0u;
        const int n_valid = __popc(__ballot_sync(FULL_MASK, valid));
        const int my_run = head ? (later ? __ffs(later) : n_valid - lane) : 0;
        const int longest = __reduce_max_sync(FULL_MASK, my_run);
        for (int t = 1; t < longest; ++t) {  // head lanes add their run in sorted (= expansion) order
            const float nv = __shfl_down_sync(FULL_MASK, v, t);
            if (t < my_run) acc += nv;
        }
        if (head) {
            const int pos = out[r] + __popc(heads & ((1u << lane) - 1u));
            c_col[pos] = (int32_t)col;
            c_val[pos] = acc;
        }
    }
}

// ------------------------------------------------------------------------ medium rows ----

// One CTA per row with at most MEDIUM_P products: expand into shared memory in expansion
// order, bitonic sort on (column << 32 | expansion index), then each run head sums its run.
template <bool NUMERIC>
__global__ void __launch_bounds__(MED_NT) k_esc_medium(CsrView A, CsrView B, const int32_t *__restrict__ row_list,
                                                       int32_t *__restrict__ row_count, const int32_t *__restrict__ c_rp,
                                                       int32_t *__restrict__ c_col, float *__restrict__ c_val) {
    __shared__ uint64_t keys[MEDIUM_P];
    __shared__ float vals[NUMERIC ? MEDIUM_P : 1];
    __shared__ int scan_tmp[40];
    const int tid = threadIdx.x;
    const int32_t i = ld_nc(row_list + blockIdx.x);
    const int32_t lo = ld_nc(A.rp + i), hi = ld_nc(A.rp + i + 1);

    int p_total = 0;
    for (int32_t chunk = lo; chunk < hi; chunk += MED_NT) {  // expand phase 2, MED_NT entries of A at a time
        const int32_t e = chunk + tid;
        int32_t b_lo = 0, len = 0;
        float a = 0.f;
        if (e < hi) {
            const int32_t j = ld_nc(A.col + e);
            b_lo = ld_nc(B.rp + j);
            len = ld_nc(B.rp + j + 1) - b_lo;
            if (NUMERIC) a = ld_nc(A.val + e);
        }
        int chunk_total;
        const int off = block_excl_sum<MED_NT>(len, scan_tmp, chunk_total);
        for (int q = 0; q < len; ++q) {
            const int idx = p_total + off + q;
            keys[idx] = ((uint64_t)(uint32_t)ld_nc(B.col + b_lo + q) << 32) | (uint32_t)idx;
            if (NUMERIC) vals[idx] = a * ld_nc(B.val + b_lo + q);
        }
        p_total += chunk_total;
    }
    int n2 = 2;
    while (n2 < p_total) n2 <<= 1;
    for (int p = p_total + tid; p < n2; p += MED_NT) keys[p] = ~0ull;
    __syncthreads();

    for (int k = 2; k <= n2; k <<= 1) {  // sort
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int p = tid; p < (n2 >> 1); p += MED_NT) {
                const int i1 = 2 * j * (p / j) + (p % j), i2 = i1 + j;
                const bool up = (i1 & k) == 0;
                const uint64_t x = keys[i1], y = keys[i2];
                if ((x > y) == up) {
                    keys[i1] = y;
                    keys[i2] = x;
                }
            }
            __syncthreads();
        }
    }

    // compress: thread t looks after sorted positions [t * per, (t + 1) * per)
    const int per = (n2 + MED_NT - 1) / MED_NT;
    const int p_lo = min(tid * per, p_total), p_hi = min(p_lo + per, p_total);
    int heads = 0;
    for (int p = p_lo; p < p_hi; ++p) heads += p == 0 || (uint32_t)(keys[p] >> 32) != (uint32_t)(keys[p - 1] >> 32);
    int unique;
    int rank = block_excl_sum<MED_NT>(heads, scan_tmp, unique);
    if (!NUMERIC) {
        if (tid == 0) row_count[i] = unique;
        return;
    }
    const int32_t out = ld_nc(c_rp + i);
    for (int p = p_lo; p < p_hi; ++p) {
        const uint32_t col = (uint32_t)(keys[p] >> 32);
        if (p == 0 || col != (uint32_t)(keys[p - 1] >> 32)) {
            float acc = vals[(uint32_t)keys[p]];
            for (int q = p + 1; q < p_total && (uint32_t)(keys[q] >> 32) == col; ++q) acc += vals[(uint32_t)keys[q]];
            c_col[out + rank] = (int32_t)col;
            c_val[out + rank] = acc;
            ++rank;
        }
    }
}

// ----------------------------------------------------------------- product walk ----

#ifndef ESC_WIN_ITEMS
#define ESC_WIN_ITEMS 4  // 32-product blocks a warp keeps in flight
#endif

// Walks a flat product range cut into segments: segment k covers the products
// [seg_off[k], seg_off[k + 1]) and they are the entries seg_start[k] ... of B, each multiplied
// by seg_a[k]; every segment is non-empty and seg_off[n_seg] == total. Called by all NT threads
// of the CTA. Every warp takes one contiguous share of the range (a multiple of 32 products) and
// moves through it 32 products at a time, lane = product, so the loads from B coalesce; the
// segment of the current block is warp-uniform state that only moves forward, and a block that
// lies inside one segment (the common case for long rows of B) needs no per-lane search.
// ESC_WIN_ITEMS blocks have their loads in flight together. f(column, value) gets every product.
template <int NT, bool WITH_VALUES, typename F>
__device__ __forceinline__ void walk_segments(const int *seg_off, const int *seg_start, const float *seg_a, int n_seg, int total,
                                              const CsrView &B, F f) {
    constexpr int NW = NT / 32;
    const int share = ((total + NW * 32 - 1) / (NW * 32)) * 32;
    int pb = warp_id() * share;
    const int pe = min(pb + share, total);
    if (pb >= pe) return;
    int k = 0;
    {  // largest k with seg_off[k] <= pb
        int h = n_seg - 1;
        while (k < h) {
            const int mid = (k + h + 1) >> 1;
            if (seg_off[mid] <= pb)
                k = mid;
            else
                h = mid - 1;
        }
    }
    int k_end = seg_off[k + 1];
    int delta = seg_start[k] - seg_off[k];  // position in B = delta + product index
    float k_a = WITH_VALUES ? seg_a[k] : 0.f;
    for (; pb < pe; pb += 32 * ESC_WIN_ITEMS) {
        while (pb >= k_end) {
            ++k;
            k_end = seg_off[k + 1];
            delta = seg_start[k] - seg_off[k];
            if (WITH_VALUES) k_a = seg_a[k];
        }
        if (pb + 32 * ESC_WIN_ITEMS <= min(k_end, pe)) {  // uniform: all the blocks lie inside segment k
            const int32_t *bc = B.col + (delta + pb + lane_id());
            const float *bvp = B.val + (delta + pb + lane_id());
            int32_t c[ESC_WIN_ITEMS];
            float bv[ESC_WIN_ITEMS];
#pragma unroll
            for (int it = 0; it < ESC_WIN_ITEMS; ++it) {
                c[it] = ld_nc(bc + 32 * it);
                bv[it] = WITH_VALUES ? ld_nc(bvp + 32 * it) : 0.f;
            }
#pragma unroll
            for (int it = 0; it < ESC_WIN_ITEMS; ++it) f(c[it], k_a * bv[it]);
            continue;
        }
        int32_t q[ESC_WIN_ITEMS];
        float av[ESC_WIN_ITEMS];
#pragma unroll
        for (int it = 0; it < ESC_WIN_ITEMS; ++it) {
            const int b = pb + 32 * it;
            q[it] = -1;
            av[it] = 0.f;
            if (b < pe) {
                while (b >= k_end) {
                    ++k;
                    k_end = seg_off[k + 1];
                    delta = seg_start[k] - seg_off[k];
                    if (WITH_VALUES) k_a = seg_a[k];
                }
                const int p = b + lane_id();
                if (b + 32 <= k_end) {
                    q[it] = delta + p;
                    av[it] = k_a;
                } else if (p < pe) {
                    int kk = k;
                    while (seg_off[kk + 1] <= p) ++kk;  // ends: seg_off[n_seg] == total > p
                    q[it] = seg_start[kk] + (p - seg_off[kk]);
                    if (WITH_VALUES) av[it] = seg_a[kk];
                }
            }
        }
        int32_t c[ESC_WIN_ITEMS];
        float bv[ESC_WIN_ITEMS];
#pragma unroll
        for (int it = 0; it < ESC_WIN_ITEMS; ++it) {
            c[it] = q[it] >= 0 ? ld_nc(B.col + q[it]) : 0;
            bv[it] = WITH_VALUES && q[it] >= 0 ? ld_nc(B.val + q[it]) : 0.f;
        }
#pragma unroll
        for (int it = 0; it < ESC_WIN_ITEMS; ++it)
            if (q[it] >= 0) f(c[it], av[it] * bv[it]);
    }
}

// ------------------------------------------------------------- ranked and heavy rows ----

constexpr int RK_WORDS = 8192;                     // bitmap words of one column window in shared memory
constexpr int RK_WINDOW_COLS = RK_WORDS * 32;      // 262144 columns per window
constexpr size_t RK_PTR_BUDGET = size_t(1) << 30;  // bytes of the window pointer table; beyond it windows are searched on the fly
constexpr int RK_NT = 256, HEAVY_NT = 512;         // threads of a CTA for rows up to / above RANKED_P products
constexpr size_t HEAVY_SMEM_NUMERIC = 104 * 1024;  // dynamic shared memory of a numeric heavy-row CTA: two per SM
#ifndef ESC_RANKED_SMEM_KB
#define ESC_RANKED_SMEM_KB 0                       // of a numeric ranked-row CTA; 0: bitmap and ranks only, four per SM
#endif

// First index in [lo, hi) whose column is >= key (hi if none).
__device__ __forceinline__ int32_t first_col_at_least(const int32_t *__restrict__ col, int32_t lo, int32_t hi, int64_t key) {
    while (lo < hi) {
        const int32_t mid = lo + ((hi - lo) >> 1);
        if (ld_nc(col + mid) < key)
            lo = mid + 1;
        else
            hi = mid;
    }
    return lo;
}

// Window pointer table of B, built only for matrices wider than one window:
// ptr[j * (n_win + 1) + w] = first position of row j whose column is >= w * RK_WINDOW_COLS
// (w = 0 .. n_win), so that window w of row j is [ptr[w], ptr[w + 1]).
__global__ void __launch_bounds__(256) k_esc_window_ptr(CsrView B, int32_t b_rows, int n_win, int32_t *__restrict__ ptr) {
    const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
    const int per = n_win + 1;
    if (t >= (int64_t)b_rows * per) return;
    const int32_t j = (int32_t)(t / per);
    const int w = (int)(t - (int64_t)j * per);
    const int32_t lo = ld_nc(B.rp + j), hi = ld_nc(B.rp + j + 1);
    ptr[t] = w == 0 ? lo : w == n_win ? hi : first_col_at_least(B.col, lo, hi, (int64_t)w * RK_WINDOW_COLS);
}

// One CTA per row, column window by column window (one window unless B is wider than
// RK_WINDOW_COLS). Per window: pass 1 walks the row's products and sets a bit per produced column
// in a shared-memory bitmap; a popcount scan turns the bitmap into the rank of every column within
// the result row and the columns are written out; pass 2 walks the products again and adds each
// one into its final position: the first `acc_slots` positions of the window accumulate in shared
// memory (float32 atomics there run several times faster than reductions in L2) and are stored
// with coalesced writes at the end, the positions beyond them take a float32 reduction in L2 on
// the row's own output range, which this CTA zeroed first. Symbolic: pass 1 and the count only.
//
// Ranks are kept per 64 columns, in 16 bits relative to the first word of the warp that scanned
// them (a warp scans `1 << wshift` consecutive words, at most 32768 columns), plus one base per warp.
//
// `row_list` is read from the front for the first n_front CTAs and from the back (list_len - 1
// downwards) for the others. `words`: bitmap words in use, (NT / 32) << wshift, covering a window.
// `win_ptr` is the window pointer table, or null (one window, or a table beyond its budget).
// `cache` (one window only), when given, carries the bitmaps from the symbolic launch to the
// numeric launch of one call, `words` per CTA: the symbolic launch stores them, the numeric
// launch loads them instead of walking the products a first time.
template <bool NUMERIC, int NT>
__global__ void __launch_bounds__(NT) k_esc_ranked(CsrView A, CsrView B, const int32_t *__restrict__ win_ptr, int n_win,
                                                   const int32_t *__restrict__ row_list, int32_t list_len, int n_front, int words,
                                                   int wshift, int acc_slots, uint32_t *cache, int32_t *__restrict__ row_count,
                                                   const int32_t *__restrict__ c_rp, int32_t *__restrict__ c_col,
                                                   float *__restrict__ c_val) {
    extern __shared__ __align__(16) unsigned char rk_smem[];
    uint32_t *bitmap = reinterpret_cast<uint32_t *>(rk_smem);
    const uint64_t *bitmap64 = reinterpret_cast<const uint64_t *>(rk_smem);  // the same bits, 64 columns per element
    uint16_t *rank16 = reinterpret_cast<uint16_t *>(rk_smem + (size_t)words * 4);  // one rank per 64 columns
    float *acc = reinterpret_cast<float *>(rk_smem + (size_t)words * 5);
    __shared__ int seg_off[NT + 1];
    __shared__ int seg_start[NT];
    __shared__ float seg_a[NUMERIC ? NT : 1];
    __shared__ int scan_tmp[72];
    __shared__ int warp_base[NT / 32];
    const int tid = threadIdx.x;
    const int r = blockIdx.x;
    const int32_t i = ld_nc(row_list + (r < n_front ? r : list_len - 1 - (r - n_front)));
    const int32_t lo = ld_nc(A.rp + i), hi = ld_nc(A.rp + i + 1);
    const bool one_chunk = hi - lo <= NT;  // then a thread keeps its entry, and pass 2 reuses the segments of pass 1
    const int per = n_win + 1;
    int32_t my_j = -1;
    float my_a = 0.f;
    if (one_chunk && lo + tid < hi) {
        my_j = ld_nc(A.col + lo + tid);
        if (NUMERIC) my_a = ld_nc(A.val + lo + tid);
    }
    int64_t out = NUMERIC ? (int64_t)ld_nc(c_rp + i) : 0;  // next free position of the row (count so far, symbolic)

    for (int w = 0; w < n_win; ++w) {
        const int32_t c_first = w * RK_WINDOW_COLS;  // below 2^31: it is a column of B

        // builds the segments of one chunk of the row's entries (their rows of B inside the window)
        // and walks them; returns whether the window holds any product
        auto pass = [&](bool build, auto f) -> bool {
            bool any = false;
            for (int32_t chunk = lo; chunk < hi; chunk += NT) {
                int n_seg, total;
                if (build) {
                    int32_t j = my_j;
                    float a = my_a;
                    if (!one_chunk) {
                        j = -1;
                        if (chunk + tid < hi) {
                            j = ld_nc(A.col + chunk + tid);
                            if (NUMERIC) a = ld_nc(A.val + chunk + tid);
                        }
                    }
                    int32_t s = 0, len = 0;
                    if (j >= 0) {
                        if (n_win == 1) {
                            s = ld_nc(B.rp + j);
                            len = ld_nc(B.rp + j + 1) - s;
                        } else if (win_ptr) {
                            s = ld_nc(win_ptr + (int64_t)j * per + w);
                            len = ld_nc(win_ptr + (int64_t)j * per + w + 1) - s;
                        } else {
                            const int32_t b_lo = ld_nc(B.rp + j), b_hi = ld_nc(B.rp + j + 1);
                            s = w == 0 ? b_lo : first_col_at_least(B.col, b_lo, b_hi, c_first);
                            len = (w == n_win - 1 ? b_hi : first_col_at_least(B.col, s, b_hi, (int64_t)c_first + RK_WINDOW_COLS)) - s;
                        }
                    }
                    int k_idx, off;
                    block_excl_sum2<NT>(len > 0 ? 1 : 0, len, scan_tmp, k_idx, off, n_seg, total);
                    if (len > 0) {
                        seg_off[k_idx] = off;
                        seg_start[k_idx] = s;
                        if (NUMERIC) seg_a[k_idx] = a;
                    }
                    if (tid == 0) {
                        seg_off[n_seg] = total;
                        scan_tmp[70] = n_seg;
                    }
                    __syncthreads();
                } else {
                    n_seg = scan_tmp[70];
                    total = seg_off[n_seg];
                }
                any |= total > 0;
                walk_segments<NT, NUMERIC>(seg_off, seg_start, seg_a, n_seg, total, B, f);
                __syncthreads();  // the segment arrays are rewritten by the next chunk
            }
            return any;
        };

        uint4 *cached = cache ? reinterpret_cast<uint4 *>(cache + (size_t)r * words) : nullptr;
        const bool from_cache = NUMERIC && cached != nullptr;
        if (from_cache) {
            for (int c = tid; c < words / 4; c += NT) reinterpret_cast<uint4 *>(bitmap)[c] = __ldcs(cached + c);
            __syncthreads();
        } else {
            for (int c = tid; c < words / 4; c += NT) reinterpret_cast<uint4 *>(bitmap)[c] = make_uint4(0u, 0u, 0u, 0u);
            __syncthreads();
            const bool any = pass(true, [&](int32_t col, float) {
                const uint32_t cw = (uint32_t)(col - c_first);
                atomicOr(bitmap + (cw >> 5), 1u << (cw & 31u));
            });
            if (!any) continue;  // uniform
            if (!NUMERIC && cached)
                for (int c = tid; c < words / 4; c += NT) __stcs(cached + c, reinterpret_cast<const uint4 *>(bitmap)[c]);
        }

        // warp v looks after the words [v << wshift, (v + 1) << wshift), 64 columns per lane and step
        const int groups = 1 << (wshift - 6);
        const int dbase = warp_id() << (wshift - 1);  // first 64-bit element of the warp
        int mine = 0;
#pragma unroll 4
        for (int g = 0; g < groups; ++g) mine += __popcll(bitmap64[dbase + g * 32 + lane_id()]);
        int cnt;
        const int excl = block_excl_sum<NT>(mine, scan_tmp, cnt);
        if (!NUMERIC) {
            out += cnt;
            continue;
        }
        const int my_base = __shfl_sync(FULL_MASK, excl, 0);  // columns of the window before this warp's words
        if (lane_id() == 0) warp_base[warp_id()] = my_base;
        int running = 0;
#pragma unroll 2
        for (int g = 0; g < groups; ++g) {
            const int idx = dbase + g * 32 + lane_id();
            uint64_t bits = bitmap64[idx];
            const int c = __popcll(bits);
            const int incl = warp_incl_sum(c);
            const int first = running + incl - c;
            rank16[idx] = (uint16_t)first;
            // the lane's columns, in 32-bit halves and 32-bit positions (the loop is the hot part of
            // the scan: one trip per result entry)
            int32_t *gcol = c_col + (out + my_base);
            int pos = first;
            uint32_t half = (uint32_t)bits;
            int32_t col0 = c_first + idx * 64;
            while (half) {
                gcol[pos++] = col0 + (__ffs((int)half) - 1);
                half &= half - 1u;
            }
            half = (uint32_t)(bits >> 32);
            col0 += 32;
            while (half) {
                gcol[pos++] = col0 + (__ffs((int)half) - 1);
                half &= half - 1u;
            }
            running += __shfl_sync(FULL_MASK, incl, 31);
        }
        float *row_val = c_val + out;  // the window's part of the row; its length fits 32 bits
        const int in_acc = min(cnt, acc_slots);
        for (int k = tid; k < in_acc; k += NT) acc[k] = 0.f;
        for (int k = acc_slots + tid; k < cnt; k += NT) row_val[k] = 0.f;  // positions beyond the shared accumulator
        __syncthreads();  // ranks complete, output zeroed (the reductions below come from this CTA only)
        pass(!one_chunk || from_cache, [&](int32_t col, float v) {
            const uint32_t cw = (uint32_t)(col - c_first);
            const uint32_t dw = cw >> 6;
            const uint64_t bits = bitmap64[dw];
            const uint32_t pos = (uint32_t)warp_base[dw >> (wshift - 1)] + rank16[dw] + __popcll(bits & ((1ull << (cw & 63u)) - 1ull));
            if (pos < (uint32_t)acc_slots)
                atomicAdd(acc + pos, v);      // shared memory
            else
                atomicAdd(row_val + pos, v);  // reduction in L2
        });
        // the pass ends with a barrier: every sum is in place
        for (int k = tid; k < in_acc; k += NT) row_val[k] = acc[k];
        out += cnt;
    }
    if (!NUMERIC && tid == 0) row_count[i] = (int32_t)out;
}

// Turns the exclusive prefix of the per-row counts into row offsets (rows + 1 entries).
__global__ void __launch_bounds__(256) k_esc_row_offsets(const int32_t *__restrict__ excl, const long long *__restrict__ total,
                                                         int32_t rows, int32_t *__restrict__ c_rp) {
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i < rows) c_rp[i] = excl[i];
    if (i == rows) c_rp[rows] = (int32_t)min(*total, (long long)INT32_MAX);
}

// ------------------------------------------------------------------------ host driver ----

// Bitmap words a ranked-row CTA keeps for B's column count (one window's worth at most): every
// warp scans a power of two of words, at least 64. `wshift` receives log2 of that count.
int ranked_words(int nt, int32_t b_cols, int *wshift = nullptr) {
    const int64_t need = (std::min<int64_t>(b_cols, RK_WINDOW_COLS) + 31) / 32;
    int shift = 6;
    while (((int64_t)(nt / 32) << shift) < need) ++shift;
    if (wshift) *wshift = shift;
    return (nt / 32) << shift;
}


int check_operand(const nb200_csr *m) {
    if (!m || m->rows < 0 || m->cols < 0 || m->nnz < 0 || !m->row_ptr) return NB200_E_BADARG;
    if (m->nnz > 0 && (!m->col || !m->val)) return NB200_E_BADARG;
    return NB200_OK;
}

struct EscPlan {
    Workspace *ws;
    RowLists lists;
    int32_t *row_count;    // rows entries (symbolic pass)
    uint64_t *scan_block;  // FusedCtl + one word per scan CTA
    int scan_ctas;
    EscCtl *ctl;
    int n_win;             // column windows of RK_WINDOW_COLS
    int32_t *win_ptr;      // window pointer table (null: one window, or beyond its budget)
    uint32_t *cache_ranked, *cache_heavy;  // bitmaps carried from the symbolic to the numeric pass (or null)
    Workspace *cache_ws;   // pool block of the bitmaps (null without them)
    EscCtl host;           // counters read back after the row-work kernel
};

// Bins the rows (kernel + one read-back) and carves the scratch of a symbolic pass, a numeric
// pass, or one after the other. `counts`: rows without products get their count written
// (needed by the symbolic pass).
constexpr size_t BITMAP_CACHE_BUDGET = size_t(8) << 30;  // bytes of bitmaps carried between the passes of one call

int esc_prepare(const nb200_csr *a, const nb200_csr *b, bool counts, bool carry_bitmaps, cudaStream_t stream, EscPlan *plan) {
    const int32_t rows = a->rows;
    const int64_t n_win = std::max<int64_t>(1, ((int64_t)b->cols + RK_WINDOW_COLS - 1) / RK_WINDOW_COLS);
    const size_t ptr_entries = n_win > 1 ? (size_t)b->rows * (size_t)(n_win + 1) : 0;
    const bool with_table = ptr_entries > 0 && ptr_entries * 4 <= RK_PTR_BUDGET;
    const int scan_ctas = (rows + SCAN_NT * SCAN_VT - 1) / (SCAN_NT * SCAN_VT);
    Carver sizes;
    for (int q = 0; q < 4; ++q) sizes.take<int32_t>((size_t)rows);
    sizes.take<int32_t>((size_t)rows + 1);
    sizes.take<uint64_t>((size_t)scan_ctas + 8);
    sizes.take<EscCtl>(1);
    if (with_table) sizes.take<int32_t>(ptr_entries);
    const int prefix_ctas = (int)(((int64_t)a->nnz + 1 + 2047) / 2048);
    sizes.take<unsigned long long>((size_t)a->nnz + 1);
    sizes.take<uint64_t>((size_t)prefix_ctas + 8);
    int st;
    if ((st = acquire_workspace(stream, sizes.used(), &plan->ws))) return st;
    Carver carve(plan->ws->dev);
    plan->lists.small_rows = carve.take<int32_t>((size_t)rows);
    plan->lists.medium_rows = carve.take<int32_t>((size_t)rows);
    plan->lists.ranked_rows = carve.take<int32_t>((size_t)rows);
    plan->lists.heavy_rows = carve.take<int32_t>((size_t)rows);
    plan->row_count = carve.take<int32_t>((size_t)rows + 1);
    plan->scan_block = carve.take<uint64_t>((size_t)scan_ctas + 8);
    plan->scan_ctas = scan_ctas;
    plan->ctl = carve.take<EscCtl>(1);
    plan->n_win = (int)n_win;
    plan->win_ptr = with_table ? carve.take<int32_t>(ptr_entries) : nullptr;
    unsigned long long *prefix = carve.take<unsigned long long>((size_t)a->nnz + 1);
    uint64_t *prefix_block = carve.take<uint64_t>((size_t)prefix_ctas + 8);

    NB200_CUDA(cudaMemsetAsync(plan->ctl, 0, sizeof(EscCtl), stream));
    NB200_CUDA(cudaMemsetAsync(prefix_block, 0, sizeof(uint64_t) * ((size_t)prefix_ctas + 8), stream));
    const CsrView A{a->row_ptr, a->col, a->val}, B{b->row_ptr, b->col, b->val};
    const bool short_rows = (int64_t)a->nnz <= 8 * (int64_t)rows;  // then a lane walks its row faster than a prefix pass pays
    if (rows > 0 && short_rows) {
        LaunchScope scope("esc_rowwork", stream);
        k_esc_rowwork_walk<<<(rows + 255) / 256, 256, 0, stream>>>(A, B, rows, counts ? plan->row_count : nullptr, plan->lists, plan->ctl);
        NB200_CUDA(cudaGetLastError());
    } else if (rows > 0) {
        {
            LaunchScope scope("esc_product_prefix", stream);
            k_esc_product_prefix<<<prefix_ctas, 256, 0, stream>>>(A, B, a->nnz, prefix, prefix_block + 4, reinterpret_cast<FusedCtl *>(prefix_block));
        }
        LaunchScope scope("esc_rowwork", stream);
        k_esc_rowwork<<<(rows + 255) / 256, 256, 0, stream>>>(A, prefix, rows, counts ? plan->row_count : nullptr, plan->lists, plan->ctl);
        NB200_CUDA(cudaGetLastError());
    }
    NB200_CUDA(cudaMemcpyAsync(plan->ws->host, plan->ctl, sizeof(EscCtl), cudaMemcpyDeviceToHost, stream));
    NB200_CUDA(cudaMemcpyAsync(plan->ws->host + 16, prefix_block, sizeof(FusedCtl), cudaMemcpyDeviceToHost, stream));
    NB200_CUDA(cudaStreamSynchronize(stream));
    std::memcpy(&plan->host, plan->ws->host, sizeof(EscCtl));
    {   // a prefix whose look-back gave up leaves rows with wrong product counts: nothing may be built on them
        FusedCtl hp;
        std::memcpy(&hp, plan->ws->host + 16, sizeof(hp));
        if (hp.status.error != 0) return note_timeout(hp.status.error, hp.status.detail, "spgemm product prefix");
    }
    if (with_table && plan->host.n_ranked + plan->host.n_giant + plan->host.n_heavy > 0) {
        LaunchScope scope("esc_window_ptr", stream);
        k_esc_window_ptr<<<(unsigned)((ptr_entries + 255) / 256), 256, 0, stream>>>(B, b->rows, plan->n_win, plan->win_ptr);
        NB200_CUDA(cudaGetLastError());
    }
    plan->cache_ranked = plan->cache_heavy = nullptr;
    plan->cache_ws = nullptr;
    if (carry_bitmaps && plan->n_win == 1) {
        // a second pool block: its size is only known now, and the first must not move
        const size_t ranked_bytes = (size_t)plan->host.n_ranked * ranked_words(RK_NT, b->cols) * 4;
        const size_t heavy_bytes = ((size_t)plan->host.n_giant + plan->host.n_heavy) * ranked_words(HEAVY_NT, b->cols) * 4;
        if (ranked_bytes + heavy_bytes > 0 && ranked_bytes + heavy_bytes <= BITMAP_CACHE_BUDGET) {
            Carver cache_sizes;
            cache_sizes.take<uint32_t>(ranked_bytes / 4);
            cache_sizes.take<uint32_t>(heavy_bytes / 4);
            Workspace *cache_ws = nullptr;
            const int cache_st = acquire_workspace(stream, cache_sizes.used(), &cache_ws, 3);
            if (cache_st == NB200_OK) {  // without room the numeric pass walks the products twice, as it does on its own
                Carver cache_carve(cache_ws->dev);
                plan->cache_ranked = ranked_bytes ? cache_carve.take<uint32_t>(ranked_bytes / 4) : nullptr;
                plan->cache_heavy = heavy_bytes ? cache_carve.take<uint32_t>(heavy_bytes / 4) : nullptr;
                plan->cache_ws = cache_ws;
            } else if (cache_st != NB200_E_NOMEM) {
                return cache_st;
            }
        }
    }
    return NB200_OK;
}

template <bool NUMERIC, int NT>
int launch_ranked(const CsrView &A, const CsrView &B, const EscPlan &plan, int32_t b_cols, const int32_t *list, int32_t list_len,
                  int n_front, int n_rows, uint32_t *cache, int32_t *count, const int32_t *c_rp, int32_t *c_col, float *c_val,
                  cudaStream_t stream) {
    int wshift = 5;
    const int words = ranked_words(NT, b_cols, &wshift);
    // numeric: whatever the bitmap and the ranks leave of the CTA's shared memory accumulates sums
    // The lighter rows do better without a shared accumulator: their CTAs are bound by the latency of
    // a row's short phases, and four CTAs per SM hide more of it than three with an accumulator
    // (7.7 against 9.2 ms on configuration 4a); the heavy rows gain (10.7 -> 7.5 ms).
    const size_t budget = std::max(NT == HEAVY_NT ? HEAVY_SMEM_NUMERIC : (size_t)ESC_RANKED_SMEM_KB * 1024, (size_t)words * 5);
    const int acc_slots = NUMERIC ? (int)((budget - (size_t)words * 5) / 4 / NT) * NT : 0;
    const size_t smem = NUMERIC ? (size_t)words * 5 + (size_t)acc_slots * 4 : (size_t)words * 4;
    NB200_CUDA(cudaFuncSetAttribute(k_esc_ranked<NUMERIC, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)(NUMERIC ? budget : (size_t)RK_WORDS * 4)));
    k_esc_ranked<NUMERIC, NT><<<n_rows, NT, smem, stream>>>(A, B, plan.win_ptr, plan.n_win, list, list_len, n_front, words, wshift,
                                                          acc_slots, cache, count, c_rp, c_col, c_val);
    NB200_CUDA(cudaGetLastError());
    return NB200_OK;
}

template <bool NUMERIC>
int esc_run_bins(const nb200_csr *a, const nb200_csr *b, const EscPlan &plan, const nb200_csr *c, cudaStream_t stream) {
    const CsrView A{a->row_ptr, a->col, a->val}, B{b->row_ptr, b->col, b->val};
    int32_t *count = NUMERIC ? nullptr : plan.row_count;
    const int32_t *c_rp = NUMERIC ? c->row_ptr : nullptr;
    int32_t *c_col = NUMERIC ? c->col : nullptr;
    float *c_val = NUMERIC ? c->val : nullptr;
    int st;
    const int n_heavy = plan.host.n_giant + plan.host.n_heavy;
    if (n_heavy > 0) {  // first: the heaviest rows take longest
        LaunchScope scope(NUMERIC ? "esc_heavy_numeric" : "esc_heavy_symbolic", stream);
        if ((st = launch_ranked<NUMERIC, HEAVY_NT>(A, B, plan, b->cols, plan.lists.heavy_rows, a->rows, plan.host.n_giant, n_heavy,
                                                             plan.cache_heavy, count, c_rp, c_col, c_val, stream)))
            return st;
    }
    if (plan.host.n_ranked > 0) {
        LaunchScope scope(NUMERIC ? "esc_ranked_numeric" : "esc_ranked_symbolic", stream);
        if ((st = launch_ranked<NUMERIC, RK_NT>(A, B, plan, b->cols, plan.lists.ranked_rows, a->rows, plan.host.n_ranked,
                                                          plan.host.n_ranked, plan.cache_ranked, count, c_rp, c_col, c_val, stream)))
            return st;
    }
    if (plan.host.n_medium > 0) {
        LaunchScope scope(NUMERIC ? "esc_medium_numeric" : "esc_medium_symbolic", stream);
        k_esc_medium<NUMERIC><<<plan.host.n_medium, MED_NT, 0, stream>>>(A, B, plan.lists.medium_rows, count, c_rp, c_col, c_val);
        NB200_CUDA(cudaGetLastError());
    }
    if (plan.host.n_small > 0) {
        LaunchScope scope(NUMERIC ? "esc_small_numeric" : "esc_small_symbolic", stream);
        const int warps = plan.host.n_small;  // rows on the list
        const int small_warps = (warps + ESC_SMALL_ROWS - 1) / ESC_SMALL_ROWS;
        if (b->cols < (1 << 27))
            k_esc_small<NUMERIC, true><<<(small_warps + 7) / 8, 256, 0, stream>>>(A, B, plan.lists.small_rows, warps, count, c_rp, c_col, c_val);
        else
            k_esc_small<NUMERIC, false><<<(small_warps + 7) / 8, 256, 0, stream>>>(A, B, plan.lists.small_rows, warps, count, c_rp, c_col, c_val);
        NB200_CUDA(cudaGetLastError());
    }
    return NB200_OK;
}

// The plan of the latest symbolic pass, kept for the numeric pass that normally follows it on the
// same operands: the bins, the window pointer table and the bitmaps are then not computed again.
// It is used only if the operand arrays, sizes, device and stream are the same, the result's row
// offsets are the array that symbolic pass filled (with the length it reported), and neither pool
// block was handed out to anyone in between (their generations are unchanged). The patterns of A
// and B must not have been rewritten in place between the two passes; their values may change.
struct SavedPlan {
    bool valid = false;
    EscPlan plan{};
    const void *a_rp = nullptr, *a_col = nullptr, *b_rp = nullptr, *b_col = nullptr, *c_rp = nullptr;
    int32_t a_rows = 0, a_nnz = 0, b_rows = 0, b_cols = 0, b_nnz = 0, c_nnz = 0;
    cudaStream_t stream = nullptr;
    int device = -1;
    uint64_t gen_main = 0, gen_cache = 0, epoch = 0;
};
std::mutex g_saved_mutex;
SavedPlan g_saved;

void save_plan(const nb200_csr *a, const nb200_csr *b, const nb200_csr *c, const EscPlan &plan, cudaStream_t stream) {
    std::lock_guard<std::mutex> g(g_saved_mutex);
    g_saved.valid = cudaGetDevice(&g_saved.device) == cudaSuccess;
    g_saved.plan = plan;
    g_saved.a_rp = a->row_ptr, g_saved.a_col = a->col, g_saved.b_rp = b->row_ptr, g_saved.b_col = b->col;
    g_saved.c_rp = c->row_ptr, g_saved.c_nnz = c->nnz;
    g_saved.a_rows = a->rows, g_saved.a_nnz = a->nnz, g_saved.b_rows = b->rows, g_saved.b_cols = b->cols, g_saved.b_nnz = b->nnz;
    g_saved.stream = stream;
    g_saved.epoch = workspace_epoch();
    g_saved.gen_main = plan.ws->generation;
    g_saved.gen_cache = plan.cache_ws ? plan.cache_ws->generation : 0;
}

bool take_saved_plan(const nb200_csr *a, const nb200_csr *b, const nb200_csr *c, cudaStream_t stream, EscPlan *out) {
    std::lock_guard<std::mutex> g(g_saved_mutex);
    int dev = -1;
    if (!g_saved.valid || g_saved.epoch != workspace_epoch()) return false;  // the pool blocks may be gone
    if (cudaGetDevice(&dev) != cudaSuccess || dev != g_saved.device || stream != g_saved.stream) return false;
    if (a->row_ptr != g_saved.a_rp || a->col != g_saved.a_col || b->row_ptr != g_saved.b_rp || b->col != g_saved.b_col) return false;
    if (c->row_ptr != g_saved.c_rp || c->nnz != g_saved.c_nnz) return false;  // row offsets obtained elsewhere: recompute
    if (a->rows != g_saved.a_rows || a->nnz != g_saved.a_nnz || b->rows != g_saved.b_rows || b->cols != g_saved.b_cols ||
        b->nnz != g_saved.b_nnz)
        return false;
    if (g_saved.plan.ws->generation != g_saved.gen_main) return false;
    if (g_saved.plan.cache_ws && g_saved.plan.cache_ws->generation != g_saved.gen_cache) return false;
    *out = g_saved.plan;
    return true;
}

// `keep`: if given, the plan is handed back, so that a numeric pass that follows at once
// (nothing else touching the stream's scratch in between) skips the binning.
int spgemm_symbolic(const nb200_csr *a, const nb200_csr *b, nb200_csr *c, int64_t *products, void *stream_v, EscPlan *keep = nullptr) {
    int st;
    if ((st = check_operand(a)) || (st = check_operand(b))) return st;
    if (!c || !c->row_ptr || a->cols != b->rows) return NB200_E_BADARG;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    c->rows = a->rows;
    c->cols = b->cols;
    c->nnz = 0;
    if (products) *products = 0;
    if (a->rows == 0) {
        NB200_CUDA(cudaMemsetAsync(c->row_ptr, 0, sizeof(int32_t), stream));
        return NB200_OK;
    }
    EscPlan plan{};
    if ((st = esc_prepare(a, b, true, true, stream, &plan))) return st;
    if (keep) *keep = plan;
    if (products) *products = (int64_t)plan.host.products;
    if ((st = esc_run_bins<false>(a, b, plan, nullptr, stream))) return st;
    FusedCtl *scan_ctl = reinterpret_cast<FusedCtl *>(plan.scan_block);
    NB200_CUDA(cudaMemsetAsync(plan.scan_block, 0, sizeof(uint64_t) * ((size_t)plan.scan_ctas + 4), stream));
    {
        LaunchScope scope("scan_lookback", stream);
        k_scan_lookback<<<plan.scan_ctas, SCAN_NT, 0, stream>>>(plan.row_count, a->rows, plan.scan_block + 4, scan_ctl);
        NB200_CUDA(cudaGetLastError());
    }
    {
        LaunchScope scope("esc_row_offsets", stream);
        k_esc_row_offsets<<<(a->rows + 256) / 256, 256, 0, stream>>>(plan.row_count, &scan_ctl->total, a->rows, c->row_ptr);
        NB200_CUDA(cudaGetLastError());
    }
    NB200_CUDA(cudaMemcpyAsync(plan.ws->host, scan_ctl, sizeof(FusedCtl), cudaMemcpyDeviceToHost, stream));
    NB200_CUDA(cudaStreamSynchronize(stream));
    FusedCtl h;
    std::memcpy(&h, plan.ws->host, sizeof(h));
    if (h.status.error != 0) return note_timeout(h.status.error, h.status.detail, "spgemm row scan");
    const int64_t nnz = h.total;
    if (nnz > INT32_MAX) return NB200_E_OVERFLOW;
    c->nnz = (int32_t)nnz;
    save_plan(a, b, c, plan, stream);
    return NB200_OK;
}

int spgemm_numeric(const nb200_csr *a, const nb200_csr *b, nb200_csr *c, void *stream_v, const EscPlan *kept = nullptr) {
    int st;
    if ((st = check_operand(a)) || (st = check_operand(b))) return st;
    if (!c || !c->row_ptr || a->cols != b->rows || c->nnz < 0) return NB200_E_BADARG;
    if (c->nnz > 0 && (!c->col || !c->val)) return NB200_E_BADARG;
    if (a->rows == 0 || c->nnz == 0) return NB200_OK;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    if (kept) return esc_run_bins<true>(a, b, *kept, c, stream);
    EscPlan plan{};
    if (take_saved_plan(a, b, c, stream, &plan)) return esc_run_bins<true>(a, b, plan, c, stream);
    if ((st = esc_prepare(a, b, false, false, stream, &plan))) return st;
    return esc_run_bins<true>(a, b, plan, c, stream);
}

}  // namespace

}  // namespace nb200

using namespace nb200;

extern "C" {

int nb200_spgemm_f32_symbolic(const nb200_csr *a, const nb200_csr *b, nb200_csr *c, int64_t *products, void *stream) {
    return spgemm_symbolic(a, b, c, products, stream);
}

int nb200_spgemm_f32_numeric(const nb200_csr *a, const nb200_csr *b, nb200_csr *c, void *stream) {
    return spgemm_numeric(a, b, c, stream);
}

int nb200_spgemm_f32(const nb200_csr *a, const nb200_csr *b, nb200_csr *c, int32_t, int32_t, void *stream_v) {
    if (!a || !c) return NB200_E_BADARG;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    c->row_ptr = nullptr;
    c->col = nullptr;
    c->val = nullptr;
    NB200_CUDA(cudaMallocAsync(reinterpret_cast<void **>(&c->row_ptr), sizeof(int32_t) * ((size_t)std::max(a->rows, 0) + 1), stream));
    EscPlan plan{};
    int st = spgemm_symbolic(a, b, c, nullptr, stream_v, &plan);
    if (st == NB200_OK && c->nnz > 0) {
        cudaError_t e = cudaMallocAsync(reinterpret_cast<void **>(&c->col), sizeof(int32_t) * (size_t)c->nnz, stream);
        if (e == cudaSuccess) e = cudaMallocAsync(reinterpret_cast<void **>(&c->val), sizeof(float) * (size_t)c->nnz, stream);
        if (e != cudaSuccess) st = note_cuda_error(e, "cudaMallocAsync");
        else st = spgemm_numeric(a, b, c, stream_v, &plan);
    }
    if (st != NB200_OK) {
        if (c->row_ptr) cudaFreeAsync(c->row_ptr, stream);
        if (c->col) cudaFreeAsync(c->col, stream);
        if (c->val) cudaFreeAsync(c->val, stream);
        c->row_ptr = c->col = nullptr;
        c->val = nullptr;
    }
    return st;
}

}  // extern "C"
