// SpGEMM C = A * B by expand - sort - compress, row by row.
//
// What the reference does (GPU only, compiler.cpp:145-148): expand every product
// a.values[p] * b.values[q] with key k = b.cols[q] in (i, j ascending, k ascending) order
// (src/backend/compute.cpp:526-611), sort each row's products by k with a global segmented sort
// (src/backend/stitch_and_generate_gpu.cpp:79-94), flag run heads, scan, and sum runs with
// warp shuffles plus atomics (:96-124, :257-363). All its counters are int32 and it
// materialises every product in HBM.
//
// Here rows are binned by their product count P_i (64-bit counters throughout) and each bin
// keeps its products on chip:
//   small   P_i <= 32     one warp per row: products in registers, bitonic sort by shuffles
//   medium  P_i <= 2048   one CTA per row: products in shared memory, bitonic sort there
//   long    P_i  > 2048   a dense accumulator per row in global memory (bitmap + float32 values
//                         over the column range), filled with atomics, compacted by a bitmap scan
//   huge    P_i  > 1024 per window of 16384 columns: the row is cut into column windows and
//                         each (row, window) unit accumulates in shared memory (float32 atomics
//                         there), so the products of the heaviest rows never reach L2 or HBM
// Two passes: symbolic (unique columns per row -> row offsets by a scan) and numeric (fill).
// Small and medium rows sum equal-column products in expansion order (ascending j), a fixed
// order; long and huge rows sum with float32 atomics, like the reference does for every row.
#include <algorithm>
#include <climits>
#include <cstring>

#include "merge_common.cuh"

namespace nb200 {

namespace {

constexpr int SMALL_P = 32;
#ifndef ESC_MEDIUM_P
#define ESC_MEDIUM_P 2048
#endif
constexpr int MEDIUM_P = ESC_MEDIUM_P;
constexpr int MED_NT = 128;
#ifndef ESC_LONG_NT
#define ESC_LONG_NT 512
#endif
#ifndef ESC_LONG_SLOTS
#define ESC_LONG_SLOTS (4 * 148)  // with 512 threads each: every SM fully occupied; the path is bound by atomic latency
#endif
constexpr int LONG_NT = ESC_LONG_NT;
// Accumulator type of the long-row path: float32 atomics, as in the reference's compress step
// (src/backend/stitch_and_generate_gpu.cpp:312-363); -DESC_ACC_DOUBLE switches to float64
// (about 1.4x slower on configuration 4a).
#ifdef ESC_ACC_DOUBLE
typedef double acc_t;
#else
typedef float acc_t;
#endif

struct CsrView {
    const int32_t *rp;
    const int32_t *col;
    const float *val;
};

// Device-side counters of one call.
struct EscCtl {
    unsigned long long products;
    int n_small, n_medium, n_long;
    int n_giant, n_huge;  // huge rows with more / at most GIANT_P products
    int n_ranked;
};

// huge_rows holds the giant rows from its front and the other huge rows from its back, so
// that the heaviest units are handed out first.
struct RowLists {
    int32_t *small_rows, *medium_rows, *long_rows, *huge_rows, *ranked_rows;
};

constexpr unsigned long long GIANT_P = 1ull << 20;

// Expand phase 1 (src/backend/compute.cpp:541-611): per-row product counts, and the bins.
// Rows without products get their count (0) written here.
__global__ void __launch_bounds__(256) k_esc_rowwork(CsrView A, CsrView B, int32_t rows, int32_t *__restrict__ row_count,
                                                     RowLists lists, unsigned long long huge_p, unsigned long long ranked_p, EscCtl *ctl) {
    __shared__ unsigned long long warp_p[8];
    const int i = blockIdx.x * 8 + warp_id();  // one warp per row, lanes stride over the row's entries
    unsigned long long p = 0;
    if (i < rows) {
        const int32_t lo = ld_nc(A.rp + i), hi = ld_nc(A.rp + i + 1);
        for (int32_t e = lo + lane_id(); e < hi; e += 32) {
            const int32_t j = ld_nc(A.col + e);
            p += (unsigned long long)(ld_nc(B.rp + j + 1) - ld_nc(B.rp + j));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) p += __shfl_xor_sync(FULL_MASK, p, o);
        if (lane_id() == 0) {
            if (p == 0) {
                if (row_count) row_count[i] = 0;
            } else if (p <= SMALL_P) {
                lists.small_rows[atomicAdd(&ctl->n_small, 1)] = i;
            } else if (p <= MEDIUM_P) {
                lists.medium_rows[atomicAdd(&ctl->n_medium, 1)] = i;
            } else if (p <= huge_p) {
                if (p <= ranked_p)
                    lists.ranked_rows[atomicAdd(&ctl->n_ranked, 1)] = i;
                else
                    lists.long_rows[atomicAdd(&ctl->n_long, 1)] = i;
            } else {
                if (p > GIANT_P)
                    lists.huge_rows[atomicAdd(&ctl->n_giant, 1)] = i;
                else
                    lists.huge_rows[rows - 1 - atomicAdd(&ctl->n_huge, 1)] = i;
            }
        }
    }
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

// One warp per row with at most 32 products. Lane l holds product l of the row's expansion
// order; the sort key is (column << 32 | l), so equal columns stay in expansion order.
// NARROW: B has fewer than 2^27 columns, so (column << 5 | lane) fits 32 bits and the sort
// moves half as much through the shuffles.
template <bool NUMERIC, bool NARROW>
__global__ void __launch_bounds__(256) k_esc_small(CsrView A, CsrView B, const int32_t *__restrict__ row_list, int n_rows,
                                                   int32_t *__restrict__ row_count, const int32_t *__restrict__ c_rp,
                                                   int32_t *__restrict__ c_col, float *__restrict__ c_val) {
    const int w = (blockIdx.x * 256 + threadIdx.x) >> 5;
    if (w >= n_rows) return;
    const int lane = lane_id();
    const int32_t i = ld_nc(row_list + w);
    const int32_t lo = ld_nc(A.rp + i), hi = ld_nc(A.rp + i + 1);
    uint32_t my_col = 0;
    float my_val = 0.f;
    bool have = false;
    int base = 0;
    for (int32_t e = lo; e < hi; ++e) {  // uniform across the warp
        const int32_t j = ld_nc(A.col + e);
        const int32_t b_lo = ld_nc(B.rp + j), len = ld_nc(B.rp + j + 1) - b_lo;
        if (lane >= base && lane < base + len) {
            my_col = (uint32_t)ld_nc(B.col + b_lo + (lane - base));
            if (NUMERIC) my_val = ld_nc(A.val + e) * ld_nc(B.val + b_lo + (lane - base));
            have = true;
        }
        base += len;
    }
    uint32_t col;
    int src;
    bool valid;
    if (NARROW) {
        uint32_t key = have ? ((my_col << 5) | (uint32_t)lane) : ~0u;
        key = warp_bitonic_sort32(key);
        col = key >> 5;
        src = (int)(key & 31u);
        valid = key != ~0u;
    } else {
        uint64_t key = have ? (((uint64_t)my_col << 32) | (uint32_t)lane) : ~0ull;
        key = warp_bitonic_sort(key);
        col = (uint32_t)(key >> 32);
        src = (int)(key & 31u);
        valid = key != ~0ull;
    }
    const uint32_t prev_col = __shfl_up_sync(FULL_MASK, col, 1);
    const bool head = valid && (lane == 0 || prev_col != col);
    const unsigned heads = __ballot_sync(FULL_MASK, head);
    if (!NUMERIC) {
        if (lane == 0) row_count[i] = __popc(heads);
        return;
    }
    float v = __shfl_sync(FULL_MASK, my_val, src);  // value of the product now at this lane
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
        const int pos = ld_nc(c_rp + i) + __popc(heads & ((1u << lane) - 1u));
        c_col[pos] = (int32_t)col;
        c_val[pos] = acc;
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

// -------------------------------------------------------------------------- long rows ----

// Dense accumulator of one long row: a bit per column, and (numeric pass) a float64 per column.
struct LongSlots {
    uint32_t *bitmap;  // slots x words
    acc_t *acc;        // slots x cols (numeric only)
    int32_t words;
    int32_t cols;
};

// A CTA takes long rows round-robin and owns one accumulator slot. Products are scattered
// with atomics; the row is then read off the bitmap in column order and the slot is wiped
// for the next row (only where it was touched).
template <bool NUMERIC>
__global__ void __launch_bounds__(LONG_NT) k_esc_long(CsrView A, CsrView B, const int32_t *__restrict__ row_list, int n_rows,
                                                      LongSlots slots, int32_t *__restrict__ row_count,
                                                      const int32_t *__restrict__ c_rp, int32_t *__restrict__ c_col,
                                                      float *__restrict__ c_val) {
    __shared__ int scan_tmp[72];
    const int tid = threadIdx.x;
    uint32_t *bitmap = slots.bitmap + (size_t)blockIdx.x * slots.words;
    acc_t *acc = NUMERIC ? slots.acc + (size_t)blockIdx.x * slots.cols : nullptr;
    for (int r = blockIdx.x; r < n_rows; r += gridDim.x) {
        const int32_t i = ld_nc(row_list + r);
        const int32_t lo = ld_nc(A.rp + i), hi = ld_nc(A.rp + i + 1);
        for (int32_t e = lo + warp_id(); e < hi; e += LONG_NT / 32) {
            const int32_t j = ld_nc(A.col + e);
            const int32_t b_lo = ld_nc(B.rp + j), b_hi = ld_nc(B.rp + j + 1);
            const float a = NUMERIC ? ld_nc(A.val + e) : 0.f;
            for (int32_t q = b_lo + lane_id(); q < b_hi; q += 32) {
                const uint32_t col = (uint32_t)ld_nc(B.col + q);
                atomicOr(bitmap + (col >> 5), 1u << (col & 31u));
                if (NUMERIC) atomicAdd(acc + col, (acc_t)(a * ld_nc(B.val + q)));
            }
        }
        __syncthreads();
        int base = 0;
        const int32_t out = NUMERIC ? ld_nc(c_rp + i) : 0;
        for (int w0 = 0; w0 < slots.words; w0 += LONG_NT) {
            const int w = w0 + tid;
            uint32_t bits = w < slots.words ? __ldcg(bitmap + w) : 0u;
            int chunk_total;
            int pos = block_excl_sum<LONG_NT>(__popc(bits), scan_tmp, chunk_total);
            if (bits) {
                bitmap[w] = 0u;
                if (NUMERIC) {
                    pos += out + base;
                    while (bits) {
                        const uint32_t col = (uint32_t)w * 32u + (uint32_t)(__ffs(bits) - 1);
                        bits &= bits - 1;
                        c_col[pos] = (int32_t)col;
                        c_val[pos] = (float)__ldcg(acc + col);
                        acc[col] = (acc_t)0;
                        ++pos;
                    }
                }
            }
            base += chunk_total;
        }
        if (!NUMERIC && tid == 0) row_count[i] = base;
        __syncthreads();
    }
}

// -------------------------------------------------------------------------- huge rows ----

constexpr int WIN_NT = 512;
constexpr int WIN_BYTES = 64 * 1024;                // shared-memory accumulator of one window
constexpr int WIN_COLS_NUMERIC = WIN_BYTES / 4;     // float32 sums: 16384 columns per window
constexpr int WIN_COLS_SYMBOLIC = WIN_BYTES;        // flag bytes: 65536 columns per window
constexpr int WIN_MAX_WINDOWS = 256;                // wider matrices keep every long row on the global accumulator
constexpr size_t WIN_PTR_BUDGET = size_t(1) << 30;  // bytes of the window pointer table
#ifndef ESC_WIN_P
#define ESC_WIN_P 1024                              // a row is huge when it has more products than this per window
#endif
#ifndef ESC_WIN_ITEMS
#define ESC_WIN_ITEMS 4                             // 32-product blocks a warp keeps in flight
#endif
constexpr uint32_t NEG_ZERO_BITS = 0x80000000u;

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

// Window pointer table of B: ptr[j * (n_win + 1) + w] = first position of row j whose column is
// >= w * win_cols (w = 0 .. n_win), so that window w of row j is [ptr[w], ptr[w + 1]).
__global__ void __launch_bounds__(256) k_esc_window_ptr(CsrView B, int32_t b_rows, int n_win, int win_cols, int32_t *__restrict__ ptr) {
    const int64_t t = (int64_t)blockIdx.x * 256 + threadIdx.x;
    const int per = n_win + 1;
    if (t >= (int64_t)b_rows * per) return;
    const int32_t j = (int32_t)(t / per);
    const int w = (int)(t - (int64_t)j * per);
    int32_t lo = ld_nc(B.rp + j), hi = ld_nc(B.rp + j + 1);
    if (w == n_win) {
        lo = hi;
    } else if (w > 0) {
        const int32_t key = w * win_cols;
        while (lo < hi) {
            const int32_t mid = lo + ((hi - lo) >> 1);
            if (ld_nc(B.col + mid) < key)
                lo = mid + 1;
            else
                hi = mid;
        }
    }
    ptr[t] = lo;
}

// Persistent CTAs take huge rows from a ticket and walk the row's column windows in order. In
// window w every entry (i, j) of the row contributes the slice [ptr[j][w], ptr[j][w + 1]) of B's
// row j; the non-empty slices of up to WIN_NT entries form one flat product range that the warps
// walk ESC_WIN_ITEMS x 32 products at a time, accumulating into shared memory. The window is
// then read off in column order behind the row's earlier windows.
//
// Numeric: the sums start at -0.0f and every product is added as (product + 0.0f), which is
// never -0.0f, so a word that still holds -0.0f was not touched and no separate flag is needed
// (-0.0f + x == x for every x that is not -0.0f). Symbolic: one flag byte per column, plain
// stores, four times as many columns per window.
template <bool NUMERIC>
__global__ void __launch_bounds__(WIN_NT, 2)
    k_esc_window(CsrView A, CsrView B, const int32_t *__restrict__ win_ptr, const int32_t *__restrict__ huge_rows, int32_t rows,
                 int n_giant, int n_rows, int n_win, int *ticket, int32_t *__restrict__ row_count,
                 const int32_t *__restrict__ c_rp, int32_t *__restrict__ c_col, float *__restrict__ c_val) {
    constexpr int WCOLS = NUMERIC ? WIN_COLS_NUMERIC : WIN_COLS_SYMBOLIC;
    extern __shared__ __align__(16) unsigned char win_smem[];
    float *acc = reinterpret_cast<float *>(win_smem);
    unsigned char *flags = win_smem;
    __shared__ int seg_off[WIN_NT + 1];
    __shared__ int seg_start[WIN_NT];
    __shared__ float seg_a[NUMERIC ? WIN_NT : 1];
    __shared__ int scan_tmp[72];
    __shared__ int s_row;
    const int tid = threadIdx.x;
    const int per = n_win + 1;

    if (NUMERIC) {
        for (int c = tid; c < WCOLS; c += WIN_NT) acc[c] = __uint_as_float(NEG_ZERO_BITS);
    } else {
        for (int c = tid; c < WIN_BYTES / 16; c += WIN_NT) reinterpret_cast<uint4 *>(flags)[c] = make_uint4(0u, 0u, 0u, 0u);
    }
    for (;;) {
        __syncthreads();  // the previous row is fully read off; s_row may be overwritten
        if (tid == 0) s_row = atomicAdd(ticket, 1);
        __syncthreads();
        const int r = s_row;
        if (r >= n_rows) break;
        const int32_t i = ld_nc(huge_rows + (r < n_giant ? r : rows - 1 - (r - n_giant)));
        const int32_t lo = ld_nc(A.rp + i), hi = ld_nc(A.rp + i + 1);
        const bool one_chunk = hi - lo <= WIN_NT;  // then every thread keeps its entry across the windows
        int64_t my_ptr = -1;
        float my_a = 0.f;
        if (one_chunk && lo + tid < hi) {
            my_ptr = (int64_t)ld_nc(A.col + lo + tid) * per;
            if (NUMERIC) my_a = ld_nc(A.val + lo + tid);
        }
        int64_t out = NUMERIC ? (int64_t)ld_nc(c_rp + i) : 0;  // next free position of the row (count so far, symbolic)

        for (int w = 0; w < n_win; ++w) {
            bool any = false;
            for (int32_t chunk = lo; chunk < hi; chunk += WIN_NT) {
                int32_t s = 0, len = 0;
                float a = my_a;
                int64_t pp = my_ptr;
                if (!one_chunk) {
                    pp = -1;
                    if (chunk + tid < hi) {
                        pp = (int64_t)ld_nc(A.col + chunk + tid) * per;
                        if (NUMERIC) a = ld_nc(A.val + chunk + tid);
                    }
                }
                if (pp >= 0) {
                    s = ld_nc(win_ptr + pp + w);
                    len = ld_nc(win_ptr + pp + w + 1) - s;
                }
                int k_idx, off, n_seg, total;
                block_excl_sum2<WIN_NT>(len > 0 ? 1 : 0, len, scan_tmp, k_idx, off, n_seg, total);
                if (total == 0) continue;  // uniform; the scan synchronises before it reuses scan_tmp
                any = true;
                if (len > 0) {
                    seg_off[k_idx] = off;
                    seg_start[k_idx] = s;
                    if (NUMERIC) seg_a[k_idx] = a;
                }
                if (tid == 0) seg_off[n_seg] = total;
                __syncthreads();
                const int32_t c_first = w * WCOLS;
                walk_segments<WIN_NT, NUMERIC>(seg_off, seg_start, seg_a, n_seg, total, B, [&](int32_t col, float v) {
                    if (NUMERIC)
                        atomicAdd(acc + (col - c_first), __fadd_rn(v, 0.0f));
                    else
                        flags[col - c_first] = 1;
                });
                __syncthreads();  // the segment arrays are rewritten by the next chunk
            }
            if (!any) continue;  // uniform

            if (!NUMERIC) {
                uint4 *f4 = reinterpret_cast<uint4 *>(flags);
                int mine = 0;
#pragma unroll
                for (int k = 0; k < WIN_BYTES / 16 / WIN_NT; ++k) {
                    const uint4 x = f4[k * WIN_NT + tid];
                    const int n = __popc(x.x) + __popc(x.y) + __popc(x.z) + __popc(x.w);
                    if (n) f4[k * WIN_NT + tid] = make_uint4(0u, 0u, 0u, 0u);
                    mine += n;
                }
                int cnt;
                block_excl_sum<WIN_NT>(mine, scan_tmp, cnt);
                out += cnt;
                continue;
            }

            // numeric read-off: warp v looks after columns [1024 v, 1024 v + 1024) of the window in 32
            // groups of 32; lane g keeps the touched mask of group g, every group is read and
            // written with lane = column, so shared-memory reads and the result stores coalesce
            const int wbase = warp_id() * 1024;
            uint32_t mask = 0u;
#pragma unroll 8
            for (int g = 0; g < 32; ++g) {
                const uint32_t m = __ballot_sync(FULL_MASK, __float_as_uint(acc[wbase + g * 32 + lane_id()]) != NEG_ZERO_BITS);
                if (lane_id() == g) mask = m;
            }
            int cnt;
            const int rank = block_excl_sum<WIN_NT>(__popc(mask), scan_tmp, cnt);
            const uint32_t below = (1u << lane_id()) - 1u;
            const int32_t col0 = w * WCOLS + wbase + lane_id();
#pragma unroll 4
            for (int g = 0; g < 32; ++g) {
                const uint32_t m = __shfl_sync(FULL_MASK, mask, g);
                const int base = __shfl_sync(FULL_MASK, rank, g);
                if (m == 0u) continue;
                if ((m >> lane_id()) & 1u) {
                    const int64_t pos = out + base + __popc(m & below);
                    c_col[pos] = col0 + g * 32;
                    c_val[pos] = acc[wbase + g * 32 + lane_id()];
                    acc[wbase + g * 32 + lane_id()] = __uint_as_float(NEG_ZERO_BITS);
                }
            }
            out += cnt;
        }
        if (!NUMERIC && tid == 0) row_count[i] = (int32_t)out;
    }
}

// ------------------------------------------------------------------------ ranked rows ----

constexpr int RK_NT = 256;
constexpr int RK_WORDS = 8192;                    // bitmap of the whole column range in shared memory
constexpr int RK_MAX_COLS = RK_WORDS * 32;        // 262144: wider matrices use the global accumulator
constexpr unsigned long long RK_MAX_P = 65535;    // ranks are kept in 16 bits
constexpr size_t RK_SMEM = RK_WORDS * 4 + RK_WORDS * 2;  // bitmap + ranks at the full width

// One CTA per row whose products exceed the sort in shared memory but not the window path.
// Pass 1 sets a bit per produced column in a shared-memory bitmap; a popcount scan turns the
// bitmap into the rank of every column within the result row; pass 2 walks the products again
// and adds each one straight into its final position of C (float32 reductions in L2 on the row's
// own compact output range, which pass 2 zeroes first). Symbolic: pass 1 and the count only.
template <bool NUMERIC>
__global__ void __launch_bounds__(RK_NT) k_esc_ranked(CsrView A, CsrView B, const int32_t *__restrict__ row_list,
                                                      int words, int32_t *__restrict__ row_count,
                                                      const int32_t *__restrict__ c_rp, int32_t *__restrict__ c_col,
                                                      float *__restrict__ c_val) {
    // `words`: bitmap words in use, a multiple of RK_NT that covers B's columns
    extern __shared__ __align__(16) unsigned char rk_smem[];
    uint32_t *bitmap = reinterpret_cast<uint32_t *>(rk_smem);
    uint16_t *rank16 = reinterpret_cast<uint16_t *>(rk_smem + (size_t)words * 4);
    __shared__ int seg_off[RK_NT + 1];
    __shared__ int seg_start[RK_NT];
    __shared__ float seg_a[NUMERIC ? RK_NT : 1];
    __shared__ int scan_tmp[72];
    const int tid = threadIdx.x;
    const int32_t i = ld_nc(row_list + blockIdx.x);
    const int32_t lo = ld_nc(A.rp + i), hi = ld_nc(A.rp + i + 1);
    const bool one_chunk = hi - lo <= RK_NT;  // then the segments of pass 1 serve pass 2 as well

    for (int c = tid; c < words / 4; c += RK_NT) reinterpret_cast<uint4 *>(bitmap)[c] = make_uint4(0u, 0u, 0u, 0u);

    // builds the segments of one chunk of the row's entries (whole rows of B) and walks them
    auto pass = [&](bool build, auto f) {
        for (int32_t chunk = lo; chunk < hi; chunk += RK_NT) {
            int n_seg, total;
            if (build) {
                int32_t s = 0, len = 0;
                float a = 0.f;
                if (chunk + tid < hi) {
                    const int32_t j = ld_nc(A.col + chunk + tid);
                    s = ld_nc(B.rp + j);
                    len = ld_nc(B.rp + j + 1) - s;
                    if (NUMERIC) a = ld_nc(A.val + chunk + tid);
                }
                int k_idx, off;
                block_excl_sum2<RK_NT>(len > 0 ? 1 : 0, len, scan_tmp, k_idx, off, n_seg, total);
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
            walk_segments<RK_NT, NUMERIC>(seg_off, seg_start, seg_a, n_seg, total, B, f);
            __syncthreads();
        }
    };

    __syncthreads();
    pass(true, [&](int32_t col, float) { atomicOr(bitmap + (col >> 5), 1u << (col & 31)); });

    // warp v looks after an eighth of the words, lane = word within groups of 32
    const int groups = words / RK_NT;
    const int wbase = warp_id() * groups * 32;
    int mine = 0;
#pragma unroll 4
    for (int g = 0; g < groups; ++g) mine += __popc(bitmap[wbase + g * 32 + lane_id()]);
    int cnt;
    const int excl = block_excl_sum<RK_NT>(mine, scan_tmp, cnt);
    if (!NUMERIC) {
        if (tid == 0) row_count[i] = cnt;
        return;
    }
    int running = __shfl_sync(FULL_MASK, excl, 0);  // columns before this warp's words
#pragma unroll 4
    for (int g = 0; g < groups; ++g) {
        const int c = __popc(bitmap[wbase + g * 32 + lane_id()]);
        const int incl = warp_incl_sum(c);
        rank16[wbase + g * 32 + lane_id()] = (uint16_t)(running + incl - c);
        running += __shfl_sync(FULL_MASK, incl, 31);
    }
    const int64_t out = ld_nc(c_rp + i);
    for (int k = tid; k < cnt; k += RK_NT) c_val[out + k] = 0.f;
    __syncthreads();  // ranks complete, output zeroed (the reductions below come from this CTA only)
    pass(!one_chunk, [&](int32_t col, float v) {
        const uint32_t bits = bitmap[col >> 5];
        const int64_t pos = out + rank16[col >> 5] + __popc(bits & ((1u << (col & 31)) - 1u));
        c_col[pos] = col;
        atomicAdd(c_val + pos, v);
    });
}

// Turns the exclusive prefix of the per-row counts into row offsets (rows + 1 entries).
__global__ void __launch_bounds__(256) k_esc_row_offsets(const int32_t *__restrict__ excl, const long long *__restrict__ total,
                                                         int32_t rows, int32_t *__restrict__ c_rp) {
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i < rows) c_rp[i] = excl[i];
    if (i == rows) c_rp[rows] = (int32_t)min(*total, (long long)INT32_MAX);
}

// ------------------------------------------------------------------------ host driver ----

int check_operand(const nb200_csr *m) {
    if (!m || m->rows < 0 || m->cols < 0 || m->nnz < 0 || !m->row_ptr) return NB200_E_BADARG;
    if (m->nnz > 0 && (!m->col || !m->val)) return NB200_E_BADARG;
    return NB200_OK;
}

constexpr size_t LONG_SLOT_BUDGET = size_t(4) << 30;  // bytes of accumulator slots per call

struct EscPlan {
    Workspace *ws;
    RowLists lists;
    int32_t *row_count;  // rows entries (symbolic pass)
    uint64_t *scan_block;  // FusedCtl + one word per scan CTA
    int scan_ctas;
    EscCtl *ctl;
    LongSlots slots;
    int n_slots;
    int n_win_numeric, n_win_symbolic;  // column windows per huge row in either pass (0: the window path is off for this B)
    EscCtl host;  // counters read back after the row-work kernel
};

int sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!cached[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// Bins the rows (kernel + one read-back) and carves the scratch of one pass.
// `numeric`: the global accumulator slots carry values (needed by the numeric pass);
// `counts`: rows without products get their count written (needed by the symbolic pass).
// A plan prepared with both serves a symbolic pass followed by a numeric pass.
int esc_prepare(const nb200_csr *a, const nb200_csr *b, bool numeric, bool counts, cudaStream_t stream, EscPlan *plan) {
    const int32_t rows = a->rows;
    const int32_t words = (b->cols + 31) / 32;
    const size_t slot_bytes = (size_t)words * 4 + (numeric ? (size_t)b->cols * sizeof(acc_t) : 0);
    // both passes bin the rows alike: the thresholds come from the numeric pass's windows
    const int64_t n_win_num = std::max<int64_t>(1, ((int64_t)b->cols + WIN_COLS_NUMERIC - 1) / WIN_COLS_NUMERIC);
    const int64_t n_win_sym = std::max<int64_t>(1, ((int64_t)b->cols + WIN_COLS_SYMBOLIC - 1) / WIN_COLS_SYMBOLIC);
    const bool windows_on = n_win_num <= WIN_MAX_WINDOWS && (size_t)b->rows * (size_t)(n_win_num + 1) * 4 <= WIN_PTR_BUDGET;
    const bool ranked_on = b->cols <= RK_MAX_COLS;
    const bool no_long_rows = windows_on && ranked_on && (unsigned long long)ESC_WIN_P * n_win_num <= RK_MAX_P;
    int max_slots = (int)std::min<size_t>(ESC_LONG_SLOTS, std::max<size_t>(1, LONG_SLOT_BUDGET / std::max<size_t>(slot_bytes, 1)));
    if (no_long_rows) max_slots = 0;
    Carver sizes;
    for (int q = 0; q < 5; ++q) sizes.take<int32_t>((size_t)rows);
    sizes.take<int32_t>((size_t)rows + 1);
    const int scan_ctas = (rows + SCAN_NT * SCAN_VT - 1) / (SCAN_NT * SCAN_VT);
    sizes.take<uint64_t>((size_t)scan_ctas + 8);
    sizes.take<EscCtl>(1);
    const size_t fixed = sizes.used();
    // the slots are only needed if there are long rows, which is known after the row-work
    // kernel; reserve them up front so that the pool block does not move in between
    int st;
    if ((st = acquire_workspace(stream, fixed + (size_t)max_slots * (slot_bytes + 512) + 1024, &plan->ws))) {
        if (st != NB200_E_NOMEM || max_slots <= 1) return st;
        max_slots = 1;
        if ((st = acquire_workspace(stream, fixed + slot_bytes + 2048, &plan->ws))) return st;
    }
    Carver carve(plan->ws->dev);
    plan->lists.small_rows = carve.take<int32_t>((size_t)rows);
    plan->lists.medium_rows = carve.take<int32_t>((size_t)rows);
    plan->lists.long_rows = carve.take<int32_t>((size_t)rows);
    plan->lists.huge_rows = carve.take<int32_t>((size_t)rows);
    plan->lists.ranked_rows = carve.take<int32_t>((size_t)rows);
    plan->row_count = carve.take<int32_t>((size_t)rows + 1);
    plan->scan_block = carve.take<uint64_t>((size_t)scan_ctas + 8);
    plan->scan_ctas = scan_ctas;
    plan->ctl = carve.take<EscCtl>(1);
    plan->slots.words = words;
    plan->slots.cols = b->cols;
    plan->slots.bitmap = carve.take<uint32_t>((size_t)max_slots * words);
    plan->slots.acc = numeric ? carve.take<acc_t>((size_t)max_slots * b->cols) : nullptr;
    plan->n_slots = max_slots;
    plan->n_win_numeric = windows_on ? (int)n_win_num : 0;
    plan->n_win_symbolic = windows_on ? (int)n_win_sym : 0;
    const unsigned long long huge_p = windows_on ? (unsigned long long)ESC_WIN_P * (unsigned long long)n_win_num : ULLONG_MAX;

    NB200_CUDA(cudaMemsetAsync(plan->ctl, 0, sizeof(EscCtl), stream));
    const CsrView A{a->row_ptr, a->col, a->val}, B{b->row_ptr, b->col, b->val};
    if (rows > 0) {
        LaunchScope scope("esc_rowwork", stream);
        k_esc_rowwork<<<(rows + 7) / 8, 256, 0, stream>>>(A, B, rows, counts ? plan->row_count : nullptr, plan->lists, huge_p,
                                                         ranked_on ? RK_MAX_P : 0ull, plan->ctl);
        NB200_CUDA(cudaGetLastError());
    }
    NB200_CUDA(cudaMemcpyAsync(plan->ws->host, plan->ctl, sizeof(EscCtl), cudaMemcpyDeviceToHost, stream));
    NB200_CUDA(cudaStreamSynchronize(stream));
    std::memcpy(&plan->host, plan->ws->host, sizeof(EscCtl));
    if (plan->host.n_long > 0) {
        plan->n_slots = std::min(plan->n_slots, plan->host.n_long);
        NB200_CUDA(cudaMemsetAsync(plan->slots.bitmap, 0, (size_t)plan->n_slots * words * 4, stream));
        if (numeric) NB200_CUDA(cudaMemsetAsync(plan->slots.acc, 0, (size_t)plan->n_slots * b->cols * sizeof(acc_t), stream));
    }
    return NB200_OK;
}

template <bool NUMERIC>
int esc_run_bins(const nb200_csr *a, const nb200_csr *b, const EscPlan &plan, const nb200_csr *c, cudaStream_t stream) {
    const CsrView A{a->row_ptr, a->col, a->val}, B{b->row_ptr, b->col, b->val};
    int32_t *count = NUMERIC ? nullptr : plan.row_count;
    const int32_t *c_rp = NUMERIC ? c->row_ptr : nullptr;
    int32_t *c_col = NUMERIC ? c->col : nullptr;
    float *c_val = NUMERIC ? c->val : nullptr;
    if (plan.host.n_small > 0) {
        LaunchScope scope(NUMERIC ? "esc_small_numeric" : "esc_small_symbolic", stream);
        const int warps = plan.host.n_small;
        if (b->cols < (1 << 27))
            k_esc_small<NUMERIC, true><<<(warps + 7) / 8, 256, 0, stream>>>(A, B, plan.lists.small_rows, warps, count, c_rp, c_col, c_val);
        else
            k_esc_small<NUMERIC, false><<<(warps + 7) / 8, 256, 0, stream>>>(A, B, plan.lists.small_rows, warps, count, c_rp, c_col, c_val);
        NB200_CUDA(cudaGetLastError());
    }
    if (plan.host.n_medium > 0) {
        LaunchScope scope(NUMERIC ? "esc_medium_numeric" : "esc_medium_symbolic", stream);
        k_esc_medium<NUMERIC><<<plan.host.n_medium, MED_NT, 0, stream>>>(A, B, plan.lists.medium_rows, count, c_rp, c_col, c_val);
        NB200_CUDA(cudaGetLastError());
    }
    if (plan.host.n_long > 0) {
        LaunchScope scope(NUMERIC ? "esc_long_numeric" : "esc_long_symbolic", stream);
        k_esc_long<NUMERIC><<<plan.n_slots, LONG_NT, 0, stream>>>(A, B, plan.lists.long_rows, plan.host.n_long, plan.slots, count, c_rp,
                                                                 c_col, c_val);
        NB200_CUDA(cudaGetLastError());
    }
    if (plan.host.n_ranked > 0) {
        static bool attr_set[2] = {false, false};
        if (!attr_set[NUMERIC]) {
            NB200_CUDA(cudaFuncSetAttribute(k_esc_ranked<NUMERIC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RK_SMEM));
            attr_set[NUMERIC] = true;
        }
        LaunchScope scope(NUMERIC ? "esc_ranked_numeric" : "esc_ranked_symbolic", stream);
        const int rk_words = (((b->cols + 31) / 32 + RK_NT - 1) / RK_NT) * RK_NT;
        k_esc_ranked<NUMERIC><<<plan.host.n_ranked, RK_NT, (size_t)rk_words * 6, stream>>>(A, B, plan.lists.ranked_rows, rk_words, count, c_rp,
                                                                                        c_col, c_val);
        NB200_CUDA(cudaGetLastError());
    }
    const int64_t n_huge = (int64_t)plan.host.n_giant + plan.host.n_huge;
    if (n_huge > 0) {
        constexpr int WCOLS = NUMERIC ? WIN_COLS_NUMERIC : WIN_COLS_SYMBOLIC;
        const int n_win = NUMERIC ? plan.n_win_numeric : plan.n_win_symbolic;
        const int64_t ptr_entries = (int64_t)b->rows * (n_win + 1);
        Carver sizes;
        sizes.take<int>(1);
        sizes.take<int32_t>((size_t)ptr_entries);
        Workspace *ws = nullptr;
        int st;
        if ((st = acquire_workspace(stream, sizes.used(), &ws, 3))) return st;
        Carver carve(ws->dev);
        int *ticket = carve.take<int>(1);
        int32_t *win_ptr = carve.take<int32_t>((size_t)ptr_entries);
        NB200_CUDA(cudaMemsetAsync(ticket, 0, sizeof(int), stream));
        {
            LaunchScope scope("esc_window_ptr", stream);
            k_esc_window_ptr<<<(unsigned)((ptr_entries + 255) / 256), 256, 0, stream>>>(B, b->rows, n_win, WCOLS, win_ptr);
            NB200_CUDA(cudaGetLastError());
        }
        static bool attr_set[2] = {false, false};
        if (!attr_set[NUMERIC]) {
            NB200_CUDA(cudaFuncSetAttribute(k_esc_window<NUMERIC>, cudaFuncAttributeMaxDynamicSharedMemorySize, WIN_BYTES));
            attr_set[NUMERIC] = true;
        }
        int per_sm = 0;
        NB200_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_esc_window<NUMERIC>, WIN_NT, WIN_BYTES));
        const int grid = (int)std::min<int64_t>(n_huge, (int64_t)sm_count() * std::max(per_sm, 1));
        LaunchScope scope(NUMERIC ? "esc_window_numeric" : "esc_window_symbolic", stream);
        k_esc_window<NUMERIC><<<grid, WIN_NT, WIN_BYTES, stream>>>(A, B, win_ptr, plan.lists.huge_rows, a->rows, plan.host.n_giant, (int)n_huge,
                                                                  n_win, ticket, count, c_rp, c_col, c_val);
        NB200_CUDA(cudaGetLastError());
    }
    return NB200_OK;
}

// `keep`: if given, the plan is prepared for both passes and handed back, so that a numeric
// pass that follows at once (nothing else touching the stream's scratch) skips the binning.
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
    if ((st = esc_prepare(a, b, keep != nullptr, true, stream, &plan))) return st;
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
    if (h.status.error != 0) return NB200_E_TIMEOUT;
    const int64_t nnz = h.total;
    if (nnz > INT32_MAX) return NB200_E_OVERFLOW;
    c->nnz = (int32_t)nnz;
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
    if ((st = esc_prepare(a, b, true, false, stream, &plan))) return st;
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
