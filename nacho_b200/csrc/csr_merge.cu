// CSR + CSR element-wise kernels: sorted union (add) and intersection (multiply) of two CSR
// operands, as flat merge-path over the (row, column) order.
//
// The merged sequence of all stored entries of A and B, ordered by (row, column) with A first
// on ties, is cut into tiles of TILE_STEP entries. A partition kernel finds every cut with
// warp-wide 32-ary searches (rows on the summed row offsets, then the merge-path diagonal
// inside the row). One CTA then owns one tile: the copy engine stages the tile's column indices
// and values in shared memory, the columns are turned into composite (row-in-tile, column) keys
// so that row boundaries need no special casing, the tile is split among the threads with an
// in-shared-memory merge-path search, every thread merges its entries in registers (a bitonic
// network), and the survivors are compacted through shared memory and written back coalesced.
// Row offsets of the result are produced by the same pass: a tile owns the offsets of the rows
// that begin inside it.
//
// Reference behaviour restated (not its code): partition src/backend/partition.cpp:813-993
// (equal columns never split, :964-983), count src/backend/compute.cpp:152-271, fill
// :273-411, value expressions :426-440, empty-result path
// src/backend/stitch_and_generate.cpp:168-220.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "csr_common.cuh"
#include "warp_merge.cuh"

namespace nb200 {

namespace {

// Tuning knobs (compile-time): merged entries per worker thread, and the number of CTAs per SM the
// register allocator is asked to leave room for. The CTA always has 256 worker threads and one
// scan warp.
#ifndef CSR2_V
#define CSR2_V 19            // merged entries per worker thread; (V + 1) rounded up to 4 must be an odd multiple of 4
#endif
#ifndef CSR2_LB_DEPTH
#define CSR2_LB_DEPTH 1      // predecessors read per round of the look-back, in units of 32
#endif
#ifndef CSR2_LB_HURRY
#define CSR2_LB_HURRY 1000  // ns between polls of the look-back once the tile itself waits for the result (faster polling
                            // was measured: 64 ns costs 5 %, the poll traffic slows the workers of the other tiles)
#endif
#ifndef CSR2_LB_SLEEP
#define CSR2_LB_SLEEP 2000  // nanoseconds between polls of the predecessors' tile words (shorter polls measurably slow the workers)
#endif
#ifndef CSR2_MIN_CTAS
#define CSR2_MIN_CTAS 3
#endif
constexpr int NT = CSR_NT;

// Tile cuts: for cut t, the row it falls in and the absolute positions in A and B.
struct Cuts {
    int32_t *row;
    int32_t *a;
    int32_t *b;
};

// Result words of an asynchronous call (CsrOut::result), written from inside the tile kernel.
__device__ __forceinline__ void publish_length(long long *result, long long total) {
    if (!result) return;
    result[0] = total;
    if (total > INT32_MAX) atomicMax(result + 1, (long long)NB200_E_OVERFLOW);
}
__device__ __forceinline__ void publish_timeout(long long *result) {
    if (result) atomicMax(result + 1, (long long)NB200_E_TIMEOUT);
}

// ------------------------------------------------------------------------- partition ----

// One warp per cut. Cut t sits at merged position min(t * tile_step, total).
__global__ void __launch_bounds__(NT) k_csr2_partition(CsrIn A, CsrIn B, int32_t rows, int64_t total,
                                                       int32_t tile_step, int32_t num_tiles, Cuts cuts, long long *result,
                                                       uint64_t *zero_block, int zero_words) {
    if (result && blockIdx.x == 0 && threadIdx.x == 0) {  // the tile kernel that follows fills in the rest
        result[1] = NB200_OK;
        result[2] = rows;
    }
    // the control block and the tile words of the kernel that follows start from zero (the grid has at
    // least 32 threads per tile word, so one word per thread covers them)
    if (blockIdx.x * NT + threadIdx.x < zero_words) zero_block[blockIdx.x * NT + threadIdx.x] = 0;
    const int t = (blockIdx.x * NT + threadIdx.x) >> 5;
    if (t > num_tiles) return;
    const int32_t a_base = ld_nc(A.rp), b_base = ld_nc(B.rp);
    int64_t d = (int64_t)t * tile_step;
    int32_t row, pa, pb;
    if (t == 0) {
        row = 0;
        pa = a_base;
        pb = b_base;
    } else if (t == num_tiles || d >= total) {
        row = rows;
        pa = a_base + A.nnz;
        pb = b_base + B.nnz;
    } else {
        // Row holding merged position d: the largest i with work(i) <= d, where work(i) is the
        // number of entries of A and B in rows before i.
        auto work = [&](int64_t i) -> int64_t {
            return (int64_t)(ld_nc(A.rp + i) - a_base) + (int64_t)(ld_nc(B.rp + i) - b_base);
        };
        row = (int32_t)warp_last_true(0, (int64_t)rows - 1, [&](int64_t i) { return work(i) <= d; });
        const int32_t a_lo = ld_nc(A.rp + row), a_hi = ld_nc(A.rp + row + 1);
        const int32_t b_lo = ld_nc(B.rp + row), b_hi = ld_nc(B.rp + row + 1);
        const int64_t dd = d - ((int64_t)(a_lo - a_base) + (int64_t)(b_lo - b_base));
        const int64_t len_a = a_hi - a_lo, len_b = b_hi - b_lo;
        // Merge-path diagonal dd inside the row: x entries of A and dd - x of B come first.
        const int64_t x_lo = dd - len_b > 0 ? dd - len_b : 0;
        const int64_t x_hi = dd < len_a ? dd : len_a;
        const int64_t x = warp_count_true(x_lo, x_hi, [&](int64_t m) {
            return ld_nc(A.col + a_lo + m) <= ld_nc(B.col + b_lo + (dd - 1 - m));
        });
        int64_t y = dd - x;
        // Keep a column present in both operands on one side of the cut.
        if (x > 0 && y < len_b && ld_nc(A.col + a_lo + x - 1) == ld_nc(B.col + b_lo + y)) ++y;
        pa = a_lo + (int32_t)x;
        pb = b_lo + (int32_t)y;
    }
    if (lane_id() == 0) {
        cuts.row[t] = row;
        cuts.a[t] = pa;
        cuts.b[t] = pb;
    }
}

// ------------------------------------------------------------------------ tile kernel ----


// Tiles whose rows do not fit a 32-bit composite key (long runs of empty rows) take this body:
// 64-bit keys (row in tile, column), plain loads, a sequential merge of VT entries per thread,
// values fetched from global memory. It is rarely taken and kept simple; the common case is
// csr2_tile_blocked below.
template <int VT, int OP, int MODE>
// (Not inlined, so the structs are taken by address: the kernel declares them __grid_constant__,
// which lets that address point at the parameter space instead of a per-thread stack copy.)
__device__ __noinline__ void csr2_tile_wide(const CsrIn &A, const CsrIn &B, const Cuts &cuts, const int t, int32_t *tile_count,
                                            volatile uint64_t *tile_state, FusedCtl *ctl, const CsrOut &Z, unsigned char *smem_raw,
                                            const int num_tiles, const int poll_limit) {
    constexpr uint64_t INF = ~0ull;
    __shared__ int scan_tmp[72];
    __shared__ int thread_rank[NT];
    __shared__ unsigned thread_emit[NT];
    __shared__ long long s_base;
    const int tid = threadIdx.x;
    const int32_t i0 = cuts.row[t], i1 = cuts.row[t + 1];
    const int32_t a0 = cuts.a[t], b0 = cuts.b[t];
    const int na = cuts.a[t + 1] - a0, nb = cuts.b[t + 1] - b0;
    const int n = na + nb;

    // Shared layout: keys of A, a sentinel, keys of B, a sentinel, then VT words of slack so
    // that the merge may read a little past the end.
    constexpr int KEY_SLOTS = NT * VT + 2 + VT;
    uint64_t *kx = reinterpret_cast<uint64_t *>(smem_raw);
    uint64_t *ky = kx + na + 1;
    unsigned *kx_hi = reinterpret_cast<unsigned *>(kx) + 1, *ky_hi = reinterpret_cast<unsigned *>(ky) + 1;

    for (int i = tid; i < na; i += NT) kx[i] = (uint64_t)(uint32_t)ld_nc(A.col + a0 + i);
    for (int i = tid; i < nb; i += NT) ky[i] = (uint64_t)(uint32_t)ld_nc(B.col + b0 + i);
    WorkerBar::sync();

    // ---- mark the first entry of every row that starts inside the tile with its row number
    // relative to i0 in the key's upper word (max wins where empty rows share a start), then spread
    // it forward with a running maximum so that every entry carries its row.
    for (int64_t r = (int64_t)i0 + 1 + tid; r <= i1; r += NT) {
        const uint32_t rr = (uint32_t)(r - i0);
        const int sa = ld_nc(A.rp + r) - a0, sb = ld_nc(B.rp + r) - b0;
        if (sa < na) atomicMax(kx_hi + 2 * sa, rr);
        if (sb < nb) atomicMax(ky_hi + 2 * sb, rr);
    }
    WorkerBar::sync();
    {
        // thread tid owns merged-array slots [tid*VT, tid*VT+VT): first the A part, then B
        const int lo = tid * VT, hi = min(lo + VT, n);
        unsigned ma = 0, mb = 0;
        for (int i = lo; i < hi; ++i) {
            if (i < na) ma = max(ma, kx_hi[2 * i]); else mb = max(mb, ky_hi[2 * (i - na)]);
        }
        unsigned ea, eb;
        block_excl_max2<NT, WorkerBar>(ma, mb, reinterpret_cast<unsigned *>(scan_tmp), ea, eb);
        for (int i = lo; i < hi; ++i) {
            if (i < na) {
                ea = max(ea, kx_hi[2 * i]);
                kx_hi[2 * i] = ea;
            } else {
                eb = max(eb, ky_hi[2 * (i - na)]);
                ky_hi[2 * (i - na)] = eb;
            }
        }
        if (tid < VT + 1) ky[nb + tid] = INF;
        if (tid == 0) kx[na] = INF;
    }
    WorkerBar::sync();

    // ---- split the tile among threads: merge-path diagonal tid * VT, ties take A first
    const int diag = min(tid * VT, n);
    int x, y;
    {
        int lo = max(0, diag - nb), hi = min(diag, na);
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (kx[mid] <= ky[diag - 1 - mid]) lo = mid + 1; else hi = mid;
        }
        x = lo;
        y = diag - lo;
    }
    const int x0 = x, y0 = y;

    // ---- merge VT entries. Bit i of `from_a` says entry i came from A, of `twin` that the same
    // column is in B too, of `emit` that the entry goes to the result.
    uint32_t col[VT];
    unsigned from_a = 0, twin = 0, emit = 0;
    {
        const int valid = min(VT, n - diag);
        uint64_t hx = kx[x], hy = ky[y];
        uint64_t last_x = x > 0 ? kx[x - 1] : INF;
#pragma unroll
        for (int i = 0; i < VT; ++i) {
            const bool ok = i < valid;
            const bool tx = hx <= hy;
            const bool both = hx == hy;
            col[i] = (uint32_t)(tx ? hx : hy);
            const bool out = OP == OP_UNION ? (tx || hy != last_x) : (tx && both);
            from_a |= (unsigned)tx << i;
            twin |= (unsigned)(tx && both) << i;
            emit |= (unsigned)(ok && out) << i;
            last_x = tx ? hx : last_x;
            x += tx;
            y += !tx;
            hx = kx[x];
            hy = ky[y];
        }
    }

    // ---- rank the survivors inside the tile
    int total;
    const int mine = __popc(emit);
    const int rank = block_excl_sum<NT, WorkerBar>(mine, scan_tmp, total);  // syncs: key reads are done
    if (MODE == MODE_COUNT) {
        if (tid == 0) tile_count[t] = total;
        return;
    }

    // ---- output base of the tile
    long long base;
    if (MODE == MODE_FILL) {
        base = tile_count[t];  // exclusive prefix over tiles, made between the two passes
    } else {
        if (warp_id() == 0) {
            if (lane_id() == 0) st_relaxed_gpu(tile_state + t, (t == 0 ? LB_PREFIX : LB_AGGREGATE) | (uint64_t)total);
            int64_t b = 0;
            if (t > 0) {
                b = lookback_predecessors(tile_state, t, &ctl->status, 32, nullptr, 64, poll_limit);
                if (lane_id() == 0) st_relaxed_gpu(tile_state + t, LB_PREFIX | (uint64_t)(b < 0 ? 0 : b + total));
            }
            if (lane_id() == 0) s_base = b;
        }
    }
    thread_rank[tid] = rank;
    thread_emit[tid] = emit;
    WorkerBar::sync();
    if (MODE == MODE_FUSED) {
        base = s_base;
        if (base < 0) {  // a bounded wait gave up; the host reports it
            if (tid == 0) publish_timeout(Z.result);
            return;
        }
        if (t == num_tiles - 1 && tid == 0) {
            ctl->total = base + total;
            publish_length(Z.result, base + total);
        }
    }

    // ---- row offsets. Result row r starts after every result entry of rows < r; inside this
    // tile those are the survivors among the first d = (A entries before row r) + (B entries
    // before row r) merged entries, read off the per-thread ranks. The tile owns rows
    // i0+1 .. i1 (the next tile's first row).
    for (int64_t r = (int64_t)i0 + 1 + tid; r <= i1; r += NT) {
        const int d = (ld_nc(A.rp + r) - a0) + (ld_nc(B.rp + r) - b0);
        const int owner = d / VT, off = d - owner * VT;
        const int before = owner >= NT ? total : thread_rank[owner] + __popc(thread_emit[owner] & ((1u << off) - 1u));
        Z.rp[r] = (int32_t)(base + before);
    }
    if (t == 0 && tid == 0) Z.rp[0] = 0;

    // ---- fetch values, compact through shared memory (the staging arrays reuse the key words:
    // the barriers above separate the last key read from the first write), store coalesced
    int32_t *out_col = reinterpret_cast<int32_t *>(smem_raw);
    float *out_val = reinterpret_cast<float *>(smem_raw) + KEY_SLOTS;
    {
        int r = rank, xi = x0, yi = y0;
#pragma unroll
        for (int i = 0; i < VT; ++i) {
            const bool tx = (from_a >> i) & 1u;
            const bool both = (twin >> i) & 1u;
            if ((emit >> i) & 1u) {
                float v;
                if (OP == OP_UNION) {
                    v = tx ? ld_nc(A.val + a0 + xi) : ld_nc(B.val + b0 + yi);
                    if (both) v = v + ld_nc(B.val + b0 + yi);
                } else {
                    v = ld_nc(A.val + a0 + xi) * ld_nc(B.val + b0 + yi);
                }
                out_col[r] = (int32_t)col[i];
                out_val[r] = v;
                ++r;
            }
            xi += tx;
            yi += !tx;
        }
    }
    WorkerBar::sync();
    for (int i = tid; i < total; i += NT) {
        Z.col[base + i] = out_col[i];
        Z.val[base + i] = out_val[i];
    }
}

// Shared-memory plan of the thread-blocked tile body, in 4-byte words. Keys and values use the
// same word positions: A's entry e sits at word oa + e and B's at word obv + e, where oa and obv
// are chosen so that a global address on a 16-byte boundary lands on a 16-byte boundary in
// shared memory too (what a bulk copy needs). The (column, value) staging pairs of the result reuse
// the key words (the keys live in registers by then) and run on into extra words.
template <int VT>
struct BlockedPlan {
    static constexpr int CAP = NT * VT;
    static constexpr int NETV = VT + 1;                          // merge-network slots in use
    static constexpr int CH = (VT + 1 + 3) & ~3;                 // words each thread scans
    static constexpr int SLOTS = NT * CH + ((NETV + 4 + 3) & ~3);  // key words = value words
    static constexpr int OUT = CAP + 8;                          // staging words per array
    static constexpr size_t BYTES = 4 * (size_t)(2 * SLOTS + OUT);
    // A thread's CH-word chunk is read and written as 16-byte vectors; an odd number of
    // vectors per chunk keeps those accesses free of shared-memory bank conflicts.
    static_assert((CH / 4) % 2 == 1, "choose VT so that (VT + 1) rounded up to 4 is an odd multiple of 4");
    static_assert(NT * CH >= CAP + 12, "scan range must cover the padded tile");
    static_assert(OUT <= SLOTS, "column staging must fit the key words it reuses");
};

// The common tile body, thread-blocked form. Keys are 32-bit composites (row in tile, column, operand bit):
//     key = ((row << cbits | column) << 1) | (0 for A, 1 for B)
// so that one unsigned compare orders entries by (row, column) with A first on ties, and
// two entries are the same position exactly when their keys differ in the last bit only.
//
// The CTA has NT worker threads and one more warp, the scan warp. Workers stage the operands
// with bulk copies, build keys (row marks, then a running maximum that every warp runs over its
// own words), split the tile by merge-path, merge VT entries each in registers with a bitonic
// network, rank the survivors (warp scans, one barrier) and compact them into shared memory. In
// the single-pass mode the scan warp meanwhile turns the tile's count into its output base by
// look-back over earlier tiles, so that this wait overlaps the workers' compaction. Six CTA-wide
// barriers per tile.
template <int VT, int OP, int MODE>
__device__ __forceinline__ void csr2_tile_blocked(const CsrIn &A, const CsrIn &B, const Cuts &cuts, const int cbits, const int t,
                                                  const int num_tiles, int32_t *tile_count, volatile uint64_t *tile_state,
                                                  FusedCtl *ctl, const CsrOut &Z, unsigned char *smem_raw, uint64_t *mbar,
                                                  const int poll_limit) {
    using P = BlockedPlan<VT>;
    constexpr int W = NT / 32;
    __shared__ int thread_rank[NT];
    __shared__ unsigned thread_emit[NT];
    __shared__ int s_wtotal[W];  // survivors of each warp
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    constexpr int NETV = P::NETV;
    constexpr bool WRITES = MODE != MODE_COUNT;
    constexpr uint32_t INF = 0xffffffffu;
    __shared__ long long s_base;
    __shared__ int s_total;
    __shared__ int s_hurry;  // set once the tile's count is out: from then on the tile waits for its base
    const int tid = threadIdx.x;
    const bool scan_warp = tid >= NT;
    const int32_t i0 = cuts.row[t], i1 = cuts.row[t + 1];
    const int32_t a0 = cuts.a[t], b0 = cuts.b[t];
    const int na = cuts.a[t + 1] - a0, nb = cuts.b[t + 1] - b0;
    const int n = na + nb;
    const uint32_t cmask = (1u << cbits) - 1u;

    // layout: values | keys | extra words. The (column, value) staging pairs of the result
    // reuse the keys (in registers by then) and run on into the extra words.
    float *vals = reinterpret_cast<float *>(smem_raw);
    uint32_t *keys = reinterpret_cast<uint32_t *>(smem_raw) + P::SLOTS;
    uint2 *out_pair = reinterpret_cast<uint2 *>(keys);
    static_assert(P::SLOTS % 2 == 0 && P::SLOTS + P::OUT >= 2 * P::OUT, "staging pairs must fit keys + extra words, 8-byte aligned");

    const int32_t *ga_col = A.col + a0, *gb_col = B.col + b0;
    const float *ga_val = A.val + a0, *gb_val = B.val + b0;
    const int ha = head_elems(ga_col), hb = head_elems(gb_col);
    const int oa = (4 - ha) & 3;                 // word of A's entry 0
    const int ob = (oa + na + 1 + 3) & ~3;       // first word of B's region (A's sentinel before it)
    const int obv = ob + ((4 - hb) & 3);         // word of B's entry 0
    const int scan_end = (obv + nb + 3) & ~3;
    uint32_t *kx = keys + oa, *ky = keys + obv;

    // ---- stage the tile. One thread hands the 16-byte-aligned interior of each array to the
    // copy engine; a few other threads load the ragged ends (at most 3 entries each side).
    // Value arrays whose alignment differs from their column arrays' take plain loads.
    const bool va_bulk = !WRITES || head_elems(ga_val) == ha, vb_bulk = !WRITES || head_elems(gb_val) == hb;
    const int head_a = min(na, ha), head_b = min(nb, hb);
    const int nva = (na - head_a) >> 2, nvb = (nb - head_b) >> 2;  // 16-byte vectors in the interior
    if (tid == 0) {
        s_hurry = 0;
        uint32_t bytes = 16u * (uint32_t)(nva + nvb);
        if (WRITES) bytes += (va_bulk ? 16u * nva : 0u) + (vb_bulk ? 16u * nvb : 0u);
        mbar_arrive_expect_tx(mbar, bytes);
        if (nva) bulk_load(kx + head_a, ga_col + head_a, 16u * nva, mbar);
        if (nvb) bulk_load(ky + head_b, gb_col + head_b, 16u * nvb, mbar);
        if (WRITES && va_bulk && nva) bulk_load(vals + oa + head_a, ga_val + head_a, 16u * nva, mbar);
        if (WRITES && vb_bulk && nvb) bulk_load(vals + obv + head_b, gb_val + head_b, 16u * nvb, mbar);
    }
    if (tid >= 32 && tid < 32 + 12) {  // ragged ends: 3 head + 3 tail slots for A, then for B
        const int k = tid - 32;
        const bool is_b = k >= 6;
        const int e = is_b ? k - 6 : k;
        const int count = is_b ? nb : na, head = is_b ? head_b : head_a, nv = is_b ? nvb : nva;
        const int idx = e < 3 ? e : head + 4 * nv + (e - 3);
        const bool live = e < 3 ? e < head : idx < count;
        if (live) {
            const int w = (is_b ? obv : oa) + idx;
            keys[w] = (uint32_t)ld_nc((is_b ? gb_col : ga_col) + idx);
            if (WRITES && (is_b ? vb_bulk : va_bulk)) vals[w] = ld_nc((is_b ? gb_val : ga_val) + idx);
        }
    }
    if (WRITES && !va_bulk && !scan_warp) for (int i = tid; i < na; i += NT) vals[oa + i] = ld_nc(ga_val + i);
    if (WRITES && !vb_bulk && !scan_warp) for (int i = tid; i < nb; i += NT) vals[obv + i] = ld_nc(gb_val + i);
    // padding words that precede live keys must read as "no row mark"; the end-of-list
    // sentinels are all-ones, which the row spreading below keeps above every live key
    if (tid >= 64 && tid < 64 + 3) { if (tid - 64 < oa) keys[tid - 64] = 0u; }
    if (tid >= 68 && tid < 68 + 3) { if (ob + (tid - 68) < obv) keys[ob + (tid - 68)] = 0u; }
    if (tid == 72) keys[oa + na] = INF;
    if (tid >= 76 && tid < 76 + NETV + 1) keys[obv + nb + (tid - 76)] = INF;
    static_assert(76 + NETV + 1 <= NT, "sentinel writers must be worker threads");

    // row offsets of the first row this thread looks after (rows i0+1 .. i1 are spread over the
    // workers); kept in registers for the row-offset pass at the end
    const int64_t my_row = (int64_t)i0 + 1 + tid;
    int32_t my_sa = 0, my_sb = 0;
    if (!scan_warp && my_row <= i1) {
        my_sa = ld_nc(A.rp + my_row) - a0;
        my_sb = ld_nc(B.rp + my_row) - b0;
    }
    // ---- the row (relative to i0) that the first key word of this warp's scan region belongs to:
    // the last row that starts at or before it. Regions that begin with an operand's first entry,
    // or in padding before it, start from row 0 of the tile. (Found while the copies fly.)
    const int w0 = wid * 32 * P::CH;
    const bool region_in_a = w0 < ob;
    unsigned carry = 0;
    if (!scan_warp) {
        const int pos = region_in_a ? w0 - oa : w0 - obv;
        if (pos > 0 && i1 > i0) {
            const int32_t *rp = region_in_a ? A.rp : B.rp;
            const int32_t start = region_in_a ? a0 : b0;
            carry = (unsigned)(warp_last_true(i0, i1, [&](int64_t r) { return ld_nc(rp + r) - start <= pos; }) - i0);
        }
    }
    const bool landed = mbar_wait_bounded(mbar, 0, MBAR_POLL_LIMIT);
    if (!__syncthreads_and(landed)) {  // the copies did not land in time: report, touch nothing
        if (tid == 0) {
            if (atomicCAS(&ctl->status.error, 0, ERR_COPY_TIMEOUT) == 0) ctl->status.detail = t;
            publish_timeout(Z.result);
            if (MODE == MODE_FUSED) tile_state[t] = LB_PREFIX;  // successors must not wait on this tile
            mbar_wait_bounded(mbar, 0, MBAR_POLL_LIMIT);        // second bounded wait for copies in flight
        }
        return;
    }

    if (scan_warp) {
        // ---- scan warp: the output base of the tile is the sum of the counts of all earlier
        // tiles, which does not depend on this tile's own count. So the walk over the
        // predecessors' words starts now, while the workers are still merging, and is usually
        // over by the time they know their count.
        if (MODE != MODE_FUSED) return;
        const int64_t bse = t == 0 ? 0 : lookback_predecessors<CSR2_LB_DEPTH>(tile_state, t, &ctl->status, CSR2_LB_SLEEP, &s_hurry,
                                                                             CSR2_LB_HURRY, poll_limit);
        CountBar::sync();  // the workers have published the tile's count by now
        const int total = s_total;
        if (lane_id() == 0) {
            if (t > 0) st_relaxed_gpu(tile_state + t, LB_PREFIX | (uint64_t)(bse < 0 ? 0 : bse + total));
            s_base = bse;
            if (bse < 0) publish_timeout(Z.result);
            if (bse >= 0 && t == num_tiles - 1) {
                ctl->total = bse + total;
                publish_length(Z.result, bse + total);
            }
        }
        __syncthreads();
        return;
    }

    // ---- mark the first entry of every row that starts inside the tile with its row number
    // relative to i0, in the bits above the column (max wins where empty rows share a start)
    for (int64_t r = my_row; r <= i1; r += NT) {
        const uint32_t rr = (uint32_t)(r - i0);
        const int sa = r == my_row ? my_sa : ld_nc(A.rp + r) - a0;
        const int sb = r == my_row ? my_sb : ld_nc(B.rp + r) - b0;
        if (sa < na) atomicMax(kx + sa, (rr << cbits) | (kx[sa] & cmask));
        if (sb < nb) atomicMax(ky + sb, (rr << cbits) | (ky[sb] & cmask));
    }
    WorkerBar::sync();

    // ---- spread the marks forward (running maximum) so that every key carries its row, and
    // append the operand bit. Each thread owns CH consecutive words, each warp 32 * CH, and a warp
    // needs nothing from the other warps (its region's first row came from the search above); A's
    // words and B's words run separately.
    {
        constexpr int NV = P::CH / 4;
        const int w_base = tid * P::CH;
        uint4 q[NV];
        unsigned ma = 0, mb = 0;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int w = w_base + 4 * j;
            q[j] = w < scan_end ? *reinterpret_cast<const uint4 *>(keys + w) : make_uint4(0, 0, 0, 0);
            const unsigned m = max(max(q[j].x & ~cmask, q[j].y & ~cmask), max(q[j].z & ~cmask, q[j].w & ~cmask));
            if (w < ob) ma = max(ma, m); else mb = max(mb, m);
        }
        // running maximum over the lanes before this one, on top of the row the warp's region starts in
        unsigned ea = __shfl_up_sync(FULL_MASK, warp_incl_max(ma), 1), eb = __shfl_up_sync(FULL_MASK, warp_incl_max(mb), 1);
        if (lane == 0) ea = eb = 0u;
        if (region_in_a) ea = max(ea, carry << cbits); else eb = max(eb, carry << cbits);
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int w = w_base + 4 * j;
            const bool in_a = w < ob;
            const unsigned src = in_a ? 0u : 1u;
            unsigned run = in_a ? ea : eb;
            uint4 v = q[j];
            run = max(run, v.x & ~cmask); v.x = ((run | (v.x & cmask)) << 1) | src;
            run = max(run, v.y & ~cmask); v.y = ((run | (v.y & cmask)) << 1) | src;
            run = max(run, v.z & ~cmask); v.z = ((run | (v.z & cmask)) << 1) | src;
            run = max(run, v.w & ~cmask); v.w = ((run | (v.w & cmask)) << 1) | src;
            if (in_a) ea = run; else eb = run;
            if (w < scan_end) *reinterpret_cast<uint4 *>(keys + w) = v;
        }
    }
    WorkerBar::sync();

    // ---- split the tile among threads: merge-path diagonal tid * VT (the operand bit makes
    // an A entry smaller than the B entry at the same position, so ties take A first)
    const int diag = min(tid * VT, n);
    int x0;
    {
        int lo = max(0, diag - nb), hi = min(diag, na);
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (kx[mid] < ky[diag - 1 - mid]) lo = mid + 1; else hi = mid;
        }
        x0 = lo;
    }
    const int y0 = diag - x0;
    const int cnt = min(VT, n - diag);
    // the next thread's split: from the next lane; the warp's last lane takes the split of the
    // warp's end diagonal, which the 32 lanes find together
    int x1 = __shfl_down_sync(FULL_MASK, x0, 1);
    {
        const int x_end = warp_count_cut(kx, na, ky, nb, min((wid + 1) * 32 * VT, n));
        if (lane == 31) x1 = x_end;
    }
    const int a = min(x1, x0 + cnt) - x0, b = cnt - a;

    // ---- merge in registers: A's entries ascending, the successor of the thread's range, an
    // all-ones plateau, B's entries descending -- a bitonic sequence -- through a merge network
    uint32_t r[NETV];
    {
        const uint32_t succ = min(kx[x0 + a], ky[y0 + b]);  // next merged key after this thread's range
#pragma unroll
        for (int i = 0; i < NETV; ++i) {
            const bool is_a = i < a, is_b = i >= NETV - b;
            const uint32_t *p = is_a ? kx + x0 + i : ky + y0 + (NETV - 1 - i);
            const uint32_t v = *p;  // stays inside the slack-padded key array either way
            r[i] = (is_a || is_b) ? v : (i == a ? succ : INF);
        }
    }
    const uint32_t prev_a = x0 > 0 ? kx[x0 - 1] : 0u;  // only an A entry can pair with a B entry
    bitonic_merge<NETV>(r);

    // Bit i of `from_a`: entry i came from A; of `same`: entries i and i+1 are one position (an A
    // entry and its B twin); of `emit`: entry i goes to the result.
    unsigned from_a = 0, same = 0;
#pragma unroll
    for (int i = 0; i < VT; ++i) {
        from_a |= (~r[i] & 1u) << i;
        same |= (unsigned)((r[i] ^ r[i + 1]) == 1u) << i;
    }
    const unsigned live = (1u << cnt) - 1u;
    const unsigned dup = (same << 1) | (unsigned)(x0 > 0 && (prev_a ^ r[0]) == 1u);  // B entries whose A twin precedes them
    const unsigned twin = same & from_a & live;
    const unsigned emit = OP == OP_UNION ? (live & ~dup) : twin;
    static_assert(VT < 32, "entry masks are 32 bits wide");

    // ---- rank the survivors inside the tile
    const int mine = __popc(emit);
    const int incl = warp_incl_sum(mine);
    if (lane == 31) s_wtotal[wid] = incl;
    WorkerBar::sync();  // also retires every thread's key reads: the staging pairs may overwrite the keys
    int total = 0, wbase = 0;
#pragma unroll
    for (int w = 0; w < W; ++w) {
        const int c = s_wtotal[w];
        wbase += w < wid ? c : 0;
        total += c;
    }
    const int rank = wbase + incl - mine;
    if (MODE == MODE_COUNT) {
        if (tid == 0) tile_count[t] = total;
        return;
    }
    thread_rank[tid] = rank;
    thread_emit[tid] = emit;
    if (MODE == MODE_FUSED) {
        if (tid == 0) {
            // successors can add this tile's count from here on
            st_relaxed_gpu(tile_state + t, (t == 0 ? LB_PREFIX : LB_AGGREGATE) | (uint64_t)total);
            s_total = total;
            *(volatile int *)&s_hurry = 1;
        }
        __threadfence_block();
        CountBar::arrive();  // the scan warp turns the count into the tile's inclusive prefix
    }

    // ---- compact (column, value) pairs of the survivors into the staging array. Entry i of the
    // thread came from A iff its key's operand bit is clear; its value sits at A's start + (A
    // entries before it) or B's start + (B entries before it), and an A entry's twin is the
    // next B entry.
    {
        const float *pa = vals + oa + x0, *pb = vals + obv + y0;
        uint2 *po = out_pair + rank;
        int ca = 0;  // A entries among the thread's first i entries
#pragma unroll
        for (int i = 0; i < VT; ++i) {
            const bool tx = (r[i] & 1u) == 0u;
            if (OP == OP_UNION) {
                float v = *(tx ? pa + ca : pb + (i - ca));
                if ((twin >> i) & 1u) v = v + pb[i - ca];  // an A entry whose twin is the next B entry
                if ((emit >> i) & 1u) {
                    *po = make_uint2((r[i] >> 1) & cmask, __float_as_uint(v));
                    ++po;
                }
            } else if ((emit >> i) & 1u) {  // intersection: only the twins need their values
                *po = make_uint2((r[i] >> 1) & cmask, __float_as_uint(pa[ca] * pb[i - ca]));
                ++po;
            }
            ca += tx;
        }
    }

    // ---- output base of the tile
    if (MODE == MODE_FUSED) __syncthreads(); else WorkerBar::sync();
    const long long base = MODE == MODE_FILL ? (long long)tile_count[t] : s_base;
    if (base < 0) return;  // a bounded wait gave up; the host reports it

    // ---- row offsets. Result row r starts after every result entry of rows < r; inside this
    // tile those are the survivors among the first d = (A entries before row r) + (B entries
    // before row r) merged entries, read off the per-thread ranks. The tile owns rows
    // i0+1 .. i1 (the next tile's first row).
    for (int64_t rw = my_row; rw <= i1; rw += NT) {
        const int sa = rw == my_row ? my_sa : ld_nc(A.rp + rw) - a0;
        const int sb = rw == my_row ? my_sb : ld_nc(B.rp + rw) - b0;
        const int d = sa + sb;
        const int owner = d / VT, off = d - owner * VT;
        const int before = owner >= NT ? total : thread_rank[owner] + __popc(thread_emit[owner] & ((1u << off) - 1u));
        Z.rp[rw] = (int32_t)(base + before);
    }
    if (t == 0 && tid == 0) Z.rp[0] = 0;

    // ---- store the compacted tile, coalesced
    int32_t *gz_col = Z.col + base;
    float *gz_val = Z.val + base;
    for (int i = tid; i < total; i += NT) {
        const uint2 p = out_pair[i];
        gz_col[i] = (int32_t)p.x;
        gz_val[i] = __uint_as_float(p.y);
    }
}

template <int V, int OP, int MODE>
__global__ void __launch_bounds__(NT + 32, CSR2_MIN_CTAS) k_csr2_tile(const __grid_constant__ CsrIn A, const __grid_constant__ CsrIn B,
                                                                         const __grid_constant__ Cuts cuts, int cbits, int32_t *tile_count,
                                                                         uint64_t *tile_state, FusedCtl *ctl,
                                                                         const __grid_constant__ CsrOut Z, int first_tile, int poll_limit) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t mbar;
    // Tiles are numbered by CTA index: CTAs are dispatched in increasing index order, so a tile
    // only ever waits on CTAs that were dispatched before it (and every such wait is bounded).
    // first_tile is 0 except in the self-test of the bounded waits, which leaves tile 0 out.
    const int t = blockIdx.x + first_tile;
    const int num_tiles = gridDim.x + first_tile;
    if (threadIdx.x == 0) {
        mbar_init(&mbar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    // 32-bit composite keys hold ((row in tile << cbits | column) << 1 | operand) when that
    // fits; tiles that span too many rows for that (long runs of empty rows) use 64-bit keys.
    const uint64_t nr = (uint64_t)(cuts.row[t + 1] - cuts.row[t]) + 1;
    const bool narrow = cbits < 31 && (nr << cbits) < 0x7fffffffull;
    if (narrow) {
        csr2_tile_blocked<V, OP, MODE>(A, B, cuts, cbits, t, num_tiles, tile_count, tile_state, ctl, Z, smem_raw, &mbar, poll_limit);
    } else {
        if (threadIdx.x >= NT) return;  // the wide-key body works with the NT worker threads alone
        csr2_tile_wide<V, OP, MODE>(A, B, cuts, t, tile_count, tile_state, ctl, Z, smem_raw, num_tiles, poll_limit);
    }
}

// ------------------------------------------------------------------------ host driver ----

constexpr int V_CSR2 = CSR2_V;
constexpr int TILE_STEP = NT * V_CSR2 - 1;  // merged entries between two tile cuts

// Dynamic shared memory of the tile kernel: the staging arrays of the common body, or the 64-bit
// keys of the wide-key body, whichever is larger.
constexpr size_t csr2_smem_bytes() {
    return std::max<size_t>(BlockedPlan<V_CSR2>::BYTES, 8 * (size_t)(NT * V_CSR2 + 2 + V_CSR2));
}

// Raises the tile kernel's dynamic shared-memory limit once per instantiation and device.
template <int OP, int MODE>
cudaError_t configure_tile_kernel() {
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(k_csr2_tile<V_CSR2, OP, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)csr2_smem_bytes());
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    return cudaSuccess;
}

// Test knobs of a launch: the first tile to run (the self-test of the bounded waits leaves tile 0
// out, so that every other tile waits for a count that never comes) and the number of polls after
// which a look-back gives up.
struct LaunchKnobs {
    int first_tile = 0;
    int poll_limit = LOOKBACK_POLL_LIMIT;
};

template <int OP, int MODE>
cudaError_t launch_tile(const CsrIn &A, const CsrIn &B, const Cuts &cuts, int cbits, int32_t *tile_count,
                        uint64_t *tile_state, FusedCtl *ctl, const CsrOut &Z, int num_tiles, cudaStream_t stream,
                        const LaunchKnobs &knobs = LaunchKnobs()) {
    cudaError_t e = configure_tile_kernel<OP, MODE>();
    if (e != cudaSuccess) return e;
    static const char *const names[2][3] = {{"csr_add_count", "csr_add_fill", "csr_add_fused"},
                                            {"csr_mul_count", "csr_mul_fill", "csr_mul_fused"}};
    if (num_tiles - knobs.first_tile <= 0) return cudaSuccess;
    LaunchScope scope(names[OP][MODE], stream);
    k_csr2_tile<V_CSR2, OP, MODE><<<num_tiles - knobs.first_tile, NT + 32, csr2_smem_bytes(), stream>>>(
        A, B, cuts, cbits, tile_count, tile_state, ctl, Z, knobs.first_tile, knobs.poll_limit);
    return cudaGetLastError();
}

// Shared driver of add and multiply. When `alloc` is set the result arrays are allocated
// here (one cudaMallocAsync each); otherwise z's arrays are the caller's, `capacity` entries.
//
// With room for the largest possible result (every operand entry for a union, the smaller
// operand for an intersection) the single-pass kernel runs. A caller-provided capacity below
// that bound takes the two-pass route, which knows the exact length before it writes.
//
// `device_result`, when given, makes the call asynchronous: the result length and the device
// status go to those two device words in stream order and the host does not wait (z->nnz stays 0).
// Only the single-pass route can do that; the call refuses a capacity below the bound.
template <int OP>
int csr2_run(const nb200_csr *a, const nb200_csr *b, nb200_csr *z, bool alloc, int64_t capacity, void *stream_v,
             int64_t *device_result = nullptr, const LaunchKnobs &knobs = LaunchKnobs()) {
    int st;
    if ((st = check_csr(a, true)) || (st = check_csr(b, true))) return st;
    if (!z || a->rows != b->rows || a->cols != b->cols) return NB200_E_BADARG;
    if (!alloc && (!z->row_ptr || capacity < 0)) return NB200_E_BADARG;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const int32_t rows = a->rows;
    const int64_t total = (int64_t)a->nnz + b->nnz;
    const int64_t tiles64 = (total + TILE_STEP - 1) / TILE_STEP;
    if (tiles64 > INT32_MAX - 1) return NB200_E_OVERFLOW;
    const int num_tiles = (int)tiles64;
    const int64_t bound = OP == OP_UNION ? total : std::min<int64_t>(a->nnz, b->nnz);
    // a caller's arrays must exist wherever the kernels may write: capacity > 0 promises col / val
    if (!alloc && capacity > 0 && total > 0 && (!z->col || !z->val)) return NB200_E_BADARG;
    if (device_result && (alloc || capacity < bound)) return NB200_E_CAPACITY;

    z->rows = rows;
    z->cols = a->cols;
    z->nnz = 0;
    if (alloc) {
        z->row_ptr = nullptr;
        z->col = nullptr;
        z->val = nullptr;
        NB200_CUDA(cudaMallocAsync(reinterpret_cast<void **>(&z->row_ptr), sizeof(int32_t) * ((size_t)rows + 1), stream));
    }
    auto fail = [&](int code) {
        if (alloc) {
            cudaFreeAsync(z->row_ptr, stream);
            if (z->col) cudaFreeAsync(z->col, stream);
            if (z->val) cudaFreeAsync(z->val, stream);
            z->row_ptr = z->col = nullptr;
            z->val = nullptr;
        }
        return code;
    };
    if (num_tiles == 0) {  // both operands empty: all-zero offsets, nothing else
        cudaError_t e = cudaMemsetAsync(z->row_ptr, 0, sizeof(int32_t) * ((size_t)rows + 1), stream);
        if (e == cudaSuccess && device_result) {
            const int64_t words[3] = {0, NB200_OK, rows};  // copied before the call returns: pageable source
            e = cudaMemcpyAsync(device_result, words, sizeof(words), cudaMemcpyDefault, stream);  // the words may be mapped host memory
        }
        if (e != cudaSuccess) return fail(note_cuda_error(e, "cudaMemsetAsync"));
        return NB200_OK;
    }

    Carver sizes;
    sizes.take<int32_t>((size_t)num_tiles + 1);
    sizes.take<int32_t>((size_t)num_tiles + 1);
    sizes.take<int32_t>((size_t)num_tiles + 1);
    sizes.take<int32_t>((size_t)num_tiles + 1);
    sizes.take<uint64_t>((size_t)num_tiles + 8);
    Workspace *ws = nullptr;
    if ((st = acquire_workspace(stream, sizes.used(), &ws))) return fail(st);
    Carver carve(ws->dev);
    Cuts cuts;
    cuts.row = carve.take<int32_t>((size_t)num_tiles + 1);
    cuts.a = carve.take<int32_t>((size_t)num_tiles + 1);
    cuts.b = carve.take<int32_t>((size_t)num_tiles + 1);
    int32_t *tile_count = carve.take<int32_t>((size_t)num_tiles + 1);
    // control block (status word, result length) and the tile words of the single-pass kernel,
    // contiguous for one memset; the two-pass route uses the control block alone
    uint64_t *fused_block = carve.take<uint64_t>((size_t)num_tiles + 8);
    static_assert(sizeof(FusedCtl) <= 4 * sizeof(uint64_t), "control block must fit its slot");
    FusedCtl *ctl = reinterpret_cast<FusedCtl *>(fused_block);
    uint64_t *tile_state = fused_block + 4;

    const CsrIn A{a->row_ptr, a->col, a->val, a->nnz}, B{b->row_ptr, b->col, b->val, b->nnz};
    const int cbits = col_bits(a->cols);
    // NACHO_B200_TWO_PASS=1 forces the count -> scan -> fill route (for comparisons).
    static const bool force_two_pass = [] { const char *e = std::getenv("NACHO_B200_TWO_PASS"); return e && e[0] == '1'; }();
    // NACHO_B200_EXACT_ALLOC=1 makes the allocating entry points count first and allocate col / val at
    // exactly nnz(Z), as the reference's drivers do (src/backend/stitch_and_generate.cpp:438-527),
    // instead of at the worst case: for callers short of memory, at the price of a second read of
    // the operands' columns.
    static const bool exact_alloc = [] { const char *e = std::getenv("NACHO_B200_EXACT_ALLOC"); return e && e[0] == '1'; }();
    const bool fused = device_result || (alloc ? !exact_alloc : (capacity >= bound && !force_two_pass));
    cudaError_t e = cudaSuccess;
    if (fused && alloc && bound > 0) {
        e = cudaMallocAsync(reinterpret_cast<void **>(&z->col), sizeof(int32_t) * (size_t)bound, stream);
        if (e == cudaSuccess) e = cudaMallocAsync(reinterpret_cast<void **>(&z->val), sizeof(float) * (size_t)bound, stream);
        if (e != cudaSuccess) return fail(note_cuda_error(e, "cudaMallocAsync"));
    }
    {
        LaunchScope scope("csr2_partition", stream);
        const int warps = num_tiles + 1;
        const int blocks = (warps * 32 + NT - 1) / NT;
        k_csr2_partition<<<blocks, NT, 0, stream>>>(A, B, rows, total, TILE_STEP, num_tiles, cuts, reinterpret_cast<long long *>(device_result),
                                                    fused_block, fused ? num_tiles + 4 : 4);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) return fail(note_cuda_error(e, "k_csr2_partition"));

    // Reads the control block back (one small copy and the call's only wait for the GPU).
    auto read_ctl = [&](FusedCtl &h) -> int {
        cudaError_t c = cudaMemcpyAsync(ws->host, ctl, sizeof(FusedCtl), cudaMemcpyDeviceToHost, stream);
        if (c == cudaSuccess) c = cudaStreamSynchronize(stream);
        if (c != cudaSuccess) return note_cuda_error(c, "read result length");
        std::memcpy(&h, ws->host, sizeof(h));
        return NB200_OK;
    };

    FusedCtl h;
    if (fused) {
        e = launch_tile<OP, MODE_FUSED>(A, B, cuts, cbits, nullptr, tile_state, ctl,
                                        CsrOut{z->row_ptr, z->col, z->val, reinterpret_cast<long long *>(device_result)}, num_tiles, stream, knobs);
        if (e != cudaSuccess) return fail(note_cuda_error(e, "k_csr2_tile<fused>"));
        if (device_result) return NB200_OK;  // length, status and rows arrive in the caller's device words, written by the kernels
        if ((st = read_ctl(h))) return fail(st);
        if (h.status.error != 0) return fail(note_timeout(h.status.error, h.status.detail, "csr merge"));
        if (h.total > INT32_MAX) return fail(NB200_E_OVERFLOW);
        z->nnz = (int32_t)h.total;
        if (alloc && h.total == 0) {  // zero-length arrays are handed over as NULL
            if (z->col) cudaFreeAsync(z->col, stream);
            if (z->val) cudaFreeAsync(z->val, stream);
            z->col = nullptr;
            z->val = nullptr;
        }
        return NB200_OK;
    }

    // count -> scan -> fill. The scan leaves the result length in the control block, whose status
    // word also collects a give-up of either tile launch (a bulk copy that did not land in time).
    e = launch_tile<OP, MODE_COUNT>(A, B, cuts, cbits, tile_count, nullptr, ctl, CsrOut{nullptr, nullptr, nullptr}, num_tiles, stream);
    if (e != cudaSuccess) return fail(note_cuda_error(e, "k_csr2_tile<count>"));
    {
        LaunchScope scope("scan_tiles", stream);
        k_scan_tiles<<<1, 1024, 0, stream>>>(tile_count, num_tiles, reinterpret_cast<int64_t *>(&ctl->total));
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) return fail(note_cuda_error(e, "k_scan_tiles"));
    if ((st = read_ctl(h))) return fail(st);
    if (h.status.error != 0) return fail(note_timeout(h.status.error, h.status.detail, "csr merge"));
    if (h.total > INT32_MAX) return fail(NB200_E_OVERFLOW);
    z->nnz = (int32_t)h.total;
    if (alloc) {
        if (h.total > 0) {
            e = cudaMallocAsync(reinterpret_cast<void **>(&z->col), sizeof(int32_t) * (size_t)h.total, stream);
            if (e == cudaSuccess) e = cudaMallocAsync(reinterpret_cast<void **>(&z->val), sizeof(float) * (size_t)h.total, stream);
            if (e != cudaSuccess) return fail(note_cuda_error(e, "cudaMallocAsync"));
        }
    } else if (h.total > capacity) {
        return NB200_E_CAPACITY;
    }
    e = launch_tile<OP, MODE_FILL>(A, B, cuts, cbits, tile_count, nullptr, ctl, CsrOut{z->row_ptr, z->col, z->val}, num_tiles, stream);
    if (e != cudaSuccess) return fail(note_cuda_error(e, "k_csr2_tile<fill>"));
    if ((st = read_ctl(h))) return fail(st);
    if (h.status.error != 0) return fail(note_timeout(h.status.error, h.status.detail, "csr merge"));
    return NB200_OK;
}

// Three-operand add Z = (A + B) + C as two chained unions (the fused kernel is in csr_add3.cu; this
// is its fallback). The association is the reference's
// (src/backend/compute.cpp:426-432 builds a + b first), so running the two-operand union twice
// gives bit-identical values to the reference's fused three-way merge: positions present in A
// and C only hold a + c, in B and C only b + c, in all three (a + b) + c, and explicit zeros
// stay. The intermediate A + B lives in the scratch pool; it costs one extra write and read of
// that intermediate compared with a single three-way pass.
int csr_add3_run(const nb200_csr *a, const nb200_csr *b, const nb200_csr *c, nb200_csr *z, bool alloc,
                 int64_t capacity, void *stream_v) {
    int st;
    if ((st = check_csr(c, true))) return st;
    if (!a || !b || a->rows != c->rows || a->cols != c->cols) return NB200_E_BADARG;
    if ((st = check_csr(a, true)) || (st = check_csr(b, true))) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    // the intermediate lives in its own pool block (slot 1), so it survives the two calls below,
    // which use slot 0, and costs no allocation after the first call
    const int64_t bound = (int64_t)a->nnz + b->nnz;
    Carver sizes;
    sizes.take<int32_t>((size_t)a->rows + 1);
    sizes.take<int32_t>((size_t)bound);
    sizes.take<float>((size_t)bound);
    Workspace *ws = nullptr;
    if ((st = acquire_workspace(stream, sizes.used(), &ws, 1))) return st;
    Carver carve(ws->dev);
    nb200_csr t{};
    t.row_ptr = carve.take<int32_t>((size_t)a->rows + 1);
    t.col = carve.take<int32_t>((size_t)bound);
    t.val = carve.take<float>((size_t)bound);
    if ((st = csr2_run<OP_UNION>(a, b, &t, false, bound, stream_v))) return st;
    return csr2_run<OP_UNION>(&t, c, z, alloc, capacity, stream_v);
}

// ------------------------------------------------------- entry point that allocates nothing ----

// Scratch of nb200_csr_add_f32_noalloc: tile cuts, the single-pass control block and one
// 8-byte word per tile, carved out of one fixed array that lives in the library's device image
// (so every GPU that loads the library holds these bytes until the process exits).
constexpr int NOALLOC_MAX_TILES = 32768;
constexpr size_t NOALLOC_SCRATCH_BYTES = 1u << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

// Device address of the array above for each device, looked up once per device. The array's
// name is only a host-side handle; kernels must be given the address from
// cudaGetSymbolAddress, taken while that device is current.
int noalloc_scratch_address(void **out) {
    static void *address[64] = {};
    static std::mutex lock;
    int dev = 0;
    NB200_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return NB200_E_UNSUPPORTED;
    std::lock_guard<std::mutex> g(lock);
    if (!address[dev]) {
        void *p = nullptr;
        NB200_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        // the tile kernel needs more dynamic shared memory than the default limit; set that
        // here too so that later calls are launches and nothing else
        NB200_CUDA(cudaFuncSetAttribute(k_csr2_tile<V_CSR2, OP_UNION, MODE_FUSED>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)csr2_smem_bytes()));
        address[dev] = p;
    }
    *out = address[dev];
    return NB200_OK;
}

int csr_add_noalloc(const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int64_t capacity, void *stream_v) {
    int st;
    if ((st = check_csr(a, true)) || (st = check_csr(b, true))) return st;
    if (!z || !z->row_ptr || capacity < 0 || a->rows != b->rows || a->cols != b->cols) return NB200_E_BADARG;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const int32_t rows = a->rows;
    const int64_t total = (int64_t)a->nnz + b->nnz;
    constexpr int tile_step = TILE_STEP;
    const int64_t tiles64 = (total + tile_step - 1) / tile_step;
    if (tiles64 > NOALLOC_MAX_TILES) return NB200_E_UNSUPPORTED;
    if (capacity < total) return NB200_E_CAPACITY;  // this entry point has the single-pass route only
    if (total > 0 && (!z->col || !z->val)) return NB200_E_BADARG;
    const int num_tiles = (int)tiles64;
    z->rows = rows;
    z->cols = a->cols;
    z->nnz = 0;
    if (num_tiles == 0) {
        NB200_CUDA(cudaMemsetAsync(z->row_ptr, 0, sizeof(int32_t) * ((size_t)rows + 1), stream));
        return NB200_OK;
    }
    void *scratch = nullptr;
    if ((st = noalloc_scratch_address(&scratch))) return st;
    Carver carve(scratch);
    uint64_t *fused_block = carve.take<uint64_t>((size_t)NOALLOC_MAX_TILES + 8);
    Cuts cuts;
    cuts.row = carve.take<int32_t>((size_t)NOALLOC_MAX_TILES + 1);
    cuts.a = carve.take<int32_t>((size_t)NOALLOC_MAX_TILES + 1);
    cuts.b = carve.take<int32_t>((size_t)NOALLOC_MAX_TILES + 1);
    static_assert(8 * (NOALLOC_MAX_TILES + 8 + 32) + 3 * (4 * (NOALLOC_MAX_TILES + 1) + 256) <= NOALLOC_SCRATCH_BYTES,
                  "scratch layout must fit the fixed array");
    FusedCtl *ctl = reinterpret_cast<FusedCtl *>(fused_block);
    uint64_t *tile_state = fused_block + 4;
    // the array keeps the previous call's contents: the ticket, the status and every tile word
    // must start at zero (the partition kernel clears them)

    const CsrIn A{a->row_ptr, a->col, a->val, a->nnz}, B{b->row_ptr, b->col, b->val, b->nnz};
    const int warps = num_tiles + 1;
    k_csr2_partition<<<(warps * 32 + NT - 1) / NT, NT, 0, stream>>>(A, B, rows, total, tile_step, num_tiles, cuts, nullptr, fused_block,
                                                                    num_tiles + 4);
    NB200_CUDA(cudaGetLastError());
    k_csr2_tile<V_CSR2, OP_UNION, MODE_FUSED><<<num_tiles, NT + 32, csr2_smem_bytes(), stream>>>(
        A, B, cuts, col_bits(a->cols), nullptr, tile_state, ctl, CsrOut{z->row_ptr, z->col, z->val}, 0, LOOKBACK_POLL_LIMIT);
    NB200_CUDA(cudaGetLastError());
    FusedCtl h;  // read back into ordinary host memory: no pinned buffer is taken for this
    NB200_CUDA(cudaMemcpyAsync(&h, ctl, sizeof(h), cudaMemcpyDeviceToHost, stream));
    NB200_CUDA(cudaStreamSynchronize(stream));
    if (h.status.error != 0) return note_timeout(h.status.error, h.status.detail, "csr merge (no-alloc)");
    if (h.total > INT32_MAX) return NB200_E_OVERFLOW;
    z->nnz = (int32_t)h.total;
    return NB200_OK;
}

}  // namespace

int csr_add3_chained(const nb200_csr *a, const nb200_csr *b, const nb200_csr *c, nb200_csr *z, bool alloc, int64_t capacity,
                     void *stream_v) {
    return csr_add3_run(a, b, c, z, alloc, capacity, stream_v);
}

}  // namespace nb200

using namespace nb200;

extern "C" {

int nb200_csr_add_f32(const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int32_t, int32_t, void *stream) {
    return csr2_run<OP_UNION>(a, b, z, true, 0, stream);
}

int nb200_csr_add_f32_into(const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int64_t capacity, void *stream) {
    return csr2_run<OP_UNION>(a, b, z, false, capacity, stream);
}

int nb200_csr_mul_f32(const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int32_t, int32_t, void *stream) {
    return csr2_run<OP_INTERSECT>(a, b, z, true, 0, stream);
}

int nb200_csr_mul_f32_into(const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int64_t capacity, void *stream) {
    return csr2_run<OP_INTERSECT>(a, b, z, false, capacity, stream);
}

int nb200_csr_add_f32_noalloc(const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int64_t capacity, void *stream) {
    return csr_add_noalloc(a, b, z, capacity, stream);
}

int nb200_csr_add_f32_async(const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int64_t capacity, int64_t *device_result,
                            void *stream) {
    if (!device_result) return NB200_E_BADARG;
    return csr2_run<OP_UNION>(a, b, z, false, capacity, stream, device_result);
}

int nb200_csr_mul_f32_async(const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int64_t capacity, int64_t *device_result,
                            void *stream) {
    if (!device_result) return NB200_E_BADARG;
    return csr2_run<OP_INTERSECT>(a, b, z, false, capacity, stream, device_result);
}

int nb200_selftest_lookback_timeout(const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int64_t capacity, int32_t polls,
                                    void *stream) {
    if (polls < 1 || !a || !b || capacity < (int64_t)a->nnz + b->nnz) return NB200_E_BADARG;
    LaunchKnobs knobs;
    knobs.first_tile = 1;
    knobs.poll_limit = polls;
    return csr2_run<OP_UNION>(a, b, z, false, capacity, stream, nullptr, knobs);
}

}  // extern "C"
