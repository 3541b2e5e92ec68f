// Fused three-operand CSR add Z = (A + B) + C in one pass over device memory: every operand entry
// is read once and every result entry written once; the intermediate A + B lives in shared memory
// only.
//
// What the reference does (restated, not its code): its partition for three operands bisects on
// the column value inside the row, with one search per operand and probe, because its merge-path
// shortcut needs exactly two operands (src/backend/partition.cpp:628-811, helper :551-584); its
// compute kernel walks the three lists together through the seven-case merge lattice
// (src/backend/compute.cpp:619-1392) and adds left to right, (a + b) + c (:426-432).
//
// Here:
//   k_csr3_partition   one warp per tile cut. The row comes from a 32-ary search on the summed row
//                      offsets of the three operands; inside the row the warp bisects on the column
//                      value, 32 columns per round, each lane counting the entries below its column
//                      in the three operands (three binary searches). A cut lies in front of a
//                      column, so entries of one position are never separated and a tile holds up
//                      to two entries fewer than the step.
//   k_csr3_tile        one CTA per tile. The copy engine stages the six arrays; the columns become
//                      composite keys (row in tile, column, one tag bit) as in the two-operand
//                      kernel. Stage 1 merges A's and B's keys (merge-path split, bitonic network in
//                      registers), adds the values of shared positions and compacts keys and values
//                      of A + B into a second pair of shared-memory arrays. Stage 2 merges that
//                      list with C's the same way, ranks the survivors, obtains the tile's output
//                      base from the scan warp's bounded look-back, and stores coalesced. Values of
//                      a position all three hold are (a + b) + c, bit-identical to the reference.
//
// Tiles whose rows do not fit the 32-bit key (long runs of empty rows) make the kernel report
// ERR_WIDE_TILE; the host then runs the chained two-operand route (csr_merge.cu), as it does for
// callers whose capacity is below nnz(A) + nnz(B) + nnz(C).
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "csr_common.cuh"
#include "warp_merge.cuh"

namespace nb200 {

namespace {

constexpr int NT = CSR_NT;
constexpr int W = NT / 32;
constexpr int VT = 11;                           // merged entries per thread and stage
constexpr int NETV = VT + 1;                     // merge-network slots in use
constexpr int CH = (VT + 1 + 3) & ~3;            // key words each thread scans
constexpr int CAP = NT * VT;                     // most merged entries of one tile
constexpr int TILE_STEP = CAP - 2;               // a cut may fall up to two entries short of its diagonal
constexpr int SLOTS = NT * CH + 64;              // staged key words = staged value words (three operands, pads, sentinels)
constexpr int MSLOTS = CAP + NETV + 4;           // keys / values of A + B
constexpr size_t SMEM_BYTES = 4 * (size_t)(2 * SLOTS + 2 * MSLOTS + 2 * CAP);
static_assert((CH / 4) % 2 == 1, "the scan chunk must be an odd number of 16-byte vectors");
static_assert(CAP + 3 * 7 + 1 + 2 * (NETV + 1) + 8 <= SLOTS, "three padded operands with their sentinels must fit");
static_assert(MSLOTS % 2 == 0 && SLOTS % 2 == 0, "the staging pairs must stay 8-byte aligned");

struct Cuts3 {
    int32_t *row, *a, *b, *c;
};

// Number of entries of the sorted segment col[lo, hi) that are below `v`.
__device__ __forceinline__ int32_t count_below(const int32_t *col, int32_t lo, int32_t hi, int32_t v) {
    const int32_t base = lo;
    while (lo < hi) {
        const int32_t mid = lo + ((hi - lo) >> 1);
        if (ld_nc(col + mid) < v) lo = mid + 1; else hi = mid;
    }
    return lo - base;
}

// One warp per cut. Cut t lies in front of the column that holds merged position
// min(t * tile_step, total) of the three operands' entries in (row, column) order.
__global__ void __launch_bounds__(NT) k_csr3_partition(CsrIn A, CsrIn B, CsrIn C, int32_t rows, int32_t cols, int64_t total,
                                                       int32_t tile_step, int32_t num_tiles, Cuts3 cuts) {
    const int t = (blockIdx.x * NT + threadIdx.x) >> 5;
    if (t > num_tiles) return;
    const int32_t a_base = ld_nc(A.rp), b_base = ld_nc(B.rp), c_base = ld_nc(C.rp);
    const int64_t d = (int64_t)t * tile_step;
    int32_t row, pa, pb, pc;
    if (t == 0) {
        row = 0, pa = a_base, pb = b_base, pc = c_base;
    } else if (t == num_tiles || d >= total) {
        row = rows, pa = a_base + A.nnz, pb = b_base + B.nnz, pc = c_base + C.nnz;
    } else {
        auto work = [&](int64_t i) -> int64_t {
            return (int64_t)(ld_nc(A.rp + i) - a_base) + (int64_t)(ld_nc(B.rp + i) - b_base) + (int64_t)(ld_nc(C.rp + i) - c_base);
        };
        row = (int32_t)warp_last_true(0, (int64_t)rows - 1, [&](int64_t i) { return work(i) <= d; });
        const int32_t a_lo = ld_nc(A.rp + row), a_hi = ld_nc(A.rp + row + 1);
        const int32_t b_lo = ld_nc(B.rp + row), b_hi = ld_nc(B.rp + row + 1);
        const int32_t c_lo = ld_nc(C.rp + row), c_hi = ld_nc(C.rp + row + 1);
        const int64_t dd = d - work(row);  // merged position inside the row
        // the largest column v with (entries of the row below v) <= dd: position dd holds column v
        const int64_t v = warp_last_true(0, (int64_t)cols - 1, [&](int64_t c) {
            return (int64_t)count_below(A.col, a_lo, a_hi, (int32_t)c) + count_below(B.col, b_lo, b_hi, (int32_t)c) +
                       count_below(C.col, c_lo, c_hi, (int32_t)c) <= dd;
        });
        pa = a_lo + count_below(A.col, a_lo, a_hi, (int32_t)v);
        pb = b_lo + count_below(B.col, b_lo, b_hi, (int32_t)v);
        pc = c_lo + count_below(C.col, c_lo, c_hi, (int32_t)v);
    }
    if (lane_id() == 0) {
        cuts.row[t] = row;
        cuts.a[t] = pa;
        cuts.b[t] = pb;
        cuts.c[t] = pc;
    }
}

// One merge stage of the tile: the sorted key lists kx[0, nx) (even keys) and ky[0, ny) (odd keys)
// in shared memory are split among the NT worker threads by merge-path, and each thread merges its
// VT entries in registers. On return r[] holds the thread's merged keys (r[VT] the key after them)
// and the masks speak about entry i in bit i: `same` -- an even key followed by its odd twin;
// `emit` -- the entry goes to the stage's output (an odd key whose twin precedes it does not);
// x0 / y0 are the thread's first entries in the two lists, cnt its number of entries.
struct StageSplit {
    int x0, y0, cnt;
    unsigned same, emit;
};

__device__ __forceinline__ StageSplit merge_stage(const uint32_t *kx, const int nx, const uint32_t *ky, const int ny,
                                                  uint32_t (&r)[NETV]) {
    constexpr uint32_t INF = 0xffffffffu;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int n = nx + ny;
    const int diag = min(tid * VT, n);
    int x0;
    {
        int lo = max(0, diag - ny), hi = min(diag, nx);
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
        const int x_end = warp_count_cut(kx, nx, ky, ny, min((wid + 1) * 32 * VT, n));
        if (lane == 31) x1 = x_end;
    }
    const int a = min(x1, x0 + cnt) - x0, b = cnt - a;
    // the thread's even keys ascending, the key that follows its range, an all-ones plateau, its
    // odd keys descending -- a bitonic sequence -- through the merge network
    {
        const uint32_t succ = min(kx[x0 + a], ky[y0 + b]);
#pragma unroll
        for (int i = 0; i < NETV; ++i) {
            const bool is_a = i < a, is_b = i >= NETV - b;
            const uint32_t *p = is_a ? kx + x0 + i : ky + y0 + (NETV - 1 - i);
            const uint32_t v = *p;  // stays inside the sentinel-padded arrays either way
            r[i] = (is_a || is_b) ? v : (i == a ? succ : INF);
        }
    }
    const uint32_t prev_a = x0 > 0 ? kx[x0 - 1] : 0u;  // only an even key can pair with the odd key after it
    bitonic_merge<NETV>(r);
    unsigned same = 0;
#pragma unroll
    for (int i = 0; i < VT; ++i) same |= (unsigned)((r[i] ^ r[i + 1]) == 1u) << i;
    const unsigned live = (1u << cnt) - 1u;
    const unsigned dup = (same << 1) | (unsigned)(x0 > 0 && (prev_a ^ r[0]) == 1u);
    StageSplit s;
    s.x0 = x0, s.y0 = y0, s.cnt = cnt;
    s.same = same & live;
    s.emit = live & ~dup;
    return s;
}

// Exclusive rank of `mine` among the worker threads and the CTA's total: warp scans, one barrier.
__device__ __forceinline__ int tile_rank(const int mine, int *s_wtotal, int &total) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int incl = warp_incl_sum(mine);
    if (lane == 31) s_wtotal[wid] = incl;
    WorkerBar::sync();
    int wbase = 0;
    total = 0;
#pragma unroll
    for (int w = 0; w < W; ++w) {
        const int c = s_wtotal[w];
        wbase += w < wid ? c : 0;
        total += c;
    }
    return wbase + incl - mine;
}

__global__ void __launch_bounds__(NT + 32, 3) k_csr3_tile(const __grid_constant__ CsrIn A, const __grid_constant__ CsrIn B,
                                                          const __grid_constant__ CsrIn C, const __grid_constant__ Cuts3 cuts,
                                                          const int cbits, uint64_t *tile_state_raw, FusedCtl *ctl,
                                                          const __grid_constant__ CsrOut Z) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t mbar;
    __shared__ int rank1[NT], rank2[NT];
    __shared__ unsigned emit1[NT], emit2[NT];
    __shared__ int s_wtotal1[W], s_wtotal2[W];
    __shared__ long long s_base;
    __shared__ int s_total, s_hurry;
    constexpr uint32_t INF = 0xffffffffu;
    volatile uint64_t *tile_state = tile_state_raw;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const bool scan_warp = tid >= NT;
    const int t = blockIdx.x;  // CTAs are dispatched in index order: a tile only waits on tiles dispatched before it
    const int num_tiles = gridDim.x;
    if (tid == 0) {
        mbar_init(&mbar, 1);
        mbar_fence_init();
        s_hurry = 0;
    }
    __syncthreads();
    const int32_t i0 = cuts.row[t], i1 = cuts.row[t + 1];
    const uint64_t nr = (uint64_t)(i1 - i0) + 1;
    if (!(cbits < 31 && (nr << cbits) < 0x7fffffffull)) {
        // the rows of this tile do not fit the key: report, let the successors through, write nothing
        if (tid == 0) {
            atomicCAS(&ctl->status.error, 0, ERR_WIDE_TILE);
            tile_state[t] = LB_PREFIX;
        }
        return;
    }
    const CsrIn *op[3] = {&A, &B, &C};
    int32_t first[3], count[3], word[3], region[3], head[3], nvec[3];
    bool val_bulk[3];
    {
        const int32_t *cut[3] = {cuts.a, cuts.b, cuts.c};
        int next = 0;
#pragma unroll
        for (int q = 0; q < 3; ++q) {
            first[q] = cut[q][t];
            count[q] = cut[q][t + 1] - first[q];
            const int h = head_elems(op[q]->col + first[q]);
            region[q] = next;                        // first word of the operand's region (16-byte aligned)
            word[q] = next + ((4 - h) & 3);          // word of the operand's entry 0
            head[q] = min(count[q], h);
            nvec[q] = (count[q] - head[q]) >> 2;     // 16-byte vectors in the interior
            val_bulk[q] = head_elems(op[q]->val + first[q]) == h;
            // sentinels behind the entries: one word for A, a merge network's worth for B and C
            next = (word[q] + count[q] + (q == 0 ? 1 : NETV + 1) + 3) & ~3;
        }
    }
    const int na = count[0], nb = count[1], nc = count[2];
    const int scan_end = (word[2] + nc + 3) & ~3;
    const uint32_t cmask = (1u << cbits) - 1u;

    // layout: staged values | staged keys | keys of A + B | values of A + B | result staging pairs
    float *vals = reinterpret_cast<float *>(smem_raw);
    uint32_t *keys = reinterpret_cast<uint32_t *>(smem_raw) + SLOTS;
    uint32_t *mk = keys + SLOTS;
    float *mv = reinterpret_cast<float *>(mk + MSLOTS);
    uint2 *out_pair = reinterpret_cast<uint2 *>(mv + MSLOTS);

    // ---- stage the tile: aligned interiors by bulk copy, ragged ends (at most three entries each
    // side) and value arrays whose alignment differs from their column array's by plain loads
    if (tid == 0) {
        uint32_t bytes = 0;
#pragma unroll
        for (int q = 0; q < 3; ++q) bytes += 16u * nvec[q] * (val_bulk[q] ? 2u : 1u);
        mbar_arrive_expect_tx(&mbar, bytes);
#pragma unroll
        for (int q = 0; q < 3; ++q) {
            if (!nvec[q]) continue;
            bulk_load(keys + word[q] + head[q], op[q]->col + first[q] + head[q], 16u * nvec[q], &mbar);
            if (val_bulk[q]) bulk_load(vals + word[q] + head[q], op[q]->val + first[q] + head[q], 16u * nvec[q], &mbar);
        }
    }
    if (tid >= 32 && tid < 32 + 18) {  // ragged ends: 3 head + 3 tail slots per operand
        const int q = (tid - 32) / 6, e = (tid - 32) % 6;
        int32_t cnt_q = 0, head_q = 0, nv_q = 0, word_q = 0, first_q = 0;
        bool bulk_q = false;
        const CsrIn *src = &A;
#pragma unroll
        for (int k = 0; k < 3; ++k)
            if (k == q) cnt_q = count[k], head_q = head[k], nv_q = nvec[k], word_q = word[k], first_q = first[k], bulk_q = val_bulk[k], src = op[k];
        const int idx = e < 3 ? e : head_q + 4 * nv_q + (e - 3);
        const bool live = e < 3 ? e < head_q : idx < cnt_q;
        if (live) {
            keys[word_q + idx] = (uint32_t)ld_nc(src->col + first_q + idx);
            if (bulk_q) vals[word_q + idx] = ld_nc(src->val + first_q + idx);
        }
    }
#pragma unroll
    for (int q = 0; q < 3; ++q)
        if (!val_bulk[q] && !scan_warp)
            for (int i = tid; i < count[q]; i += NT) vals[word[q] + i] = ld_nc(op[q]->val + first[q] + i);
    // padding words in front of live keys must read as "no row mark"; sentinels behind them as all-ones
    if (tid >= 64 && tid < 64 + 9) {
        const int q = (tid - 64) / 3, k = (tid - 64) % 3;
        int32_t region_q = 0, word_q = 0;
#pragma unroll
        for (int j = 0; j < 3; ++j)
            if (j == q) region_q = region[j], word_q = word[j];
        if (region_q + k < word_q) keys[region_q + k] = 0u;
    }
    if (tid == 80) keys[word[0] + na] = INF;
    if (tid >= 96 && tid < 96 + NETV + 1) keys[word[1] + nb + (tid - 96)] = INF;
    if (tid >= 128 && tid < 128 + NETV + 1) keys[word[2] + nc + (tid - 128)] = INF;

    // row offsets of the first row this thread looks after (rows i0+1 .. i1 are spread over the workers)
    const int64_t my_row = (int64_t)i0 + 1 + tid;
    int32_t my_s[3] = {0, 0, 0};
    if (!scan_warp && my_row <= i1) {
#pragma unroll
        for (int q = 0; q < 3; ++q) my_s[q] = ld_nc(op[q]->rp + my_row) - first[q];
    }
    // ---- the row (relative to i0) of the first key word this warp scans: the last row that starts
    // at or before it in the operand whose region the word lies in (found while the copies fly)
    const int w0 = wid * 32 * CH;
    const int start_region = w0 < region[1] ? 0 : (w0 < region[2] ? 1 : 2);
    unsigned carry = 0;
    if (!scan_warp) {
        int32_t word_q = 0, first_q = 0;
        const int32_t *rp = A.rp;
#pragma unroll
        for (int q = 0; q < 3; ++q)
            if (q == start_region) word_q = word[q], first_q = first[q], rp = op[q]->rp;
        const int pos = w0 - word_q;
        if (pos > 0 && i1 > i0)
            carry = (unsigned)(warp_last_true(i0, i1, [&](int64_t r) { return ld_nc(rp + r) - first_q <= pos; }) - i0);
    }
    const bool landed = mbar_wait_bounded(&mbar, 0, MBAR_POLL_LIMIT);
    if (!__syncthreads_and(landed)) {  // the copies did not land in time: report, touch nothing
        if (tid == 0) {
            if (atomicCAS(&ctl->status.error, 0, ERR_COPY_TIMEOUT) == 0) ctl->status.detail = t;
            tile_state[t] = LB_PREFIX;  // successors must not wait on this tile
            mbar_wait_bounded(&mbar, 0, MBAR_POLL_LIMIT);  // second bounded wait for copies in flight
        }
        return;
    }

    if (scan_warp) {
        // the tile's output base is the sum of the counts of all earlier tiles: the walk over their
        // words starts now, while the workers merge
        const int64_t bse = t == 0 ? 0 : lookback_predecessors(tile_state, t, &ctl->status, 2000, &s_hurry, 1000);
        CountBar::sync();  // the workers have published the tile's count by now
        const int total = s_total;
        if (lane == 0) {
            if (t > 0) st_relaxed_gpu(tile_state + t, LB_PREFIX | (uint64_t)(bse < 0 ? 0 : bse + total));
            s_base = bse;
            if (bse >= 0 && t == num_tiles - 1) ctl->total = bse + total;
        }
        __syncthreads();
        return;
    }

    // ---- mark the first entry of every row that starts inside the tile with its row number
    // relative to i0, in the bits above the column (max wins where empty rows share a start)
    for (int64_t r = my_row; r <= i1; r += NT) {
        const uint32_t rr = (uint32_t)(r - i0);
#pragma unroll
        for (int q = 0; q < 3; ++q) {
            const int s = r == my_row ? my_s[q] : ld_nc(op[q]->rp + r) - first[q];
            if (s < count[q]) atomicMax(keys + word[q] + s, (rr << cbits) | (keys[word[q] + s] & cmask));
        }
    }
    WorkerBar::sync();

    // ---- spread the marks forward (running maximum, each operand's words on their own) so that
    // every key carries its row, and append the tag bit: 0 for A, 1 for B and for C. A thread owns
    // CH consecutive words, a warp 32 * CH; the warp's first row came from the search above.
    {
        constexpr int NV = CH / 4;
        const int w_base = tid * CH;
        uint4 q4[NV];
        unsigned m[3] = {0u, 0u, 0u};
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int w = w_base + 4 * j;
            q4[j] = w < scan_end ? *reinterpret_cast<const uint4 *>(keys + w) : make_uint4(0, 0, 0, 0);
            const unsigned mx = max(max(q4[j].x & ~cmask, q4[j].y & ~cmask), max(q4[j].z & ~cmask, q4[j].w & ~cmask));
            const int reg = w < region[1] ? 0 : (w < region[2] ? 1 : 2);
#pragma unroll
            for (int q = 0; q < 3; ++q) m[q] = reg == q ? max(m[q], mx) : m[q];
        }
        unsigned e[3];
#pragma unroll
        for (int q = 0; q < 3; ++q) {
            e[q] = __shfl_up_sync(FULL_MASK, warp_incl_max(m[q]), 1);
            if (lane == 0) e[q] = 0u;
            if (q == start_region) e[q] = max(e[q], carry << cbits);
        }
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int w = w_base + 4 * j;
            const int reg = w < region[1] ? 0 : (w < region[2] ? 1 : 2);
            const unsigned tag = reg == 0 ? 0u : 1u;
            unsigned run = reg == 0 ? e[0] : (reg == 1 ? e[1] : e[2]);
            uint4 v = q4[j];
            run = max(run, v.x & ~cmask); v.x = ((run | (v.x & cmask)) << 1) | tag;
            run = max(run, v.y & ~cmask); v.y = ((run | (v.y & cmask)) << 1) | tag;
            run = max(run, v.z & ~cmask); v.z = ((run | (v.z & cmask)) << 1) | tag;
            run = max(run, v.w & ~cmask); v.w = ((run | (v.w & cmask)) << 1) | tag;
#pragma unroll
            for (int q = 0; q < 3; ++q) e[q] = reg == q ? run : e[q];
            if (w < scan_end) *reinterpret_cast<uint4 *>(keys + w) = v;
        }
    }
    WorkerBar::sync();

    // ---- stage 1: A + B into (mk, mv), compacted; a position both hold carries a + b
    uint32_t r[NETV];
    int total1;
    {
        const uint32_t *kx = keys + word[0], *ky = keys + word[1];
        const StageSplit s = merge_stage(kx, na, ky, nb, r);
        const int rank = tile_rank(__popc(s.emit), s_wtotal1, total1);
        rank1[tid] = rank;
        emit1[tid] = s.emit;
        const float *pa = vals + word[0] + s.x0, *pb = vals + word[1] + s.y0;
        int ca = 0, o = rank;
#pragma unroll
        for (int i = 0; i < VT; ++i) {
            const bool tx = (r[i] & 1u) == 0u;
            float v = *(tx ? pa + ca : pb + (i - ca));
            if ((s.same >> i) & 1u) v = v + pb[i - ca];  // an A entry whose twin is the next B entry
            if ((s.emit >> i) & 1u) {
                mk[o] = r[i] & ~1u;  // the sum plays the first operand's part in stage 2
                mv[o] = v;
                ++o;
            }
            ca += tx;
        }
        if (tid < NETV + 1) mk[total1 + tid] = INF;  // nobody's entries: total1 is the same in every thread
    }
    WorkerBar::sync();

    // ---- stage 2: (A + B) + C
    int total;
    const StageSplit s = merge_stage(mk, total1, keys + word[2], nc, r);
    const int rank = tile_rank(__popc(s.emit), s_wtotal2, total);
    rank2[tid] = rank;
    emit2[tid] = s.emit;
    if (tid == 0) {
        // successors can add this tile's count from here on
        st_relaxed_gpu(tile_state + t, (t == 0 ? LB_PREFIX : LB_AGGREGATE) | (uint64_t)total);
        s_total = total;
        *(volatile int *)&s_hurry = 1;
    }
    __threadfence_block();
    CountBar::arrive();  // the scan warp turns the count into the tile's inclusive prefix
    {
        const float *pa = mv + s.x0, *pb = vals + word[2] + s.y0;
        uint2 *po = out_pair + rank;
        int ca = 0;
#pragma unroll
        for (int i = 0; i < VT; ++i) {
            const bool tx = (r[i] & 1u) == 0u;
            float v = *(tx ? pa + ca : pb + (i - ca));
            if ((s.same >> i) & 1u) v = v + pb[i - ca];  // (a + b) + c
            if ((s.emit >> i) & 1u) {
                *po = make_uint2((r[i] >> 1) & cmask, __float_as_uint(v));
                ++po;
            }
            ca += tx;
        }
    }
    __syncthreads();  // the scan warp has the base; the staging pairs are complete
    const long long base = s_base;
    if (base < 0) return;  // a bounded wait gave up; the host reports it

    // ---- row offsets. Result row r starts after every result entry of rows < r: those are the
    // survivors among the first (entries of A + B before row r) + (entries of C before row r)
    // entries of stage 2, and the entries of A + B before row r are the survivors among the first
    // (A entries before r) + (B entries before r) entries of stage 1. The tile owns rows i0+1 .. i1.
    for (int64_t rw = my_row; rw <= i1; rw += NT) {
        int sq[3];
#pragma unroll
        for (int q = 0; q < 3; ++q) sq[q] = rw == my_row ? my_s[q] : ld_nc(op[q]->rp + rw) - first[q];
        const int d1 = sq[0] + sq[1];
        const int o1 = d1 / VT, f1 = d1 - o1 * VT;
        const int sm = o1 >= NT ? total1 : rank1[o1] + __popc(emit1[o1] & ((1u << f1) - 1u));
        const int d2 = sm + sq[2];
        const int o2 = d2 / VT, f2 = d2 - o2 * VT;
        const int before = o2 >= NT ? total : rank2[o2] + __popc(emit2[o2] & ((1u << f2) - 1u));
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

int csr_add3_run(const nb200_csr *a, const nb200_csr *b, const nb200_csr *c, nb200_csr *z, bool alloc, int64_t capacity,
                 void *stream_v) {
    int st;
    if ((st = check_csr(a, true)) || (st = check_csr(b, true)) || (st = check_csr(c, true))) return st;
    if (!z || a->rows != b->rows || a->cols != b->cols || a->rows != c->rows || a->cols != c->cols) return NB200_E_BADARG;
    if (!alloc && (!z->row_ptr || capacity < 0)) return NB200_E_BADARG;
    const int64_t total = (int64_t)a->nnz + b->nnz + c->nnz;
    if (total > INT32_MAX) return NB200_E_OVERFLOW;
    if (!alloc && capacity > 0 && total > 0 && (!z->col || !z->val)) return NB200_E_BADARG;
    static const bool force_chained = [] { const char *e = std::getenv("NACHO_B200_ADD3_CHAINED"); return e && e[0] == '1'; }();
    // the fused kernel writes at its final positions in one pass: it needs room for the worst case
    if (force_chained || total == 0 || (!alloc && capacity < total)) return csr_add3_chained(a, b, c, z, alloc, capacity, stream_v);

    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const int32_t rows = a->rows;
    const int num_tiles = (int)((total + TILE_STEP - 1) / TILE_STEP);
    Carver sizes;
    for (int q = 0; q < 4; ++q) sizes.take<int32_t>((size_t)num_tiles + 1);
    sizes.take<uint64_t>((size_t)num_tiles + 8);
    Workspace *ws = nullptr;
    if ((st = acquire_workspace(stream, sizes.used(), &ws, 3))) return st;  // slot 3: the chained fallback uses 0 and 1
    Carver carve(ws->dev);
    Cuts3 cuts;
    cuts.row = carve.take<int32_t>((size_t)num_tiles + 1);
    cuts.a = carve.take<int32_t>((size_t)num_tiles + 1);
    cuts.b = carve.take<int32_t>((size_t)num_tiles + 1);
    cuts.c = carve.take<int32_t>((size_t)num_tiles + 1);
    uint64_t *fused_block = carve.take<uint64_t>((size_t)num_tiles + 8);
    FusedCtl *ctl = reinterpret_cast<FusedCtl *>(fused_block);
    uint64_t *tile_state = fused_block + 4;

    nb200_csr out = *z;  // the caller's struct is filled in only once the route is settled
    out.rows = rows, out.cols = a->cols, out.nnz = 0;
    cudaError_t e;
    if (alloc) {
        out.row_ptr = out.col = nullptr;
        out.val = nullptr;
        e = cudaMallocAsync(reinterpret_cast<void **>(&out.row_ptr), sizeof(int32_t) * ((size_t)rows + 1), stream);
        if (e == cudaSuccess) e = cudaMallocAsync(reinterpret_cast<void **>(&out.col), sizeof(int32_t) * (size_t)total, stream);
        if (e == cudaSuccess) e = cudaMallocAsync(reinterpret_cast<void **>(&out.val), sizeof(float) * (size_t)total, stream);
        if (e != cudaSuccess) {
            if (out.row_ptr) cudaFreeAsync(out.row_ptr, stream);
            if (out.col) cudaFreeAsync(out.col, stream);
            return note_cuda_error(e, "cudaMallocAsync");
        }
    }
    auto release = [&]() {
        if (alloc) {
            cudaFreeAsync(out.row_ptr, stream);
            cudaFreeAsync(out.col, stream);
            cudaFreeAsync(out.val, stream);
        }
    };
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        e = cudaFuncSetAttribute(k_csr3_tile, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return release(), note_cuda_error(e, "cudaFuncSetAttribute");
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const CsrIn A{a->row_ptr, a->col, a->val, a->nnz}, B{b->row_ptr, b->col, b->val, b->nnz}, C{c->row_ptr, c->col, c->val, c->nnz};
    e = cudaMemsetAsync(fused_block, 0, sizeof(uint64_t) * ((size_t)num_tiles + 4), stream);
    if (e != cudaSuccess) return release(), note_cuda_error(e, "cudaMemsetAsync");
    {
        LaunchScope scope("csr3_partition", stream);
        const int warps = num_tiles + 1;
        k_csr3_partition<<<(warps * 32 + NT - 1) / NT, NT, 0, stream>>>(A, B, C, rows, a->cols, total, TILE_STEP, num_tiles, cuts);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) return release(), note_cuda_error(e, "k_csr3_partition");
    {
        LaunchScope scope("csr_add3_fused", stream);
        k_csr3_tile<<<num_tiles, NT + 32, SMEM_BYTES, stream>>>(A, B, C, cuts, col_bits(a->cols), tile_state, ctl,
                                                                  CsrOut{out.row_ptr, out.col, out.val});
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) return release(), note_cuda_error(e, "k_csr3_tile");
    e = cudaMemcpyAsync(ws->host, ctl, sizeof(FusedCtl), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return release(), note_cuda_error(e, "read result length");
    FusedCtl h;
    std::memcpy(&h, ws->host, sizeof(h));
    if (h.status.error == ERR_WIDE_TILE) {  // long runs of empty rows: the two-operand kernels have a wide-key body
        release();
        return csr_add3_chained(a, b, c, z, alloc, capacity, stream_v);
    }
    if (h.status.error != 0) return release(), note_timeout(h.status.error, h.status.detail, "csr add3");
    if (h.total > INT32_MAX) return release(), NB200_E_OVERFLOW;
    *z = out;
    z->nnz = (int32_t)h.total;
    if (alloc && h.total == 0) {  // zero-length arrays are handed over as NULL
        cudaFreeAsync(z->col, stream);
        cudaFreeAsync(z->val, stream);
        z->col = nullptr;
        z->val = nullptr;
    }
    return NB200_OK;
}

}  // namespace

}  // namespace nb200

using namespace nb200;

extern "C" {

int nb200_csr_add_3_f32(const nb200_csr *a, const nb200_csr *b, const nb200_csr *c, nb200_csr *z, int32_t, int32_t,
                        void *stream) {
    return csr_add3_run(a, b, c, z, true, 0, stream);
}

int nb200_csr_add_3_f32_into(const nb200_csr *a, const nb200_csr *b, const nb200_csr *c, nb200_csr *z,
                             int64_t capacity, void *stream) {
    return csr_add3_run(a, b, c, z, false, capacity, stream);
}

}  // extern "C"
