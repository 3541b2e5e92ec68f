// COO3 tensor add: sorted union of two 3-mode tensors stored as parallel (i, j, k) coordinate
// arrays, as one flat merge-path over lexicographic coordinate order.
//
// The reference flattens the three COO levels into one merged coordinate and compares
// tuples (src/Compile.cpp:66-154, src/backend/tensor.cpp:447-560); its partition is the 2-way
// merge-path with the rule that equal coordinates are never split
// (src/backend/partition.cpp:813-993, :964-983). Here each coordinate is packed into one
// 64-bit key, i in the top bits, then j, then k, using just enough bits for each extent, so
// that tuple order is integer order. Tensors whose three extents need more than 63 bits in
// total take a second, simpler tile kernel that compares (i, j) and k as a 64-bit and a 32-bit
// word, i.e. the full three-int32 tuple compare of the reference for any extents.
//
// Kernels: k_coo3_partition (one warp per tile cut, 32-ary diagonal search) and k_coo3_tile
// (one CTA per tile: pack keys into shared memory, split by merge-path, merge VT entries per
// thread, rank survivors, obtain the output base -- single pass with bounded look-back, or
// from the scanned counts of a first pass -- compact through shared memory, store coalesced).
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "merge_common.cuh"
#include "tma.cuh"

namespace nb200 {

namespace {

#ifndef COO3_NT
#define COO3_NT 256
#endif
#ifndef COO3_VT
#define COO3_VT 11
#endif
#ifndef COO3_MIN_CTAS
#define COO3_MIN_CTAS 4
#endif
constexpr int NT = COO3_NT;
constexpr int VT = COO3_VT;
constexpr int CAP = NT * VT;
constexpr int KEY_SLOTS = CAP + 2 + VT;
constexpr uint64_t INF = ~0ull;

struct Coo3In {
    const int32_t *i, *j, *k;
    const float *val;
    int32_t nnz;
};

struct Coo3Out {
    int32_t *i, *j, *k;
    float *val;
};

struct Packing {
    using Key = uint64_t;
    int bj, bk;  // bits of j and k; i takes the rest
    __host__ __device__ uint64_t pack(int32_t i, int32_t j, int32_t k) const {
        return ((((uint64_t)(uint32_t)i << bj) | (uint32_t)j) << bk) | (uint32_t)k;
    }
    __host__ __device__ int32_t i_of(uint64_t key) const { return (int32_t)(key >> (bj + bk)); }
    __host__ __device__ int32_t j_of(uint64_t key) const { return (int32_t)((key >> bk) & ((1ull << bj) - 1ull)); }
    __host__ __device__ int32_t k_of(uint64_t key) const { return (int32_t)(key & ((1ull << bk) - 1ull)); }
};

// Coordinates too wide for one 64-bit word: (i, j) in one word, k in another, compared in that
// order -- the three-int32 tuple order of the reference (src/backend/tensor.cpp:447-560).
struct Key96 {
    uint64_t ij;
    uint32_t k;
    __device__ bool operator<=(const Key96 &o) const { return ij < o.ij || (ij == o.ij && k <= o.k); }
    __device__ bool operator==(const Key96 &o) const { return ij == o.ij && k == o.k; }
};
struct WidePacking {
    using Key = Key96;
    __device__ Key96 pack(int32_t i, int32_t j, int32_t k) const {
        return Key96{((uint64_t)(uint32_t)i << 32) | (uint32_t)j, (uint32_t)k};
    }
};

struct Cuts2 {
    int32_t *a;
    int32_t *b;
};

template <typename PK>
__device__ __forceinline__ typename PK::Key key_at(const Coo3In &T, const PK &pk, int64_t p) {
    return pk.pack(ld_nc(T.i + p), ld_nc(T.j + p), ld_nc(T.k + p));
}

// Tile cuts, found in two levels so that the searches read little: every COARSE-th cut by one
// warp with a 32-ary search over the whole diagonal (few cuts, many probes each), then every
// other cut by one thread with a binary search between its two coarse neighbours (many cuts,
// few probes each). Cut t sits at merged position min(t * tile_step, total); equal coordinates
// stay on one side of a cut.
constexpr int COARSE = 32;

template <typename PK>
__device__ __forceinline__ void finish_cut(const Coo3In &A, const Coo3In &B, const PK &pk, int64_t d, int64_t x,
                                           int32_t *pa, int32_t *pb) {
    int64_t y = d - x;
    if (x > 0 && y < B.nnz && key_at(A, pk, x - 1) == key_at(B, pk, y)) ++y;
    *pa = (int32_t)x;
    *pb = (int32_t)y;
}

template <typename PK>
__global__ void __launch_bounds__(NT) k_coo3_partition_coarse(Coo3In A, Coo3In B, PK pk, int64_t total, int32_t tile_step,
                                                              int32_t num_tiles, Cuts2 cuts) {
    const int c = (blockIdx.x * NT + threadIdx.x) >> 5;
    const int64_t t64 = (int64_t)c * COARSE;
    if (t64 > num_tiles + COARSE - 1) return;
    const int t = (int)min(t64, (int64_t)num_tiles);  // the last coarse cut is the end of the data
    const int64_t d = (int64_t)t * tile_step;
    int32_t pa, pb;
    if (t == 0) {
        pa = pb = 0;
    } else if (t == num_tiles || d >= total) {
        pa = A.nnz;
        pb = B.nnz;
    } else {
        const int64_t x_lo = d - B.nnz > 0 ? d - B.nnz : 0;
        const int64_t x_hi = d < A.nnz ? d : A.nnz;
        const int64_t x = warp_count_true(x_lo, x_hi, [&](int64_t m) { return key_at(A, pk, m) <= key_at(B, pk, d - 1 - m); });
        finish_cut(A, B, pk, d, x, &pa, &pb);
    }
    if (lane_id() == 0) {
        cuts.a[t] = pa;
        cuts.b[t] = pb;
    }
}

template <typename PK>
__global__ void __launch_bounds__(NT) k_coo3_partition_fine(Coo3In A, Coo3In B, PK pk, int64_t total, int32_t tile_step,
                                                            int32_t num_tiles, Cuts2 cuts) {
    const int t = blockIdx.x * NT + threadIdx.x;
    if (t >= num_tiles || t % COARSE == 0) return;
    const int64_t d = (int64_t)t * tile_step;
    int32_t pa, pb;
    if (d >= total) {
        pa = A.nnz;
        pb = B.nnz;
    } else {
        const int c0 = t / COARSE * COARSE, c1 = min(c0 + COARSE, num_tiles);
        int64_t lo = max((int64_t)cuts.a[c0], d - B.nnz > 0 ? d - B.nnz : 0);
        int64_t hi = min((int64_t)cuts.a[c1], d < A.nnz ? d : (int64_t)A.nnz);
        while (lo < hi) {  // first m with key_A(m) > key_B(d - 1 - m)
            const int64_t mid = (lo + hi) >> 1;
            if (key_at(A, pk, mid) <= key_at(B, pk, d - 1 - mid)) lo = mid + 1; else hi = mid;
        }
        finish_cut(A, B, pk, d, lo, &pa, &pb);
    }
    cuts.a[t] = pa;
    cuts.b[t] = pb;
}

// Hardware barriers of the tile kernel: 0 = whole CTA, 1 = the NT worker threads, 2 = workers
// arrive / the scan warp waits ("the tile's count is known").
using WorkerBar = NamedBarrier<1, NT>;
using CountBar = NamedBarrier<2, NT + 32>;
using LevelBar = NamedBarrier<3, NT + 32>;  // second hand-over to the scan warp (CSF3 levels)

constexpr int RAW_SLOTS = CAP + 16;  // words per staged raw array (i, j, k, value)
static_assert(RAW_SLOTS >= KEY_SLOTS, "packed keys reuse the raw i and j arrays");
constexpr int MBAR_POLL_LIMIT = 1 << 24;
constexpr int ERR_COPY_TIMEOUT = 2;

// Number of 4-byte elements from `p` up to the next 16-byte boundary (0..3).
__device__ __forceinline__ int head_elems(const void *p) {
    return (int)(((16u - (unsigned)(reinterpret_cast<uintptr_t>(p) & 15u)) & 15u) >> 2);
}

template <int MODE, bool CSF_OUT>
__global__ void __launch_bounds__(NT + 32, COO3_MIN_CTAS) k_coo3_tile(Coo3In A, Coo3In B, Packing pk, Cuts2 cuts, int32_t *tile_count,
                                                                 uint64_t *tile_state_raw, FusedCtl *ctl, Coo3Out Z,
                                                                 CsfLevelsOut csf) {
    static_assert(!CSF_OUT || MODE == MODE_FUSED, "the CSF3 levels are written by the single-pass launch only");
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ int scan_tmp[72];
    __shared__ long long s_base, s_base_levels, s_levels;
    __shared__ int s_hurry, s_hurry_levels;  // set once the tile's count / packed level count is out
    __shared__ unsigned long long s_prev_key;
    __shared__ __align__(8) uint64_t mbar;
    __shared__ int s_total;
    constexpr bool WRITES = MODE != MODE_COUNT;
    volatile uint64_t *tile_state = tile_state_raw;
    const int tid = threadIdx.x;
    const bool scan_warp = tid >= NT;  // one extra warp: it only turns counts into output bases
    int t = blockIdx.x;
    if (tid == 0) {
        mbar_init(&mbar, 1);
        mbar_fence_init();
        s_hurry = 0;
        s_hurry_levels = 0;
    }
    __syncthreads();
    // tiles are numbered by CTA index: CTAs are dispatched in increasing index order, so a tile
    // only waits on CTAs dispatched before it (and every such wait is bounded)
    const int32_t a0 = cuts.a[t], b0 = cuts.b[t];
    const int na = cuts.a[t + 1] - a0, nb = cuts.b[t + 1] - b0;
    const int n = na + nb;
    if (CSF_OUT && tid == NT - 1) {
        // the coordinate that precedes the tile's first result entry: the larger of the last
        // entries before the cut (a cut never separates equal coordinates); all-ones if none
        uint64_t prev = INF;
        if (a0 > 0) prev = key_at(A, pk, (int64_t)a0 - 1);
        if (b0 > 0) {
            const uint64_t pb = key_at(B, pk, (int64_t)b0 - 1);
            prev = prev == INF ? pb : max(prev, pb);
        }
        s_prev_key = prev;
    }

    // Shared layout, in 4-byte words: four raw arrays of RAW_SLOTS words each (i, j, k, value),
    // where A's entry e sits at word oa + e and B's at word ob + e, chosen so that 16-byte
    // boundaries of global memory fall on 16-byte boundaries here (what a bulk copy needs).
    // Once the coordinates are packed, the 64-bit keys take the place of the raw i and j arrays,
    // and the value staging array of the result takes the place of the raw k array.
    uint32_t *raw = reinterpret_cast<uint32_t *>(smem_raw);
    uint64_t *kx = reinterpret_cast<uint64_t *>(smem_raw);
    uint64_t *ky = kx + na + 1;
    float *out_val = reinterpret_cast<float *>(raw + 2 * RAW_SLOTS);
    uint64_t *out_key = kx;
    const int ha = head_elems(A.i + a0), hb = head_elems(B.i + b0);
    const int oa = (4 - ha) & 3;
    const int ob = ((oa + na + 3) & ~3) + ((4 - hb) & 3);
    const float *vx = reinterpret_cast<const float *>(raw + 3 * RAW_SLOTS) + oa;
    const float *vy = reinterpret_cast<const float *>(raw + 3 * RAW_SLOTS) + ob;

    // ---- stage the eight operand arrays: aligned interiors by bulk copy, ragged ends (at most
    // three entries each side) and arrays whose alignment differs from their i array's by
    // plain loads
    {
        const void *src[8] = {A.i + a0, A.j + a0, A.k + a0, A.val + a0, B.i + b0, B.j + b0, B.k + b0, B.val + b0};
        const int head_a = min(na, ha), head_b = min(nb, hb);
        const int nva = (na - head_a) >> 2, nvb = (nb - head_b) >> 2;
        bool bulk[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) bulk[q] = head_elems(src[q]) == (q < 4 ? ha : hb) && (WRITES || (q & 3) != 3);
        if (tid == 0) {
            uint32_t bytes = 0;
#pragma unroll
            for (int q = 0; q < 8; ++q) bytes += bulk[q] ? 16u * (q < 4 ? nva : nvb) : 0u;
            mbar_arrive_expect_tx(&mbar, bytes);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const int nv = q < 4 ? nva : nvb, head = q < 4 ? head_a : head_b;
                if (bulk[q] && nv)
                    bulk_load(raw + (q & 3) * RAW_SLOTS + (q < 4 ? oa : ob) + head,
                              static_cast<const uint32_t *>(src[q]) + head, 16u * nv, &mbar);
            }
        }
        if (tid >= 32 && tid < 32 + 48) {  // ragged ends: 8 arrays x (3 head + 3 tail)
            const int q = (tid - 32) / 6, e = (tid - 32) % 6;
            const int count = q < 4 ? na : nb, head = q < 4 ? head_a : head_b, nv = q < 4 ? nva : nvb;
            const int idx = e < 3 ? e : head + 4 * nv + (e - 3);
            const bool live = (e < 3 ? e < head : idx < count) && (WRITES || (q & 3) != 3);
            bool is_bulk = false;
#pragma unroll
            for (int qq = 0; qq < 8; ++qq) is_bulk = qq == q ? bulk[qq] : is_bulk;
            if (live && is_bulk) {
                const uint32_t *g = nullptr;
#pragma unroll
                for (int qq = 0; qq < 8; ++qq) g = qq == q ? static_cast<const uint32_t *>(src[qq]) : g;
                raw[(q & 3) * RAW_SLOTS + (q < 4 ? oa : ob) + idx] = ld_nc(g + idx);
            }
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            if (!bulk[q] && (WRITES || (q & 3) != 3)) {
                const int count = q < 4 ? na : nb;
                for (int e = tid; e < count && !scan_warp; e += NT)
                    raw[(q & 3) * RAW_SLOTS + (q < 4 ? oa : ob) + e] = ld_nc(static_cast<const uint32_t *>(src[q]) + e);
            }
        }
    }
    const bool landed = mbar_wait_bounded(&mbar, 0, MBAR_POLL_LIMIT);
    if (!__syncthreads_and(landed)) {  // the copies did not land in time: report, touch nothing
        if (tid == 0) {
            if (atomicCAS(&ctl->status.error, 0, ERR_COPY_TIMEOUT) == 0) ctl->status.detail = t;
            if (MODE == MODE_FUSED) tile_state[t] = LB_PREFIX;
            mbar_wait_bounded(&mbar, 0, MBAR_POLL_LIMIT);  // second bounded wait for copies in flight
        }
        return;
    }

    if (scan_warp) {
        // the output base is the sum of the counts of all earlier tiles and does not depend on
        // this tile's count: walk the predecessors' words while the workers merge
        if (MODE != MODE_FUSED) return;
        const int64_t bse = t == 0 ? 0 : lookback_predecessors(tile_state, t, &ctl->status, 1000, &s_hurry, 1000);
        CountBar::sync();  // the workers have published the tile's count by now
        const int total = s_total;
        if (lane_id() == 0) {
            if (t > 0) st_relaxed_gpu(tile_state + t, LB_PREFIX | (uint64_t)(bse < 0 ? 0 : bse + total));
            s_base = bse;
            if (bse >= 0 && t == (int)gridDim.x - 1) ctl->total = bse + total;
        }
        __syncthreads();
        if (CSF_OUT) {
            // second walk: slices and fibres of all earlier tiles (packed), while the workers store
            volatile uint64_t *level_state = csf.tile_state;
            const int64_t lv = t == 0 ? 0 : lookback_predecessors(level_state, t, &ctl->status, 1000, &s_hurry_levels, 1000);
            LevelBar::sync();  // the workers have published the tile's packed count by now
            const long long packed = s_levels;
            if (lane_id() == 0) {
                if (t > 0) st_relaxed_gpu(level_state + t, LB_PREFIX | (uint64_t)(lv < 0 ? 0 : lv + packed));
                s_base_levels = lv;
            }
            __syncthreads();
        }
        return;
    }

    // ---- pack the coordinates into 64-bit keys (registers first: the keys overwrite the raw
    // i and j arrays)
    {
        uint64_t packed[VT];
#pragma unroll
        for (int q = 0; q < VT; ++q) {
            const int e = tid + q * NT;  // merged staging slot: A's entries first, then B's
            const int w = e < na ? oa + e : ob + (e - na);
            packed[q] = e < n ? pk.pack((int32_t)raw[w], (int32_t)raw[RAW_SLOTS + w], (int32_t)raw[2 * RAW_SLOTS + w]) : INF;
        }
        WorkerBar::sync();
#pragma unroll
        for (int q = 0; q < VT; ++q) {
            const int e = tid + q * NT;
            if (e < na) kx[e] = packed[q];
            else if (e < n) ky[e - na] = packed[q];
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

    // ---- merge VT entries, straight-line. Bit i of `from_a`: entry i came from A; of `twin`:
    // the same coordinate is in B too; of `emit`: the entry goes to the result (B's copy of a
    // shared coordinate does not).
    uint64_t key[VT];
    unsigned from_a = 0, twin = 0, emit = 0;
    {
        const int valid = min(VT, n - diag);
        uint64_t hx = kx[x], hy = ky[y];
        uint64_t last_x = x > 0 ? kx[x - 1] : INF;
#pragma unroll
        for (int i = 0; i < VT; ++i) {
            const bool tx = hx <= hy;
            const bool both = hx == hy;
            key[i] = tx ? hx : hy;
            from_a |= (unsigned)tx << i;
            twin |= (unsigned)(tx && both) << i;
            emit |= (unsigned)(i < valid && (tx || hy != last_x)) << i;
            last_x = tx ? hx : last_x;
            x += tx;
            y += !tx;
            hx = kx[x];
            hy = ky[y];
        }
    }

    if (MODE == MODE_REDUCE) {
        // ---- inner product: sum a * b over the coordinates both operands hold, in double; one
        // atomic per tile into the control block (the order of the tiles' sums is not fixed, as
        // with the reference's atomic accumulation, src/backend/compute.cpp:498-525)
        double sum = 0.0;
        int xi = x0, yi = y0;
#pragma unroll
        for (int i = 0; i < VT; ++i) {
            const bool tx = (from_a >> i) & 1u;
            if ((twin >> i) & 1u && i < min(VT, n - diag)) sum += (double)(vx[xi] * vy[yi]);
            xi += tx;
            yi += !tx;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(FULL_MASK, sum, o);
        double *partial = reinterpret_cast<double *>(scan_tmp);  // 72 ints = room for 8 doubles and more
        WorkerBar::sync();
        if (lane_id() == 0) partial[warp_id()] = sum;
        WorkerBar::sync();
        if (tid == 0) {
            double s = 0.0;
            for (int w = 0; w < NT / 32; ++w) s += partial[w];
            atomicAdd(reinterpret_cast<double *>(&ctl->total), s);
        }
        return;
    }

    // ---- rank the survivors inside the tile
    int total;
    const int mine = __popc(emit);
    const int rank = block_excl_sum<NT, WorkerBar>(mine, scan_tmp, total);  // syncs: key reads are done
    if (MODE == MODE_COUNT) {
        if (tid == 0) tile_count[t] = total;
        return;
    }
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

    // ---- compact through shared memory, then unpack and store coalesced
    {
        int r = rank, xi = x0, yi = y0;
#pragma unroll
        for (int i = 0; i < VT; ++i) {
            const bool tx = (from_a >> i) & 1u;
            const bool both = (twin >> i) & 1u;
            const bool out = (emit >> i) & 1u;
            float v = tx ? vx[xi] : vy[yi];
            if (both) v = v + vy[yi];
            if (out) {
                out_key[r] = key[i];
                out_val[r] = v;
            }
            r += out;
            xi += tx;
            yi += !tx;
        }
    }
    // ---- CSF3 levels above k, first half: thread t looks after the staged result entries
    // [t VT, t VT + VT); bit q of `new_i` / `new_ij`: entry q opens a new i slice / a new (i, j)
    // fibre. The tile's packed count goes out before the tile waits for anything.
    const int e0 = tid * VT;
    unsigned new_i = 0, new_ij = 0;
    int rank_i = 0, rank_ij = 0;
    if (CSF_OUT) {
        WorkerBar::sync();  // the staged entries of the other workers are in place
        const int mine_n = max(0, min(VT, total - e0));
        const int sh_ij = pk.bk, sh_i = pk.bj + pk.bk;
        uint64_t prev = e0 == 0 ? (uint64_t)s_prev_key : (mine_n > 0 ? out_key[e0 - 1] : 0ull);
#pragma unroll
        for (int q = 0; q < VT; ++q) {
            if (q < mine_n) {
                const uint64_t cur = out_key[e0 + q];
                new_i |= (unsigned)((cur >> sh_i) != (prev >> sh_i)) << q;
                new_ij |= (unsigned)((cur >> sh_ij) != (prev >> sh_ij)) << q;
                prev = cur;
            }
        }
        int tot_i, tot_ij;
        block_excl_sum2<NT, WorkerBar>(__popc(new_i), __popc(new_ij), scan_tmp, rank_i, rank_ij, tot_i, tot_ij);
        if (tid == 0) {
            const long long packed = ((long long)tot_i << 31) | (long long)tot_ij;
            st_relaxed_gpu(csf.tile_state + t, (t == 0 ? LB_PREFIX : LB_AGGREGATE) | (uint64_t)packed);
            s_levels = packed;
            *(volatile int *)&s_hurry_levels = 1;
        }
        __threadfence_block();
        LevelBar::arrive();  // the scan warp turns the packed count into the tile's inclusive prefix
    }

    // ---- output base of the tile (from the scan warp, or from the scanned counts)
    if (MODE == MODE_FUSED) __syncthreads(); else WorkerBar::sync();
    const long long base = MODE == MODE_FILL ? (long long)tile_count[t] : s_base;
    if (base < 0) {  // a bounded wait gave up; the host reports it
        if (CSF_OUT) __syncthreads();  // the scan warp still waits at the levels barrier
        return;
    }
    for (int i = tid; i < total; i += NT) {
        const uint64_t kq = out_key[i];
        if (!CSF_OUT) {
            Z.i[base + i] = pk.i_of(kq);
            Z.j[base + i] = pk.j_of(kq);
        }
        Z.k[base + i] = pk.k_of(kq);
        Z.val[base + i] = out_val[i];
    }
    if (!CSF_OUT) return;

    // ---- CSF3 levels above k, second half: slices / fibres of the earlier tiles, then the scatter
    __syncthreads();
    const long long levels_base = s_base_levels;
    if (levels_base < 0) return;
    int r = (int)(levels_base >> 31) + rank_i;
    int f = (int)(levels_base & 0x7fffffff) + rank_ij;
#pragma unroll
    for (int q = 0; q < VT; ++q) {
        if ((new_ij >> q) & 1u) {
            const uint64_t cur = out_key[e0 + q];
            if (f < csf.cap_j) {
                csf.j_idx[f] = pk.j_of(cur);
                csf.k_ptr[f] = (int32_t)(base + e0 + q);
            }
            if ((new_i >> q) & 1u) {
                if (r < csf.cap_i) {
                    csf.i_idx[r] = pk.i_of(cur);
                    csf.j_ptr[r] = f;
                }
                ++r;
            }
            ++f;
        }
    }
    if (t == (int)gridDim.x - 1 && tid == NT - 1) {  // the last worker of the last tile holds the totals
        csf.totals->n_i = r;
        csf.totals->n_j = f;
        if (f <= csf.cap_j) csf.k_ptr[f] = (int32_t)(base + total);
        if (r <= csf.cap_i) csf.j_ptr[r] = f;
    }
}

// ---------------------------------------------------------------- wide coordinates ----

// Tile kernel for extents that need more than 63 bits together. One CTA of WNT threads per tile of
// WNT * WVT - 1 merged entries: (i, j) words and k words staged in shared memory with plain loads,
// merge-path split with the two-word compare, sequential merge of WVT entries per thread, values
// fetched from global memory, compaction through shared memory, coalesced stores. Single pass with
// bounded look-back, or count / fill around a scan, like the packed-key kernel.
constexpr int WNT = 256, WVT = 7, WCAP = WNT * WVT, WKS = WCAP + 2 + WVT;

template <int MODE>
__global__ void __launch_bounds__(WNT) k_coo3_tile_wide(Coo3In A, Coo3In B, Cuts2 cuts, int32_t *tile_count, uint64_t *tile_state_raw,
                                                         FusedCtl *ctl, Coo3Out Z) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ int scan_tmp[40];
    __shared__ long long s_base;
    volatile uint64_t *tile_state = tile_state_raw;
    const WidePacking pk;
    const int tid = threadIdx.x;
    const int t = blockIdx.x;  // CTAs are dispatched in index order; waits on earlier tiles are bounded
    const int32_t a0 = cuts.a[t], b0 = cuts.b[t];
    const int na = cuts.a[t + 1] - a0, nb = cuts.b[t + 1] - b0;
    const int n = na + nb;
    uint64_t *hx = reinterpret_cast<uint64_t *>(smem_raw), *hy = hx + na + 1;
    uint32_t *lx = reinterpret_cast<uint32_t *>(hx + WKS), *ly = lx + na + 1;
    float *out_val = reinterpret_cast<float *>(lx + WKS);
    for (int e = tid; e < na; e += WNT) {
        const Key96 q = key_at(A, pk, (int64_t)a0 + e);
        hx[e] = q.ij;
        lx[e] = q.k;
    }
    for (int e = tid; e < nb; e += WNT) {
        const Key96 q = key_at(B, pk, (int64_t)b0 + e);
        hy[e] = q.ij;
        ly[e] = q.k;
    }
    if (tid < WVT + 1) hy[nb + tid] = ~0ull, ly[nb + tid] = ~0u;  // all-ones orders after every coordinate
    if (tid == 0) hx[na] = ~0ull, lx[na] = ~0u;
    __syncthreads();
    auto kx = [&](int p) { return Key96{hx[p], lx[p]}; };
    auto ky = [&](int p) { return Key96{hy[p], ly[p]}; };

    // ---- split the tile among threads: merge-path diagonal tid * WVT, ties take A first
    const int diag = min(tid * WVT, n);
    int x, y;
    {
        int lo = max(0, diag - nb), hi = min(diag, na);
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (kx(mid) <= ky(diag - 1 - mid)) lo = mid + 1; else hi = mid;
        }
        x = lo;
        y = diag - lo;
    }
    const int x0 = x, y0 = y;

    // ---- merge WVT entries; bit i of `from_a`: entry i came from A; of `twin`: the same
    // coordinate is in B too; of `emit`: the entry goes to the result
    Key96 key[WVT];
    unsigned from_a = 0, twin = 0, emit = 0;
    {
        const int valid = min(WVT, n - diag);
        Key96 cx = kx(x), cy = ky(y);
        Key96 last_x = x > 0 ? kx(x - 1) : Key96{~0ull, ~0u};
#pragma unroll
        for (int i = 0; i < WVT; ++i) {
            const bool tx = cx <= cy;
            const bool both = cx == cy;
            key[i] = tx ? cx : cy;
            from_a |= (unsigned)tx << i;
            twin |= (unsigned)(tx && both) << i;
            emit |= (unsigned)(i < valid && (tx || !(cy == last_x))) << i;
            last_x = tx ? cx : last_x;
            x += tx;
            y += !tx;
            cx = kx(x);
            cy = ky(y);
        }
    }
    int total;
    const int rank = block_excl_sum<WNT>(__popc(emit), scan_tmp, total);  // syncs: key reads are done
    if (MODE == MODE_COUNT) {
        if (tid == 0) tile_count[t] = total;
        return;
    }
    if (MODE == MODE_FUSED && warp_id() == 0) {
        const int64_t b = lookback_exclusive(tile_state, t, total, &ctl->status);
        if (lane_id() == 0) {
            s_base = b;
            if (b >= 0 && t == (int)gridDim.x - 1) ctl->total = b + total;
        }
    }
    // ---- compact through shared memory (the staging arrays reuse the key words), store coalesced
    {
        int r = rank, xi = x0, yi = y0;
#pragma unroll
        for (int i = 0; i < WVT; ++i) {
            const bool tx = (from_a >> i) & 1u;
            if ((emit >> i) & 1u) {
                float v = tx ? ld_nc(A.val + a0 + xi) : ld_nc(B.val + b0 + yi);
                if ((twin >> i) & 1u) v = v + ld_nc(B.val + b0 + yi);
                hx[r] = key[i].ij;
                lx[r] = key[i].k;
                out_val[r] = v;
                ++r;
            }
            xi += tx;
            yi += !tx;
        }
    }
    __syncthreads();
    const long long base = MODE == MODE_FILL ? (long long)tile_count[t] : s_base;
    if (base < 0) return;  // a bounded wait gave up; the host reports it
    for (int e = tid; e < total; e += WNT) {
        const uint64_t ij = hx[e];
        Z.i[base + e] = (int32_t)(ij >> 32);
        Z.j[base + e] = (int32_t)(uint32_t)ij;
        Z.k[base + e] = (int32_t)lx[e];
        Z.val[base + e] = out_val[e];
    }
}

constexpr size_t coo3_wide_smem_bytes() { return 12 * (size_t)WKS + 4 * (size_t)WCAP; }

template <int MODE>
cudaError_t launch_coo3_tile_wide(const Coo3In &A, const Coo3In &B, const Cuts2 &cuts, int32_t *tile_count, uint64_t *tile_state,
                                  FusedCtl *ctl, const Coo3Out &Z, int num_tiles, cudaStream_t stream) {
    static const char *const names[3] = {"coo3_add_wide_count", "coo3_add_wide_fill", "coo3_add_wide_fused"};
    LaunchScope scope(names[MODE], stream);
    k_coo3_tile_wide<MODE><<<num_tiles, WNT, coo3_wide_smem_bytes(), stream>>>(A, B, cuts, tile_count, tile_state, ctl, Z);
    return cudaGetLastError();
}

constexpr size_t coo3_smem_bytes() { return 16 * (size_t)RAW_SLOTS; }
static_assert(coo3_wide_smem_bytes() <= 48 * 1024, "the wide tile kernel stays within the default shared-memory limit");


int bits_for(int32_t extent) {
    int b = 1;
    while (b < 32 && (int64_t(1) << b) < (int64_t)extent) ++b;
    return b;
}

template <int MODE, bool CSF_OUT = false>
cudaError_t launch_coo3_tile(const Coo3In &A, const Coo3In &B, const Packing &pk, const Cuts2 &cuts, int32_t *tile_count,
                             uint64_t *tile_state, FusedCtl *ctl, const Coo3Out &Z, int num_tiles, cudaStream_t stream,
                             const CsfLevelsOut &csf = CsfLevelsOut{}) {
    auto kernel = k_coo3_tile<MODE, CSF_OUT>;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)coo3_smem_bytes());
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    static const char *const names[4] = {"coo3_add_count", "coo3_add_fill", "coo3_add_fused", "coo3_inner_prod"};
    LaunchScope scope(CSF_OUT ? "coo3_add_fused_csf" : names[MODE], stream);
    kernel<<<num_tiles, NT + 32, coo3_smem_bytes(), stream>>>(A, B, pk, cuts, tile_count, tile_state, ctl, Z, csf);
    return cudaGetLastError();
}

int check_coo3(const nb200_coo3 *t) {
    if (!t || t->nnz < 0 || t->dims[0] < 0 || t->dims[1] < 0 || t->dims[2] < 0) return NB200_E_BADARG;
    if (t->nnz > 0 && (!t->i || !t->j || !t->k || !t->val)) return NB200_E_BADARG;
    return NB200_OK;
}

}  // namespace

// Shared by the COO3 entry points and the CSF3 add (which merges expanded coordinates).
// When `alloc` is set the four result arrays are allocated here (one cudaMallocAsync each, at
// the worst-case length nnz(A) + nnz(B)); otherwise they are the caller's, `capacity` entries.
//
// `scratch` / `host_slot`, when given, replace the library's pooled workspace (the caller then
// owns a block of coo3_add_scratch_bytes() bytes and a pinned int64[8]); the CSF3 add uses this
// to keep its own temporaries and this function's in one pool block.
//
// `csf`, when given, asks the single-pass launch to write the CSF3 levels above k instead of the
// merged i and j columns (z->i and z->j may then be null); `*csf_done` tells whether that
// happened (the count -> scan -> fill route does not do it).
// (Both sized for the smaller tile of the wide-coordinate kernel, an upper bound for the other.)
int64_t coo3_add_tiles(int64_t total_entries) { return (total_entries + (WCAP - 1) - 1) / (WCAP - 1); }

size_t coo3_add_scratch_bytes(int64_t total_entries) {
    const int64_t tiles = coo3_add_tiles(total_entries);
    Carver sizes;
    sizes.take<int32_t>((size_t)tiles + 1);
    sizes.take<int32_t>((size_t)tiles + 1);
    sizes.take<int32_t>((size_t)tiles + 1);
    sizes.take<int64_t>(1);
    sizes.take<uint64_t>((size_t)tiles + 8);
    return sizes.used();
}

int coo3_add_run(const nb200_coo3 *a, const nb200_coo3 *b, nb200_coo3 *z, bool alloc, int64_t capacity, void *stream_v,
                 void *scratch, int64_t *host_slot, const CsfLevelsOut *csf, bool *csf_done) {
    int st;
    if (csf_done) *csf_done = false;
    if ((st = check_coo3(a)) || (st = check_coo3(b))) return st;
    if (!z || a->dims[0] != b->dims[0] || a->dims[1] != b->dims[1] || a->dims[2] != b->dims[2]) return NB200_E_BADARG;
    if (!alloc && capacity < 0) return NB200_E_BADARG;
    const int bi = bits_for(a->dims[0]), bj = bits_for(a->dims[1]), bk = bits_for(a->dims[2]);
    const bool wide = bi + bj + bk > 63;  // the coordinates do not pack into one 64-bit key
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const int64_t total = (int64_t)a->nnz + b->nnz;
    const int tile_step = wide ? WCAP - 1 : CAP - 1;
    const int64_t tiles64 = (total + tile_step - 1) / tile_step;
    if (tiles64 > INT32_MAX - 1) return NB200_E_OVERFLOW;
    const int num_tiles = (int)tiles64;
    for (int d = 0; d < 3; ++d) z->dims[d] = a->dims[d];
    z->nnz = 0;
    if (alloc) z->i = z->j = z->k = nullptr, z->val = nullptr;
    if (num_tiles == 0) return NB200_OK;
    if (!alloc && capacity > 0 && (!z->k || !z->val)) return NB200_E_BADARG;

    auto fail = [&](int code) {
        if (alloc) {
            if (z->i) cudaFreeAsync(z->i, stream);
            if (z->j) cudaFreeAsync(z->j, stream);
            if (z->k) cudaFreeAsync(z->k, stream);
            if (z->val) cudaFreeAsync(z->val, stream);
            z->i = z->j = z->k = nullptr;
            z->val = nullptr;
        }
        return code;
    };

    if (!scratch) {
        Workspace *ws = nullptr;
        if ((st = acquire_workspace(stream, coo3_add_scratch_bytes(total), &ws))) return st;
        scratch = ws->dev;
        host_slot = ws->host;
    }
    Carver carve(scratch);
    Cuts2 cuts;
    cuts.a = carve.take<int32_t>((size_t)num_tiles + 1);
    cuts.b = carve.take<int32_t>((size_t)num_tiles + 1);
    int32_t *tile_count = carve.take<int32_t>((size_t)num_tiles + 1);
    carve.take<int64_t>(1);
    uint64_t *fused_block = carve.take<uint64_t>((size_t)num_tiles + 8);
    FusedCtl *ctl = reinterpret_cast<FusedCtl *>(fused_block);
    uint64_t *tile_state = fused_block + 4;

    const Coo3In A{a->i, a->j, a->k, a->val, a->nnz}, B{b->i, b->j, b->k, b->val, b->nnz};
    const Packing pk{bj, bk};
    static const bool force_two_pass = [] { const char *e = std::getenv("NACHO_B200_TWO_PASS"); return e && e[0] == '1'; }();
    const bool fused = alloc || (capacity >= total && !force_two_pass);
    const bool levels = fused && csf != nullptr && !alloc && !wide;  // the wide kernel writes coordinates only
    if (!levels && !alloc && capacity > 0 && (!z->i || !z->j)) return NB200_E_BADARG;
    cudaError_t e = cudaMemsetAsync(fused_block, 0, sizeof(uint64_t) * (fused ? (size_t)num_tiles + 4 : 4), stream);
    if (e != cudaSuccess) return note_cuda_error(e, "cudaMemsetAsync");
    if (fused) {
        if (alloc) {
            void **arrays[4] = {reinterpret_cast<void **>(&z->i), reinterpret_cast<void **>(&z->j),
                                reinterpret_cast<void **>(&z->k), reinterpret_cast<void **>(&z->val)};
            for (auto p : arrays) {
                e = cudaMallocAsync(p, 4 * (size_t)total, stream);
                if (e != cudaSuccess) return fail(note_cuda_error(e, "cudaMallocAsync"));
            }
        }
    }
    {
        LaunchScope scope("coo3_partition", stream);
        const int warps = num_tiles / COARSE + 2;
        if (wide) {
            k_coo3_partition_coarse<<<(warps * 32 + NT - 1) / NT, NT, 0, stream>>>(A, B, WidePacking{}, total, tile_step, num_tiles, cuts);
            k_coo3_partition_fine<<<(num_tiles + NT - 1) / NT, NT, 0, stream>>>(A, B, WidePacking{}, total, tile_step, num_tiles, cuts);
        } else {
            k_coo3_partition_coarse<<<(warps * 32 + NT - 1) / NT, NT, 0, stream>>>(A, B, pk, total, tile_step, num_tiles, cuts);
            k_coo3_partition_fine<<<(num_tiles + NT - 1) / NT, NT, 0, stream>>>(A, B, pk, total, tile_step, num_tiles, cuts);
        }
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) return fail(note_cuda_error(e, "k_coo3_partition"));
    const Coo3Out Z{z->i, z->j, z->k, z->val};
    if (fused) {
        if (wide) {
            e = launch_coo3_tile_wide<MODE_FUSED>(A, B, cuts, nullptr, tile_state, ctl, Z, num_tiles, stream);
        } else if (levels) {
            e = launch_coo3_tile<MODE_FUSED, true>(A, B, pk, cuts, nullptr, tile_state, ctl, Z, num_tiles, stream, *csf);
            if (csf_done) *csf_done = true;
        } else {
            e = launch_coo3_tile<MODE_FUSED>(A, B, pk, cuts, nullptr, tile_state, ctl, Z, num_tiles, stream);
        }
        if (e != cudaSuccess) return fail(note_cuda_error(e, "k_coo3_tile<fused>"));
        e = cudaMemcpyAsync(host_slot, ctl, sizeof(FusedCtl), cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) return fail(note_cuda_error(e, "read result length"));
        FusedCtl h;
        std::memcpy(&h, host_slot, sizeof(h));
        if (h.status.error != 0) return fail(note_timeout(h.status.error, h.status.detail, "coo3 merge"));
        if (h.total > INT32_MAX) return fail(NB200_E_OVERFLOW);
        z->nnz = (int32_t)h.total;
        return NB200_OK;
    }
    // count -> scan -> fill. The scan leaves the result length in the control block, whose status
    // word also collects a give-up of either tile launch (a bulk copy that did not land in time).
    auto read_ctl = [&](FusedCtl &h) -> int {
        cudaError_t c = cudaMemcpyAsync(host_slot, ctl, sizeof(FusedCtl), cudaMemcpyDeviceToHost, stream);
        if (c == cudaSuccess) c = cudaStreamSynchronize(stream);
        if (c != cudaSuccess) return note_cuda_error(c, "read result length");
        std::memcpy(&h, host_slot, sizeof(h));
        return NB200_OK;
    };
    FusedCtl h;
    e = wide ? launch_coo3_tile_wide<MODE_COUNT>(A, B, cuts, tile_count, nullptr, ctl, Coo3Out{}, num_tiles, stream)
             : launch_coo3_tile<MODE_COUNT>(A, B, pk, cuts, tile_count, nullptr, ctl, Coo3Out{}, num_tiles, stream);
    if (e != cudaSuccess) return note_cuda_error(e, "k_coo3_tile<count>");
    {
        LaunchScope scope("scan_tiles", stream);
        k_scan_tiles<<<1, 1024, 0, stream>>>(tile_count, num_tiles, reinterpret_cast<int64_t *>(&ctl->total));
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) return note_cuda_error(e, "k_scan_tiles");
    if ((st = read_ctl(h))) return st;
    if (h.status.error != 0) return note_timeout(h.status.error, h.status.detail, "coo3 merge");
    if (h.total > INT32_MAX) return NB200_E_OVERFLOW;
    z->nnz = (int32_t)h.total;
    if (h.total > capacity) return NB200_E_CAPACITY;
    e = wide ? launch_coo3_tile_wide<MODE_FILL>(A, B, cuts, tile_count, nullptr, ctl, Z, num_tiles, stream)
             : launch_coo3_tile<MODE_FILL>(A, B, pk, cuts, tile_count, nullptr, ctl, Z, num_tiles, stream);
    if (e != cudaSuccess) return note_cuda_error(e, "k_coo3_tile<fill>");
    if ((st = read_ctl(h))) return st;
    if (h.status.error != 0) return note_timeout(h.status.error, h.status.detail, "coo3 merge");
    return NB200_OK;
}

__global__ void k_store_scalar(const FusedCtl *ctl, float *out) {
    out[0] = (float)__longlong_as_double(ctl->total);
}

// Inner product of two COO3 tensors: sum over the coordinates both hold of a * b, written as one
// float32 to the device word `z` (the reference returns a one-element tensor: compiler.cpp:141-143,
// append-reduction src/backend/compute.cpp:498-525). The same partition and tile kernel as the add,
// in a mode that writes no tensor. Products are float32 (as the reference's), their sum is kept in
// double until the end. Extents that do not pack into 64 bits are not supported here.
// `scratch` / `host_slot` as for coo3_add_run.
int coo3_inner_run(const nb200_coo3 *a, const nb200_coo3 *b, float *z, void *stream_v, void *scratch, int64_t *host_slot) {
    int st;
    if ((st = check_coo3(a)) || (st = check_coo3(b))) return st;
    if (!z || a->dims[0] != b->dims[0] || a->dims[1] != b->dims[1] || a->dims[2] != b->dims[2]) return NB200_E_BADARG;
    const int bi = bits_for(a->dims[0]), bj = bits_for(a->dims[1]), bk = bits_for(a->dims[2]);
    if (bi + bj + bk > 63) return NB200_E_UNSUPPORTED;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const int64_t total = (int64_t)a->nnz + b->nnz;
    constexpr int tile_step = CAP - 1;
    const int64_t tiles64 = (total + tile_step - 1) / tile_step;
    if (tiles64 > INT32_MAX - 1) return NB200_E_OVERFLOW;
    const int num_tiles = (int)tiles64;
    if (a->nnz == 0 || b->nnz == 0) {
        NB200_CUDA(cudaMemsetAsync(z, 0, sizeof(float), stream));
        return NB200_OK;
    }
    if (!scratch) {
        Workspace *ws = nullptr;
        if ((st = acquire_workspace(stream, coo3_add_scratch_bytes(total), &ws))) return st;
        scratch = ws->dev;
        host_slot = ws->host;
    }
    Carver carve(scratch);
    Cuts2 cuts;
    cuts.a = carve.take<int32_t>((size_t)num_tiles + 1);
    cuts.b = carve.take<int32_t>((size_t)num_tiles + 1);
    carve.take<int32_t>((size_t)num_tiles + 1);
    carve.take<int64_t>(1);
    FusedCtl *ctl = reinterpret_cast<FusedCtl *>(carve.take<uint64_t>((size_t)num_tiles + 8));
    const Coo3In A{a->i, a->j, a->k, a->val, a->nnz}, B{b->i, b->j, b->k, b->val, b->nnz};
    const Packing pk{bj, bk};
    NB200_CUDA(cudaMemsetAsync(ctl, 0, 4 * sizeof(uint64_t), stream));
    {
        LaunchScope scope("coo3_partition", stream);
        const int warps = num_tiles / COARSE + 2;
        k_coo3_partition_coarse<<<(warps * 32 + NT - 1) / NT, NT, 0, stream>>>(A, B, pk, total, tile_step, num_tiles, cuts);
        k_coo3_partition_fine<<<(num_tiles + NT - 1) / NT, NT, 0, stream>>>(A, B, pk, total, tile_step, num_tiles, cuts);
        NB200_CUDA(cudaGetLastError());
    }
    cudaError_t e = launch_coo3_tile<MODE_REDUCE>(A, B, pk, cuts, nullptr, nullptr, ctl, Coo3Out{}, num_tiles, stream);
    if (e != cudaSuccess) return note_cuda_error(e, "k_coo3_tile<reduce>");
    k_store_scalar<<<1, 1, 0, stream>>>(ctl, z);
    NB200_CUDA(cudaGetLastError());
    NB200_CUDA(cudaMemcpyAsync(host_slot, ctl, sizeof(FusedCtl), cudaMemcpyDeviceToHost, stream));
    NB200_CUDA(cudaStreamSynchronize(stream));
    FusedCtl h;
    std::memcpy(&h, host_slot, sizeof(h));
    return h.status.error != 0 ? note_timeout(h.status.error, h.status.detail, "coo3 inner product") : NB200_OK;
}

}  // namespace nb200

using namespace nb200;

extern "C" {

int nb200_coo3d_add_f32(const nb200_coo3 *a, const nb200_coo3 *b, nb200_coo3 *z, int32_t, int32_t, void *stream) {
    return coo3_add_run(a, b, z, true, 0, stream, nullptr, nullptr, nullptr, nullptr);
}

int nb200_coo3d_add_f32_into(const nb200_coo3 *a, const nb200_coo3 *b, nb200_coo3 *z, int64_t capacity, void *stream) {
    return coo3_add_run(a, b, z, false, capacity, stream, nullptr, nullptr, nullptr, nullptr);
}

int nb200_inner_prod_coo_f32(const nb200_coo3 *a, const nb200_coo3 *b, float *z, void *stream) {
    return coo3_inner_run(a, b, z, stream, nullptr, nullptr);
}

}  // extern "C"
