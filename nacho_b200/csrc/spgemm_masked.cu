// Masked SpGEMM ("sssmm"): Z_ik = sum_j a_ij * b_jk * c_ik on the positions the mask C stores and
// at least one product reaches. The reference declares it as one fused kernel
// (compiler.cpp:150-153: Sum_j a_ij * b_jk * c_ik) and runs it through the same expand / sort /
// compress machinery as its SpGEMM (src/backend/stitch_and_generate_gpu.cpp:14-139), on the products
// that survive the three-way intersection.
//
// Here the mask drives the accumulation, so nothing outside it is ever formed, sorted or written:
//   k_sssmm_classify    one warp per row: does the row have fewer than LIGHT_P products (counted
//                       only until that is known), and how wide (first to last column) and how
//                       long is its mask row? The row goes on one of five lists.
//   k_sssmm_bitmap      rows with many products, one CTA per row taken from a ticket: the mask row
//                       becomes a bitmap over its column span in shared memory plus, per 64-bit
//                       word, the count of set bits before it. A product tests one bit; a hit finds
//                       its position in the mask row as rank + popcount and adds
//                       (a_ij * b_jk) * c_ik -- the reference's expression, left to right -- to a
//                       shared-memory accumulator (rows whose mask row is too long for that, or
//                       whose span needs the whole shared memory, accumulate in global memory).
//                       Three list classes, by the shared memory a row needs.
//   k_sssmm_search_*    rows with few products (one warp per row) and rows whose span exceeds the
//                       largest bitmap (one CTA per row): binary search of the product's column in
//                       the mask row, float atomics on the global accumulators.
//   k_scan_lookback     exclusive scan of the "reached" flags: the result position of every mask
//                       position.
//   k_sssmm_compact     reached positions move to their result slot (column, value); the result's
//                       row offsets are the scanned flags at the mask's row starts.
// The sums are float32 atomics in arrival order, as the reference's compress is for every row.
#include <algorithm>
#include <cstring>

#include "block_utils.cuh"
#include "merge_common.cuh"

namespace nb200 {

namespace {

constexpr int LIGHT_P = 256;    // rows with fewer products than this are searched by one warp
constexpr int SEARCH_NT = 128;  // threads of a searching CTA
// lists: bitmap classes 0..2, wide rows (searched by a CTA), light rows (searched by a warp)
constexpr int LIST_WIDE = 3, LIST_LIGHT = 4;
constexpr int WARP_ENTRIES = 8; // entries of A's row one warp of a unit takes

// Work classes. A unit of work is a run of `unit` consecutive entries of one row of A (a row with
// more entries becomes several units, so a hub row spreads over the SMs), worked by one CTA of
// `nt` threads. The bitmap classes keep `words` 64-bit bitmap words and `entries` accumulators of
// the mask row in shared memory: bytes = 12 * words + 5 * entries (bitmap, ranks; sums, flags).
struct WorkClass {
    int words, entries, nt;
    __host__ __device__ constexpr int unit() const { return WARP_ENTRIES * (nt / 32); }
    constexpr size_t smem() const { return size_t(12) * words + size_t(5) * entries + 16; }
};
constexpr WorkClass CLASS[4] = {
    {1024, 2048, 256},    //  65536 columns of span, 22.5 KB: eight CTAs per SM
    {4096, 8192, 1024},   // 262144 columns, 88 KB: two CTAs per SM
    {16384, 0, 1024},     // 2^20 columns, 192 KB, sums in global memory: one CTA per SM
    {0, 0, SEARCH_NT},    // wider still: no bitmap, binary search
};

struct CsrView {
    const int32_t *rp, *col;
    const float *val;
};

struct SssmmCtl {
    int count[8];   // units (light list: rows) on each list
    int ticket[8];  // next list position to hand out
};

__global__ void __launch_bounds__(256) k_sssmm_classify(CsrView A, CsrView B, CsrView C, int32_t rows, int64_t list_cap,
                                                       int2 *__restrict__ units, int32_t *__restrict__ light,
                                                       SssmmCtl *__restrict__ ctl) {
    const int lane = lane_id();
    const int64_t warps = (int64_t)gridDim.x * (256 / 32);
    for (int64_t i = (int64_t)blockIdx.x * (256 / 32) + warp_id(); i < rows; i += warps) {
        const int32_t c_lo = ld_nc(C.rp + i), c_hi = ld_nc(C.rp + i + 1);
        const int32_t a_lo = ld_nc(A.rp + i), a_hi = ld_nc(A.rp + i + 1);
        if (c_lo == c_hi || a_lo == a_hi) continue;
        unsigned products = 0;  // exact below LIGHT_P, a lower bound beyond
        for (int32_t p0 = a_lo; p0 < a_hi && products < LIGHT_P; p0 += 32) {
            unsigned mine = 0;
            if (p0 + lane < a_hi) {
                const int32_t j = ld_nc(A.col + p0 + lane);
                mine = min((unsigned)(ld_nc(B.rp + j + 1) - ld_nc(B.rp + j)), (unsigned)LIGHT_P);
            }
            products += __reduce_add_sync(0xffffffffu, mine);
        }
        if (products == 0) continue;
        if (products < LIGHT_P) {
            if (lane == 0) light[atomicAdd(&ctl->count[LIST_LIGHT], 1)] = (int32_t)i;
            continue;
        }
        const int32_t words = (ld_nc(C.col + c_hi - 1) >> 6) - (ld_nc(C.col + c_lo) >> 6) + 1, entries = c_hi - c_lo;
        int list = LIST_WIDE;
        if (words <= CLASS[0].words && entries <= CLASS[0].entries) list = 0;
        else if (words <= CLASS[1].words && entries <= CLASS[1].entries) list = 1;
        else if (words <= CLASS[2].words) list = 2;
        const int unit = list == 0 ? CLASS[0].unit() : list == LIST_WIDE ? CLASS[LIST_WIDE].unit() : CLASS[1].unit();
        const int n_units = (a_hi - a_lo + unit - 1) / unit;
        int base = 0;
        if (lane == 0) base = atomicAdd(&ctl->count[list], n_units);
        base = __shfl_sync(0xffffffffu, base, 0);
        for (int u = lane; u < n_units; u += 32) units[list * list_cap + base + u] = make_int2((int)i, a_lo + u * unit);
    }
}

// One product column k of the mask row [c_lo, c_hi) by binary search; on a hit the product goes to
// the global sums.
__device__ __forceinline__ void search_product(const CsrView &B, const CsrView &C, int32_t q, int32_t k, float av, int32_t c_lo,
                                               int32_t c_hi, int32_t c0, float *__restrict__ acc, int32_t *__restrict__ hit) {
    int32_t lo = c_lo, hi = c_hi;  // first position of the mask's row with column >= k
    while (lo < hi) {
        const int32_t mid = lo + ((hi - lo) >> 1);
        if (ld_nc(C.col + mid) < k) lo = mid + 1; else hi = mid;
    }
    if (lo < c_hi && ld_nc(C.col + lo) == k) {
        atomicAdd(acc + (lo - c0), (av * ld_nc(B.val + q)) * ld_nc(C.val + lo));
        hit[lo - c0] = 1;
    }
}

__global__ void __launch_bounds__(256) k_sssmm_search_warp(CsrView A, CsrView B, CsrView C, const int32_t *__restrict__ list,
                                                          SssmmCtl *__restrict__ ctl, float *__restrict__ acc,
                                                          int32_t *__restrict__ hit) {
    const int lane = lane_id();
    const int32_t c0 = ld_nc(C.rp);  // the mask may be a row block of a larger matrix: positions count from its first entry
    const int count = ctl->count[LIST_LIGHT];
    for (;;) {
        int t = 0;
        if (lane == 0) t = atomicAdd(&ctl->ticket[LIST_LIGHT], 1);
        t = __shfl_sync(0xffffffffu, t, 0);
        if (t >= count) return;
        const int64_t i = ld_nc(list + t);
        const int32_t c_lo = ld_nc(C.rp + i), c_hi = ld_nc(C.rp + i + 1);
        for (int32_t p = ld_nc(A.rp + i), a_hi = ld_nc(A.rp + i + 1); p < a_hi; ++p) {
            const int32_t j = ld_nc(A.col + p);
            const float av = ld_nc(A.val + p);
            for (int32_t q = ld_nc(B.rp + j) + lane, b_hi = ld_nc(B.rp + j + 1); q < b_hi; q += 32)
                search_product(B, C, q, ld_nc(B.col + q), av, c_lo, c_hi, c0, acc, hit);
        }
    }
}

constexpr int CHUNK = 128;  // products one warp takes at a time: four loads per lane in flight

// Shared memory of unit_products: for every entry of the unit, the bounds of its row of B, its
// value, and the number of chunks in front of it.
template <int NT>
struct UnitRows {
    static constexpr int E = WARP_ENTRIES * (NT / 32);
    int32_t lo[E], hi[E], first[E];
    float av[E];
    int tmp[34];
};

// The products of the entries [p_begin, p_end) of A's row, spread evenly over the warps of the CTA:
// the rows of B the entries select are cut into chunks of CHUNK products, the chunks are numbered
// through (an exclusive sum over the entries) and warp w takes chunks w, w + warps, ...; a chunk
// finds its entry by binary search in the shared-memory sums. The columns of a warp's next chunk
// are requested before the current one is worked. The CTA must be in step on entry; `product(q, k,
// a)` receives the position in B, the column and A's value.
template <int NT, typename Product>
__device__ __forceinline__ void unit_products(const CsrView &A, const CsrView &B, int32_t p_begin, int32_t p_end, UnitRows<NT> &rows,
                                              Product product) {
    constexpr int NW = NT / 32;
    const int tid = threadIdx.x, lane = lane_id(), n_e = p_end - p_begin;
    int chunks = 0;
    if (tid < n_e) {
        const int32_t j = ld_nc(A.col + p_begin + tid);
        const int32_t lo = ld_nc(B.rp + j), hi = ld_nc(B.rp + j + 1);
        rows.av[tid] = ld_nc(A.val + p_begin + tid);
        rows.lo[tid] = lo;
        rows.hi[tid] = hi;
        chunks = (hi - lo + CHUNK - 1) / CHUNK;
    }
    int total;
    const int before = block_excl_sum<NT>(chunks, rows.tmp, total);
    if (tid < n_e) rows.first[tid] = before;
    __syncthreads();

    struct Fetched {
        int32_t k[4], q;
        float a;
    };
    auto fetch = [&](int c, Fetched &f) {
        int e = 0, above = n_e;  // the last entry whose first chunk is <= c
        while (above - e > 1) {
            const int mid = (e + above) >> 1;
            if (rows.first[mid] <= c) e = mid; else above = mid;
        }
        const int32_t hi = rows.hi[e];
        f.q = rows.lo[e] + (c - rows.first[e]) * CHUNK + lane;
        f.a = rows.av[e];
#pragma unroll
        for (int u = 0; u < 4; ++u) f.k[u] = f.q + 32 * u < hi ? ld_nc(B.col + f.q + 32 * u) : -1;
    };
    Fetched cur, next;
    int c = warp_id();
    if (c < total) fetch(c, cur);
    for (; c < total; c += NW) {
        if (c + NW < total) fetch(c + NW, next);
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (cur.k[u] >= 0) product(cur.q + 32 * u, cur.k[u], cur.a);
        cur = next;
    }
}

__global__ void __launch_bounds__(SEARCH_NT) k_sssmm_search_cta(CsrView A, CsrView B, CsrView C, const int2 *__restrict__ units,
                                                               SssmmCtl *__restrict__ ctl, float *__restrict__ acc,
                                                               int32_t *__restrict__ hit) {
    __shared__ UnitRows<SEARCH_NT> s_rows;
    const int32_t c0 = ld_nc(C.rp);
    const int count = ctl->count[LIST_WIDE];
    for (int t = blockIdx.x; t < count; t += gridDim.x) {
        const int2 unit = units[t];
        const int64_t i = unit.x;
        const int32_t c_lo = ld_nc(C.rp + i), c_hi = ld_nc(C.rp + i + 1);
        unit_products<SEARCH_NT>(A, B, unit.y, min(unit.y + CLASS[LIST_WIDE].unit(), ld_nc(A.rp + i + 1)), s_rows,
                                 [&](int32_t q, int32_t k, float av) { search_product(B, C, q, k, av, c_lo, c_hi, c0, acc, hit); });
        __syncthreads();
    }
}

template <int NT, bool SHARED_ACC>
__global__ void __launch_bounds__(NT) k_sssmm_bitmap(CsrView A, CsrView B, CsrView C, const int2 *__restrict__ units,
                                                    SssmmCtl *__restrict__ ctl, int which, int words_cap, int entries_cap,
                                                    float *__restrict__ acc, int32_t *__restrict__ hit) {
    extern __shared__ uint64_t sm_words[];
    uint64_t *bm = sm_words;                                         // bit (k - 64 * w0) set: the mask row stores column k
    uint32_t *bm32 = reinterpret_cast<uint32_t *>(bm);               // the same bits, for 32-bit shared-memory atomics
    uint32_t *rank = reinterpret_cast<uint32_t *>(bm + words_cap);   // set bits in front of each 64-bit word
    float *acc_s = reinterpret_cast<float *>(rank + words_cap);
    unsigned char *flag_s = reinterpret_cast<unsigned char *>(acc_s + entries_cap);
    __shared__ int2 s_unit;
    __shared__ UnitRows<NT> s_rows;
    const int tid = threadIdx.x;
    const int32_t c0 = ld_nc(C.rp);
    const int count = ctl->count[which];
    for (;;) {
        if (tid == 0) {
            const int t = atomicAdd(&ctl->ticket[which], 1);
            s_unit = t < count ? units[t] : make_int2(-1, 0);
        }
        __syncthreads();
        const int2 unit = s_unit;
        const int64_t i = unit.x;
        if (i < 0) return;
        const int32_t c_lo = ld_nc(C.rp + i), c_hi = ld_nc(C.rp + i + 1);
        const int32_t w0 = ld_nc(C.col + c_lo) >> 6;
        const int32_t words = (ld_nc(C.col + c_hi - 1) >> 6) - w0 + 1, entries = c_hi - c_lo;
        for (int w = tid; w < words; w += NT) bm[w] = 0;
        if (SHARED_ACC)
            for (int p = tid; p < entries; p += NT) {
                acc_s[p] = 0.0f;
                flag_s[p] = 0;
            }
        __syncthreads();
        for (int32_t p = c_lo + tid; p < c_hi; p += NT) {
            const int32_t k = ld_nc(C.col + p) - (w0 << 6);
            atomicOr(bm32 + (k >> 5), 1u << (k & 31));
        }
        __syncthreads();
        {   // ranks: every thread counts a run of consecutive words, the CTA scans the runs
            const int per = (words + NT - 1) / NT;
            const int w_lo = min(tid * per, words), w_hi = min(w_lo + per, words);
            int mine = 0, total;
            for (int w = w_lo; w < w_hi; ++w) mine += __popcll(bm[w]);
            int before = block_excl_sum<NT>(mine, s_rows.tmp, total);
            for (int w = w_lo; w < w_hi; ++w) {
                rank[w] = (uint32_t)before;
                before += __popcll(bm[w]);
            }
        }
        __syncthreads();
        const int32_t col0 = w0 << 6;
        const uint32_t span = (uint32_t)words << 6;
        unit_products<NT>(A, B, unit.y, min(unit.y + WARP_ENTRIES * (NT / 32), ld_nc(A.rp + i + 1)), s_rows, [&](int32_t q, int32_t k, float av) {
            const uint32_t bit = (uint32_t)(k - col0);
            if (bit >= span || !((bm32[bit >> 5] >> (bit & 31)) & 1)) return;  // most products end here
            const uint32_t w = bit >> 6, sh = bit & 63;
            const int32_t pos = (int32_t)rank[w] + __popcll(bm[w] & ((1ull << sh) - 1));
            const float v = (av * ld_nc(B.val + q)) * ld_nc(C.val + c_lo + pos);
            if (SHARED_ACC) {
                atomicAdd(acc_s + pos, v);
                flag_s[pos] = 1;
            } else {
                atomicAdd(acc + (c_lo - c0 + pos), v);
                hit[c_lo - c0 + pos] = 1;
            }
        });
        __syncthreads();
        if (SHARED_ACC) {  // other units of the same row add to the same sums
            for (int p = tid; p < entries; p += NT)
                if (flag_s[p]) {
                    atomicAdd(acc + (c_lo - c0 + p), acc_s[p]);
                    hit[c_lo - c0 + p] = 1;
                }
            __syncthreads();
        }
    }
}

// `pos` holds the exclusive scan of the flags over nnz + 1 entries (the last flag is 0, so
// pos[nnz] is the total).
__global__ void __launch_bounds__(256) k_sssmm_compact(const int32_t *__restrict__ pos, const float *__restrict__ acc,
                                                      const int32_t *__restrict__ c_rp, const int32_t *__restrict__ c_col, int32_t nnz,
                                                      int32_t *__restrict__ z_col, float *__restrict__ z_val) {
    const int64_t p = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (p >= nnz) return;
    const int32_t at = ld_nc(pos + p);
    if (ld_nc(pos + p + 1) > at) {
        z_col[at] = ld_nc(c_col + ld_nc(c_rp) + p);
        z_val[at] = ld_nc(acc + p);
    }
}

__global__ void __launch_bounds__(256) k_sssmm_row_offsets(const int32_t *__restrict__ pos, const int32_t *__restrict__ c_rp,
                                                          int32_t rows, int32_t *__restrict__ z_rp) {
    const int64_t r = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (r > rows) return;
    z_rp[r] = ld_nc(pos + (ld_nc(c_rp + r) - ld_nc(c_rp)));
}

int check(const nb200_csr *m) {
    if (!m || m->rows < 0 || m->cols < 0 || m->nnz < 0 || !m->row_ptr) return NB200_E_BADARG;
    if (m->nnz > 0 && (!m->col || !m->val)) return NB200_E_BADARG;
    return NB200_OK;
}

int sssmm_run(const nb200_csr *a, const nb200_csr *b, const nb200_csr *c, nb200_csr *z, int64_t capacity, void *stream_v) {
    int st;
    if ((st = check(a)) || (st = check(b)) || (st = check(c))) return st;
    if (!z || !z->row_ptr || capacity < 0 || a->cols != b->rows || c->rows != a->rows || c->cols != b->cols) return NB200_E_BADARG;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const int32_t rows = a->rows, nnz = c->nnz;
    z->rows = rows;
    z->cols = b->cols;
    z->nnz = 0;
    if (nnz == 0 || a->nnz == 0 || b->nnz == 0) {
        NB200_CUDA(cudaMemsetAsync(z->row_ptr, 0, sizeof(int32_t) * ((size_t)rows + 1), stream));
        return NB200_OK;
    }
    // per device, so set on every call: cheap next to the launches that follow
    NB200_CUDA(cudaFuncSetAttribute(k_sssmm_bitmap<1024, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CLASS[1].smem()));
    NB200_CUDA(cudaFuncSetAttribute(k_sssmm_bitmap<1024, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CLASS[2].smem()));
    int device = 0, sms = 148;
    NB200_CUDA(cudaGetDevice(&device));
    NB200_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));

    const int scan_ctas = (int)(((int64_t)nnz + 1 + SCAN_NT * SCAN_VT - 1) / (SCAN_NT * SCAN_VT));
    const int64_t list_cap = (int64_t)rows + a->nnz / CLASS[LIST_WIDE].unit() + 1;  // the smallest unit bounds every list
    Carver sizes;
    sizes.take<float>((size_t)nnz);
    sizes.take<int32_t>((size_t)nnz + 1);
    sizes.take<uint64_t>((size_t)scan_ctas + 8);
    sizes.take<SssmmCtl>(1);
    sizes.take<int2>((size_t)4 * list_cap);
    sizes.take<int32_t>((size_t)rows);
    Workspace *ws = nullptr;
    if ((st = acquire_workspace(stream, sizes.used(), &ws, 1))) return st;
    Carver carve(ws->dev);
    float *acc = carve.take<float>((size_t)nnz);
    int32_t *hit = carve.take<int32_t>((size_t)nnz + 1);
    uint64_t *scan_block = carve.take<uint64_t>((size_t)scan_ctas + 8);
    SssmmCtl *sctl = carve.take<SssmmCtl>(1);
    int2 *units = carve.take<int2>((size_t)4 * list_cap);
    int32_t *light = carve.take<int32_t>((size_t)rows);
    FusedCtl *ctl = reinterpret_cast<FusedCtl *>(scan_block);
    NB200_CUDA(cudaMemsetAsync(acc, 0, sizeof(float) * (size_t)nnz, stream));
    NB200_CUDA(cudaMemsetAsync(hit, 0, sizeof(int32_t) * ((size_t)nnz + 1), stream));
    NB200_CUDA(cudaMemsetAsync(scan_block, 0, sizeof(uint64_t) * ((size_t)scan_ctas + 4), stream));
    NB200_CUDA(cudaMemsetAsync(sctl, 0, sizeof(SssmmCtl), stream));
    const CsrView A{a->row_ptr, a->col, a->val}, B{b->row_ptr, b->col, b->val}, C{c->row_ptr, c->col, c->val};
    const int row_warps_grid = (int)std::min<int64_t>(((int64_t)rows + 7) / 8, (int64_t)sms * 8);
    const int most = (int)std::min<int64_t>(list_cap, 1 << 30);
    {
        LaunchScope scope("sssmm_classify", stream);
        k_sssmm_classify<<<row_warps_grid, 256, 0, stream>>>(A, B, C, rows, list_cap, units, light, sctl);
    }
    // Every list is worked by resident CTAs that take units from a ticket; a list's length stays on
    // the device, so an empty list costs one launch of CTAs that leave at once.
    {
        LaunchScope scope("sssmm_bitmap_wide", stream);
        k_sssmm_bitmap<1024, false><<<std::min(sms, most), 1024, CLASS[2].smem(), stream>>>(A, B, C, units + 2 * list_cap, sctl, 2,
                                                                                           CLASS[2].words, 0, acc, hit);
    }
    {
        LaunchScope scope("sssmm_bitmap_medium", stream);
        k_sssmm_bitmap<1024, true><<<std::min(2 * sms, most), 1024, CLASS[1].smem(), stream>>>(A, B, C, units + list_cap, sctl, 1,
                                                                                              CLASS[1].words, CLASS[1].entries, acc, hit);
    }
    {
        LaunchScope scope("sssmm_bitmap_narrow", stream);
        k_sssmm_bitmap<256, true><<<std::min(8 * sms, most), 256, CLASS[0].smem(), stream>>>(A, B, C, units, sctl, 0, CLASS[0].words,
                                                                                            CLASS[0].entries, acc, hit);
    }
    {
        LaunchScope scope("sssmm_search_wide", stream);
        k_sssmm_search_cta<<<std::min(16 * sms, most), SEARCH_NT, 0, stream>>>(A, B, C, units + (size_t)LIST_WIDE * list_cap, sctl, acc, hit);
    }
    {
        LaunchScope scope("sssmm_search_light", stream);
        k_sssmm_search_warp<<<row_warps_grid, 256, 0, stream>>>(A, B, C, light, sctl, acc, hit);
    }
    {
        LaunchScope scope("scan_lookback", stream);
        k_scan_lookback<<<scan_ctas, SCAN_NT, 0, stream>>>(hit, nnz + 1, scan_block + 4, ctl);
    }
    {
        LaunchScope scope("sssmm_row_offsets", stream);
        k_sssmm_row_offsets<<<(int)(((int64_t)rows + 1 + 255) / 256), 256, 0, stream>>>(hit, c->row_ptr, rows, z->row_ptr);
    }
    NB200_CUDA(cudaGetLastError());
    NB200_CUDA(cudaMemcpyAsync(ws->host, ctl, sizeof(FusedCtl), cudaMemcpyDeviceToHost, stream));
    NB200_CUDA(cudaStreamSynchronize(stream));
    FusedCtl h;
    std::memcpy(&h, ws->host, sizeof(h));
    if (h.status.error != 0) return note_timeout(h.status.error, h.status.detail, "sssmm scan");
    z->nnz = (int32_t)h.total;
    if (h.total > capacity) return NB200_E_CAPACITY;
    if (h.total > 0) {
        if (!z->col || !z->val) return NB200_E_BADARG;
        LaunchScope scope("sssmm_compact", stream);
        k_sssmm_compact<<<(int)(((int64_t)nnz + 255) / 256), 256, 0, stream>>>(hit, acc, c->row_ptr, c->col, nnz, z->col, z->val);
        NB200_CUDA(cudaGetLastError());
    }
    return NB200_OK;
}

}  // namespace

}  // namespace nb200

using namespace nb200;

extern "C" {

int nb200_sssmm_f32_into(const nb200_csr *a, const nb200_csr *b, const nb200_csr *c, nb200_csr *z, int64_t capacity, void *stream) {
    return sssmm_run(a, b, c, z, capacity, stream);
}

}  // extern "C"
