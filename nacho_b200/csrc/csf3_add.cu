// CSF3 tensor add: Z = A + B for tensors stored as three compressed levels (i list, j fibres
// under each i, k fibres under each (i, j)). The reference emits a three-level nested union
// (src/backend/compute.cpp:619-1392 with the runtime-exclusion partition of
// src/backend/partition.cpp:286-328, 586-811): merge the i lists, under equal i merge the j
// fibres, under equal (i, j) merge k, otherwise copy the subtree. The result is the unique
// canonical tree of the union of the coordinate sets, so it is produced here from flat merges, by
// one of two routes (two_level_pays chooses; NACHO_B200_CSF_TWO_LEVEL=0 / 1 forces one).
// Route over expanded coordinates (fibres of about one entry):
//   1. k_csf_expand    every stored entry gets its (i, j) written out next to its k: one warp
//                      per 32 (i, j) fibres finds their i by binary search and fills their ranges;
//   2. coo3_add_run    the sorted-union merge of the two coordinate lists (coo3_merge.cu); k and
//                      the values go straight into the result's k_idx / val arrays. On its
//                      single-pass route the merge also writes i_idx / j_ptr / j_idx / k_ptr
//                      itself (CsfLevelsOut) and nothing else is left to do;
//   3. k_csf_compress  only after the count -> scan -> fill route of the merge: one pass over
//                      the merged (i, j) columns: head flags for new i and new (i, j), a packed
//                      two-counter scan across tiles by bounded look-back, and the scatter of
//                      i_idx / j_ptr / j_idx / k_ptr.
// Two-level route (fibres of several entries; described above csf_add_two_level): the fibre lists
// are merged by the route above, which yields the upper levels and tells which operand holds which
// fibre; the entries then go through the CSR union with one row per result fibre, so that no
// per-entry (i, j) is ever written.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "merge_common.cuh"

namespace nb200 {

int coo3_add_run(const nb200_coo3 *a, const nb200_coo3 *b, nb200_coo3 *z, bool alloc, int64_t capacity, void *stream_v,
                 void *scratch, int64_t *host_slot, const CsfLevelsOut *csf, bool *csf_done);
int coo3_inner_run(const nb200_coo3 *a, const nb200_coo3 *b, float *z, void *stream_v, void *scratch, int64_t *host_slot);
size_t coo3_add_scratch_bytes(int64_t total_entries);
int64_t coo3_add_tiles(int64_t total_entries);

namespace {

constexpr int NT = 256;

// One warp per 32 consecutive (i, j) fibres. Each lane looks up its fibre's i (the last
// fibre-list start <= q, by binary search) and j; the warp then walks the entries of its 32
// fibres together, 32 entries at a time, each lane taking the (i, j) of its entry's fibre from
// the lane that holds it, so that the writes are coalesced however short the fibres are.
__global__ void __launch_bounds__(NT) k_csf_expand(int32_t n_i, int32_t n_j, const int32_t *__restrict__ i_idx,
                                                   const int32_t *__restrict__ j_ptr, const int32_t *__restrict__ j_idx,
                                                   const int32_t *__restrict__ k_ptr, int32_t *__restrict__ out_i,
                                                   int32_t *__restrict__ out_j) {
    const int w = (blockIdx.x * NT + threadIdx.x) >> 5;
    const int q0 = w * 32;
    if (q0 >= n_j) return;
    const int lane = lane_id();
    const int q = q0 + lane;
    int32_t start = INT32_MAX, i = 0, j = 0;
    if (q < n_j) {
        int lo = 0, hi = n_i - 1;  // largest r with j_ptr[r] <= q
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (ld_nc(j_ptr + mid) <= q) lo = mid; else hi = mid - 1;
        }
        i = ld_nc(i_idx + lo);
        j = ld_nc(j_idx + q);
        start = ld_nc(k_ptr + q);
    }
    const int32_t p_begin = __shfl_sync(FULL_MASK, start, 0);
    const int32_t p_end = ld_nc(k_ptr + min(q0 + 32, n_j));
    // Within a block of 32 entries the fibre starts form a bit mask, and an entry's fibre is the
    // number of fibres started at or before it. An empty fibre shares its start with its
    // successor; a block that sees one falls back to a search over the 32 starts by shuffles.
    for (int32_t base = p_begin; base < p_end; base += 32) {
        const int32_t rel = start - base;  // INT32_MAX - base for lanes past the last fibre: never in range
        const bool in_block = rel >= 0 && rel < 32;
        const int started = __popc(__ballot_sync(FULL_MASK, rel < 0));  // fibres that start before the block
        const unsigned starts = __reduce_or_sync(FULL_MASK, in_block ? 1u << rel : 0u);
        const int32_t p = base + lane;
        int f = started + __popc(starts & (0xffffffffu >> (31 - lane))) - 1;
        if (__popc(__ballot_sync(FULL_MASK, in_block)) != __popc(starts)) {  // uniform: an empty fibre in the block
            int lo = 0, hi = 31;  // largest lane whose fibre starts at or before p
#pragma unroll
            for (int step = 0; step < 5; ++step) {
                const int mid = (lo + hi + 1) >> 1;
                const int32_t sm = __shfl_sync(FULL_MASK, start, mid);
                if (sm <= p) lo = mid; else hi = mid - 1;
            }
            f = lo;
        }
        const int32_t vi = __shfl_sync(FULL_MASK, i, f), vj = __shfl_sync(FULL_MASK, j, f);
        if (p < p_end) {
            out_i[p] = vi;
            out_j[p] = vj;
        }
    }
}

struct CompressCtl {
    int ticket;
    DeviceStatus status;
    int n_i, n_j;
};

constexpr int CVT = 32;  // entries per thread in the compress pass (one bit each in the head masks)
constexpr int CCH = 8;   // entries per load step: two 16-byte loads per coordinate array

// Loads entries [p, p + CCH) of `z` (-1 beyond the end). p is a multiple of CCH, so the fast
// path is two aligned 16-byte loads.
__device__ __forceinline__ void load_chunk(const int32_t *__restrict__ z, int64_t p, int32_t nnz, int32_t (&out)[CCH]) {
    if (p + CCH <= nnz) {
        const int4 lo = __ldg(reinterpret_cast<const int4 *>(z + p)), hi = __ldg(reinterpret_cast<const int4 *>(z + p) + 1);
        out[0] = lo.x, out[1] = lo.y, out[2] = lo.z, out[3] = lo.w, out[4] = hi.x, out[5] = hi.y, out[6] = hi.z, out[7] = hi.w;
    } else {
#pragma unroll
        for (int q = 0; q < CCH; ++q) out[q] = p + q < nnz ? ld_nc(z + p + q) : -1;
    }
}

// Head flags + packed scan + scatter. A tile's count is (new i's << 31 | new (i, j)'s).
__global__ void __launch_bounds__(NT) k_csf_compress(int32_t nnz, const int32_t *__restrict__ zi,
                                                     const int32_t *__restrict__ zj, int32_t cap_i, int32_t cap_j,
                                                     int32_t *__restrict__ i_idx, int32_t *__restrict__ j_ptr,
                                                     int32_t *__restrict__ j_idx, int32_t *__restrict__ k_ptr,
                                                     uint64_t *tile_state_raw, CompressCtl *ctl) {
    __shared__ int scan_tmp[72];
    __shared__ int s_tile;
    __shared__ long long s_base;
    volatile uint64_t *tile_state = tile_state_raw;
    const int tid = threadIdx.x;
    const int t = blockIdx.x;  // CTAs are dispatched in index order; waits on earlier tiles are bounded
    const int64_t p0 = ((int64_t)t * NT + tid) * CVT;
    unsigned head_i = 0, head_ij = 0;
    {
        int32_t prev_i = p0 > 0 && p0 - 1 < nnz ? ld_nc(zi + p0 - 1) : -1;
        int32_t prev_j = p0 > 0 && p0 - 1 < nnz ? ld_nc(zj + p0 - 1) : -1;
#pragma unroll
        for (int c = 0; c < CVT / CCH; ++c) {
            int32_t ci[CCH], cj[CCH];
            load_chunk(zi, p0 + c * CCH, nnz, ci);
            load_chunk(zj, p0 + c * CCH, nnz, cj);
#pragma unroll
            for (int q = 0; q < CCH; ++q) {
                const bool live = p0 + c * CCH + q < nnz;
                const bool ni = live && ci[q] != prev_i;
                const bool nij = live && (ni || cj[q] != prev_j);
                head_i |= (unsigned)ni << (c * CCH + q);
                head_ij |= (unsigned)nij << (c * CCH + q);
                prev_i = ci[q];
                prev_j = cj[q];
            }
        }
    }
    int tot_i, tot_ij;
    int rank_i = block_excl_sum<NT>(__popc(head_i), scan_tmp, tot_i);
    int rank_ij = block_excl_sum<NT>(__popc(head_ij), scan_tmp, tot_ij);
    if (warp_id() == 0) {
        const int64_t packed = ((int64_t)tot_i << 31) | (int64_t)tot_ij;
        const int64_t b = lookback_exclusive(tile_state, t, packed, &ctl->status);
        if (lane_id() == 0) s_base = b;
    }
    __syncthreads();
    const long long base = s_base;
    if (base < 0) return;
    int r = (int)(base >> 31) + rank_i;
    int f = (int)(base & 0x7fffffff) + rank_ij;
#pragma unroll
    for (int c = 0; c < CVT / CCH; ++c) {
        if (((head_ij >> (c * CCH)) & 0xffu) == 0) continue;  // no fibre starts in this chunk
        int32_t ci[CCH], cj[CCH];
        load_chunk(zi, p0 + c * CCH, nnz, ci);  // second read, from cache
        load_chunk(zj, p0 + c * CCH, nnz, cj);
#pragma unroll
        for (int q = 0; q < CCH; ++q) {
            const int bit = c * CCH + q;
            if ((head_ij >> bit) & 1u) {
                if (f < cap_j) {
                    j_idx[f] = cj[q];
                    k_ptr[f] = (int32_t)(p0 + bit);
                }
                if ((head_i >> bit) & 1u) {
                    if (r < cap_i) {
                        i_idx[r] = ci[q];
                        j_ptr[r] = f;
                    }
                    ++r;
                }
                ++f;
            }
        }
    }
    if (t == (int)gridDim.x - 1 && tid == NT - 1) {  // last thread of the last tile holds the totals
        ctl->n_i = r;
        ctl->n_j = f;
        if (f <= cap_j) k_ptr[f] = nnz;
        if (r <= cap_i) j_ptr[r] = f;
    }
}

constexpr int FS_VT = 8;  // fibres per thread in k_fibre_slices

// i of every fibre. A CTA takes NT * FS_VT consecutive fibres; they lie in at most that many + 1
// consecutive stored slices (a stored slice has at least one fibre), so warp 0 finds the slice of the
// first fibre with a 32-ary search, the CTA copies that window of j_ptr / i_idx to shared memory and
// every thread finds its fibres' slices there.
__global__ void __launch_bounds__(NT) k_fibre_slices(int32_t n_i, int32_t n_j, const int32_t *__restrict__ i_idx,
                                                    const int32_t *__restrict__ j_ptr, int32_t *__restrict__ out_i) {
    constexpr int SPAN = NT * FS_VT;
    __shared__ int32_t s_start[SPAN + 1], s_i[SPAN + 1];
    __shared__ int s_first;
    const int tid = threadIdx.x;
    const int64_t q0 = (int64_t)blockIdx.x * SPAN;
    if (tid < 32) {
        const int64_t r = warp_last_true(0, (int64_t)n_i - 1, [&](int64_t x) { return ld_nc(j_ptr + x) <= q0; });
        if (tid == 0) s_first = (int)r;
    }
    __syncthreads();
    const int first = s_first;
    const int need = (int)min((int64_t)SPAN, (int64_t)n_j - q0);  // fibres of this CTA: slices first .. first + need at most
    for (int w = tid; w <= need; w += NT) {
        const bool live = first + w < n_i;
        s_start[w] = live ? ld_nc(j_ptr + first + w) : INT32_MAX;
        s_i[w] = live ? ld_nc(i_idx + first + w) : 0;
    }
    __syncthreads();
#pragma unroll
    for (int v = 0; v < FS_VT; ++v) {
        const int64_t q = q0 + tid + v * NT;
        if (q >= n_j) return;
        int lo = 0, hi = need;  // largest w with s_start[w] <= q
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (s_start[mid] <= q) lo = mid; else hi = mid - 1;
        }
        out_i[q] = s_i[lo];
    }
}

// The route over expanded coordinates: steps 1-3 of the file comment. `z`'s arrays exist and hold
// cap_i / cap_j / cap_k entries (cap_k >= n_k(A) + n_k(B)); nothing is freed here on failure.
// `unit_fibres`: every fibre of the operands holds exactly one entry (n_k == n_j) and their k_ptr
// arrays are not read: the j column of the entries is j_idx itself and only i is written out.
int csf_add_expanded(const nb200_csf3 *a, const nb200_csf3 *b, nb200_csf3 *z, int64_t cap_i, int64_t cap_j, int64_t cap_k,
                     cudaStream_t stream, int slot, bool unit_fibres = false) {
    const int64_t total = (int64_t)a->n_k + b->n_k;
    cudaError_t e;
    int st;
    (void)cap_k;
    // one pool block: expanded (i, j) of A, of B and of the merged list, the merge's own scratch
    // and the compress pass's control block and tile words
    const int64_t compress_tiles = std::max<int64_t>((total + NT * CVT - 1) / (NT * CVT), coo3_add_tiles(total));
    Carver sizes;
    sizes.take<int32_t>((size_t)a->n_k);
    sizes.take<int32_t>((size_t)a->n_k);
    sizes.take<int32_t>((size_t)b->n_k);
    sizes.take<int32_t>((size_t)b->n_k);
    sizes.take<int32_t>((size_t)total);
    sizes.take<int32_t>((size_t)total);
    sizes.take<uint64_t>((size_t)compress_tiles + 8);
    const size_t own = sizes.used();
    Workspace *ws = nullptr;
    if ((st = acquire_workspace(stream, own + coo3_add_scratch_bytes(total) + 256, &ws, slot))) return (st);
    Carver carve(ws->dev);
    int32_t *ai = carve.take<int32_t>((size_t)a->n_k), *aj = carve.take<int32_t>((size_t)a->n_k);
    int32_t *bi = carve.take<int32_t>((size_t)b->n_k), *bj = carve.take<int32_t>((size_t)b->n_k);
    int32_t *zi = carve.take<int32_t>((size_t)total), *zj = carve.take<int32_t>((size_t)total);
    uint64_t *compress_block = carve.take<uint64_t>((size_t)compress_tiles + 8);
    void *merge_scratch = static_cast<unsigned char *>(ws->dev) + own;

    if (unit_fibres) {
        aj = a->j_idx;
        bj = b->j_idx;
        if (a->n_j > 0) {
            LaunchScope scope("csf_fibre_slices", stream);
            k_fibre_slices<<<(int)(((int64_t)a->n_j + NT * FS_VT - 1) / (NT * FS_VT)), NT, 0, stream>>>(a->n_i, a->n_j, a->i_idx, a->j_ptr, ai);
        }
        if (b->n_j > 0) {
            LaunchScope scope("csf_fibre_slices", stream);
            k_fibre_slices<<<(int)(((int64_t)b->n_j + NT * FS_VT - 1) / (NT * FS_VT)), NT, 0, stream>>>(b->n_i, b->n_j, b->i_idx, b->j_ptr, bi);
        }
    } else {
        if (a->n_j > 0) {
            LaunchScope scope("csf_expand", stream);
            k_csf_expand<<<(int)(((int64_t)a->n_j + 31) / 32 * 32 + NT - 1) / NT, NT, 0, stream>>>(a->n_i, a->n_j, a->i_idx, a->j_ptr, a->j_idx, a->k_ptr, ai, aj);
        }
        if (b->n_j > 0) {
            LaunchScope scope("csf_expand", stream);
            k_csf_expand<<<(int)(((int64_t)b->n_j + 31) / 32 * 32 + NT - 1) / NT, NT, 0, stream>>>(b->n_i, b->n_j, b->i_idx, b->j_ptr, b->j_idx, b->k_ptr, bi, bj);
        }
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return (note_cuda_error(e, "k_csf_expand"));

    nb200_coo3 ca{{a->dims[0], a->dims[1], a->dims[2]}, a->n_k, ai, aj, a->k_idx, a->val};
    nb200_coo3 cb{{b->dims[0], b->dims[1], b->dims[2]}, b->n_k, bi, bj, b->k_idx, b->val};
    nb200_coo3 cz{{0, 0, 0}, 0, zi, zj, z->k_idx, z->val};
    CompressCtl *ctl = reinterpret_cast<CompressCtl *>(compress_block);
    static_assert(sizeof(CompressCtl) <= 4 * sizeof(uint64_t), "control block must fit its slot");
    uint64_t *tile_state = compress_block + 4;

    // single-pass route: the merge writes the levels above k itself (no merged i / j columns, no
    // compress pass); its second look-back runs over `tile_state`, its totals land in ctl
    e = cudaMemsetAsync(compress_block, 0, sizeof(uint64_t) * ((size_t)coo3_add_tiles(total) + 4), stream);
    if (e != cudaSuccess) return (note_cuda_error(e, "cudaMemsetAsync"));
    const CsfLevelsOut levels{z->i_idx, z->j_ptr, z->j_idx, z->k_ptr, (int32_t)std::min<int64_t>(cap_i, INT32_MAX),
                              (int32_t)std::min<int64_t>(cap_j, INT32_MAX), tile_state, reinterpret_cast<CsfTotals *>(&ctl->n_i)};
    bool levels_done = false;
    if ((st = coo3_add_run(&ca, &cb, &cz, false, total, stream, merge_scratch, ws->host, &levels, &levels_done))) return (st);
    const int32_t nnz = cz.nnz;
    z->n_k = nnz;
    if (levels_done) {
        e = cudaMemcpyAsync(ws->host, ctl, sizeof(CompressCtl), cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) return (note_cuda_error(e, "read result lengths"));
        CompressCtl h;
        std::memcpy(&h, ws->host, sizeof(h));
        z->n_i = h.n_i;
        z->n_j = h.n_j;
        if (h.n_i > cap_i || h.n_j > cap_j) return (NB200_E_CAPACITY);
        return NB200_OK;
    }

    const int tiles = (int)(((int64_t)nnz + NT * CVT - 1) / (NT * CVT));
    e = cudaMemsetAsync(compress_block, 0, sizeof(uint64_t) * ((size_t)tiles + 4), stream);
    if (e != cudaSuccess) return (note_cuda_error(e, "cudaMemsetAsync"));
    {
        LaunchScope scope("csf_compress", stream);
        k_csf_compress<<<tiles, NT, 0, stream>>>(nnz, zi, zj, (int32_t)std::min<int64_t>(cap_i, INT32_MAX),
                                                 (int32_t)std::min<int64_t>(cap_j, INT32_MAX), z->i_idx, z->j_ptr, z->j_idx,
                                                 z->k_ptr, tile_state, ctl);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) return (note_cuda_error(e, "k_csf_compress"));
    e = cudaMemcpyAsync(ws->host, ctl, sizeof(CompressCtl), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return (note_cuda_error(e, "read result lengths"));
    CompressCtl h;
    std::memcpy(&h, ws->host, sizeof(h));
    if (h.status.error != 0) return note_timeout(h.status.error, h.status.detail, "csf3 level compress");
    z->n_i = h.n_i;
    z->n_j = h.n_j;
    if (h.n_i > cap_i || h.n_j > cap_j) return (NB200_E_CAPACITY);
    return NB200_OK;
}

// ------------------------------------------------------------------ the two-level route ----
//
// When the fibres hold several entries each, expanding (i, j) for every entry moves more bytes
// than the tensor has. The same union then comes from two smaller merges:
//   1. the fibre lists of A and B -- every (i, j) fibre as one entry of a tensor whose third level
//      is a single position -- go through the expanded route above with the values 1 (A) and 2 (B):
//      the result is Z's i_idx / j_ptr / j_idx, and per fibre of Z the sum 1, 2 or 3 says which
//      operands hold it;
//   2. an exclusive count of the A flags (and of the B flags) is the fibre of A (of B) that a
//      fibre of Z corresponds to, or the next one if the operand lacks it: k_ptr[that fibre] is a
//      row-offset array over Z's fibres in which a missing fibre is an empty row;
//   3. with those offsets A's and B's (k_idx, val) arrays are CSR matrices with one row per fibre
//      of Z, and the CSR union (csr_merge.cu) writes Z's k_ptr, k_idx and val in one pass.

__global__ void __launch_bounds__(NT) k_fill_float(float *__restrict__ p, int32_t n, float v) {
    const int64_t i = (int64_t)blockIdx.x * NT + threadIdx.x;
    if (i < n) p[i] = v;
}

constexpr int OVT = 16;  // fibres per thread in the offsets pass
constexpr int32_t DCSR_FIBRE_ROWS = 1 << 24;  // first extent up to which the fibre lists go through the DCSR union

// flags[u] in {1, 2, 3} for the n fibres of Z: which operand holds fibre u. Writes, for u = 0 .. n,
// off_a[u] = a_kptr[fibres of A before u] and off_b[u] likewise: one pass, the two running counts
// packed into one word and carried across tiles by bounded look-back.
__global__ void __launch_bounds__(NT) k_fibre_offsets(const float *__restrict__ flags, int32_t n, const int32_t *__restrict__ a_kptr,
                                                     const int32_t *__restrict__ b_kptr, int32_t *__restrict__ off_a,
                                                     int32_t *__restrict__ off_b, uint64_t *state_raw, FusedCtl *ctl) {
    __shared__ int scan_tmp[72];
    __shared__ long long s_base;
    volatile uint64_t *state = state_raw;
    const int tid = threadIdx.x, t = blockIdx.x;  // CTAs are dispatched in index order; waits on earlier tiles are bounded
    const int64_t p0 = ((int64_t)t * NT + tid) * OVT;
    int f[OVT], mine_a = 0, mine_b = 0;
    if (p0 + OVT <= n) {  // 16-byte loads: a thread's fibres are consecutive
#pragma unroll
        for (int q = 0; q < OVT; q += 4) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(flags + p0 + q));
            f[q] = (int)v.x, f[q + 1] = (int)v.y, f[q + 2] = (int)v.z, f[q + 3] = (int)v.w;
        }
    } else {
#pragma unroll
        for (int q = 0; q < OVT; ++q) f[q] = p0 + q < n ? (int)ld_nc(flags + p0 + q) : 0;
    }
#pragma unroll
    for (int q = 0; q < OVT; ++q) {
        mine_a += f[q] & 1;
        mine_b += f[q] >> 1;
    }
    int before_a, before_b, tot_a, tot_b;
    block_excl_sum2<NT>(mine_a, mine_b, scan_tmp, before_a, before_b, tot_a, tot_b);
    if (warp_id() == 0) {
        const int64_t b = lookback_exclusive(state, t, ((int64_t)tot_a << 31) | (int64_t)tot_b, &ctl->status);
        if (lane_id() == 0) s_base = b;
    }
    __syncthreads();
    const long long base = s_base;
    if (base < 0) return;
    int ca = (int)(base >> 31) + before_a, cb = (int)(base & 0x7fffffff) + before_b;
    int32_t va[OVT], vb[OVT];
#pragma unroll
    for (int q = 0; q < OVT; ++q) {
        const bool live = p0 + q <= n;
        va[q] = live ? ld_nc(a_kptr + ca) : 0;
        vb[q] = live ? ld_nc(b_kptr + cb) : 0;
        ca += f[q] & 1;
        cb += f[q] >> 1;
    }
    if (p0 + OVT <= (int64_t)n + 1) {
#pragma unroll
        for (int q = 0; q < OVT; q += 4) {
            *reinterpret_cast<int4 *>(off_a + p0 + q) = make_int4(va[q], va[q + 1], va[q + 2], va[q + 3]);
            *reinterpret_cast<int4 *>(off_b + p0 + q) = make_int4(vb[q], vb[q + 1], vb[q + 2], vb[q + 3]);
        }
    } else {
#pragma unroll
        for (int q = 0; q < OVT; ++q)
            if (p0 + q <= n) off_a[p0 + q] = va[q], off_b[p0 + q] = vb[q];
    }
}

// The expanded route moves 8 bytes of (i, j) per entry out and back in; the two-level route moves
// about as much per FIBRE. It pays once fibres hold a few entries on average.
bool two_level_pays(const nb200_csf3 *a, const nb200_csf3 *b) {
    if (a->n_j == 0 || b->n_j == 0) return false;
    if (const char *e = std::getenv("NACHO_B200_CSF_TWO_LEVEL")) return e[0] != '0';  // read per call: tests take both routes
    return 3 * ((int64_t)a->n_j + b->n_j) <= (int64_t)a->n_k + b->n_k;
}

int csf_add_two_level(const nb200_csf3 *a, const nb200_csf3 *b, nb200_csf3 *z, int64_t cap_i, int64_t cap_j, int64_t cap_k,
                      cudaStream_t stream) {
    const int32_t nja = a->n_j, njb = b->n_j;
    const int64_t bound_j = (int64_t)nja + njb;
    if (bound_j > INT32_MAX - 1) return NB200_E_OVERFLOW;
    const int32_t most = std::max(nja, njb);
    const int tiles_cap = (int)((bound_j + 1 + NT * OVT - 1) / (NT * OVT));
    Carver sizes;
    sizes.take<int32_t>((size_t)most);          // k_idx of the fibre tensors: zeros
    sizes.take<float>((size_t)nja);             // 1 per fibre of A
    sizes.take<float>((size_t)njb);             // 2 per fibre of B
    sizes.take<int32_t>((size_t)bound_j + 1);   // fibre tensor of Z: k_ptr
    sizes.take<int32_t>((size_t)bound_j);       //                     k_idx
    sizes.take<float>((size_t)bound_j);         //                     flags
    sizes.take<int32_t>((size_t)bound_j + 1);   // offsets of A's entries over Z's fibres
    sizes.take<int32_t>((size_t)bound_j + 1);   // the same for B
    sizes.take<uint64_t>((size_t)tiles_cap + 8);
    Workspace *ws = nullptr;
    int st;
    if ((st = acquire_workspace(stream, sizes.used(), &ws, 3))) return st;
    Carver carve(ws->dev);
    int32_t *zeros = carve.take<int32_t>((size_t)most);
    float *ones = carve.take<float>((size_t)nja), *twos = carve.take<float>((size_t)njb);
    int32_t *zf_kptr = carve.take<int32_t>((size_t)bound_j + 1), *zf_kidx = carve.take<int32_t>((size_t)bound_j);
    float *flags = carve.take<float>((size_t)bound_j);
    int32_t *off_a = carve.take<int32_t>((size_t)bound_j + 1), *off_b = carve.take<int32_t>((size_t)bound_j + 1);
    uint64_t *scan_block = carve.take<uint64_t>((size_t)tiles_cap + 8);
    auto grid = [](int64_t n) { return (int)((n + NT - 1) / NT); };

    NB200_CUDA(cudaMemsetAsync(zeros, 0, sizeof(int32_t) * (size_t)most, stream));
    {
        LaunchScope scope("csf_fibre_setup", stream);
        k_fill_float<<<grid(nja), NT, 0, stream>>>(ones, nja, 1.0f);
    }
    {
        LaunchScope scope("csf_fibre_setup", stream);
        k_fill_float<<<grid(njb), NT, 0, stream>>>(twos, njb, 2.0f);
    }
    NB200_CUDA(cudaGetLastError());

    // ---- 1. union of the fibre lists. They are DCSR matrices as they lie (slices x j): where the
    // first extent allows scratch per slice number and the caller's i capacity covers the one-pass
    // worst case, the DCSR union (CSR merge kernels, formats2d.cu) takes them; otherwise the route
    // over expanded coordinates does, with every fibre as one entry.
    const int64_t bound_i = std::min<int64_t>((int64_t)a->n_i + b->n_i, a->dims[0]);
    nb200_csf3 fz = *z;
    if (a->dims[0] <= DCSR_FIBRE_ROWS && cap_i >= bound_i) {
        const nb200_dcsr da{a->dims[0], a->dims[1], a->n_i, nja, a->i_idx, a->j_ptr, a->j_idx, ones};
        const nb200_dcsr db{b->dims[0], b->dims[1], b->n_i, njb, b->i_idx, b->j_ptr, b->j_idx, twos};
        nb200_dcsr dz{0, 0, 0, 0, z->i_idx, z->j_ptr, z->j_idx, flags};
        st = nb200_dcsr_add_f32_into(&da, &db, &dz, cap_i, std::min<int64_t>(cap_j, bound_j), stream);
        fz.n_i = dz.n_i;
        fz.n_j = dz.nnz;
    } else {
        nb200_csf3 fa = *a, fb = *b;
        fa.n_k = nja, fa.k_ptr = nullptr, fa.k_idx = zeros, fa.val = ones;
        fb.n_k = njb, fb.k_ptr = nullptr, fb.k_idx = zeros, fb.val = twos;
        fz.k_ptr = zf_kptr, fz.k_idx = zf_kidx, fz.val = flags;
        st = csf_add_expanded(&fa, &fb, &fz, cap_i, std::min<int64_t>(cap_j, bound_j), bound_j, stream, 0, true);
    }
    z->n_i = fz.n_i;
    z->n_j = fz.n_j;
    if (st != NB200_OK) return st;
    const int32_t nz = fz.n_j;  // fibres of Z

    // ---- 2. offsets of A's and B's entries over Z's fibres
    NB200_CUDA(cudaMemsetAsync(scan_block, 0, sizeof(uint64_t) * ((size_t)tiles_cap + 8), stream));
    {
        LaunchScope scope("csf_fibre_offsets", stream);
        k_fibre_offsets<<<(int)(((int64_t)nz + 1 + NT * OVT - 1) / (NT * OVT)), NT, 0, stream>>>(
            flags, nz, a->k_ptr, b->k_ptr, off_a, off_b, scan_block + 4, reinterpret_cast<FusedCtl *>(scan_block));
    }
    NB200_CUDA(cudaGetLastError());
    {   // a look-back of the offsets pass that gave up leaves offsets unwritten: they must not be used
        NB200_CUDA(cudaMemcpyAsync(ws->host, scan_block, sizeof(FusedCtl), cudaMemcpyDeviceToHost, stream));
        NB200_CUDA(cudaStreamSynchronize(stream));
        FusedCtl h;
        std::memcpy(&h, ws->host, sizeof(h));
        if (h.status.error != 0) return note_timeout(h.status.error, h.status.detail, "csf3 fibre offsets");
    }

    // ---- 3. the entries: a CSR union with one row per fibre of Z
    const nb200_csr ma{nz, a->dims[2], a->n_k, off_a, a->k_idx, a->val};
    const nb200_csr mb{nz, b->dims[2], b->n_k, off_b, b->k_idx, b->val};
    nb200_csr mz{0, 0, 0, z->k_ptr, z->k_idx, z->val};
    st = nb200_csr_add_f32_into(&ma, &mb, &mz, cap_k, stream);
    z->n_k = mz.nnz;
    return st;
}

int check_csf3(const nb200_csf3 *t) {
    if (!t || t->n_i < 0 || t->n_j < 0 || t->n_k < 0) return NB200_E_BADARG;
    if (t->n_k > 0 && (!t->i_idx || !t->j_ptr || !t->j_idx || !t->k_ptr || !t->k_idx || !t->val)) return NB200_E_BADARG;
    return NB200_OK;
}

int csf_add_run(const nb200_csf3 *a, const nb200_csf3 *b, nb200_csf3 *z, bool alloc, int64_t cap_i, int64_t cap_j,
                int64_t cap_k, void *stream_v) {
    int st;
    if ((st = check_csf3(a)) || (st = check_csf3(b))) return st;
    if (!z || a->dims[0] != b->dims[0] || a->dims[1] != b->dims[1] || a->dims[2] != b->dims[2]) return NB200_E_BADARG;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const int64_t total = (int64_t)a->n_k + b->n_k;
    if (total > INT32_MAX) return NB200_E_OVERFLOW;
    const int64_t bound_i = (int64_t)a->n_i + b->n_i, bound_j = (int64_t)a->n_j + b->n_j;
    for (int d = 0; d < 3; ++d) z->dims[d] = a->dims[d];
    z->n_i = z->n_j = z->n_k = 0;
    cudaError_t e;
    if (alloc) {
        z->i_idx = z->j_ptr = z->j_idx = z->k_ptr = z->k_idx = nullptr;
        z->val = nullptr;
        cap_i = bound_i;
        cap_j = bound_j;
        cap_k = total;
        struct { void **p; size_t n; } arrays[6] = {
            {reinterpret_cast<void **>(&z->i_idx), (size_t)bound_i}, {reinterpret_cast<void **>(&z->j_ptr), (size_t)bound_i + 1},
            {reinterpret_cast<void **>(&z->j_idx), (size_t)bound_j}, {reinterpret_cast<void **>(&z->k_ptr), (size_t)bound_j + 1},
            {reinterpret_cast<void **>(&z->k_idx), (size_t)total},   {reinterpret_cast<void **>(&z->val), (size_t)total}};
        for (auto &arr : arrays) {
            if (arr.n == 0) continue;
            e = cudaMallocAsync(arr.p, 4 * arr.n, stream);
            if (e != cudaSuccess) {
                for (auto &other : arrays) {
                    if (*other.p) cudaFreeAsync(*other.p, stream);
                    *other.p = nullptr;
                }
                return note_cuda_error(e, "cudaMallocAsync");
            }
        }
    } else {
        if (cap_i < 0 || cap_j < 0 || cap_k < 0 || !z->j_ptr || !z->k_ptr) return NB200_E_BADARG;
        if (cap_k < total) return NB200_E_CAPACITY;  // the merge needs room for every operand entry
        if (total > 0 && (!z->i_idx || !z->j_idx || !z->k_idx || !z->val)) return NB200_E_BADARG;
    }
    auto fail = [&](int code) {
        if (alloc) {
            void **ps[6] = {reinterpret_cast<void **>(&z->i_idx), reinterpret_cast<void **>(&z->j_ptr),
                            reinterpret_cast<void **>(&z->j_idx), reinterpret_cast<void **>(&z->k_ptr),
                            reinterpret_cast<void **>(&z->k_idx), reinterpret_cast<void **>(&z->val)};
            for (auto p : ps) {
                if (*p) cudaFreeAsync(*p, stream);
                *p = nullptr;
            }
        }
        return code;
    };
    if (total == 0) {  // empty result: the two offset arrays hold their single leading zero
        e = cudaMemsetAsync(z->j_ptr, 0, sizeof(int32_t), stream);
        if (e == cudaSuccess) e = cudaMemsetAsync(z->k_ptr, 0, sizeof(int32_t), stream);
        if (e != cudaSuccess) return fail(note_cuda_error(e, "cudaMemsetAsync"));
        return NB200_OK;
    }

    st = two_level_pays(a, b) ? csf_add_two_level(a, b, z, cap_i, cap_j, cap_k, stream) : csf_add_expanded(a, b, z, cap_i, cap_j, cap_k, stream, 0);
    return st == NB200_OK ? NB200_OK : fail(st);
}

// Inner product of two CSF3 tensors (compiler.cpp:141): every entry gets its (i, j) written out
// next to its k (k_csf_expand), then the coordinate lists go through the inner-product mode of the
// COO3 tile kernel.
int csf_inner_run(const nb200_csf3 *a, const nb200_csf3 *b, float *z, void *stream_v) {
    int st;
    if ((st = check_csf3(a)) || (st = check_csf3(b))) return st;
    if (!z || a->dims[0] != b->dims[0] || a->dims[1] != b->dims[1] || a->dims[2] != b->dims[2]) return NB200_E_BADARG;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    if (a->n_k == 0 || b->n_k == 0) {
        NB200_CUDA(cudaMemsetAsync(z, 0, sizeof(float), stream));
        return NB200_OK;
    }
    const int64_t total = (int64_t)a->n_k + b->n_k;
    if (total > INT32_MAX) return NB200_E_OVERFLOW;
    Carver sizes;
    sizes.take<int32_t>((size_t)a->n_k);
    sizes.take<int32_t>((size_t)a->n_k);
    sizes.take<int32_t>((size_t)b->n_k);
    sizes.take<int32_t>((size_t)b->n_k);
    const size_t own = sizes.used();
    Workspace *ws = nullptr;
    if ((st = acquire_workspace(stream, own + coo3_add_scratch_bytes(total) + 256, &ws))) return st;
    Carver carve(ws->dev);
    int32_t *ai = carve.take<int32_t>((size_t)a->n_k), *aj = carve.take<int32_t>((size_t)a->n_k);
    int32_t *bi = carve.take<int32_t>((size_t)b->n_k), *bj = carve.take<int32_t>((size_t)b->n_k);
    void *merge_scratch = static_cast<unsigned char *>(ws->dev) + own;
    {
        LaunchScope scope("csf_expand", stream);
        k_csf_expand<<<(int)(((int64_t)a->n_j + 31) / 32 * 32 + NT - 1) / NT, NT, 0, stream>>>(a->n_i, a->n_j, a->i_idx, a->j_ptr, a->j_idx, a->k_ptr, ai, aj);
    }
    {
        LaunchScope scope("csf_expand", stream);
        k_csf_expand<<<(int)(((int64_t)b->n_j + 31) / 32 * 32 + NT - 1) / NT, NT, 0, stream>>>(b->n_i, b->n_j, b->i_idx, b->j_ptr, b->j_idx, b->k_ptr, bi, bj);
    }
    NB200_CUDA(cudaGetLastError());
    nb200_coo3 ca{{a->dims[0], a->dims[1], a->dims[2]}, a->n_k, ai, aj, a->k_idx, a->val};
    nb200_coo3 cb{{b->dims[0], b->dims[1], b->dims[2]}, b->n_k, bi, bj, b->k_idx, b->val};
    return coo3_inner_run(&ca, &cb, z, stream_v, merge_scratch, ws->host);
}

}  // namespace

}  // namespace nb200

using namespace nb200;

extern "C" {

int nb200_csf_add_f32(const nb200_csf3 *a, const nb200_csf3 *b, nb200_csf3 *z, int32_t, int32_t, void *stream) {
    return csf_add_run(a, b, z, true, 0, 0, 0, stream);
}

int nb200_csf_add_f32_into(const nb200_csf3 *a, const nb200_csf3 *b, nb200_csf3 *z, int64_t cap_i, int64_t cap_j,
                           int64_t cap_k, void *stream) {
    return csf_add_run(a, b, z, false, cap_i, cap_j, cap_k, stream);
}

int nb200_inner_prod_f32(const nb200_csf3 *a, const nb200_csf3 *b, float *z, void *stream) {
    return csf_inner_run(a, b, z, stream);
}

}  // extern "C"
