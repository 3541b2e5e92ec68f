// The 2-D formats beside CSR: coordinate lists (COO) and doubly compressed rows (DCSR), and the
// element-wise kernels the reference declares over them (compiler.cpp:118-126):
//   coo_add, coo_mul        COO  (+|.*) COO  -> COO
//   coo_csr_add             CSR  +      COO  -> CSR
//   dcsr_add, dcsr_mul      DCSR (+|.*) DCSR -> DCSR
// A sorted coordinate list and a DCSR matrix are both a CSR matrix whose row offsets are not
// stored: their column and value arrays are already in CSR order. So each kernel here builds the
// missing row offsets (one small pass over the rows), runs the CSR merge kernels of csr_merge.cu
// on the caller's own column / value arrays, and converts the result's row level back:
//   COO   the row index of every result entry is written out (one warp per 32 rows);
//   DCSR  the rows that the reference keeps are selected and compressed (scan + scatter):
//         for the sum, the rows that hold a result entry; for the product, the rows that BOTH
//         operands store -- also those whose columns do not meet, which the reference keeps as
//         an empty fibre (its intersection works level by level: src/backend/compute.cpp:619-1392
//         run on the i level first, then on j inside the matched rows).
// Scratch: three row-offset arrays of rows + 1 entries (and one flag array for DCSR).
#include <algorithm>
#include <cstring>

#include "merge_common.cuh"

namespace nb200 {

namespace {

constexpr int NT = 256;

// rp[r] = ptr[q(r)] where q(r) is the number of ids below r (ids sorted ascending, n of them);
// ptr == nullptr stands for ptr[q] = q. Thread q writes the rows in (ids[q - 1], ids[q]]; the rows
// after the last id get ptr[n]. With repeated ids (a coordinate list) a thread whose id equals its
// predecessor's has no row to write.
__global__ void __launch_bounds__(NT) k_row_offsets(const int32_t *__restrict__ ids, const int32_t *__restrict__ ptr, int32_t n,
                                                   int32_t rows, int32_t *__restrict__ rp) {
    const int64_t q = (int64_t)blockIdx.x * NT + threadIdx.x;
    if (q > n) return;
    const int64_t first = q == 0 ? 0 : (int64_t)ld_nc(ids + q - 1) + 1;
    const int64_t last = q == n ? rows : ld_nc(ids + q);
    const int32_t v = ptr ? ld_nc(ptr + q) : (int32_t)q;
    for (int64_t r = first; r <= last && r <= rows; ++r) rp[r] = v;
}

// out[p] = the row of entry p, for every entry of a CSR structure: one warp per 32 consecutive
// rows walks their entries 32 at a time; an entry's row is the last of the 32 whose start is at
// or before it (found with five shuffles), so the writes are coalesced however short the rows are.
__global__ void __launch_bounds__(NT) k_expand_rows(const int32_t *__restrict__ rp, int32_t rows, int32_t *__restrict__ out) {
    const int w = (blockIdx.x * NT + threadIdx.x) >> 5;
    const int64_t r0 = (int64_t)w * 32;
    if (r0 >= rows) return;
    const int lane = lane_id();
    const int32_t start = r0 + lane < rows ? ld_nc(rp + r0 + lane) : INT32_MAX;
    const int32_t p_begin = __shfl_sync(FULL_MASK, start, 0);
    const int32_t p_end = ld_nc(rp + min(r0 + 32, (int64_t)rows));
    for (int32_t base = p_begin; base < p_end; base += 32) {
        const int32_t p = base + lane;
        int lo = 0, hi = 31;  // largest lane whose row starts at or before p
#pragma unroll
        for (int step = 0; step < 5; ++step) {
            const int mid = (lo + hi + 1) >> 1;
            const int32_t sm = __shfl_sync(FULL_MASK, start, mid);
            if (sm <= p) lo = mid; else hi = mid - 1;
        }
        if (p < p_end) out[p] = (int32_t)(r0 + lo);
    }
}

// keep[r] = 1 for the rows the result stores. Sum: a row with a result entry. Product: a row
// that both operands store (whatever its result holds).
__global__ void __launch_bounds__(NT) k_dcsr_keep(const int32_t *__restrict__ rpa, const int32_t *__restrict__ rpb,
                                                 const int32_t *__restrict__ rpz, int32_t rows, int product, int32_t *__restrict__ keep) {
    const int64_t r = (int64_t)blockIdx.x * NT + threadIdx.x;
    if (r >= rows) return;
    const bool in_a = ld_nc(rpa + r + 1) > ld_nc(rpa + r), in_b = ld_nc(rpb + r + 1) > ld_nc(rpb + r);
    keep[r] = product ? (in_a && in_b) : (ld_nc(rpz + r + 1) > ld_nc(rpz + r));
}

// After the exclusive scan of keep[]: row r, if kept, is result row pos[r]. The flag is recomputed
// (pos[r + 1] > pos[r], with the total after the last row).
__global__ void __launch_bounds__(NT) k_dcsr_scatter(const int32_t *__restrict__ pos, const long long *__restrict__ total,
                                                    const int32_t *__restrict__ rpz, int32_t rows, int32_t *__restrict__ i_idx,
                                                    int32_t *__restrict__ j_ptr) {
    const int64_t r = (int64_t)blockIdx.x * NT + threadIdx.x;
    if (r > rows) return;
    const int32_t n = (int32_t)*total;
    if (r == rows) {
        j_ptr[n] = ld_nc(rpz + rows);
        return;
    }
    const int32_t at = ld_nc(pos + r);
    const int32_t next = r + 1 < rows ? ld_nc(pos + r + 1) : n;
    if (next > at) {
        i_idx[at] = (int32_t)r;
        j_ptr[at] = ld_nc(rpz + r);
    }
}

int check_coo(const nb200_coo *m) {
    if (!m || m->rows < 0 || m->cols < 0 || m->nnz < 0) return NB200_E_BADARG;
    if (m->nnz > 0 && (!m->i || !m->j || !m->val)) return NB200_E_BADARG;
    return NB200_OK;
}

int check_dcsr(const nb200_dcsr *m) {
    if (!m || m->rows < 0 || m->cols < 0 || m->n_i < 0 || m->nnz < 0 || m->n_i > m->rows) return NB200_E_BADARG;
    if (!m->j_ptr || (m->n_i > 0 && !m->i_idx) || (m->nnz > 0 && (!m->j_idx || !m->val))) return NB200_E_BADARG;
    return NB200_OK;
}

cudaError_t launch_row_offsets(const int32_t *ids, const int32_t *ptr, int32_t n, int32_t rows, int32_t *rp, cudaStream_t stream) {
    LaunchScope scope("row_offsets", stream);
    k_row_offsets<<<(int)(((int64_t)n + 1 + NT - 1) / NT), NT, 0, stream>>>(ids, ptr, n, rows, rp);
    return cudaGetLastError();
}

typedef int (*csr_into_fn)(const nb200_csr *, const nb200_csr *, nb200_csr *, int64_t, void *);

// Scratch of one call: three row-offset arrays, the keep / position array and a control block
// with the scan's tile words (DCSR only). Pool slot 1: the CSR kernels underneath use slot 0.
struct Scratch2d {
    int32_t *rpa, *rpb, *rpz, *keep;
    uint64_t *scan_block;
    Workspace *ws;
};

int take_scratch(int32_t rows, cudaStream_t stream, Scratch2d *s) {
    const size_t scan_ctas = ((size_t)rows + SCAN_NT * SCAN_VT - 1) / (SCAN_NT * SCAN_VT) + 1;
    Carver sizes;
    for (int q = 0; q < 4; ++q) sizes.take<int32_t>((size_t)rows + 2);
    sizes.take<uint64_t>(scan_ctas + 8);
    int st;
    if ((st = acquire_workspace(stream, sizes.used(), &s->ws, 1))) return st;
    Carver carve(s->ws->dev);
    s->rpa = carve.take<int32_t>((size_t)rows + 2);
    s->rpb = carve.take<int32_t>((size_t)rows + 2);
    s->rpz = carve.take<int32_t>((size_t)rows + 2);
    s->keep = carve.take<int32_t>((size_t)rows + 2);
    s->scan_block = carve.take<uint64_t>(scan_ctas + 8);
    return NB200_OK;
}

int coo2_run(csr_into_fn op, bool is_union, const nb200_coo *a, const nb200_coo *b, nb200_coo *z, int64_t capacity, void *stream_v) {
    int st;
    if ((st = check_coo(a)) || (st = check_coo(b))) return st;
    if (!z || a->rows != b->rows || a->cols != b->cols || capacity < 0) return NB200_E_BADARG;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    z->rows = a->rows;
    z->cols = a->cols;
    z->nnz = 0;
    const int64_t total = (int64_t)a->nnz + b->nnz;
    if (total == 0 || (!is_union && (a->nnz == 0 || b->nnz == 0))) return NB200_OK;
    if (capacity > 0 && (!z->i || !z->j || !z->val)) return NB200_E_BADARG;
    Scratch2d s;
    if ((st = take_scratch(a->rows, stream, &s))) return st;
    cudaError_t e = launch_row_offsets(a->i, nullptr, a->nnz, a->rows, s.rpa, stream);
    if (e == cudaSuccess) e = launch_row_offsets(b->i, nullptr, b->nnz, b->rows, s.rpb, stream);
    if (e != cudaSuccess) return note_cuda_error(e, "k_row_offsets");
    const nb200_csr ca{a->rows, a->cols, a->nnz, s.rpa, a->j, a->val}, cb{b->rows, b->cols, b->nnz, s.rpb, b->j, b->val};
    nb200_csr cz{a->rows, a->cols, 0, s.rpz, z->j, z->val};
    st = op(&ca, &cb, &cz, capacity, stream_v);
    z->nnz = cz.nnz;
    if (st != NB200_OK) return st;
    if (cz.nnz > 0) {
        LaunchScope scope("expand_rows", stream);
        const int64_t warps = ((int64_t)a->rows + 31) / 32;
        k_expand_rows<<<(int)((warps * 32 + NT - 1) / NT), NT, 0, stream>>>(s.rpz, a->rows, z->i);
        e = cudaGetLastError();
        if (e != cudaSuccess) return note_cuda_error(e, "k_expand_rows");
    }
    return NB200_OK;
}

int dcsr2_run(csr_into_fn op, bool is_union, const nb200_dcsr *a, const nb200_dcsr *b, nb200_dcsr *z, int64_t cap_i, int64_t capacity,
              void *stream_v) {
    int st;
    if ((st = check_dcsr(a)) || (st = check_dcsr(b))) return st;
    if (!z || a->rows != b->rows || a->cols != b->cols || capacity < 0 || cap_i < 0 || !z->j_ptr) return NB200_E_BADARG;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const int32_t rows = a->rows;
    z->rows = rows;
    z->cols = a->cols;
    z->n_i = z->nnz = 0;
    const int64_t bound_i = is_union ? std::min<int64_t>((int64_t)a->n_i + b->n_i, rows) : std::min(a->n_i, b->n_i);
    if (cap_i < bound_i) return NB200_E_CAPACITY;  // the row level is written in one pass: room for the worst case
    if (bound_i > 0 && !z->i_idx) return NB200_E_BADARG;
    if (bound_i == 0) {  // no row survives: one leading zero in the offsets
        NB200_CUDA(cudaMemsetAsync(z->j_ptr, 0, sizeof(int32_t), stream));
        return NB200_OK;
    }
    if (capacity > 0 && (!z->j_idx || !z->val)) return NB200_E_BADARG;
    Scratch2d s;
    if ((st = take_scratch(rows, stream, &s))) return st;
    cudaError_t e = launch_row_offsets(a->i_idx, a->j_ptr, a->n_i, rows, s.rpa, stream);
    if (e == cudaSuccess) e = launch_row_offsets(b->i_idx, b->j_ptr, b->n_i, rows, s.rpb, stream);
    if (e != cudaSuccess) return note_cuda_error(e, "k_row_offsets");
    const nb200_csr ca{rows, a->cols, a->nnz, s.rpa, a->j_idx, a->val}, cb{rows, b->cols, b->nnz, s.rpb, b->j_idx, b->val};
    nb200_csr cz{rows, a->cols, 0, s.rpz, z->j_idx, z->val};
    st = op(&ca, &cb, &cz, capacity, stream_v);
    z->nnz = cz.nnz;
    if (st != NB200_OK) return st;
    // select the rows the result stores, number them, write the compressed row level
    const int scan_ctas = (int)(((int64_t)rows + SCAN_NT * SCAN_VT - 1) / (SCAN_NT * SCAN_VT));
    FusedCtl *ctl = reinterpret_cast<FusedCtl *>(s.scan_block);
    NB200_CUDA(cudaMemsetAsync(s.scan_block, 0, sizeof(uint64_t) * ((size_t)scan_ctas + 4), stream));
    {
        LaunchScope scope("dcsr_keep", stream);
        k_dcsr_keep<<<(int)(((int64_t)rows + NT - 1) / NT), NT, 0, stream>>>(s.rpa, s.rpb, s.rpz, rows, is_union ? 0 : 1, s.keep);
    }
    {
        LaunchScope scope("scan_lookback", stream);
        k_scan_lookback<<<scan_ctas, SCAN_NT, 0, stream>>>(s.keep, rows, s.scan_block + 4, ctl);
    }
    {
        LaunchScope scope("dcsr_scatter", stream);
        k_dcsr_scatter<<<(int)(((int64_t)rows + 1 + NT - 1) / NT), NT, 0, stream>>>(s.keep, &ctl->total, s.rpz, rows, z->i_idx, z->j_ptr);
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return note_cuda_error(e, "dcsr row level");
    NB200_CUDA(cudaMemcpyAsync(s.ws->host, ctl, sizeof(FusedCtl), cudaMemcpyDeviceToHost, stream));
    NB200_CUDA(cudaStreamSynchronize(stream));
    FusedCtl h;
    std::memcpy(&h, s.ws->host, sizeof(h));
    if (h.status.error != 0) return note_timeout(h.status.error, h.status.detail, "dcsr row compress");
    z->n_i = (int32_t)h.total;
    return NB200_OK;
}

}  // namespace

}  // namespace nb200

using namespace nb200;

extern "C" {

int nb200_coo_add_f32_into(const nb200_coo *a, const nb200_coo *b, nb200_coo *z, int64_t capacity, void *stream) {
    return coo2_run(nb200_csr_add_f32_into, true, a, b, z, capacity, stream);
}

int nb200_coo_mul_f32_into(const nb200_coo *a, const nb200_coo *b, nb200_coo *z, int64_t capacity, void *stream) {
    return coo2_run(nb200_csr_mul_f32_into, false, a, b, z, capacity, stream);
}

int nb200_coo_csr_add_f32_into(const nb200_csr *a, const nb200_coo *b, nb200_csr *z, int64_t capacity, void *stream_v) {
    int st;
    if ((st = check_coo(b))) return st;
    if (!a || a->rows != b->rows || a->cols != b->cols) return NB200_E_BADARG;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    Scratch2d s;
    if ((st = take_scratch(b->rows, stream, &s))) return st;
    cudaError_t e = launch_row_offsets(b->i, nullptr, b->nnz, b->rows, s.rpb, stream);
    if (e != cudaSuccess) return note_cuda_error(e, "k_row_offsets");
    const nb200_csr cb{b->rows, b->cols, b->nnz, s.rpb, b->j, b->val};
    return nb200_csr_add_f32_into(a, &cb, z, capacity, stream_v);
}

int nb200_dcsr_add_f32_into(const nb200_dcsr *a, const nb200_dcsr *b, nb200_dcsr *z, int64_t cap_i, int64_t capacity, void *stream) {
    return dcsr2_run(nb200_csr_add_f32_into, true, a, b, z, cap_i, capacity, stream);
}

int nb200_dcsr_mul_f32_into(const nb200_dcsr *a, const nb200_dcsr *b, nb200_dcsr *z, int64_t cap_i, int64_t capacity, void *stream) {
    return dcsr2_run(nb200_csr_mul_f32_into, false, a, b, z, cap_i, capacity, stream);
}

}  // extern "C"
