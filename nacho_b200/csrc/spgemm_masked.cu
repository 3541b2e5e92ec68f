// Masked SpGEMM ("sssmm"): Z_ik = sum_j a_ij * b_jk * c_ik on the positions the mask C stores and
// at least one product reaches. The reference declares it as one fused kernel
// (compiler.cpp:150-153: Sum_j a_ij * b_jk * c_ik) and runs it through the same expand / sort /
// compress machinery as its SpGEMM (src/backend/stitch_and_generate_gpu.cpp:14-139), on the products
// that survive the three-way intersection.
//
// Here the mask drives the accumulation, so nothing outside it is ever formed:
//   k_sssmm_accumulate  one CTA per row i. Its warps take the entries a_ij of the row, the lanes of
//                       a warp the entries b_jk of row j of B; each product looks its column k up in
//                       the (sorted) columns of row i of C by binary search and, if the mask holds
//                       it, adds (a_ij * b_jk) * c_ik -- the reference's expression, left to right --
//                       to that position's accumulator and flags the position. Accumulators and
//                       flags are two scratch arrays of nnz(C) entries.
//   k_scan_lookback     exclusive scan of the flags: the result position of every mask position.
//   k_sssmm_compact     flagged positions move to their result slot (column, value); the result's
//                       row offsets are the scanned flags at the mask's row starts.
// The sums are float32 atomics in arrival order, as the reference's compress is for every row.
#include <algorithm>
#include <cstring>

#include "merge_common.cuh"

namespace nb200 {

namespace {

constexpr int NT = 128;

struct CsrView {
    const int32_t *rp, *col;
    const float *val;
};

__global__ void __launch_bounds__(NT) k_sssmm_accumulate(CsrView A, CsrView B, CsrView C, int32_t rows, float *__restrict__ acc,
                                                        int32_t *__restrict__ hit) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int32_t c0 = ld_nc(C.rp);  // the mask may be a row block of a larger matrix: positions count from its first entry
    for (int64_t i = blockIdx.x; i < rows; i += gridDim.x) {
        const int32_t c_lo = ld_nc(C.rp + i), c_hi = ld_nc(C.rp + i + 1);
        const int32_t a_lo = ld_nc(A.rp + i), a_hi = ld_nc(A.rp + i + 1);
        if (c_lo == c_hi || a_lo == a_hi) continue;
        for (int32_t p = a_lo + warp; p < a_hi; p += NT / 32) {
            const int32_t j = ld_nc(A.col + p);
            const float av = ld_nc(A.val + p);
            const int32_t b_lo = ld_nc(B.rp + j), b_hi = ld_nc(B.rp + j + 1);
            for (int32_t q = b_lo + lane; q < b_hi; q += 32) {
                const int32_t k = ld_nc(B.col + q);
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
    const int scan_ctas = (int)(((int64_t)nnz + 1 + SCAN_NT * SCAN_VT - 1) / (SCAN_NT * SCAN_VT));
    Carver sizes;
    sizes.take<float>((size_t)nnz);
    sizes.take<int32_t>((size_t)nnz + 1);
    sizes.take<uint64_t>((size_t)scan_ctas + 8);
    Workspace *ws = nullptr;
    if ((st = acquire_workspace(stream, sizes.used(), &ws, 1))) return st;
    Carver carve(ws->dev);
    float *acc = carve.take<float>((size_t)nnz);
    int32_t *hit = carve.take<int32_t>((size_t)nnz + 1);
    uint64_t *scan_block = carve.take<uint64_t>((size_t)scan_ctas + 8);
    FusedCtl *ctl = reinterpret_cast<FusedCtl *>(scan_block);
    NB200_CUDA(cudaMemsetAsync(acc, 0, sizeof(float) * (size_t)nnz, stream));
    NB200_CUDA(cudaMemsetAsync(hit, 0, sizeof(int32_t) * ((size_t)nnz + 1), stream));
    NB200_CUDA(cudaMemsetAsync(scan_block, 0, sizeof(uint64_t) * ((size_t)scan_ctas + 4), stream));
    const CsrView A{a->row_ptr, a->col, a->val}, B{b->row_ptr, b->col, b->val}, C{c->row_ptr, c->col, c->val};
    {
        LaunchScope scope("sssmm_accumulate", stream);
        k_sssmm_accumulate<<<std::min<int64_t>(rows, 1 << 20), NT, 0, stream>>>(A, B, C, rows, acc, hit);
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
    if (h.status.error != 0) return NB200_E_TIMEOUT;
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
