// Types and small helpers shared by the CSR element-wise kernels (two-operand kernels in
// csr_merge.cu, the fused three-operand add in csr_add3.cu).
#pragma once

#include <stdint.h>

#include "block_utils.cuh"
#include "common.cuh"
#include "merge_common.cuh"
#include "tma.cuh"

namespace nb200 {

constexpr int CSR_NT = 256;  // worker threads of a CSR tile CTA (one more warp scans)

struct CsrIn {
    const int32_t *rp;
    const int32_t *col;
    const float *val;
    int32_t nnz;
};

struct CsrOut {
    int32_t *rp;
    int32_t *col;
    float *val;
    // Asynchronous calls only: three device words {result entries, status, rows} the kernels fill
    // themselves. The partition kernel writes rows and a status of 0, the last tile the length, and
    // any tile whose bounded wait gives up (or a length beyond int32) raises the status.
    long long *result = nullptr;
};

// Hardware barriers of the tile kernels: 0 = the whole CTA (__syncthreads), 1 = the worker
// threads, 2 = workers arrive / the scan warp waits ("the tile's count is known").
using WorkerBar = NamedBarrier<1, CSR_NT>;
using CountBar = NamedBarrier<2, CSR_NT + 32>;

constexpr int MBAR_POLL_LIMIT = 1 << 24;
constexpr int ERR_COPY_TIMEOUT = 2;
constexpr int ERR_WIDE_TILE = 3;  // a tile's rows do not fit the 32-bit composite key of a kernel without a wide-key body

// Number of 4-byte elements from `p` up to the next 16-byte boundary (0..3).
__device__ __forceinline__ int head_elems(const void *p) {
    return (int)(((16u - (unsigned)(reinterpret_cast<uintptr_t>(p) & 15u)) & 15u) >> 2);
}

inline int col_bits(int32_t cols) {
    int b = 1;
    while (b < 32 && (int64_t(1) << b) < (int64_t)cols) ++b;
    return b;
}

inline int check_csr(const nb200_csr *m, bool need_arrays) {
    if (!m || m->rows < 0 || m->cols < 0 || m->nnz < 0) return NB200_E_BADARG;
    if (need_arrays && (!m->row_ptr || (m->nnz > 0 && (!m->col || !m->val)))) return NB200_E_BADARG;
    return NB200_OK;
}

// Two chained two-operand unions (A + B) + C through a pool intermediate: the route of callers
// whose capacity is below the worst case, and of inputs the fused kernel does not take.
int csr_add3_chained(const nb200_csr *a, const nb200_csr *b, const nb200_csr *c, nb200_csr *z, bool alloc, int64_t capacity,
                     void *stream_v);

}  // namespace nb200
