// Helpers shared by the per-kernel wrappers of the reference-GPU checker library.
#pragma once
#include <cuda_runtime.h>

#include "ref_gpu_abi.h"

// The emitted CSR operand/result structs all hold (size, size, offsets*, length, indices*,
// values*, nnz) in this order under kernel-specific field names (emitter
// src/backend/tensor.cpp:13-61), so they are filled and read by position.
template <typename T>
static T csr_pos_view(const ref_csr *m) {
    return T{m->rows, m->cols, m->row_ptr, m->nnz, m->col, m->val, m->nnz};
}

template <typename T>
static void csr_pos_out(const T &Z, ref_csr *z) {
    struct Plain {
        int32_t rows, cols;
        int32_t *row_ptr;
        int32_t nnz_len;
        int32_t *col;
        float *val;
        int32_t nnz;
    };
    static_assert(sizeof(Plain) == sizeof(T), "CSR struct layout differs from the emitter's");
    Plain p;
    __builtin_memcpy(&p, &Z, sizeof(p));
    z->rows = p.rows;
    z->cols = p.cols;
    z->nnz = p.nnz_len;
    z->row_ptr = p.row_ptr;
    z->col = p.col;
    z->val = p.val;
}

static inline int ref_gpu_finish() {
    cudaError_t e = cudaDeviceSynchronize();
    cudaError_t l = cudaGetLastError();
    return (int)(e != cudaSuccess ? e : l);
}
