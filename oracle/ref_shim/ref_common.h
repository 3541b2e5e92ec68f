// Helpers shared by the per-kernel wrappers of the reference-CPU checker library.
#pragma once
#include "ref_abi.h"

// The emitted headers declare one POD struct type per operand with identical CSR fields
// (emitter src/backend/tensor.cpp:13-61); these fill any of them from the C-ABI view.
template <typename T>
static T csr_view(const ref_csr *m) {
    T t = {};
    t.dim_i_size = m->rows;
    t.dim_j_size = m->cols;
    t.dim_j_offsets = m->row_ptr;
    t.dim_j_length = m->nnz;
    t.dim_j_indices = m->col;
    t.values = m->val;
    t.nnz = m->nnz;
    return t;
}

template <typename T>
static void csr_out(const T &Z, ref_csr *z) {
    z->rows = Z.dim_i_size;
    z->cols = Z.dim_j_size;
    z->nnz = Z.dim_j_length;
    z->row_ptr = Z.dim_j_offsets;
    z->col = Z.dim_j_indices;
    z->val = Z.values;
}
