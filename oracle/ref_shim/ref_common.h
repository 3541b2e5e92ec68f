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

// 2-D COO operands and results (Compressed_non_unique + Singleton levels of compiler.cpp:50-58).
template <typename T>
static T coo_view(const ref_coo *m) {
    T t = {};
    t.dim_i_size = m->rows;
    t.dim_j_size = m->cols;
    t.dim_i_length = m->nnz;
    t.dim_i_indices = m->i;
    t.dim_j_length = m->nnz;
    t.dim_j_indices = m->j;
    t.values = m->val;
    t.nnz = m->nnz;
    return t;
}

template <typename T>
static void coo_out(const T &Z, ref_coo *z) {
    z->rows = Z.dim_i_size;
    z->cols = Z.dim_j_size;
    z->nnz = Z.dim_j_length;
    z->i = Z.dim_i_indices;
    z->j = Z.dim_j_indices;
    z->val = Z.values;
}

// DCSR: both levels compressed (compiler.cpp:38-42).
template <typename T>
static T dcsr_view(const ref_dcsr *m) {
    T t = {};
    t.dim_i_size = m->rows;
    t.dim_j_size = m->cols;
    t.dim_i_length = m->n_i;
    t.dim_i_indices = m->i_idx;
    t.dim_j_offsets = m->j_ptr;
    t.dim_j_length = m->nnz;
    t.dim_j_indices = m->j_idx;
    t.values = m->val;
    t.nnz = m->nnz;
    return t;
}

template <typename T>
static void dcsr_out(const T &Z, ref_dcsr *z) {
    z->rows = Z.dim_i_size;
    z->cols = Z.dim_j_size;
    z->n_i = Z.dim_i_length;
    z->nnz = Z.dim_j_length;
    z->i_idx = Z.dim_i_indices;
    z->j_ptr = Z.dim_j_offsets;
    z->j_idx = Z.dim_j_indices;
    z->val = Z.values;
}

template <typename T>
static T coo3_view_of(const ref_coo3 *m) {
    T t = {};
    t.dim_i_size = m->dims[0];
    t.dim_j_size = m->dims[1];
    t.dim_k_size = m->dims[2];
    t.dim_i_length = m->nnz;
    t.dim_i_indices = m->i;
    t.dim_j_length = m->nnz;
    t.dim_j_indices = m->j;
    t.dim_k_length = m->nnz;
    t.dim_k_indices = m->k;
    t.values = m->val;
    t.nnz = m->nnz;
    return t;
}

template <typename T>
static T csf3_view_of(const ref_csf3 *m) {
    T t = {};
    t.dim_i_size = m->dims[0];
    t.dim_j_size = m->dims[1];
    t.dim_k_size = m->dims[2];
    t.dim_i_length = m->n_i;
    t.dim_i_indices = m->i_idx;
    t.dim_j_offsets = m->j_ptr;
    t.dim_j_length = m->n_j;
    t.dim_j_indices = m->j_idx;
    t.dim_k_offsets = m->k_ptr;
    t.dim_k_length = m->n_k;
    t.dim_k_indices = m->k_idx;
    t.values = m->val;
    t.nnz = m->n_k;
    return t;
}
