// C ABI of the reference-CPU checker library (test infrastructure only).
//
// Each ref_* function wraps one CPU driver emitted by the reference's compiler
// (<kernel>_cpu_i32_f32; emitter src/backend/stitch_and_generate_cpu.cpp:18) so that tests
// and the CPU-baseline leg of the benchmark can call it through ctypes. Result arrays are
// malloc'd by the emitted driver; release them with ref_free().
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
    int32_t rows, cols;
    int32_t nnz;
    int32_t *row_ptr;  // rows + 1
    int32_t *col;      // nnz
    float *val;        // nnz
} ref_csr;

typedef struct {
    int32_t dims[3];
    int32_t nnz;
    int32_t *i, *j, *k;  // nnz each
    float *val;
} ref_coo3;

typedef struct {
    int32_t dims[3];
    int32_t n_i, n_j, n_k;
    int32_t *i_idx;  // n_i
    int32_t *j_ptr;  // n_i + 1
    int32_t *j_idx;  // n_j
    int32_t *k_ptr;  // n_j + 1
    int32_t *k_idx;  // n_k
    float *val;      // n_k
} ref_csf3;

typedef struct {
    int32_t rows, cols;
    int32_t nnz;
    int32_t *i, *j;  // nnz each
    float *val;
} ref_coo;

typedef struct {
    int32_t rows, cols;
    int32_t n_i, nnz;
    int32_t *i_idx;  // n_i: the rows that hold entries
    int32_t *j_ptr;  // n_i + 1
    int32_t *j_idx;  // nnz
    float *val;      // nnz
} ref_dcsr;

int ref_threads(void);
void ref_free(void *p);
void ref_csr_add(const ref_csr *a, const ref_csr *b, ref_csr *z);
void ref_csr_mul(const ref_csr *a, const ref_csr *b, ref_csr *z);
void ref_csr_add_3(const ref_csr *a, const ref_csr *b, const ref_csr *c, ref_csr *z);
void ref_coo3d_add(const ref_coo3 *a, const ref_coo3 *b, ref_coo3 *z);
void ref_csf_add(const ref_csf3 *a, const ref_csf3 *b, ref_csf3 *z);
void ref_coo_add(const ref_coo *a, const ref_coo *b, ref_coo *z);
void ref_coo_mul(const ref_coo *a, const ref_coo *b, ref_coo *z);
void ref_coo_csr_add(const ref_csr *a, const ref_coo *b, ref_csr *z);
void ref_dcsr_add(const ref_dcsr *a, const ref_dcsr *b, ref_dcsr *z);
void ref_dcsr_mul(const ref_dcsr *a, const ref_dcsr *b, ref_dcsr *z);
float ref_inner_prod(const ref_csf3 *a, const ref_csf3 *b);
float ref_inner_prod_coo(const ref_coo3 *a, const ref_coo3 *b);

#ifdef __cplusplus
}
#endif
