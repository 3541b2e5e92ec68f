/*
 * CPU oracle: a plain-C restatement of the algorithms behind the reference's sparse-kernel
 * hot path (CSR union add, fused 3-operand add, CSR intersection multiply, COO3 / CSF3 tensor
 * add, expand-sort-compress SpGEMM).
 *
 * TEST INFRASTRUCTURE ONLY. The tests, the smoke check and the CPU-baseline leg of the
 * benchmark call this to check the CUDA path; no product code links, loads or calls it.
 *
 * Parity of this restatement is pinned in two ways: (1) against the reference's own emitted
 * CPU kernels (csr_add / csr_add_3 / csr_mul / coo3d_add / csf_add _cpu_i32_f32), built by
 * the `ref` target of the Makefile beside this file and compared bit-for-bit on seeded
 * inputs and on every edge case of the test-suite; (2) against golden vectors produced by
 * those kernels and committed with the tests. SpGEMM has no CPU implementation in the
 * reference (compiler.cpp:145-148 targets the GPU only), so its restatement is pinned
 * against a float64 Gustavson product and the integer pattern product instead.
 *
 * All indices are int32 and all values float32, as in the reference
 * (src/backend/stitch_and_generate.cpp:235-236). Operands must have sorted, duplicate-free
 * columns / coordinates. Explicit zeros are kept in every result.
 *
 * Output arrays are caller-allocated at the stated capacity; every function returns the
 * number of stored entries (or -1 on a bad argument).
 */
#ifndef NACHO_B200_ORACLE_H
#define NACHO_B200_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Union add Z = A + B. Capacity of z_col / z_val: nnz(A) + nnz(B). z_row_ptr: rows + 1.
 * Follows the emitted csr_add kernels: row bisection on summed row offsets
 * (src/backend/partition.cpp:628-811), sorted two-way merge per row with the "both present"
 * branch adding a + b and the tails copying (src/backend/compute.cpp:426-432, 619-1392),
 * count -> serial exclusive prefix -> fill (src/backend/stitch_and_generate_cpu.cpp:156-215). */
int64_t orc_csr_add(int32_t rows, const int32_t *a_row_ptr, const int32_t *a_col,
                    const float *a_val, const int32_t *b_row_ptr, const int32_t *b_col,
                    const float *b_val, int32_t *z_row_ptr, int32_t *z_col, float *z_val,
                    int nthreads);

/* Intersection multiply Z = A .* B. Capacity: min(nnz(A), nnz(B)), at least 1.
 * Same skeleton with only the "both present" branch, value a * b
 * (src/backend/compute.cpp:434-440). An empty result has an all-zero row_ptr
 * (src/backend/stitch_and_generate.cpp:168-220). */
int64_t orc_csr_mul(int32_t rows, const int32_t *a_row_ptr, const int32_t *a_col,
                    const float *a_val, const int32_t *b_row_ptr, const int32_t *b_col,
                    const float *b_val, int32_t *z_row_ptr, int32_t *z_col, float *z_val,
                    int nthreads);

/* Fused three-operand union add Z = (A + B) + C with left-to-right association
 * (src/backend/compute.cpp:426-432). Capacity: nnz(A) + nnz(B) + nnz(C). */
int64_t orc_csr_add3(int32_t rows, const int32_t *a_row_ptr, const int32_t *a_col,
                     const float *a_val, const int32_t *b_row_ptr, const int32_t *b_col,
                     const float *b_val, const int32_t *c_row_ptr, const int32_t *c_col,
                     const float *c_val, int32_t *z_row_ptr, int32_t *z_col, float *z_val,
                     int nthreads);

/* COO3 union add over lexicographically sorted unique (i, j, k) triples: the three levels
 * are flattened into one merged coordinate (src/Compile.cpp:66-154) and compared as tuples
 * (src/backend/tensor.cpp:447-560). Capacity: na + nb. */
int64_t orc_coo3_add(int32_t na, const int32_t *ai, const int32_t *aj, const int32_t *ak,
                     const float *av, int32_t nb, const int32_t *bi, const int32_t *bj,
                     const int32_t *bk, const float *bv, int32_t *zi, int32_t *zj, int32_t *zk,
                     float *zv, int nthreads);

/* CSF3 (three compressed levels) union add: merge the i lists; under equal i merge the j
 * fibres; under equal (i, j) merge k; otherwise copy the subtree
 * (src/backend/compute.cpp:619-1392 emitted three levels deep).
 * Capacities: z_i_idx na_i+nb_i; z_j_ptr that+1; z_j_idx na_j+nb_j; z_k_ptr that+1;
 * z_k_idx / z_val na_k+nb_k. counts[3] receives (n_i, n_j, n_k). Returns n_k. */
int64_t orc_csf3_add(int32_t na_i, const int32_t *a_i_idx, const int32_t *a_j_ptr,
                     const int32_t *a_j_idx, const int32_t *a_k_ptr, const int32_t *a_k_idx,
                     const float *a_val, int32_t nb_i, const int32_t *b_i_idx,
                     const int32_t *b_j_ptr, const int32_t *b_j_idx, const int32_t *b_k_ptr,
                     const int32_t *b_k_idx, const float *b_val, int32_t *z_i_idx,
                     int32_t *z_j_ptr, int32_t *z_j_idx, int32_t *z_k_ptr, int32_t *z_k_idx,
                     float *z_val, int32_t *counts);

/* Expand-sort-compress SpGEMM C = A * B, restating the GPU-only reference path:
 * products a.values[p] * b.values[q] with key k = b.cols[q] in (i, j ascending, k ascending)
 * order (src/backend/compute.cpp:434-440, 526-538), per-row sort by k and sum of equal-k runs
 * with explicit zeros kept and product-free rows left empty
 * (src/backend/stitch_and_generate_gpu.cpp:14-139, 257-363).
 *
 * orc_spgemm_symbolic fills c_row_ptr (rows + 1), stores the product count in *products and
 * returns nnz(C). orc_spgemm_numeric then fills c_col and c_val (float32 sums taken in
 * ascending-j order, one valid order of the reference's order-free atomic sum) and, when
 * non-NULL, c_val64 (float64 sums of float64 products) and c_abs64 (sum of |a*b|, the
 * conditioning bound used by the tolerance test). */
int64_t orc_spgemm_symbolic(int32_t rows, int32_t b_cols, const int32_t *a_row_ptr,
                            const int32_t *a_col, const int32_t *b_row_ptr,
                            const int32_t *b_col, int32_t *c_row_ptr, int64_t *products,
                            int nthreads);
int64_t orc_spgemm_numeric(int32_t rows, int32_t b_cols, const int32_t *a_row_ptr,
                           const int32_t *a_col, const float *a_val, const int32_t *b_row_ptr,
                           const int32_t *b_col, const float *b_val, const int32_t *c_row_ptr,
                           int32_t *c_col, float *c_val, double *c_val64, double *c_abs64,
                           int nthreads);

#ifdef __cplusplus
}
#endif
#endif
