/*
 * nacho_b200 — C ABI of the B200 (sm_100a) sparse-kernel library.
 *
 * Drop-in boundary for the GPU hot path of the nacho sparse tensor algebra compiler: each
 * entry point below stands where one of nacho's emitted host drivers
 * `<kernel>::<kernel>_gpu_i32_f32(a, b[, c], num_blocks, threads_per_block)` stands today
 * (emitter: src/backend/stitch_and_generate_gpu.cpp:142-185, signature
 * src/backend/stitch_and_generate.cpp:278-290), and is what the emitted nanobind wrappers
 * `gpu_<kernel>_f32` (src/backend/generate_bindings.cpp:288-331) would call instead.
 *
 * Conventions shared by every entry point
 *   - All indices are int32 and all values float32 (src/backend/stitch_and_generate.cpp:235-236).
 *   - Every array pointer is a DEVICE pointer on the current CUDA device, 4-byte aligned,
 *     contiguous. Operands are borrowed and never written (runtime/nacho_nb.h:73-78).
 *   - Operands must hold sorted, duplicate-free columns / coordinates, as nacho requires.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream, which is
 *     what nacho's drivers use, src/backend/stitch_and_generate_gpu.cpp:163-167).
 *   - Every call returns an nb200_status; 0 is success. Nothing throws and nothing aborts.
 *   - The calls block the host until the result lengths are known (one small device-to-host
 *     read), like nacho's drivers do; on return the result is complete in stream order.
 *   - num_blocks / threads_per_block are accepted for signature compatibility
 *     (src/backend/generate_bindings.cpp:317-327); the kernels size their own grids, so the
 *     two values are ignored.
 *
 * Two flavours per operator
 *   nb200_<op>_f32       allocates each result array separately with cudaMallocAsync on
 *                        `stream`, so that each can be released independently with
 *                        nb200_free_async (= cudaFreeAsync), the ownership nacho's adopt_gpu
 *                        capsules expect (runtime/nacho_nb.h:50-58,
 *                        runtime/cuda_utils/cuda_utils.cu:7-11). A zero-length array is
 *                        returned as NULL (runtime/nacho_nb.h:37-45).
 *   nb200_<op>_f32_into  writes into caller-owned arrays of a stated capacity (for callers
 *                        whose framework owns device memory, e.g. torch tensors) and reports
 *                        the used lengths. If a capacity is too small the call returns
 *                        NB200_E_CAPACITY with the needed lengths filled in and the value /
 *                        index arrays untouched.
 */
#ifndef NACHO_B200_H
#define NACHO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NB200_VERSION 100

typedef enum nb200_status {
    NB200_OK = 0,
    NB200_E_BADARG = 1,     /* null pointer, negative size, mismatched shapes */
    NB200_E_CUDA = 2,       /* a CUDA runtime call failed; see nb200_last_cuda_error() */
    NB200_E_OVERFLOW = 3,   /* a result length or work count does not fit int32 */
    NB200_E_CAPACITY = 4,   /* caller-provided result arrays are too small */
    NB200_E_TIMEOUT = 5,    /* a bounded device-side wait gave up (no hang, context intact) */
    NB200_E_NOMEM = 6,      /* device allocation failed */
    NB200_E_UNSUPPORTED = 7 /* size beyond a documented limit of the entry point */
} nb200_status;

/* CSR matrix: the field set of nacho's emitted CSR structs
 * {dim_i_size, dim_j_size, dim_j_offsets, dim_j_length, dim_j_indices, values, nnz}
 * (src/backend/tensor.cpp:13-61, include/backend/tensor.h:78-81). */
typedef struct nb200_csr {
    int32_t rows;     /* dim_i_size */
    int32_t cols;     /* dim_j_size */
    int32_t nnz;      /* dim_j_length */
    int32_t *row_ptr; /* dim_j_offsets, rows + 1 entries */
    int32_t *col;     /* dim_j_indices, nnz entries */
    float *val;       /* values, nnz entries */
} nb200_csr;

/* COO3 tensor: three parallel coordinate arrays + values
 * (src/backend/tensor.cpp:13-61 for the Compressed_non_unique, Singleton, Singleton levels of
 * compiler.cpp:60-64). */
typedef struct nb200_coo3 {
    int32_t dims[3];
    int32_t nnz;
    int32_t *i, *j, *k; /* dim_{i,j,k}_indices, nnz entries each */
    float *val;
} nb200_coo3;

/* CSF3 tensor: three compressed levels (compiler.cpp:44-48); the outermost level has no
 * offsets array (src/backend/tensor.cpp:35-39). */
typedef struct nb200_csf3 {
    int32_t dims[3];
    int32_t n_i, n_j, n_k; /* dim_{i,j,k}_length */
    int32_t *i_idx;        /* dim_i_indices, n_i */
    int32_t *j_ptr;        /* dim_j_offsets, n_i + 1 */
    int32_t *j_idx;        /* dim_j_indices, n_j */
    int32_t *k_ptr;        /* dim_k_offsets, n_j + 1 */
    int32_t *k_idx;        /* dim_k_indices, n_k */
    float *val;            /* values, n_k */
} nb200_csf3;

/* 2-D coordinate list: the field set of nacho's emitted COO structs (Compressed_non_unique +
 * Singleton_unique levels, compiler.cpp:50-53): parallel row / column arrays sorted by (i, j). */
typedef struct nb200_coo {
    int32_t rows, cols;
    int32_t nnz;
    int32_t *i, *j; /* dim_{i,j}_indices, nnz entries each */
    float *val;
} nb200_coo;

/* DCSR matrix: both levels compressed (compiler.cpp:38-42): only the rows that hold entries are
 * stored, with their row numbers. */
typedef struct nb200_dcsr {
    int32_t rows, cols;
    int32_t n_i, nnz; /* dim_i_length, dim_j_length */
    int32_t *i_idx;   /* dim_i_indices, n_i */
    int32_t *j_ptr;   /* dim_j_offsets, n_i + 1 */
    int32_t *j_idx;   /* dim_j_indices, nnz */
    float *val;       /* values, nnz */
} nb200_dcsr;

/* ---- library -------------------------------------------------------------------------- */

int nb200_version(void);
const char *nb200_strerror(int status);
/* Text of the last CUDA error seen by the calling thread's most recent failing call; after
 * NB200_E_TIMEOUT, which bounded device-side wait gave up and at which tile. */
const char *nb200_last_cuda_error(void);
/* Release a result array of an allocating entry point: cudaFreeAsync(p, stream); NULL is
 * ignored. Replaces cudaFreeWrapper (runtime/cuda_utils/cuda_utils.cu:7-11). */
int nb200_free_async(void *p, void *stream);
/* Release the per-device scratch pools the library keeps between calls. */
int nb200_release_workspaces(void);
/* Number of kernels this library has launched in this process so far. */
uint64_t nb200_launch_count(void);

/* Per-kernel device timing. While enabled, every kernel launch of the library is bracketed
 * by CUDA events on its stream. nb200_profile_read synchronises those events and reports,
 * for the kernel called `name`, the launches and their summed duration since the last
 * nb200_profile_reset; nb200_profile_names writes a comma-separated list of kernel names. */
int nb200_profile_enable(int on);
int nb200_profile_reset(void);
int nb200_profile_read(const char *name, int64_t *launches, double *total_ms);
int nb200_profile_names(char *buf, size_t buf_len);

/* ---- CSR element-wise ------------------------------------------------------------------- */

/* Z = A + B, sorted union per row; a position present in both holds a + b, explicit zeros
 * are kept. Replaces csr_add::csr_add_gpu_i32_f32 (kernel declared at compiler.cpp:112;
 * partition src/backend/partition.cpp:813-993, count/fill src/backend/compute.cpp:152-411).
 * Result: row_ptr rows+1, col/val nnz. Capacity that always suffices: nnz(A) + nnz(B). */
int nb200_csr_add_f32(const nb200_csr *a, const nb200_csr *b, nb200_csr *z,
                      int32_t num_blocks, int32_t threads_per_block, void *stream);
int nb200_csr_add_f32_into(const nb200_csr *a, const nb200_csr *b, nb200_csr *z,
                           int64_t capacity, void *stream);

/* Z = A + B for callers that must not trigger any device or pinned-host allocation while they
 * run -- code inside a framework's memory-pool callback or an out-of-memory handler, plug-ins
 * living under a fixed memory budget that the host application has already handed out, and
 * latency-critical loops where an allocator call could take a lock or synchronise the device.
 * Has no counterpart in the reference, whose drivers allocate on every call.
 *
 * Same result as nb200_csr_add_f32_into, but the scratch memory of the kernels (tile cuts and
 * the cross-tile counters) is a fixed 1 MiB array inside the library's device image instead of
 * a pool that grows on demand. The call makes no cudaMalloc / cudaFree / cudaHostAlloc and
 * calls no allocating library routine; the caller provides every operand and result array.
 * Limits and rules:
 *   - nnz(A) + nnz(B) may not exceed 32768 tiles' worth of entries (about 159 million);
 *     larger inputs return NB200_E_UNSUPPORTED and nothing is launched.
 *   - `capacity` (entries in z->col / z->val) must be at least nnz(A) + nnz(B); otherwise
 *     NB200_E_CAPACITY. z->row_ptr holds rows + 1 entries.
 *   - The first call on each device looks up the array's device address and raises the
 *     kernel's shared-memory limit; make that first call before any stream capture begins.
 *   - All calls on a device share the one array: it is re-zeroed at the start of each call,
 *     and two calls that overlap on the GPU (different streams, different host threads)
 *     would corrupt each other. Serialise them.
 *   - Launches made here are not counted by nb200_launch_count nor timed by the profile. */
int nb200_csr_add_f32_noalloc(const nb200_csr *a, const nb200_csr *b, nb200_csr *z,
                              int64_t capacity, void *stream);

/* Asynchronous forms of add and multiply: like the _into forms with a capacity of at least the
 * worst case (nnz(A) + nnz(B) for add, min(nnz(A), nnz(B)) for multiply; less returns
 * NB200_E_CAPACITY), but the call returns as soon as its kernels are queued. The result length and
 * the device-side status arrive, in stream order, in three int64 DEVICE words:
 * device_result[0] = nnz(Z), device_result[1] = an nb200_status (NB200_OK, NB200_E_TIMEOUT or
 * NB200_E_OVERFLOW), device_result[2] = the row count (so that the three words are a row block's
 * whole contribution to a stitch and can be all-gathered as they are). z->nnz is left 0. For callers that consume the length on the device -- a
 * multi-GPU stitch that all-gathers the block lengths, a pipeline that launches the next operator
 * from the same stream -- and must not stall the host once per call. The reference has no
 * counterpart: its drivers read every length back (src/backend/stitch_and_generate_gpu.cpp:660-671). */
int nb200_csr_add_f32_async(const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int64_t capacity,
                            int64_t *device_result, void *stream);
int nb200_csr_mul_f32_async(const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int64_t capacity,
                            int64_t *device_result, void *stream);

/* Z = A .* B, sorted intersection per row, value a * b. Replaces
 * csr_mul::csr_mul_gpu_i32_f32 (compiler.cpp:116; src/backend/compute.cpp:434-440). An empty
 * result has an all-zero row_ptr (src/backend/stitch_and_generate.cpp:168-220).
 * Capacity that always suffices: min(nnz(A), nnz(B)). */
int nb200_csr_mul_f32(const nb200_csr *a, const nb200_csr *b, nb200_csr *z,
                      int32_t num_blocks, int32_t threads_per_block, void *stream);
int nb200_csr_mul_f32_into(const nb200_csr *a, const nb200_csr *b, nb200_csr *z,
                           int64_t capacity, void *stream);

/* Host-buffer forms of add and multiply: every pointer in a, b and z is a HOST pointer (pinned
 * memory gives full PCIe speed; pageable memory works but copies synchronously). The matrices
 * are streamed through the current device in row blocks of about 12 M operand entries on three
 * internal streams, so that the upload of one block, the merge of the previous one and the
 * download of the one before overlap. z->row_ptr (rows + 1), z->col and z->val (`capacity`
 * entries each) are the caller's; on return z->nnz is the result length and the arrays are
 * complete (the call synchronises its own streams). NB200_E_CAPACITY if the result does not fit.
 * Calls on one device take turns (the library holds a per-device lock for the whole call); on any
 * error return the call has first waited for every copy it had queued, so the host buffers are no
 * longer read or written once it is back.
 * The reference has no counterpart: its operators take device tensors only. */
int nb200_csr_add_f32_host(const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int64_t capacity);
int nb200_csr_mul_f32_host(const nb200_csr *a, const nb200_csr *b, nb200_csr *z, int64_t capacity);

/* Z = (A + B) + C, left-to-right association, in one call. Replaces
 * csr_add_3::csr_add_3_gpu_i32_f32 (compiler.cpp:114; src/backend/compute.cpp:426-432).
 * Capacity that always suffices: nnz(A) + nnz(B) + nnz(C). */
int nb200_csr_add_3_f32(const nb200_csr *a, const nb200_csr *b, const nb200_csr *c,
                        nb200_csr *z, int32_t num_blocks, int32_t threads_per_block,
                        void *stream);
int nb200_csr_add_3_f32_into(const nb200_csr *a, const nb200_csr *b, const nb200_csr *c,
                             nb200_csr *z, int64_t capacity, void *stream);

/* ---- SpGEMM ----------------------------------------------------------------------------- */

/* C = A * B by expand-sort-compress; columns sorted per row, explicit zeros kept, rows
 * without products empty. Replaces spgemm::spgemm_gpu_i32_f32 (compiler.cpp:145-148;
 * expand src/backend/compute.cpp:526-611, sort/compress
 * src/backend/stitch_and_generate_gpu.cpp:14-139,257-363). Unlike the reference, product
 * counts are 64-bit (a product count above 2^31 is fine as long as nnz(C) fits int32) and
 * rows with at most 256 products sum equal-column products in a fixed order (ascending j);
 * longer rows accumulate with float32 atomics (as the reference does for every row). No
 * product is written to device memory; scratch is a few int32 per row, plus, for matrices wider
 * than 262144 columns, a pointer table of one int32 per row of B and 262144 columns of width. */
int nb200_spgemm_f32(const nb200_csr *a, const nb200_csr *b, nb200_csr *c, int32_t num_blocks,
                     int32_t threads_per_block, void *stream);
/* Two-step form for caller-owned memory: _symbolic fills c->row_ptr (rows + 1, caller-owned)
 * and c->nnz; the caller then provides col/val of c->nnz entries to _numeric.
 * `products` (may be NULL) receives the number of scalar products. A _numeric call that follows
 * a _symbolic call on the same arrays, device and stream, with no other call of this library on
 * that stream in between, reuses what _symbolic left in the scratch pool (row bins and the column
 * bitmaps of the long rows, up to 8 GiB) instead of computing it again; any other order of calls
 * is equally valid and recomputes. That reuse assumes the patterns of A and B (row offsets and
 * columns) are unchanged between the two calls -- their values may differ -- and that c->row_ptr is
 * the array _symbolic filled; a caller that rewrites a pattern in place must call _symbolic again. */
int nb200_spgemm_f32_symbolic(const nb200_csr *a, const nb200_csr *b, nb200_csr *c,
                              int64_t *products, void *stream);
int nb200_spgemm_f32_numeric(const nb200_csr *a, const nb200_csr *b, nb200_csr *c,
                             void *stream);

/* Masked SpGEMM: Z_ik = sum_j a_ij * b_jk * c_ik on the positions the mask C stores and at least
 * one product reaches (explicit zeros kept, columns in C's order). Replaces
 * sssmm::sssmm_gpu_i32_f32 (compiler.cpp:150-153). The mask drives the accumulation: every product
 * looks its column up in C's row and is added -- as (a * b) * c, the reference's expression -- to
 * that position or dropped, so nothing outside the mask is formed; float32 atomics in arrival
 * order, as the reference's compress. z->row_ptr holds rows(A) + 1 entries; `capacity` entries in
 * z->col / z->val, nnz(C) always suffices (less returns NB200_E_CAPACITY with z->nnz filled in).
 * Scratch: 8 bytes per entry of C. */
int nb200_sssmm_f32_into(const nb200_csr *a, const nb200_csr *b, const nb200_csr *c, nb200_csr *z,
                         int64_t capacity, void *stream);

/* ---- 3-mode tensor add ------------------------------------------------------------------ */

/* Z = A + B over lexicographically sorted unique (i, j, k). Replaces
 * coo3d_add::coo3d_add_gpu_i32_f32 (compiler.cpp:138; merged coordinate level
 * src/Compile.cpp:66-154). Capacity that always suffices: nnz(A) + nnz(B). */
int nb200_coo3d_add_f32(const nb200_coo3 *a, const nb200_coo3 *b, nb200_coo3 *z,
                        int32_t num_blocks, int32_t threads_per_block, void *stream);
int nb200_coo3d_add_f32_into(const nb200_coo3 *a, const nb200_coo3 *b, nb200_coo3 *z,
                             int64_t capacity, void *stream);

/* Z = A + B for CSF3 operands. Replaces csf_add::csf_add_gpu_i32_f32 (compiler.cpp:135).
 * Capacities that always suffice (for _into): i_idx n_i(A)+n_i(B); j_ptr that + 1;
 * j_idx n_j(A)+n_j(B); k_ptr that + 1; k_idx / val n_k(A)+n_k(B). The _into form takes the
 * three capacities (entries of i_idx, j_idx, k_idx); j_ptr / k_ptr must hold one entry more
 * than cap_i / cap_j, and cap_k must be at least n_k(A)+n_k(B) (the merge works in place in
 * the result's k_idx / val arrays). Any extents up to 2^31 - 1 per mode work, here and for COO3:
 * coordinates that fit 63 bits together are merged as packed 64-bit keys, wider ones as
 * (i, j) / k word pairs (the reference's three-int32 tuple compare, src/backend/tensor.cpp:447-560). */
int nb200_csf_add_f32(const nb200_csf3 *a, const nb200_csf3 *b, nb200_csf3 *z,
                      int32_t num_blocks, int32_t threads_per_block, void *stream);
int nb200_csf_add_f32_into(const nb200_csf3 *a, const nb200_csf3 *b, nb200_csf3 *z,
                           int64_t cap_i, int64_t cap_j, int64_t cap_k, void *stream);

/* ---- the rest of the element-wise family, and the inner products ------------------------- */

/* The kernels nacho declares beside the six above over 2-D coordinate lists and doubly compressed
 * rows (compiler.cpp:118-126) and the two full reductions (compiler.cpp:141-143), in the
 * caller-owned-memory form only. Results are bit-identical to nacho's CPU kernels: sorted union /
 * intersection, explicit zeros kept.
 *   coo_add / coo_mul    Z = A (+|.*) B over sorted unique (i, j) lists; `capacity` entries in
 *                        z->i / z->j / z->val (always enough: nnz(A)+nnz(B), min(nnz(A), nnz(B))).
 *   coo_csr_add          Z = A + B with A in CSR and B a coordinate list; Z in CSR.
 *   dcsr_add / dcsr_mul  DCSR operands and result. `cap_i` entries in z->i_idx (z->j_ptr one more)
 *                        must cover the worst case, min(n_i(A)+n_i(B), rows) for the sum and
 *                        min(n_i(A), n_i(B)) for the product; `capacity` as for CSR. The product
 *                        keeps every row that BOTH operands store, with an empty column range where
 *                        their columns do not meet, as nacho's level-by-level intersection does.
 * These run the CSR merge kernels on the operands' own column / value arrays after rebuilding the
 * row offsets, so they need scratch of a few int32 per matrix ROW (not per stored row). */
int nb200_coo_add_f32_into(const nb200_coo *a, const nb200_coo *b, nb200_coo *z, int64_t capacity, void *stream);
int nb200_coo_mul_f32_into(const nb200_coo *a, const nb200_coo *b, nb200_coo *z, int64_t capacity, void *stream);
int nb200_coo_csr_add_f32_into(const nb200_csr *a, const nb200_coo *b, nb200_csr *z, int64_t capacity, void *stream);
int nb200_dcsr_add_f32_into(const nb200_dcsr *a, const nb200_dcsr *b, nb200_dcsr *z, int64_t cap_i, int64_t capacity,
                            void *stream);
int nb200_dcsr_mul_f32_into(const nb200_dcsr *a, const nb200_dcsr *b, nb200_dcsr *z, int64_t cap_i, int64_t capacity,
                            void *stream);

/* z[0] = sum over the coordinates both tensors hold of a * b, one float32 in DEVICE memory (nacho
 * returns a one-element tensor). Replaces inner_prod::inner_prod_gpu_i32_f32 (CSF3 operands) and
 * inner_prod_coo::inner_prod_coo_gpu_i32_f32 (COO3 operands); append-reduction
 * src/backend/compute.cpp:498-525. Each product is a float32 multiply as in nacho; the products
 * are summed in double and rounded once, where nacho adds float32 atomically in arrival order, so
 * the two agree to float32 rounding of the sum, not bit for bit. Extents must pack into 63 bits. */
int nb200_inner_prod_f32(const nb200_csf3 *a, const nb200_csf3 *b, float *z, void *stream);
int nb200_inner_prod_coo_f32(const nb200_coo3 *a, const nb200_coo3 *b, float *z, void *stream);

/* ---- self-test -------------------------------------------------------------------------- */

/* Exercises the give-up path of the bounded device-side waits without faulting or hanging the
 * GPU: runs the single-pass CSR add on (a, b) WITHOUT its first tile and with a look-back limit of
 * `polls` polls, so that the second tile waits for a count nobody publishes, gives up, records it
 * and lets its successors through. Needs operands of at least three tiles (a few thousand entries
 * each); `capacity` >= nnz(A) + nnz(B). Returns NB200_E_TIMEOUT when the path works (the contents
 * of z are then meaningless, but every write stayed inside its arrays); the context stays usable.
 * Has no counterpart in the reference, which has no device-side waits. */
int nb200_selftest_lookback_timeout(const nb200_csr *a, const nb200_csr *b, nb200_csr *z,
                                    int64_t capacity, int32_t polls, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* NACHO_B200_H */
