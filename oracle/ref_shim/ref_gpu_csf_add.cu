// Wrapper around the reference's emitted csf_add_gpu_i32_f32 (test infrastructure only).
#include "csf_add_gpu.h"
#include "ref_gpu_common.h"

template <typename T>
static T csf3_view(const ref_csf3 *m) {
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

extern "C" int ref_gpu_csf_add(const ref_csf3 *a, const ref_csf3 *b, ref_csf3 *z, int num_blocks, int threads_per_block) {
    using namespace csf_add;
    auto Z = csf_add_gpu_i32_f32(csf3_view<a_tensor_format<index_t, value_t>>(a), csf3_view<b_tensor_format<index_t, value_t>>(b),
                                 num_blocks, threads_per_block);
    z->dims[0] = Z.dim_i_size;
    z->dims[1] = Z.dim_j_size;
    z->dims[2] = Z.dim_k_size;
    z->n_i = Z.dim_i_length;
    z->n_j = Z.dim_j_length;
    z->n_k = Z.dim_k_length;
    z->i_idx = Z.dim_i_indices;
    z->j_ptr = Z.dim_j_offsets;
    z->j_idx = Z.dim_j_indices;
    z->k_ptr = Z.dim_k_offsets;
    z->k_idx = Z.dim_k_indices;
    z->val = Z.values;
    return ref_gpu_finish();
}
