// Wrapper around the reference's emitted coo3d_add_gpu_i32_f32 (test infrastructure only).
#include "coo3d_add_gpu.h"
#include "ref_gpu_common.h"

template <typename T>
static T coo3_view(const ref_coo3 *m) {
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

extern "C" int ref_gpu_coo3d_add(const ref_coo3 *a, const ref_coo3 *b, ref_coo3 *z, int num_blocks, int threads_per_block) {
    using namespace coo3d_add;
    auto Z = coo3d_add_gpu_i32_f32(coo3_view<a_tensor_format<index_t, value_t>>(a), coo3_view<b_tensor_format<index_t, value_t>>(b),
                                   num_blocks, threads_per_block);
    z->dims[0] = Z.dim_i_size;
    z->dims[1] = Z.dim_j_size;
    z->dims[2] = Z.dim_k_size;
    z->nnz = Z.dim_k_length;
    z->i = Z.dim_i_indices;
    z->j = Z.dim_j_indices;
    z->k = Z.dim_k_indices;
    z->val = Z.values;
    return ref_gpu_finish();
}
