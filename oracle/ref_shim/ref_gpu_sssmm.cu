// Wrapper around the reference's emitted sssmm_gpu_i32_f32 (test infrastructure only).
#include "sssmm_gpu.h"
#include "ref_gpu_common.h"

extern "C" int ref_gpu_sssmm(const ref_csr *a, const ref_csr *b, const ref_csr *c, ref_csr *z, int num_blocks,
                             int threads_per_block) {
    using namespace sssmm;
    auto Z = sssmm_gpu_i32_f32(csr_pos_view<a_tensor_format<index_t, value_t>>(a), csr_pos_view<b_tensor_format<index_t, value_t>>(b),
                               csr_pos_view<c_tensor_format<index_t, value_t>>(c), num_blocks, threads_per_block);
    csr_pos_out(Z, z);
    return ref_gpu_finish();
}
