// Wrapper around the reference's emitted spgemm_gpu_i32_f32 (test infrastructure only).
#include "spgemm_gpu.h"
#include "ref_gpu_common.h"

extern "C" int ref_gpu_spgemm(const ref_csr *a, const ref_csr *b, ref_csr *z, int num_blocks, int threads_per_block) {
    using namespace spgemm;
    auto Z = spgemm_gpu_i32_f32(csr_pos_view<a_tensor_format<index_t, value_t>>(a), csr_pos_view<b_tensor_format<index_t, value_t>>(b),
                              num_blocks, threads_per_block);
    csr_pos_out(Z, z);
    return ref_gpu_finish();
}
