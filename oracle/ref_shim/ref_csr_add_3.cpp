// Wrapper around the reference's emitted csr_add_3_cpu_i32_f32 (test infrastructure only).
#include "csr_add_3_cpu.h"
#include "ref_common.h"

extern "C" void ref_csr_add_3(const ref_csr *a, const ref_csr *b, const ref_csr *c, ref_csr *z) {
    using namespace csr_add_3;
    auto Z = csr_add_3_cpu_i32_f32(csr_view<a_tensor_format<index_t, value_t>>(a),
                                   csr_view<b_tensor_format<index_t, value_t>>(b),
                                   csr_view<c_tensor_format<index_t, value_t>>(c));
    csr_out(Z, z);
}
