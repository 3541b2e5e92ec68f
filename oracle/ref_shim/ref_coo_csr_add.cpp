// Wrapper around the reference's emitted coo_csr_add_cpu_i32_f32 (test infrastructure only).
#include "coo_csr_add_cpu.h"
#include "ref_common.h"

extern "C" void ref_coo_csr_add(const ref_csr *a, const ref_coo *b, ref_csr *z) {
    using namespace coo_csr_add;
    auto Z = coo_csr_add_cpu_i32_f32(csr_view<a_tensor_format<index_t, value_t>>(a),
                                  coo_view<b_tensor_format<index_t, value_t>>(b));
    csr_out(Z, z);
}
