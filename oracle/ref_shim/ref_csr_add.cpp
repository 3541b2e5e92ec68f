// Wrapper around the reference's emitted csr_add_cpu_i32_f32 (test infrastructure only).
#include "csr_add_cpu.h"
#include "ref_common.h"

extern "C" void ref_csr_add(const ref_csr *a, const ref_csr *b, ref_csr *z) {
    using namespace csr_add;
    auto Z = csr_add_cpu_i32_f32(csr_view<a_tensor_format<index_t, value_t>>(a),
                              csr_view<b_tensor_format<index_t, value_t>>(b));
    csr_out(Z, z);
}
