// Wrapper around the reference's emitted csr_mul_cpu_i32_f32 (test infrastructure only).
#include "csr_mul_cpu.h"
#include "ref_common.h"

extern "C" void ref_csr_mul(const ref_csr *a, const ref_csr *b, ref_csr *z) {
    using namespace csr_mul;
    auto Z = csr_mul_cpu_i32_f32(csr_view<a_tensor_format<index_t, value_t>>(a),
                              csr_view<b_tensor_format<index_t, value_t>>(b));
    csr_out(Z, z);
}
