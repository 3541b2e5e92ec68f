// Wrapper around the reference's emitted coo_mul_cpu_i32_f32 (test infrastructure only).
#include "coo_mul_cpu.h"
#include "ref_common.h"

extern "C" void ref_coo_mul(const ref_coo *a, const ref_coo *b, ref_coo *z) {
    using namespace coo_mul;
    auto Z = coo_mul_cpu_i32_f32(coo_view<a_tensor_format<index_t, value_t>>(a),
                                  coo_view<b_tensor_format<index_t, value_t>>(b));
    coo_out(Z, z);
}
