// Wrapper around the reference's emitted dcsr_add_cpu_i32_f32 (test infrastructure only).
#include "dcsr_add_cpu.h"
#include "ref_common.h"

extern "C" void ref_dcsr_add(const ref_dcsr *a, const ref_dcsr *b, ref_dcsr *z) {
    using namespace dcsr_add;
    auto Z = dcsr_add_cpu_i32_f32(dcsr_view<a_tensor_format<index_t, value_t>>(a),
                                  dcsr_view<b_tensor_format<index_t, value_t>>(b));
    dcsr_out(Z, z);
}
