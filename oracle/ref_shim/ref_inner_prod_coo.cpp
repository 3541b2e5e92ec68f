// Wrapper around the reference's emitted inner_prod_coo_cpu_i32_f32 (test infrastructure only).
#include <cstdlib>

#include "inner_prod_coo_cpu.h"
#include "ref_common.h"

extern "C" float ref_inner_prod_coo(const ref_coo3 *a, const ref_coo3 *b) {
    using namespace inner_prod_coo;
    auto Z = inner_prod_coo_cpu_i32_f32(coo3_view_of<a_tensor_format<index_t, value_t>>(a),
                                  coo3_view_of<b_tensor_format<index_t, value_t>>(b));
    const float v = Z.values[0];
    std::free(Z.values);
    return v;
}
