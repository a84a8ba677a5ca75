// Compiled (syntax only) by tests/test_abi.py against the reference's own headers: every forwarding function of
// include/shims/quantizer_shim.hpp must have exactly the type of the reference's declaration it replaces
// (src/gpu.hpp:222-292), so that a drift of either side fails this build.
#include <type_traits>

#include "shims/quantizer_shim.hpp"

#define SAME(f) static_assert(std::is_same_v<decltype(&qtip::f), decltype(&qtip_b200_shim::f)>, #f " differs from src/gpu.hpp")
SAME(k_scale_rows_cols);
SAME(k_scale);
SAME(k_sub);
SAME(k_transpose);
SAME(k_hadamard_rows);
SAME(k_sumsq);
SAME(k_add_diag);
SAME(k_diag_sum);
SAME(k_split_bf16);
SAME(k_diff_split_bf16);
SAME(k_dot);
SAME(k_ldlq_prep);
SAME(k_viterbi_fwd);
SAME(k_viterbi_overlap);
SAME(k_viterbi_finish);
SAME(k_decode_states);
int main() { return 0; }
