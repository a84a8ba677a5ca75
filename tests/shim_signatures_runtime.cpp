// Compiled (syntax only) by tests/test_abi.py against the reference's own headers: every forwarding function of
// include/shims/runtime_shim.hpp must have exactly the type of the reference's declaration it replaces
// (runtime/cuda/kernels.hpp, runtime/cuda/batch_kernels.hpp), and qtip_matrix must be laid out like QtipMatrix.
#include <cstddef>
#include <type_traits>

#include "shims/runtime_shim.hpp"

namespace rt = behemoth::cuda_runtime;
#define SAME(f) static_assert(std::is_same_v<decltype(&rt::f), decltype(&qtip_b200_shim::f)>, #f " differs from the reference's header")
SAME(initialize_tables);
SAME(qtip_prepare);
SAME(qtip_multiply);
SAME(qtip_finish);
SAME(qtip_finish_b16);
SAME(qtip_forward);
SAME(fp8_forward);
SAME(qtip_multiply_batch);
SAME(qtip_decode_matrix);
SAME(reduce_products);
SAME(reduce_to_b16);
SAME(decode_fp8_matrix);
static_assert(sizeof(qtip_matrix) == sizeof(rt::QtipMatrix) && offsetof(qtip_matrix, trellis) == offsetof(rt::QtipMatrix, trellis) &&
                  offsetof(qtip_matrix, su) == offsetof(rt::QtipMatrix, su) && offsetof(qtip_matrix, sv) == offsetof(rt::QtipMatrix, sv) &&
                  offsetof(qtip_matrix, lut) == offsetof(rt::QtipMatrix, lut) && offsetof(qtip_matrix, in) == offsetof(rt::QtipMatrix, in) &&
                  offsetof(qtip_matrix, out) == offsetof(rt::QtipMatrix, out),
              "qtip_matrix is not laid out like QtipMatrix");
static_assert(sizeof(rt::B16) == sizeof(uint16_t), "B16 is not a 16-bit type");
int main() { return 0; }
