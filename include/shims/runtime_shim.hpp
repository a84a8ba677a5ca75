// Reference-side binding of the runtime's QTIP linear operator to libqtip_b200: one forwarding function per declaration
// of the reference's runtime/cuda/kernels.hpp:11-24 and runtime/cuda/batch_kernels.hpp:5-8,22-25 that belongs to the
// trellis-decode path, same names, same argument lists, errors as std::runtime_error like the reference's. A maintainer
// compiles this in place of the definitions in runtime/cuda/kernels.cu / batch_kernels.cu with
// QTIP_B200_SHIM_NAMESPACE set to `behemoth::cuda_runtime`; the signature test of this repository compiles it in a
// namespace of its own and compares every function's type with the reference's declaration.
#pragma once
#include <stdexcept>

#include "../qtip_b200.h"
#include "batch_kernels.hpp"  // reference: QtipMatrix, B16, Stream and the declarations being bound

#ifndef QTIP_B200_SHIM_NAMESPACE
#define QTIP_B200_SHIM_NAMESPACE qtip_b200_shim
#endif

namespace QTIP_B200_SHIM_NAMESPACE {
using ::behemoth::cuda_runtime::B16;
using ::behemoth::cuda_runtime::QtipMatrix;
using ::behemoth::cuda_runtime::Stream;
inline qtip_matrix pod(const QtipMatrix& w) { return qtip_matrix{w.trellis, w.su, w.sv, w.lut, w.in, w.out}; }
inline void qb(int rc) {
  if (rc != 0) throw std::runtime_error(qtip_last_error());
}
inline void initialize_tables() { qb(qtip_init()); }
inline void qtip_prepare(QtipMatrix w, const B16* x, float* scratch, B16* rotated, Stream s, int tokens, bool rank_major) {
  qb(::qtip_prepare(pod(w), reinterpret_cast<const uint16_t*>(x), scratch, reinterpret_cast<uint16_t*>(rotated), s, tokens,
                    rank_major ? 1 : 0));
}
inline void qtip_multiply(QtipMatrix w, const B16* rotated, float* z, int stride, int splits, Stream s, int tokens) {
  qb(::qtip_multiply(pod(w), reinterpret_cast<const uint16_t*>(rotated), z, stride, splits, s, tokens));
}
inline void qtip_finish(QtipMatrix w, const float* z, B16* y, float* scratch, bool round_z, int splits, Stream s, int tokens,
                        bool rank_major) {
  qb(::qtip_finish(pod(w), z, reinterpret_cast<uint16_t*>(y), scratch, round_z ? 1 : 0, splits, s, tokens,
                   rank_major ? 1 : 0));
}
inline void qtip_finish_b16(QtipMatrix w, const B16* z, B16* y, float* scratch, int tokens, Stream s, bool rank_major) {
  qb(::qtip_finish_b16(pod(w), reinterpret_cast<const uint16_t*>(z), reinterpret_cast<uint16_t*>(y), scratch, tokens, s,
                       rank_major ? 1 : 0));
}
inline void qtip_forward(QtipMatrix w, const B16* x, B16* y, float* scratch, B16* rotated, float* z, bool round_z, Stream s,
                         int splits) {
  qb(::qtip_forward(pod(w), reinterpret_cast<const uint16_t*>(x), reinterpret_cast<uint16_t*>(y), scratch,
                    reinterpret_cast<uint16_t*>(rotated), z, round_z ? 1 : 0, s, splits));
}
inline void fp8_forward(const uint8_t* w, const float* scale, const B16* x, B16* y, int in, int out, Stream s) {
  qb(::qtip_fp8_forward(w, scale, reinterpret_cast<const uint16_t*>(x), reinterpret_cast<uint16_t*>(y), in, out, 1, s));
}
inline void qtip_multiply_batch(QtipMatrix w, const B16* x, float* z, int stride, int splits, int tokens, Stream s,
                                int implementation) {
  qb(::qtip_multiply_batch(pod(w), reinterpret_cast<const uint16_t*>(x), z, stride, splits, tokens, s, implementation));
}
inline void qtip_decode_matrix(QtipMatrix w, B16* out, Stream s) {
  qb(::qtip_decode_matrix(pod(w), reinterpret_cast<uint16_t*>(out), s));
}
inline void reduce_products(float* x, size_t elements, int splits, Stream s) { qb(::qtip_reduce_products(x, elements, splits, s)); }
inline void reduce_to_b16(const float* x, const float* scale, B16* y, size_t elements, int width, int splits, Stream s) {
  qb(::qtip_reduce_to_b16(x, scale, reinterpret_cast<uint16_t*>(y), elements, width, splits, s));
}
inline void decode_fp8_matrix(const uint8_t* w, B16* out, size_t elements, Stream s) {
  qb(::qtip_decode_fp8_matrix(w, reinterpret_cast<uint16_t*>(out), elements, s));
}
}  // namespace QTIP_B200_SHIM_NAMESPACE
