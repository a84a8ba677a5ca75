// Reference-side binding of the quantizer's GPU interface to libqtip_b200: one forwarding function per k_* wrapper of the
// reference's src/gpu.hpp:222-292, same names, same argument lists. A maintainer of the reference drops the definitions
// of src/viterbi.hip / src/kernels.hip for these functions and includes this header with QTIP_B200_SHIM_NAMESPACE set to
// `qtip`; the signature test of this repository compiles it in a namespace of its own and compares every function's type
// with the reference's declaration.
#pragma once
#include <string>

#include "../qtip_b200.h"
#include "common.hpp"  // reference: QCHECK / die
#include "gpu.hpp"     // reference: hipStream_t, the declarations being bound

#ifndef QTIP_B200_SHIM_NAMESPACE
#define QTIP_B200_SHIM_NAMESPACE qtip_b200_shim
#endif

namespace QTIP_B200_SHIM_NAMESPACE {
inline void qb(int rc) {
  if (rc != 0) ::qtip::die(std::string("qtip_b200: ") + qtip_last_error());
}
inline void k_scale_rows_cols(float* X, long rows, long cols, long ld, const float* rs, const float* cs, hipStream_t s) {
  qb(qtip_k_scale_rows_cols(X, rows, cols, ld, rs, cs, s));
}
inline void k_scale(float* X, long rows, long cols, long ld, float a, hipStream_t s) { qb(qtip_k_scale(X, rows, cols, ld, a, s)); }
inline void k_sub(const float* A, const float* B, float* D, long rows, long cols, long ld, hipStream_t s) {
  qb(qtip_k_sub(A, B, D, rows, cols, ld, s));
}
inline void k_transpose(const float* in, long rows, long cols, long ld_in, float* out, long ld_out, hipStream_t s) {
  qb(qtip_k_transpose(in, rows, cols, ld_in, out, ld_out, s));
}
inline void k_hadamard_rows(float* X, long rows, int n, long ld, bool transpose, hipStream_t s) {
  qb(qtip_k_hadamard_rows(X, rows, n, ld, transpose ? 1 : 0, s));
}
inline void k_sumsq(const float* X, long rows, long cols, long ld, double* out, hipStream_t s) {
  qb(qtip_k_sumsq(X, rows, cols, ld, out, s));
}
inline void k_add_diag(float* H, long n, float a, hipStream_t s) { qb(qtip_k_add_diag(H, n, a, s)); }
inline void k_diag_sum(const float* H, long n, double* out, hipStream_t s) { qb(qtip_k_diag_sum(H, n, out, s)); }
inline void k_split_bf16(const float* X, long rows, long cols, long ld_in, uint16_t* hi, uint16_t* lo, long ld_out,
                         hipStream_t s) {
  qb(qtip_k_split_bf16(X, rows, cols, ld_in, hi, lo, ld_out, s));
}
inline void k_diff_split_bf16(const float* A, const float* B, long rows, long cols, long ld, uint16_t* hi, uint16_t* lo,
                              long ld_out, hipStream_t s) {
  qb(qtip_k_diff_split_bf16(A, B, rows, cols, ld, hi, lo, ld_out, s));
}
inline void k_dot(const float* A, long lda, const float* B, long ldb, long rows, long cols, double* out, hipStream_t s) {
  qb(qtip_k_dot(A, lda, B, ldb, rows, cols, out, s));
}
inline void k_ldlq_prep(const float* WT, const float* hatWT, const float* prod, const float* L, long n, long m, int col0,
                        int bufend, float* X, hipStream_t s) {
  qb(qtip_k_ldlq_prep(WT, hatWT, prod, L, n, m, col0, bufend, X, s));
}
inline void k_viterbi_fwd(const float* X, const int* overlap, int roll, int B, uint16_t* A, uint16_t* final_state,
                          const uint32_t* lut_h2, hipStream_t s) {
  qb(qtip_k_viterbi_fwd(X, overlap, roll, B, A, final_state, lut_h2, s));
}
inline void k_viterbi_overlap(const uint16_t* A, const uint16_t* final_state, int B, int* overlap, hipStream_t s) {
  qb(qtip_k_viterbi_overlap(A, final_state, B, overlap, s));
}
inline void k_viterbi_finish(const uint16_t* A, const uint16_t* final_state, int B, int b0, uint16_t* Q, int nblk, int blk,
                             float* hatWT, long m, int col0, const uint32_t* lut_h2, hipStream_t s) {
  qb(qtip_k_viterbi_finish(A, final_state, B, b0, Q, nblk, blk, hatWT, m, col0, lut_h2, s));
}
inline void k_decode_states(const uint16_t* states, int B, float* hat, const uint32_t* lut_h2, hipStream_t s) {
  qb(qtip_k_decode_states(states, B, hat, lut_h2, s));
}
}  // namespace QTIP_B200_SHIM_NAMESPACE
