// TEST INFRASTRUCTURE ONLY -- C-ABI wrappers around the reference's own GPU encode kernels (src/viterbi.hip, CUDA branch
// selected by QTIP_CUDA), compiled from the reference tree where it lies (see Makefile target `refgpu`). The GPU parity
// tests use it to check that this repository's kernels give the same bits as the reference's kernels on the same GPU, and
// the bench reports its rate beside ours. Never part of the product library. Arguments as src/gpu.hpp:276-292; errors
// abort the process (the reference's HIP_CHECK convention).
#include <cstdint>

#include "gpu.hpp"

extern "C" {
void refgpu_ldlq_prep(const float* WT, const float* hatWT, const float* prod, const float* L, long n, long m, int col0,
                      int bufend, float* X, void* s) {
  qtip::k_ldlq_prep(WT, hatWT, prod, L, n, m, col0, bufend, X, static_cast<hipStream_t>(s));
}
void refgpu_viterbi_fwd(const float* X, const int* overlap, int roll, int B, uint16_t* A, uint16_t* final_state,
                        const uint32_t* lut_h2, void* s) {
  qtip::k_viterbi_fwd(X, overlap, roll, B, A, final_state, lut_h2, static_cast<hipStream_t>(s));
}
void refgpu_viterbi_overlap(const uint16_t* A, const uint16_t* final_state, int B, int* overlap, void* s) {
  qtip::k_viterbi_overlap(A, final_state, B, overlap, static_cast<hipStream_t>(s));
}
void refgpu_viterbi_finish(const uint16_t* A, const uint16_t* final_state, int B, int b0, uint16_t* Q, int nblk, int blk,
                           float* hatWT, long m, int col0, const uint32_t* lut_h2, void* s) {
  qtip::k_viterbi_finish(A, final_state, B, b0, Q, nblk, blk, hatWT, m, col0, lut_h2, static_cast<hipStream_t>(s));
}
void refgpu_decode_states(const uint16_t* states, int B, float* hat, const uint32_t* lut_h2, void* s) {
  qtip::k_decode_states(states, B, hat, lut_h2, static_cast<hipStream_t>(s));
}
}
