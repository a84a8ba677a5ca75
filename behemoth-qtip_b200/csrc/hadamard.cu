// Random-Hadamard transforms x <- (hadK^(T) (x) H_P) x / sqrt(n), n = K * P, K in {1, 12, 20, 28}, P a power of two.
//
// (hadK (x) H_P) = (I (x) H_P)(hadK (x) I): the order-K mix across the K chunks is done first, then a natural-order
// fast Walsh-Hadamard transform on each chunk of P. Every variant below uses that order and the same summation order,
// so the whole-row kernel and the chunk-per-CTA kernel give identical bits.
//
//  * had_row_kernel: one CTA per row, the whole row (up to 57,344 floats = 224 KiB) in shared memory, read and written
//    once. Used for the quantizer's fp32 matrices and for prefill-sized token batches.
//  * had_chunk_kernel: K CTAs per row, each mixing its own chunk from the full row (served by L2) and transforming it.
//    No inter-CTA step; used for a few tokens where latency, not traffic, decides.
//
// Sources/destinations (Mode): fp32 in place (quantizer); bf16 x times SU -> bf16 (operator input); fp32 partial
// products summed over K-splits, optionally rounded to bf16 -> times SV -> bf16 (operator output); bf16 z -> same.
#include "hadamard.cuh"

namespace qb {

int epilogue_residual_device_setup();   // epilogue_residual.cu
int epilogue_gateup_device_setup();  // epilogue_gateup.cu

template <int K, bool T>
static int configure_modes() {
  int rc;
  if ((rc = configure<K, T, Mode::F32Inplace>())) return rc;
  if ((rc = configure<K, T, Mode::Prepare>())) return rc;
  if ((rc = configure<K, T, Mode::Finish>())) return rc;
  return configure<K, T, Mode::FinishB16>();
}
int hadamard_device_setup() {
  int rc;
  if ((rc = configure_modes<1, false>())) return rc;
  if ((rc = configure_modes<12, false>()) || (rc = configure_modes<12, true>())) return rc;
  if ((rc = configure_modes<20, false>()) || (rc = configure_modes<20, true>())) return rc;
  if ((rc = configure_modes<28, false>()) || (rc = configure_modes<28, true>())) return rc;
  if ((rc = epilogue_residual_device_setup()) || (rc = epilogue_gateup_device_setup())) return rc;
  return QTIP_OK;
}

// Operator-side entry points used by decode.cu. ranks: 0/1 = row-major source, R >= 2 = gathered [rank][row][n/R].
int hadamard_prepare(const uint16_t* x, const float* su, uint16_t* rotated, int n, int tokens, int ranks,
                     cudaStream_t s) {
  HadArgs a{};
  a.src = x, a.dst = rotated, a.sign = su, a.ld = n, a.n = n, a.splits = 1, a.ranks = ranks;
  return dispatch<Mode::Prepare>(a, tokens, true, false, s);
}
int hadamard_finish(const float* z, const float* sv, uint16_t* y, int n, int tokens, int splits, long split_stride,
                    int round_z, int ranks, cudaStream_t s) {
  HadArgs a{};
  a.src = z, a.dst = y, a.sign = sv, a.ld = n, a.n = n, a.splits = splits, a.split_stride = split_stride;
  a.round_z = round_z, a.ranks = ranks;
  return dispatch<Mode::Finish>(a, tokens, false, false, s);
}
int hadamard_finish_b16(const uint16_t* z, const float* sv, uint16_t* y, int n, int tokens, int ranks, cudaStream_t s) {
  HadArgs a{};
  a.src = z, a.dst = y, a.sign = sv, a.ld = n, a.n = n, a.splits = 1, a.ranks = ranks;
  return dispatch<Mode::FinishB16>(a, tokens, false, false, s);
}


}  // namespace qb

using namespace qb;

extern "C" int qtip_k_hadamard_rows(float* X_d, long rows, int n, long ld, int transpose, void* stream) {
  QB_REQUIRE(X_d && rows >= 0 && n > 0 && ld >= n, QTIP_E_ARG, "qtip_k_hadamard_rows: bad argument");
  if (!device_info()) return QTIP_E_DEVICE;
  HadArgs a{};
  a.src = X_d, a.dst = X_d, a.ld = ld, a.n = n, a.splits = 1;
  return dispatch<Mode::F32Inplace>(a, rows, transpose != 0, true, as_stream(stream));
}
