// TEST INFRASTRUCTURE ONLY -- C-ABI wrappers around the reference's own encode-side CPU code (src/qtip_core.cpp),
// compiled from the reference tree where it lies (see Makefile target `ref`). Used to validate the restated oracle
// and as the CPU baseline; never part of the product library.
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "qtip_core.hpp"
#include "safetensors.hpp"

extern "C" {
// codebook(): the reference's committed HYB table. src/qtip_core.cpp:18-50.
void ref_codebook(uint16_t* tlut_h /*1024*/, uint32_t* lut_h2 /*65536*/, double* lut_rms) {
  const qtip::Codebook& cb = qtip::codebook();
  if (tlut_h) std::memcpy(tlut_h, cb.tlut_h, sizeof cb.tlut_h);
  if (lut_h2) std::memcpy(lut_h2, cb.lut_h2.data(), 65536 * 4);
  if (lut_rms) *lut_rms = cb.lut_rms;
}
void ref_perm(int* perm, int* inv) {
  std::memcpy(perm, qtip::perm256(), 256 * sizeof(int));
  std::memcpy(inv, qtip::inv_perm256(), 256 * sizeof(int));
}
int ref_had_K(int n) { return qtip::had_K(n); }
// had_table(K) of src/qtip_constants.hpp; returns 0 if the reference has no table of that order.
int ref_had_table(int K, int8_t* out);
void ref_hadamard_rows(double* X, long rows, int n, long ld, int transpose) {
  qtip::hadamard_rows_ref(X, rows, n, ld, transpose != 0);
}
// quantize_seq_ref over B sequences (OpenMP over sequences). src/qtip_core.cpp:180-191.
void ref_quantize_seqs(const float* X, int B, uint16_t* states, float* hat, double* cost) {
#pragma omp parallel for schedule(dynamic, 1)
  for (int b = 0; b < B; ++b) {
    float h[256];
    double c = qtip::quantize_seq_ref(X + size_t(b) * 256, states + size_t(b) * 128, h);
    if (hat) std::memcpy(hat + size_t(b) * 256, h, sizeof h);
    if (cost) cost[b] = c;
  }
}
double ref_viterbi(const float* X, int overlap, uint16_t* states) { return qtip::viterbi_ref(X, overlap, states); }
double ref_path_cost(const float* X, const uint16_t* states) { return qtip::path_cost(X, states); }
void ref_decode_states(const uint16_t* states, float* hat) { qtip::decode_states(states, hat); }
void ref_pack_trellis(const uint16_t* states, long B, uint16_t* packed) { qtip::pack_trellis(states, B, packed); }
void ref_unpack_trellis(const uint16_t* packed, long B, uint16_t* states) { qtip::unpack_trellis(packed, B, states); }
void ref_swizzle(const uint16_t* packed, int m, int n, uint16_t* out) { qtip::swizzle_for_kernel(packed, m, n, out); }
void ref_unswizzle(const uint16_t* in, int m, int n, uint16_t* packed) { qtip::unswizzle_for_kernel(in, m, n, packed); }
int ref_block_ldl(double* A, int n, float* L, int threads) { return qtip::block_ldl_to_L(A, n, L, threads) ? 0 : -1; }
// One linear's checkpoint tensors through the reference's own container writer (SafeTensorsWriter, src/safetensors.cpp:93-136),
// with the tensor names, dtypes and shapes of write_layer_file (src/pipeline.cpp:329-340). `sv` already holds sign * Wscale.
void ref_write_layer_file(const char* path, int layer, int count, const char* const* names, const int* m, const int* n,
                          const uint16_t* const* trellis, const uint16_t* const* su_bf16, const float* const* sv,
                          const uint16_t* tlut) {
  qtip::SafeTensorsWriter w;
  const int64_t zero = 0, eight = 8;
  for (int i = 0; i < count; ++i) {
    const std::string b = "model.layers." + std::to_string(layer) + "." + names[i] + ".";
    const long tiles = long(m[i] / 16) * (n[i] / 16);
    w.add(b + "trellis", "I16", {tiles, 32}, trellis[i], size_t(tiles) * 64);
    w.add(b + "SU", "BF16", {n[i]}, su_bf16[i], size_t(n[i]) * 2);
    w.add(b + "SV", "F32", {m[i]}, sv[i], size_t(m[i]) * 4);
    w.add(b + "tlut", "F16", {512, 2}, tlut, 2048);
    w.add(b + "rcp", "I64", {}, &zero, 8);
    w.add(b + "tp_rank", "I64", {}, &eight, 8);
  }
  w.write(path);
}
}
