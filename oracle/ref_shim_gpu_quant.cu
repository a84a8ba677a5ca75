// TEST INFRASTRUCTURE ONLY -- C-ABI wrappers around the reference's own GPU quantizer (src/quantizer.cpp: ldlq_gpu,
// rotate_hessian / ldl_hessian / quantize_group, with its kernels src/kernels.hip and src/viterbi.hip and its library
// GEMM wrapper src/gemm.cpp), compiled from the reference tree where it lies (Makefile target `refquant`). The GPU parity
// tests compare this repository's LDLQ and group quantizer with it on the same inputs, and the bench reports its time
// beside ours. Never part of the product library. Errors abort the process (the reference's QCHECK convention).
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "quantizer.hpp"

extern "C" {
// ldlq_gpu (src/quantizer.cpp:30-89) on device buffers; the reference's compiled-in codebook.
void refq_ldlq_gpu(const float* WT, const float* L, long n, long m, float* hatWT, uint16_t* Q, int vit_batch,
                   double* vit_seconds, void* s) {
  qtip::Gemm gemm(static_cast<hipStream_t>(s));
  qtip::ldlq_gpu(static_cast<hipStream_t>(s), gemm, WT, L, n, m, hatWT, Q, vit_batch, qtip::device_lut(), vit_seconds);
}
// quantize_group (src/quantizer.cpp:166-346) for `count` dense fp32 linears [m_i][n] sharing the Hessian H [n][n], all on
// the HOST. Outputs, per linear, into caller-sized host arrays: trellis (m/16)(n/16)*32 words, su (bf16 bits, n), sv (m),
// wscale, proxy, proxy_rot_reg; timing[8] = GroupTiming fields in declaration order.
void refq_quantize_group(int count, const int* m, const float* const* W, int n, const float* H, uint64_t seed,
                         double sigma_reg, double scale_override, int ldl_threads, uint16_t* const* trellis,
                         uint16_t* const* su_bf16, float* const* sv, float* wscale, double* proxy, double* proxy_rot_reg,
                         double* timing, void* s) {
  qtip::Gemm gemm(static_cast<hipStream_t>(s));
  std::vector<qtip::LinearIn> lins(static_cast<size_t>(count));
  for (int i = 0; i < count; ++i) {
    lins[size_t(i)].name = "linear" + std::to_string(i);
    lins[size_t(i)].m = m[i];
    lins[size_t(i)].w_f32 = W[i];
  }
  qtip::QuantOpts opt;
  opt.sigma_reg = sigma_reg;
  opt.scale_override = scale_override;
  opt.ldl_threads = ldl_threads;
  qtip::GroupTiming tm;
  std::vector<qtip::LinearOut> out = qtip::quantize_group(static_cast<hipStream_t>(s), gemm, lins, n, H, seed, opt, &tm, "test");
  for (int i = 0; i < count; ++i) {
    const qtip::LinearOut& o = out[size_t(i)];
    std::memcpy(trellis[i], o.trellis.data(), o.trellis.size() * 2);
    std::memcpy(su_bf16[i], o.su_bf16.data(), o.su_bf16.size() * 2);
    std::memcpy(sv[i], o.sv.data(), o.sv.size() * 4);
    wscale[i] = o.wscale, proxy[i] = o.proxy, proxy_rot_reg[i] = o.proxy_rot_reg;
  }
  if (timing) {
    const double t[8] = {tm.load, tm.rht, tm.ldl_cpu, tm.ldlq, tm.viterbi, tm.proxy, tm.pack, tm.total};
    std::memcpy(timing, t, sizeof t);
  }
}
}
