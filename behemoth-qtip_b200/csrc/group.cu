// quantize_group of the reference (src/quantizer.cpp:166-346) on device buffers: several linears that share one input
// Hessian -- hence one SU, one L -- are rotated into ONE transposed matrix WT [n][mt] (mt = sum of their rows), quantised
// by one LDLQ + Viterbi run over all mt rows (every column step then carries mt / 16 sequences), scored with the
// proxy error tr(D HR D^T) / tr(W HR W^T), and packed into the checkpoint layout, linear by linear.
//
// The proxy traces follow the reference's scheme (src/quantizer.cpp:90-109,272-301): fp32 operands are split into bf16
// hi + lo, three of the four partial products are kept (hi hi + hi lo + lo hi) by concatenating along K, and the
// product runs on the tensor cores with fp32 accumulation -- here through this library's tcgen05 GEMM
// (qtip_prefill_gemm) instead of a vendor GEMM. Y = X HR for a chunk X of rotated weight rows, then <X, Y> in fp64.
#include <cmath>

#include "common.cuh"

namespace qb {

static size_t align256g(size_t x) { return (x + 255) / 256 * 256; }
constexpr long kProxyChunk = 2048;  // rotated weight rows per trace product

struct GroupLayout {
  size_t ldlq, packed, hcat, dt, xt, xcat, y, acc, total;
};
static GroupLayout group_layout(long n, long mt, long m_max) {
  GroupLayout g;
  const long mc = m_max < kProxyChunk ? m_max : kProxyChunk;
  g.ldlq = qtip_ldlq_workspace_bytes(n, mt);
  g.packed = align256g(size_t(m_max / 16) * (n / 16) * 32 * 2);
  g.hcat = align256g(size_t(n) * 3 * n * 2);
  g.dt = align256g(size_t(n) * mt * 4);
  g.xt = align256g(size_t(mc) * n * 4);
  g.xcat = align256g(size_t(mc) * 3 * n * 2);
  g.y = align256g(size_t(mc) * n * 4);
  g.acc = 256;
  g.total = g.ldlq + g.packed + g.hcat + g.dt + g.xt + g.xcat + g.y + g.acc;
  return g;
}

// tr(X HR X^T) for the rotated weight rows held as columns [c0, c0 + mc) of XT [n][ld]: transpose the chunk to rows,
// split, one K-concatenated tensor-core product, fp64 dot. Synchronises the stream (the value is returned to the host).
static int quad_trace(const float* XT, long n, long ld, long c0, long mc, const uint16_t* hcat, float* xt, uint16_t* xcat,
                      float* y, double* acc, int* status, cudaStream_t s, double* out) {
  void* st = s;
  int rc;
  if ((rc = qtip_k_transpose(XT + c0, n, mc, ld, xt, n, st))) return rc;                       // xt [mc][n]
  if ((rc = qtip_k_split_bf16(xt, mc, n, n, xcat, xcat + 2 * n, 3 * n, st))) return rc;         // [hi | . | lo]
  if ((rc = qtip_k_split_bf16(xt, mc, n, n, xcat + n, nullptr, 3 * n, st))) return rc;          // [hi | hi | lo]
  if ((rc = qtip_prefill_gemm(hcat, xcat, y, int(n), int(3 * n), int(n), int(mc), status, st))) return rc;  // y [mc][n]
  QB_CUDA(cudaMemsetAsync(acc, 0, sizeof(double), s));
  if ((rc = qtip_k_dot(xt, n, y, n, mc, n, acc, st))) return rc;
  QB_CUDA(cudaMemcpyAsync(out, acc, sizeof(double), cudaMemcpyDeviceToHost, s));
  QB_CUDA(cudaStreamSynchronize(s));
  return QTIP_OK;
}
static int sumsq_sync(const float* X, long rows, long cols, long ld, double* acc, cudaStream_t s, double* out) {
  QB_CUDA(cudaMemsetAsync(acc, 0, sizeof(double), s));
  int rc = qtip_k_sumsq(X, rows, cols, ld, acc, s);
  if (rc) return rc;
  QB_CUDA(cudaMemcpyAsync(out, acc, sizeof(double), cudaMemcpyDeviceToHost, s));
  QB_CUDA(cudaStreamSynchronize(s));
  return QTIP_OK;
}

}  // namespace qb

using namespace qb;

extern "C" size_t qtip_quantize_group_workspace_bytes(long n, long mt, long m_max) {
  if (n <= 0 || mt <= 0 || m_max <= 0 || m_max > mt) return 0;
  return group_layout(n, mt, m_max).total;
}

extern "C" int qtip_quantize_group(qtip_group_linear* lins, int count, long n, const float* HR_d, const float* L_d,
                                   const float* su_d, double creg, const uint32_t* lut_h2_d, double lut_rms,
                                   double scale_override, float* WT_d, float* hatWT_d, uint16_t* Q_d, void* workspace_d,
                                   size_t workspace_bytes, void* stream) {
  QB_REQUIRE(lins && count >= 1 && HR_d && L_d && su_d && lut_h2_d && WT_d && hatWT_d && Q_d && workspace_d, QTIP_E_ARG,
             "qtip_quantize_group: null pointer or empty group");
  QB_REQUIRE(n > 0 && n % 128 == 0, QTIP_E_GEOMETRY, "qtip_quantize_group needs n %% 128 == 0 (n = %ld)", n);
  QB_REQUIRE(lut_rms > 0 && scale_override > 0, QTIP_E_ARG, "qtip_quantize_group: lut_rms and scale_override must be > 0");
  long mt = 0, m_max = 0;
  for (int i = 0; i < count; ++i) {
    QB_REQUIRE(lins[i].W_d && lins[i].sv_d && lins[i].trellis_d, QTIP_E_ARG, "qtip_quantize_group: linear %d has a null pointer", i);
    QB_REQUIRE(lins[i].m > 0 && lins[i].m % 32 == 0, QTIP_E_GEOMETRY, "qtip_quantize_group: linear %d has m = %ld (needs m %% 32 == 0)", i,
               lins[i].m);
    mt += lins[i].m;
    m_max = lins[i].m > m_max ? lins[i].m : m_max;
  }
  const GroupLayout g = group_layout(n, mt, m_max);
  QB_REQUIRE(workspace_bytes >= g.total, QTIP_E_WORKSPACE, "qtip_quantize_group: workspace of %zu bytes is too small (need %zu)",
             workspace_bytes, g.total);
  if (!device_info()) return QTIP_E_DEVICE;
  unsigned char* p = static_cast<unsigned char*>(workspace_d);
  uint16_t* packed = reinterpret_cast<uint16_t*>(p + g.ldlq);
  uint16_t* hcat = reinterpret_cast<uint16_t*>(p + g.ldlq + g.packed);
  float* DT = reinterpret_cast<float*>(p + g.ldlq + g.packed + g.hcat);
  float* xt = reinterpret_cast<float*>(p + g.ldlq + g.packed + g.hcat + g.dt);
  uint16_t* xcat = reinterpret_cast<uint16_t*>(p + g.ldlq + g.packed + g.hcat + g.dt + g.xt);
  float* y = reinterpret_cast<float*>(p + g.ldlq + g.packed + g.hcat + g.dt + g.xt + g.xcat);
  double* acc = reinterpret_cast<double*>(p + g.ldlq + g.packed + g.hcat + g.dt + g.xt + g.xcat + g.y);
  int* gemm_status = reinterpret_cast<int*>(acc + 1);
  cudaStream_t s = as_stream(stream);
  int rc;

  // ---- weights -> Wr^T (n x mt), each linear's column block divided by its Wscale (src/quantizer.cpp:236-250)
  long off = 0;
  for (int i = 0; i < count; ++i) {
    qtip_group_linear& l = lins[i];
    float* wt = WT_d + off;
    if ((rc = qtip_k_scale_rows_cols(l.W_d, l.m, n, n, l.sv_d, su_d, stream))) return rc;
    if ((rc = qtip_k_hadamard_rows(l.W_d, l.m, int(n), n, 1, stream))) return rc;
    if ((rc = qtip_k_transpose(l.W_d, l.m, n, n, wt, mt, stream))) return rc;
    if ((rc = qtip_k_hadamard_rows(wt, n, int(l.m), mt, 1, stream))) return rc;
    double ss = 0;
    if ((rc = sumsq_sync(wt, n, l.m, mt, acc, s, &ss))) return rc;
    const double rms = std::sqrt(ss / (double(n) * double(l.m)));
    l.wscale = float(rms / (double(float(lut_rms)) * scale_override));
    QB_REQUIRE(l.wscale > 0 && std::isfinite(l.wscale), QTIP_E_ARG, "qtip_quantize_group: linear %d has rotated rms %g", i, rms);
    if ((rc = qtip_k_scale(wt, n, l.m, mt, float(1.0 / double(l.wscale)), stream))) return rc;
    off += l.m;
  }

  // ---- LDLQ + Viterbi over all rows at once (src/quantizer.cpp:258-267)
  if ((rc = qtip_ldlq(WT_d, L_d, n, mt, 0, mt, hatWT_d, Q_d, lut_h2_d, workspace_d, g.ldlq, stream))) return rc;

  // ---- proxy errors in the rotated, scaled domain (Wscale cancels), src/quantizer.cpp:269-301
  QB_CUDA(cudaMemsetAsync(gemm_status, 0, sizeof(int), s));
  if ((rc = qtip_k_split_bf16(HR_d, n, n, n, hcat, hcat + n, 3 * n, stream))) return rc;   // [Hh | Hl | .]
  if ((rc = qtip_k_split_bf16(HR_d, n, n, n, hcat + 2 * n, nullptr, 3 * n, stream))) return rc;  // [Hh | Hl | Hh]
  if ((rc = qtip_k_sub(WT_d, hatWT_d, DT, n, mt, mt, stream))) return rc;  // D^T = (W - hatW)^T, all linears
  off = 0;
  for (int i = 0; i < count; ++i) {
    qtip_group_linear& l = lins[i];
    double num = 0, den = 0, wn2 = 0, dn2 = 0;
    for (long c = 0; c < l.m; c += kProxyChunk) {
      const long mc = l.m - c < kProxyChunk ? l.m - c : kProxyChunk;
      double t = 0;
      if ((rc = quad_trace(WT_d, n, mt, off + c, mc, hcat, xt, xcat, y, acc, gemm_status, s, &t))) return rc;
      den += t;
      if ((rc = quad_trace(DT, n, mt, off + c, mc, hcat, xt, xcat, y, acc, gemm_status, s, &t))) return rc;
      num += t;
    }
    if ((rc = sumsq_sync(WT_d + off, n, l.m, mt, acc, s, &wn2))) return rc;
    if ((rc = sumsq_sync(DT + off, n, l.m, mt, acc, s, &dn2))) return rc;
    // HR = rot(H) + creg I and the rotation is orthogonal: the unregularised proxy follows by removing creg |.|^2
    l.proxy_rot_reg = num / den;
    l.proxy = (num - creg * dn2) / (den - creg * wn2);
    off += l.m;
  }
  int gs = 0;
  QB_CUDA(cudaMemcpyAsync(&gs, gemm_status, sizeof(int), cudaMemcpyDeviceToHost, s));
  QB_CUDA(cudaStreamSynchronize(s));
  QB_REQUIRE(gs == 0, QTIP_E_KERNEL, "qtip_quantize_group: a bounded pipeline wait of the trace product ran out (status %d)", gs);

  // ---- states -> bit stream -> kernel layout, linear by linear (src/quantizer.cpp:303-320)
  off = 0;
  const long nblk = n / 16;
  for (int i = 0; i < count; ++i) {
    qtip_group_linear& l = lins[i];
    const long tiles = (l.m / 16) * nblk;
    const uint16_t* q = Q_d + size_t(off / 16) * nblk * 128;
    if ((rc = qtip_pack_trellis(q, tiles, packed, stream))) return rc;
    if ((rc = qtip_swizzle_for_kernel(packed, int(l.m), int(n), l.trellis_d, stream))) return rc;
    off += l.m;
  }
  return QTIP_OK;
}
