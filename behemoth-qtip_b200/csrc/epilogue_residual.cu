// Fused decode-step epilogues around the residual stream (reference: runtime/include/behemoth/qtip_gpu.hpp:199-285,
// kernels runtime/src/qtip.hip:713-786,826-889,1025-1163): RMSNorm + SU + hadUt in one kernel, the o / down residual
// epilogue, and that epilogue fused with the next block's input transform. Instantiates the PrepareNorm / PrepareSmem / FinishResidual modes
// of the shared Hadamard templates for the orders the model shapes use (1, 12, 28).
#include "hadamard.cuh"

namespace qb {

template <int K>
static int configure_in() {
  int rc;
  if ((rc = configure<K, K != 1, Mode::PrepareNorm>())) return rc;
  if ((rc = configure<K, false, Mode::FinishResidual>())) return rc;
  QB_CUDA(cudaFuncSetAttribute(had_row_residual_input_kernel<K>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (kMaxRowFloats - 1024) * 4));
  return QTIP_OK;
}
int epilogue_residual_device_setup() {
  int rc;
  if ((rc = configure_in<1>()) || (rc = configure_in<12>()) || (rc = configure_in<28>())) return rc;
  return QTIP_OK;
}

static int prepare_dims(HadArgs& a, long rows) {
  const int K = had_order(a.n);
  QB_REQUIRE(K > 0, QTIP_E_GEOMETRY, "unsupported Hadamard size %d", a.n);
  a.P = a.n / K;
  a.rows = int(rows);
  a.scale = 1.0f / std::sqrt(float(a.n));
  return K;
}
int hadamard_input_transform(const uint16_t* x, long ldx, const uint16_t* norm, float eps, const float* su, int n,
                             int rows, uint16_t* u, long ldu, uint16_t* xn, cudaStream_t s) {
  HadArgs a{};
  a.src = x, a.dst = u, a.sign = su, a.ld = ldx, a.ld_dst = ldu, a.n = n, a.splits = 1;
  a.norm = norm, a.eps = eps, a.xn = xn, a.factor = 1.f;
  return dispatch_epilogue<Mode::PrepareNorm>(a, rows, true, s);
}
int hadamard_output_residual(const float* z, int splits, long split_stride, int round_z, int ranks, const float* sv,
                             int n, int rows, uint16_t* state, cudaStream_t s) {
  HadArgs a{};
  a.src = z, a.dst = state, a.sign = sv, a.ld = n, a.n = n, a.splits = splits, a.split_stride = split_stride;
  a.round_z = round_z, a.ranks = ranks;
  return dispatch_epilogue<Mode::FinishResidual>(a, rows, false, s);
}
// state += epilogue(z), then u = input transform of the updated state (same width). One kernel per row when the batch
// is large enough for the whole-row kernels, else the two separate launches: identical results either way.
int hadamard_output_residual_input(const float* z, int splits, long split_stride, int round_z, int ranks, const float* sv,
                                   int n, int rows, uint16_t* state, const uint16_t* norm, float eps, const float* su,
                                   uint16_t* u, long ldu, uint16_t* xn, cudaStream_t s) {
  HadArgs fin{};
  fin.src = z, fin.dst = state, fin.sign = sv, fin.ld = n, fin.n = n, fin.splits = splits, fin.split_stride = split_stride;
  fin.round_z = round_z, fin.ranks = ranks;
  const int K = prepare_dims(fin, rows);
  if (K <= 0) return K;
  QB_REQUIRE(K != 20, QTIP_E_GEOMETRY, "the fused epilogues carry the Hadamard orders 1, 12 and 28 (n = %d needs 20)", n);
  if (rows == 0) return QTIP_OK;
  if (fin.ranks > 1) QB_REQUIRE(n % fin.ranks == 0, QTIP_E_GEOMETRY, "n = %d is not divisible by %d ranks", n, fin.ranks);
  const bool chunks = K > 1 && rows < kChunkRowsBelow && fin.P <= 8192;
  if (chunks || n > kMaxRowFloats - 1024) {
    int rc = hadamard_output_residual(z, splits, split_stride, round_z, ranks, sv, n, rows, state, s);
    if (rc) return rc;
    return hadamard_input_transform(state, n, norm, eps, su, n, rows, u, ldu, xn, s);
  }
  HadArgs prep{};
  prep.dst = u, prep.sign = su, prep.ld_dst = ldu, prep.n = n, prep.splits = 1, prep.P = fin.P, prep.rows = fin.rows;
  prep.scale = fin.scale, prep.norm = norm, prep.eps = eps, prep.xn = xn, prep.factor = 1.f;
  switch (K) {
    case 1: had_row_residual_input_kernel<1><<<unsigned(rows), 1024, size_t(n) * 4, s>>>(fin, prep); break;
    case 12: had_row_residual_input_kernel<12><<<unsigned(rows), 1024, size_t(n) * 4, s>>>(fin, prep); break;
    default: had_row_residual_input_kernel<28><<<unsigned(rows), 1024, size_t(n) * 4, s>>>(fin, prep); break;
  }
  QB_LAUNCHED();
  return QTIP_OK;
}

}  // namespace qb

using namespace qb;

extern "C" int qtip_input_transform(const uint16_t* x_d, long ldx, const uint16_t* norm_d, float epsilon, const float* su_d,
                                    int n, int rows, uint16_t* u_d, long ldu, uint16_t* xn_d, void* stream) {
  QB_REQUIRE(x_d && su_d && u_d && n > 0 && rows >= 0 && ldx >= n && ldu >= n, QTIP_E_ARG, "qtip_input_transform: bad argument");
  QB_REQUIRE(!xn_d || norm_d, QTIP_E_ARG, "qtip_input_transform: xn is the normalised row and needs a norm weight");
  if (!device_info()) return QTIP_E_DEVICE;
  return hadamard_input_transform(x_d, ldx, norm_d, epsilon, su_d, n, rows, u_d, ldu, xn_d, as_stream(stream));
}
extern "C" int qtip_output_residual(const float* z_d, int splits, int rows, int rank_major, const float* sv_d, int n,
                                    uint16_t* state_d, void* stream) {
  QB_REQUIRE(z_d && sv_d && state_d && n > 0 && rows >= 0, QTIP_E_ARG, "qtip_output_residual: bad argument");
  QB_REQUIRE(splits >= 1 && splits <= 32, QTIP_E_GEOMETRY, "qtip_output_residual: splits = %d", splits);
  if (!device_info()) return QTIP_E_DEVICE;
  const int ranks = (rank_major && rows > 1) ? (rank_major == 1 ? 2 : rank_major) : 0;
  return hadamard_output_residual(z_d, splits, long(rows) * n, 0, ranks, sv_d, n, rows, state_d, as_stream(stream));
}
extern "C" int qtip_output_residual_input(const float* z_d, int splits, int rows, int rank_major, const float* sv_d, int n,
                                          uint16_t* state_d, const uint16_t* norm_d, float epsilon, const float* su_d,
                                          uint16_t* u_d, long ldu, uint16_t* xn_d, void* stream) {
  QB_REQUIRE(z_d && sv_d && state_d && su_d && u_d && n > 0 && rows >= 0 && ldu >= n, QTIP_E_ARG,
             "qtip_output_residual_input: bad argument");
  QB_REQUIRE(!xn_d || norm_d, QTIP_E_ARG, "qtip_output_residual_input: xn is the normalised row and needs a norm weight");
  QB_REQUIRE(splits >= 1 && splits <= 32, QTIP_E_GEOMETRY, "qtip_output_residual_input: splits = %d", splits);
  if (!device_info()) return QTIP_E_DEVICE;
  const int ranks = (rank_major && rows > 1) ? (rank_major == 1 ? 2 : rank_major) : 0;
  return hadamard_output_residual_input(z_d, splits, long(rows) * n, 0, ranks, sv_d, n, rows, state_d, norm_d, epsilon,
                                        su_d, u_d, ldu, xn_d, as_stream(stream));
}
