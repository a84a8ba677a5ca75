// The gate/up epilogue of a decode step (reference: output_gateup, runtime/include/behemoth/qtip_gpu.hpp:243-247, kernel
// runtime/src/qtip.hip:891-930): h = bf16(silu(g) * u) with g, u the two output transforms of the stacked gate/up
// products. Instantiates the FinishGateUp mode of the shared Hadamard templates for the orders the model shapes use
// (1, 12, 28).
#include "hadamard.cuh"

namespace qb {

template <int K>
static int configure_out() {
  QB_CUDA(cudaFuncSetAttribute(had_row_gateup_kernel<K>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxRowFloats * 4));
  QB_CUDA(cudaFuncSetAttribute(had_chunk_gateup_kernel<K>, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * 8192 * 4));
  return QTIP_OK;
}
int epilogue_gateup_device_setup() {
  int rc;
  if ((rc = configure_out<1>()) || (rc = configure_out<12>()) || (rc = configure_out<28>())) return rc;
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
// z [split][rows][2 F] (gate | up), h [rows][F]
int hadamard_output_gateup(const float* z, int splits, long split_stride, int round_z, const float* sv_gate,
                           const float* sv_up, int F, int rows, uint16_t* h, cudaStream_t s) {
  HadArgs a{};
  a.src = z, a.dst = h, a.sign = sv_gate, a.ld = 2L * F, a.ld_dst = F, a.n = F, a.splits = splits;
  a.split_stride = split_stride, a.round_z = round_z;
  const int K = prepare_dims(a, rows);
  if (K <= 0) return K;
  QB_REQUIRE(K != 20, QTIP_E_GEOMETRY, "the fused epilogues carry the Hadamard orders 1, 12 and 28 (F = %d needs 20)", F);
  if (rows == 0) return QTIP_OK;
  const bool chunks = K > 1 && rows < kChunkRowsBelow && a.P <= 8192;
  QB_REQUIRE(chunks || 2L * F <= kMaxRowFloats, QTIP_E_GEOMETRY, "gate/up rows of 2 x %d floats do not fit a CTA", F);
  QB_REQUIRE(rows <= 65535, QTIP_E_GEOMETRY, "too many rows");
  const int threads = a.P >= 1024 ? 1024 : (a.P < 64 ? 64 : a.P);
  const size_t chunk_smem = (size_t(a.P > 1024 ? a.P : 1024) + a.P) * 4, row_smem = size_t(F) * 8;
  // few rows: a link of a decode step's kernel chain (programmatic dependent launch, like the other chunk kernels)
#define QB_GATEUP(K_)                                                                                                  \
  if (chunks)                                                                                                          \
    QB_CUDA(launch_chained(had_chunk_gateup_kernel<K_>, dim3(K_, unsigned(rows)), dim3(threads), chunk_smem, s, a, sv_up)); \
  else had_row_gateup_kernel<K_><<<unsigned(rows), 1024, row_smem, s>>>(a, sv_up)
  switch (K) {
    case 1: had_row_gateup_kernel<1><<<unsigned(rows), 1024, row_smem, s>>>(a, sv_up); break;
    case 12: QB_GATEUP(12); break;
    default: QB_GATEUP(28); break;
  }
#undef QB_GATEUP
  QB_LAUNCHED();
  return QTIP_OK;
}
}  // namespace qb

using namespace qb;

extern "C" int qtip_output_gateup(const float* z_d, int splits, int rows, const float* sv_gate_d, const float* sv_up_d,
                                  int features, uint16_t* h_d, void* stream) {
  QB_REQUIRE(z_d && sv_gate_d && sv_up_d && h_d && features > 0 && rows >= 0, QTIP_E_ARG, "qtip_output_gateup: bad argument");
  QB_REQUIRE(splits >= 1 && splits <= 32, QTIP_E_GEOMETRY, "qtip_output_gateup: splits = %d", splits);
  if (!device_info()) return QTIP_E_DEVICE;
  return hadamard_output_gateup(z_d, splits, long(rows) * 2 * features, 1, sv_gate_d, sv_up_d, features, rows, h_d,
                                as_stream(stream));
}
