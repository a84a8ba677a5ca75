// Shared helpers of the qtip_b200 library: status/error plumbing, per-device state, small device functions.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/qtip_b200.h"

namespace qb {

// Sets the calling thread's error message and returns `code`.
int fail(int code, const char* fmt, ...);
// Records a CUDA failure; returns the (positive) cudaError_t value.
int cuda_fail(cudaError_t e, const char* what, const char* file, int line);

#define QB_CUDA(x)                                                        \
  do {                                                                    \
    cudaError_t e_ = (x);                                                 \
    if (e_ != cudaSuccess) return qb::cuda_fail(e_, #x, __FILE__, __LINE__); \
  } while (0)
#define QB_LAUNCHED() QB_CUDA(cudaGetLastError())
#define QB_REQUIRE(cond, code, ...)                   \
  do {                                                \
    if (!(cond)) return qb::fail(code, __VA_ARGS__); \
  } while (0)

inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

// Per-device facts filled by qtip_init().
struct DeviceInfo {
  bool ready = false;
  int sm_count = 0;
  int max_clusters = 0;  // co-resident 8-CTA clusters of the Viterbi kernel
};
DeviceInfo* device_info();  // for the current device; nullptr + error set if qtip_init() has not run there
int viterbi_device_setup(DeviceInfo* info);  // viterbi.cu
int decode_device_setup(DeviceInfo* info);   // decode.cu
int gemm_tc_device_setup();                   // gemm_tc.cu
int trellis_tc_device_setup();                // trellis_tc.cu
// viterbi.cu: status words of the kernel-level cluster launches and of the built-in scratch; read, then cleared, on `s`
int viterbi_read_status(int* kernel_level, int* noalloc, cudaStream_t s);
int viterbi_set_status(int which, int value, cudaStream_t s);  // test hook behind qtip_debug_set_status
int block_ldl_device_setup();                // block_ldl.cu
int hadamard_device_setup();                 // hadamard.cu: uploads the order-12/20/28 factors

// Order-K Hadamard factor (Paley construction), K in {12, 20, 28}; row-major +-1. Returns false otherwise.
bool had_factor(int K, int8_t* H);
// get_hadK restricted to the carried orders: 12, 20, 28, 1 (power of two) or 0 (unsupported).
int had_order(long n);

// ---- device helpers
__device__ __forceinline__ float bf16_to_f32(uint16_t x) { return __uint_as_float(uint32_t(x) << 16); }
__device__ __forceinline__ uint16_t f32_to_bf16(float x) {  // round to nearest even, finite inputs
  uint32_t u = __float_as_uint(x);
  return uint16_t((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}
__device__ __forceinline__ float half_lo(uint32_t u) { return __half2float(__ushort_as_half(uint16_t(u))); }
__device__ __forceinline__ float half_hi(uint32_t u) { return __half2float(__ushort_as_half(uint16_t(u >> 16))); }
__device__ __forceinline__ float round_half(float x) { return __half2float(__float2half_rn(x)); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

// Tile permutation: sequence position p <-> tile index 16 r + c.
__device__ __forceinline__ int perm_fwd(int p) {
  return ((p >> 1) & 1) * 128 + ((p >> 5) & 7) * 16 + ((p >> 2) & 1) * 8 + ((p >> 3) & 3) * 2 + (p & 1);
}
__device__ __forceinline__ int perm_inv(int q) {
  return ((((((q >> 4) & 7) * 4 + ((q >> 1) & 3)) * 2 + ((q >> 3) & 1)) * 2 + (q >> 7)) * 2) + (q & 1);
}
// LUT entry (sign << 9 | index) of a trellis state; bits above 15 are ignored.
__device__ __forceinline__ uint32_t lut_entry(uint32_t s) {
  s &= 0xffffu;
  return ((s * (s + 1u)) >> 6) & 1023u;
}

inline unsigned blocks_for(long n, int per) { return unsigned((n + per - 1) / per); }

// Programmatic dependent launch for the chains of short kernels of a decode step (input transform, product, output
// transform, ...): a kernel launched through launch_chained() may become resident while the kernel before it in the
// stream is still draining, runs whatever does not depend on that kernel (table set-up), and blocks in
// chain_wait() until the earlier kernel has completed and its writes are visible. Every kernel of a chain calls
// chain_release() first (its successor may then be scheduled as SMs free up) and chain_wait() before its first read
// of an activation or first write of an output. Without the launch attribute both calls do nothing.
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
bool chained_launches_enabled();  // QTIP_PDL=0 turns the attribute off (plain stream order), tables.cu
template <typename... Params, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                  Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = s;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = chained_launches_enabled() ? 1 : 0;
  cfg.attrs = &attr, cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

}  // namespace qb
