// TEST INFRASTRUCTURE ONLY -- C-ABI wrappers around the reference's own CUDA runtime operator
// (runtime/cuda/kernels.cu, runtime/cuda/batch_kernels.cu), compiled from the reference tree where it lies (see Makefile
// target `refgpu`). Used by the GPU parity tests and reported beside this repository's kernels by the bench. Never part
// of the product library. The reference throws std::runtime_error; the wrappers return 1 and keep the message.
#include <cstdint>
#include <stdexcept>
#include <string>

#include "batch_kernels.hpp"

namespace rt = behemoth::cuda_runtime;
static thread_local std::string g_err;
template <class F>
static int guarded(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::exception& e) {
    g_err = e.what();
    return 1;
  }
}
static rt::QtipMatrix mat(const uint16_t* trellis, const float* su, const float* sv, const uint32_t* lut, int in, int out) {
  return rt::QtipMatrix{trellis, su, sv, lut, in, out};
}

extern "C" {
const char* refgpu_last_error() { return g_err.c_str(); }
int refgpu_initialize_tables() { return guarded([&] { rt::initialize_tables(); }); }
int refgpu_qtip_prepare(const uint16_t* trellis, const float* su, const float* sv, const uint32_t* lut, int in, int out,
                        const uint16_t* x, float* scratch, uint16_t* rotated, void* s, int tokens, int rank_major) {
  return guarded([&] {
    rt::qtip_prepare(mat(trellis, su, sv, lut, in, out), x, scratch, rotated, static_cast<rt::Stream>(s), tokens,
                     rank_major != 0);
  });
}
int refgpu_qtip_multiply(const uint16_t* trellis, const float* su, const float* sv, const uint32_t* lut, int in, int out,
                         const uint16_t* rotated, float* z, int stride, int splits, void* s, int tokens) {
  return guarded([&] {
    rt::qtip_multiply(mat(trellis, su, sv, lut, in, out), rotated, z, stride, splits, static_cast<rt::Stream>(s), tokens);
  });
}
int refgpu_qtip_finish(const uint16_t* trellis, const float* su, const float* sv, const uint32_t* lut, int in, int out,
                       const float* z, uint16_t* y, float* scratch, int round_z, int splits, void* s, int tokens,
                       int rank_major) {
  return guarded([&] {
    rt::qtip_finish(mat(trellis, su, sv, lut, in, out), z, y, scratch, round_z != 0, splits, static_cast<rt::Stream>(s),
                    tokens, rank_major != 0);
  });
}
int refgpu_qtip_forward(const uint16_t* trellis, const float* su, const float* sv, const uint32_t* lut, int in, int out,
                        const uint16_t* x, uint16_t* y, float* scratch, uint16_t* rotated, float* z, int round_z, void* s,
                        int splits) {
  return guarded([&] {
    rt::qtip_forward(mat(trellis, su, sv, lut, in, out), x, y, scratch, rotated, z, round_z != 0,
                     static_cast<rt::Stream>(s), splits);
  });
}
int refgpu_qtip_multiply_batch(const uint16_t* trellis, const float* su, const float* sv, const uint32_t* lut, int in,
                               int out, const uint16_t* rotated, float* z, int stride, int splits, int tokens, void* s,
                               int implementation) {
  return guarded([&] {
    rt::qtip_multiply_batch(mat(trellis, su, sv, lut, in, out), rotated, z, stride, splits, tokens,
                            static_cast<rt::Stream>(s), implementation);
  });
}
int refgpu_qtip_decode_matrix(const uint16_t* trellis, const float* su, const float* sv, const uint32_t* lut, int in,
                              int out, uint16_t* dense, void* s) {
  return guarded([&] { rt::qtip_decode_matrix(mat(trellis, su, sv, lut, in, out), dense, static_cast<rt::Stream>(s)); });
}
int refgpu_fp8_forward(const uint8_t* w, const float* scale, const uint16_t* x, uint16_t* y, int in, int out, void* s) {
  return guarded([&] { rt::fp8_forward(w, scale, x, y, in, out, static_cast<rt::Stream>(s)); });
}
}
