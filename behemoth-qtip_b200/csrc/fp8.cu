// W8A16 projection for the FP8 (e4m3, OCP "fn": 0x7f / 0xff are NaN) K/V weights that sit beside the QTIP linears of a
// layer: y[t][o] = bf16( (sum_i fp8(w[o][i]) * bf16(x[t][i])) * scale[o] ), fp32 accumulation.
// HBM-bound (one byte per weight): a warp owns an output row, each lane streams 16 weights per 16-byte load, keeps one
// fp32 accumulator per token (up to 8 tokens per pass) and the row is reduced with shuffles at the end.
#include <cuda_fp8.h>

#include "common.cuh"

namespace qb {

constexpr int kFp8Tokens = 8;

__device__ __forceinline__ float2 fp8x2_to_float2(uint16_t v) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(__nv_fp8x2_storage_t(v), __NV_E4M3);
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}

__global__ __launch_bounds__(256) void fp8_gemv_kernel(const uint8_t* __restrict__ w, const float* __restrict__ scale,
                                                       const uint16_t* __restrict__ x, uint16_t* __restrict__ y, int in,
                                                       int out, int tokens) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= out) return;
  const int t0 = blockIdx.y * kFp8Tokens, nt = min(kFp8Tokens, tokens - t0);
  float acc[kFp8Tokens];
#pragma unroll
  for (int t = 0; t < kFp8Tokens; ++t) acc[t] = 0.f;
  const uint4* wr = reinterpret_cast<const uint4*>(w + size_t(row) * in);
  for (int c = lane; c < in / 16; c += 32) {
    const uint4 wv = wr[c];
    const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
    float wf[16];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 a = fp8x2_to_float2(uint16_t(ww[q])), b = fp8x2_to_float2(uint16_t(ww[q] >> 16));
      wf[4 * q] = a.x, wf[4 * q + 1] = a.y, wf[4 * q + 2] = b.x, wf[4 * q + 3] = b.y;
    }
#pragma unroll
    for (int t = 0; t < kFp8Tokens; ++t) {
      if (t < nt) {
        const uint4* xr = reinterpret_cast<const uint4*>(x + size_t(t0 + t) * in) + 2 * c;
        const uint4 x0 = __ldg(xr), x1 = __ldg(xr + 1);
        const uint32_t xx[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          acc[t] = fmaf(wf[2 * q], __uint_as_float(xx[q] << 16), acc[t]);
          acc[t] = fmaf(wf[2 * q + 1], __uint_as_float(xx[q] & 0xffff0000u), acc[t]);
        }
      }
    }
  }
  const float sc = scale[row];
#pragma unroll
  for (int t = 0; t < kFp8Tokens; ++t) {
    float s = acc[t];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (lane == 0 && t < nt) y[size_t(t0 + t) * out + row] = f32_to_bf16(s * sc);
  }
}

}  // namespace qb

using namespace qb;

extern "C" int qtip_fp8_forward(const uint8_t* w_d, const float* scale_d, const uint16_t* x_d, uint16_t* y_d, int in,
                                int out, int tokens, void* stream) {
  QB_REQUIRE(w_d && scale_d && x_d && y_d && tokens >= 1, QTIP_E_ARG, "qtip_fp8_forward: bad argument");
  QB_REQUIRE(in > 0 && out > 0 && in % 16 == 0, QTIP_E_GEOMETRY, "qtip_fp8_forward: in = %d must be a multiple of 16", in);
  const dim3 grid(blocks_for(out, 8), blocks_for(tokens, kFp8Tokens));
  QB_REQUIRE(grid.y <= 65535, QTIP_E_GEOMETRY, "qtip_fp8_forward: too many tokens (%d)", tokens);
  fp8_gemv_kernel<<<grid, 256, 0, as_stream(stream)>>>(w_d, scale_d, x_d, y_d, in, out, tokens);
  QB_LAUNCHED();
  return QTIP_OK;
}
