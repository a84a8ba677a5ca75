// W8A16 projection for the FP8 (e4m3, OCP "fn": 0x7f / 0xff are NaN) K/V weights that sit beside the QTIP linears of a
// layer: y[t][o] = bf16( (sum_i fp8(w[o][i]) * bf16(x[t][i])) * scale[o] ), fp32 accumulation.
// HBM-bound (one byte per weight): four warps share an output row, each lane streams 16 weights per 16-byte load (two
// loads in flight), keeps one fp32 accumulator per token (up to 8 tokens per pass); shuffles and shared memory reduce.
#include <cuda_fp8.h>

#include "common.cuh"

namespace qb {

constexpr int kFp8Tokens = 8;

__device__ __forceinline__ float2 fp8x2_to_float2(uint16_t v) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(__nv_fp8x2_storage_t(v), __NV_E4M3);
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}

// Four warps share a row (a quarter of K each), two rows per 256-thread CTA; partial sums meet in shared memory.
constexpr int kFp8Split = 4;
__global__ __launch_bounds__(256) void fp8_gemv_kernel(const uint8_t* __restrict__ w, const float* __restrict__ scale,
                                                       const uint16_t* __restrict__ x, uint16_t* __restrict__ y, int in,
                                                       int out, int tokens) {
  __shared__ float part[8][kFp8Tokens];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.x * 2 + (warp >> 2), quarter = warp & 3;
  const int t0 = blockIdx.y * kFp8Tokens, nt = min(kFp8Tokens, tokens - t0);
  float acc[kFp8Tokens];
#pragma unroll
  for (int t = 0; t < kFp8Tokens; ++t) acc[t] = 0.f;
  chain_release();
  chain_wait();  // x may come from the kernel before this one, y may still be read by it
  if (row < out) {
    const int chunks = in / 16, c_lo = chunks * quarter / kFp8Split, c_hi = chunks * (quarter + 1) / kFp8Split;
    const uint4* wr = reinterpret_cast<const uint4*>(w + size_t(row) * in);
    for (int c0 = c_lo + lane; c0 < c_hi; c0 += 64) {
      // two independent 16-byte weight loads in flight per lane
      const int c1 = c0 + 32;
      const uint4 wa = wr[c0];
      const uint4 wb = c1 < c_hi ? wr[c1] : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const uint4 wv = half ? wb : wa;
        const int c = half ? c1 : c0;
        if (c >= c_hi) break;
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
    }
  }
#pragma unroll
  for (int t = 0; t < kFp8Tokens; ++t) {
    float s = acc[t];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (lane == 0) part[warp][t] = s;
  }
  __syncthreads();
  if (threadIdx.x < 2 * kFp8Tokens) {
    const int r = threadIdx.x / kFp8Tokens, t = threadIdx.x % kFp8Tokens, orow = blockIdx.x * 2 + r;
    if (orow < out && t < nt) {
      const float s = ((part[4 * r][t] + part[4 * r + 1][t]) + part[4 * r + 2][t]) + part[4 * r + 3][t];
      y[size_t(t0 + t) * out + orow] = f32_to_bf16(s * scale[orow]);
    }
  }
}

// Exact bf16 value of every e4m3 byte (e4m3 has 3 mantissa bits: bf16 holds it exactly); 16 bytes per thread.
__global__ void fp8_to_bf16_kernel(const uint8_t* __restrict__ in, uint16_t* __restrict__ out, size_t n16) {
  const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n16) return;
  const uint4 v = reinterpret_cast<const uint4*>(in)[i];
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint32_t o[8];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float2 a = fp8x2_to_float2(uint16_t(w[q])), b = fp8x2_to_float2(uint16_t(w[q] >> 16));
    o[2 * q] = (__float_as_uint(a.x) >> 16) | (__float_as_uint(a.y) & 0xffff0000u);
    o[2 * q + 1] = (__float_as_uint(b.x) >> 16) | (__float_as_uint(b.y) & 0xffff0000u);
  }
  uint4* dst = reinterpret_cast<uint4*>(out) + 2 * i;
  dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
  dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

}  // namespace qb

using namespace qb;

extern "C" int qtip_decode_fp8_matrix(const uint8_t* w_d, uint16_t* out_d, size_t elements, void* stream) {
  QB_REQUIRE(w_d && out_d, QTIP_E_ARG, "qtip_decode_fp8_matrix: null pointer");
  QB_REQUIRE(elements % 16 == 0, QTIP_E_GEOMETRY, "qtip_decode_fp8_matrix: element count must be a multiple of 16");
  if (elements == 0) return QTIP_OK;
  fp8_to_bf16_kernel<<<blocks_for(long(elements / 16), 256), 256, 0, as_stream(stream)>>>(w_d, out_d, elements / 16);
  QB_LAUNCHED();
  return QTIP_OK;
}

extern "C" int qtip_fp8_forward(const uint8_t* w_d, const float* scale_d, const uint16_t* x_d, uint16_t* y_d, int in,
                                int out, int tokens, void* stream) {
  QB_REQUIRE(w_d && scale_d && x_d && y_d && tokens >= 1, QTIP_E_ARG, "qtip_fp8_forward: bad argument");
  QB_REQUIRE(in > 0 && out > 0 && in % 16 == 0, QTIP_E_GEOMETRY, "qtip_fp8_forward: in = %d must be a multiple of 16", in);
  const dim3 grid(blocks_for(out, 2), blocks_for(tokens, kFp8Tokens));
  QB_REQUIRE(grid.y <= 65535, QTIP_E_GEOMETRY, "qtip_fp8_forward: too many tokens (%d)", tokens);
  QB_CUDA(launch_chained(fp8_gemv_kernel, grid, dim3(256), 0, as_stream(stream), w_d, scale_d, x_d, y_d, in, out, tokens));
  QB_LAUNCHED();
  return QTIP_OK;
}
