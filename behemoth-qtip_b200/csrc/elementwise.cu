// Elementwise, reduction and layout kernels around LDLQ and the weight rotation (fp32 matrices with a row stride),
// and the device-side trellis bitstream packing. All are HBM-bound: vectorised where the layout allows, grid-stride
// with a few CTAs per SM elsewhere.
#include "common.cuh"

namespace qb {

constexpr int kEwThreads = 256;
static inline unsigned ew_grid(long n) {
  long b = (n + kEwThreads - 1) / kEwThreads;
  const long cap = 148L * 16;
  return unsigned(b < 1 ? 1 : (b > cap ? cap : b));
}

__global__ void scale_rc_kernel(float* X, long rows, long cols, long ld, const float* rs, const float* cs, float a) {
  const long n = rows * cols;
  for (long i = long(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += long(gridDim.x) * blockDim.x) {
    const long r = i / cols, c = i - r * cols;
    float v = X[r * ld + c];
    if (rs) v *= rs[r];
    if (cs) v *= cs[c];
    X[r * ld + c] = v * a;
  }
}
__global__ void sub_kernel(const float* A, const float* B, float* D, long rows, long cols, long ld) {
  const long n = rows * cols;
  for (long i = long(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += long(gridDim.x) * blockDim.x) {
    const long r = i / cols, o = r * ld + (i - r * cols);
    D[o] = A[o] - B[o];
  }
}

// Sum of one double per thread over the CTA (at most 1,024 threads), valid in thread 0. Lanes fold with
// __reduce-style butterfly steps on the two 32-bit halves; one slot per warp in shared memory carries the warp totals to
// warp 0, which folds them the same way.
__device__ __forceinline__ double warp_total(double v) {
#pragma unroll
  for (int step = 1; step < 32; step <<= 1) v += __shfl_down_sync(0xffffffffu, v, step);
  return v;  // complete in lane 0
}
__device__ __forceinline__ double block_sum(double v) {
  __shared__ double warp_totals[32];
  const int lane = threadIdx.x % 32, warp = threadIdx.x / 32, warps = (blockDim.x + 31) / 32;
  v = warp_total(v);
  if (lane == 0) warp_totals[warp] = v;
  __syncthreads();
  if (warp != 0) return 0.0;
  return warp_total(lane < warps ? warp_totals[lane] : 0.0);
}
// out += sum over the block of A .* B (B == nullptr: A .* A); fp64 accumulation, one atomic per CTA.
__global__ void dot_kernel(const float* A, long lda, const float* B, long ldb, long rows, long cols, double* out) {
  double acc = 0;
  const long n = rows * cols;
  for (long i = long(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += long(gridDim.x) * blockDim.x) {
    const long r = i / cols, c = i - r * cols;
    const double a = A[r * lda + c];
    acc += a * (B ? double(B[r * ldb + c]) : a);
  }
  acc = block_sum(acc);
  if (threadIdx.x == 0) atomicAdd(out, acc);
}
__global__ void add_diag_kernel(float* H, long n, float a) {
  const long i = long(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) H[i * n + i] += a;
}
__global__ void diag_sum_kernel(const float* H, long n, double* out) {
  double acc = 0;
  for (long i = long(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += long(gridDim.x) * blockDim.x)
    acc += H[i * n + i];
  acc = block_sum(acc);
  if (threadIdx.x == 0) atomicAdd(out, acc);
}
// v = A - B (B may be null) -> bf16 hi and (optionally) bf16 lo of the remainder.
__global__ void split_kernel(const float* A, const float* B, long rows, long cols, long ld, uint16_t* hi, uint16_t* lo,
                             long ld_out) {
  const long n = rows * cols;
  for (long i = long(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += long(gridDim.x) * blockDim.x) {
    const long r = i / cols, c = i - r * cols;
    float v = A[r * ld + c];
    if (B) v -= B[r * ld + c];
    const uint16_t h = f32_to_bf16(v);
    hi[r * ld_out + c] = h;
    if (lo) lo[r * ld_out + c] = f32_to_bf16(v - bf16_to_f32(h));
  }
}
// out[c][r] = in[r][c] through a padded 32x32 shared tile.
__global__ void transpose_kernel(const float* in, long rows, long cols, long ld_in, float* out, long ld_out) {
  __shared__ float tile[32][33];
  const long c0 = long(blockIdx.x) * 32, r0 = long(blockIdx.y) * 32;
  const int tx = threadIdx.x, ty = threadIdx.y;
  for (int k = ty; k < 32; k += 8) {
    const long r = r0 + k, c = c0 + tx;
    if (r < rows && c < cols) tile[k][tx] = in[r * ld_in + c];
  }
  __syncthreads();
  for (int k = ty; k < 32; k += 8) {
    const long c = c0 + k, r = r0 + tx;
    if (r < rows && c < cols) out[c * ld_out + r] = tile[tx][k];
  }
}

// Sequences of all 16x16 tiles of a row-major matrix (row stride ld): X[(tr * (n/16) + tc)][p] = W[16 tr + r][16 tc + c]
// with 16 r + c = perm_fwd(p). One thread per output element; a warp writes 128 contiguous bytes.
__global__ void tiles_from_matrix_kernel(const float* __restrict__ W, long m, long n, long ld, float* __restrict__ X) {
  const long total = m * n;
  for (long i = long(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
    const long tile = i >> 8;
    const int q = perm_fwd(int(i & 255));
    const long tr = tile / (n >> 4), tc = tile - tr * (n >> 4);
    X[i] = W[(tr * 16 + (q >> 4)) * ld + tc * 16 + (q & 15)];
  }
}

// ---- trellis bitstream: word w of a sequence holds stream bits [16 w, 16 w + 16), MSB first. State t is the 16-bit
// window at bit 4 t, so word w = state[4 w] (its 16 bits are exactly that window). One thread per word.
__global__ void pack_kernel(const uint16_t* __restrict__ states, long nwords, uint16_t* __restrict__ packed) {
  const long i = long(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= nwords) return;
  const long b = i >> 5;
  const int w = int(i & 31);
  packed[i] = states[b * 128 + 4 * w];
}
// state t = window at bit 4 t (wrapping): from words t >> 2 and (t >> 2) + 1 mod 32. One thread per state.
__global__ void unpack_kernel(const uint16_t* __restrict__ packed, long nstates, uint16_t* __restrict__ states) {
  const long i = long(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= nstates) return;
  const long b = i >> 7;
  const int t = int(i & 127), w = t >> 2, sh = 4 * (t & 3);
  const uint32_t u = uint32_t(packed[b * 32 + w]) << 16 | packed[b * 32 + ((w + 1) & 31)];
  states[i] = uint16_t(u >> (16 - sh));
}
// Kernel layout: out[(((i0*N2 + j0)*32 + c)*2 + j1)*2 + i1] = packed[((2 i0 + i1) * (n/16) + 2 j0 + j1) * 32 + c].
template <bool Forward>
__global__ void swizzle_kernel(const uint16_t* __restrict__ in, long total, int N2, uint16_t* __restrict__ out) {
  const long o = long(blockIdx.x) * blockDim.x + threadIdx.x;  // index in kernel layout
  if (o >= total) return;
  const int i1 = int(o & 1), j1 = int((o >> 1) & 1), c = int((o >> 2) & 31);
  const long blk = o >> 7, j0 = blk % N2, i0 = blk / N2;
  const long p = ((2 * i0 + i1) * (2L * N2) + 2 * j0 + j1) * 32 + c;  // index in plain packed order
  if (Forward) out[o] = in[p];
  else out[p] = in[o];
}

}  // namespace qb

using namespace qb;

extern "C" int qtip_k_scale_rows_cols(float* X_d, long rows, long cols, long ld, const float* rs_d, const float* cs_d,
                                      void* stream) {
  QB_REQUIRE(X_d && rows >= 0 && cols >= 0 && ld >= cols, QTIP_E_ARG, "qtip_k_scale_rows_cols: bad argument");
  if (rows * cols == 0) return QTIP_OK;
  scale_rc_kernel<<<ew_grid(rows * cols), kEwThreads, 0, as_stream(stream)>>>(X_d, rows, cols, ld, rs_d, cs_d, 1.f);
  QB_LAUNCHED();
  return QTIP_OK;
}
extern "C" int qtip_k_scale(float* X_d, long rows, long cols, long ld, float a, void* stream) {
  QB_REQUIRE(X_d && rows >= 0 && cols >= 0 && ld >= cols, QTIP_E_ARG, "qtip_k_scale: bad argument");
  if (rows * cols == 0) return QTIP_OK;
  scale_rc_kernel<<<ew_grid(rows * cols), kEwThreads, 0, as_stream(stream)>>>(X_d, rows, cols, ld, nullptr, nullptr, a);
  QB_LAUNCHED();
  return QTIP_OK;
}
extern "C" int qtip_k_sub(const float* A_d, const float* B_d, float* D_d, long rows, long cols, long ld, void* stream) {
  QB_REQUIRE(A_d && B_d && D_d && rows >= 0 && cols >= 0 && ld >= cols, QTIP_E_ARG, "qtip_k_sub: bad argument");
  if (rows * cols == 0) return QTIP_OK;
  sub_kernel<<<ew_grid(rows * cols), kEwThreads, 0, as_stream(stream)>>>(A_d, B_d, D_d, rows, cols, ld);
  QB_LAUNCHED();
  return QTIP_OK;
}
extern "C" int qtip_k_sumsq(const float* X_d, long rows, long cols, long ld, double* out_d, void* stream) {
  QB_REQUIRE(X_d && out_d && rows >= 0 && cols >= 0 && ld >= cols, QTIP_E_ARG, "qtip_k_sumsq: bad argument");
  if (rows * cols == 0) return QTIP_OK;
  dot_kernel<<<ew_grid(rows * cols), kEwThreads, 0, as_stream(stream)>>>(X_d, ld, nullptr, 0, rows, cols, out_d);
  QB_LAUNCHED();
  return QTIP_OK;
}
extern "C" int qtip_k_dot(const float* A_d, long lda, const float* B_d, long ldb, long rows, long cols, double* out_d,
                          void* stream) {
  QB_REQUIRE(A_d && B_d && out_d && rows >= 0 && cols >= 0, QTIP_E_ARG, "qtip_k_dot: bad argument");
  if (rows * cols == 0) return QTIP_OK;
  dot_kernel<<<ew_grid(rows * cols), kEwThreads, 0, as_stream(stream)>>>(A_d, lda, B_d, ldb, rows, cols, out_d);
  QB_LAUNCHED();
  return QTIP_OK;
}
extern "C" int qtip_k_add_diag(float* H_d, long n, float a, void* stream) {
  QB_REQUIRE(H_d && n >= 0, QTIP_E_ARG, "qtip_k_add_diag: bad argument");
  if (n == 0) return QTIP_OK;
  add_diag_kernel<<<blocks_for(n, kEwThreads), kEwThreads, 0, as_stream(stream)>>>(H_d, n, a);
  QB_LAUNCHED();
  return QTIP_OK;
}
extern "C" int qtip_k_diag_sum(const float* H_d, long n, double* out_d, void* stream) {
  QB_REQUIRE(H_d && out_d && n >= 0, QTIP_E_ARG, "qtip_k_diag_sum: bad argument");
  if (n == 0) return QTIP_OK;
  diag_sum_kernel<<<64, kEwThreads, 0, as_stream(stream)>>>(H_d, n, out_d);
  QB_LAUNCHED();
  return QTIP_OK;
}
extern "C" int qtip_k_split_bf16(const float* X_d, long rows, long cols, long ld_in, uint16_t* hi_d, uint16_t* lo_d,
                                 long ld_out, void* stream) {
  QB_REQUIRE(X_d && hi_d && rows >= 0 && cols >= 0, QTIP_E_ARG, "qtip_k_split_bf16: bad argument");
  if (rows * cols == 0) return QTIP_OK;
  split_kernel<<<ew_grid(rows * cols), kEwThreads, 0, as_stream(stream)>>>(X_d, nullptr, rows, cols, ld_in, hi_d, lo_d,
                                                                           ld_out);
  QB_LAUNCHED();
  return QTIP_OK;
}
extern "C" int qtip_k_diff_split_bf16(const float* A_d, const float* B_d, long rows, long cols, long ld, uint16_t* hi_d,
                                      uint16_t* lo_d, long ld_out, void* stream) {
  QB_REQUIRE(A_d && B_d && hi_d && rows >= 0 && cols >= 0, QTIP_E_ARG, "qtip_k_diff_split_bf16: bad argument");
  if (rows * cols == 0) return QTIP_OK;
  split_kernel<<<ew_grid(rows * cols), kEwThreads, 0, as_stream(stream)>>>(A_d, B_d, rows, cols, ld, hi_d, lo_d, ld_out);
  QB_LAUNCHED();
  return QTIP_OK;
}
extern "C" int qtip_k_transpose(const float* in_d, long rows, long cols, long ld_in, float* out_d, long ld_out,
                                void* stream) {
  QB_REQUIRE(in_d && out_d && rows >= 0 && cols >= 0, QTIP_E_ARG, "qtip_k_transpose: bad argument");
  if (rows * cols == 0) return QTIP_OK;
  const dim3 grid(blocks_for(cols, 32), blocks_for(rows, 32));
  QB_REQUIRE(grid.y <= 65535, QTIP_E_GEOMETRY, "qtip_k_transpose: more than 2,097,120 rows");
  transpose_kernel<<<grid, dim3(32, 8), 0, as_stream(stream)>>>(in_d, rows, cols, ld_in, out_d, ld_out);
  QB_LAUNCHED();
  return QTIP_OK;
}

extern "C" int qtip_tiles_from_matrix(const float* W_d, long m, long n, long ld, float* X_d, void* stream) {
  QB_REQUIRE(W_d && X_d && ld >= n, QTIP_E_ARG, "qtip_tiles_from_matrix: bad argument");
  QB_REQUIRE(m >= 0 && n >= 0 && m % 16 == 0 && n % 16 == 0, QTIP_E_GEOMETRY,
             "qtip_tiles_from_matrix: %ld x %ld is not a whole number of 16x16 tiles", m, n);
  if (m * n == 0) return QTIP_OK;
  tiles_from_matrix_kernel<<<ew_grid(m * n), kEwThreads, 0, as_stream(stream)>>>(W_d, m, n, ld, X_d);
  QB_LAUNCHED();
  return QTIP_OK;
}

extern "C" int qtip_pack_trellis(const uint16_t* states_d, long B, uint16_t* packed_d, void* stream) {
  QB_REQUIRE(states_d && packed_d && B >= 0, QTIP_E_ARG, "qtip_pack_trellis: bad argument");
  if (B == 0) return QTIP_OK;
  pack_kernel<<<blocks_for(B * 32, 256), 256, 0, as_stream(stream)>>>(states_d, B * 32, packed_d);
  QB_LAUNCHED();
  return QTIP_OK;
}
extern "C" int qtip_unpack_trellis(const uint16_t* packed_d, long B, uint16_t* states_d, void* stream) {
  QB_REQUIRE(states_d && packed_d && B >= 0, QTIP_E_ARG, "qtip_unpack_trellis: bad argument");
  if (B == 0) return QTIP_OK;
  unpack_kernel<<<blocks_for(B * 128, 256), 256, 0, as_stream(stream)>>>(packed_d, B * 128, states_d);
  QB_LAUNCHED();
  return QTIP_OK;
}
static int swizzle_common(const uint16_t* in, int m, int n, uint16_t* out, bool forward, void* stream) {
  QB_REQUIRE(in && out, QTIP_E_ARG, "swizzle: null pointer");
  QB_REQUIRE(m > 0 && n > 0 && m % 32 == 0 && n % 32 == 0, QTIP_E_GEOMETRY,
             "kernel layout needs m, n multiples of 32 (got %d x %d)", m, n);
  const long total = long(m / 16) * (n / 16) * 32;
  if (forward)
    swizzle_kernel<true><<<blocks_for(total, 256), 256, 0, as_stream(stream)>>>(in, total, n / 32, out);
  else
    swizzle_kernel<false><<<blocks_for(total, 256), 256, 0, as_stream(stream)>>>(in, total, n / 32, out);
  QB_LAUNCHED();
  return QTIP_OK;
}
extern "C" int qtip_swizzle_for_kernel(const uint16_t* packed_d, int m, int n, uint16_t* out_d, void* stream) {
  return swizzle_common(packed_d, m, n, out_d, true, stream);
}
extern "C" int qtip_unswizzle_for_kernel(const uint16_t* in_d, int m, int n, uint16_t* packed_d, void* stream) {
  return swizzle_common(in_d, m, n, packed_d, false, stream);
}
