// Block LDL of the rotated, damped Hessian on the GPU, in fp64: H = (Lb + I) D (Lb + I)^T with 16 x 16 diagonal blocks,
// delivered as the strictly block-lower factor Lb in fp32 -- what LDLQ consumes. The reference computes it on the host
// (src/qtip_core.cpp:321-487: cholesky_inplace + block_ldl_to_L, fp64, OpenMP); at n = 28,672 that is the longest stage
// of a Hessian group once the Viterbi runs on a B200.
//
// Method (same algebra as the reference): symmetrise in fp64, A = (H + H^T) / 2; Cholesky A = C C^T (lower); for every
// 16-column block bj, Lb[:, bj] = C[:, bj] * inv(C[bj, bj]) below the diagonal block, zero on and above it.
// The Cholesky is right-looking with 128-column panels:
//   1. chol_diag_kernel   one CTA factors the 128 x 128 diagonal block in shared memory;
//   2. chol_panel_kernel  rows below: x L11^T = a by forward substitution, 64 rows per CTA, L11 and the rows in shared
//                         memory, four partial sums per row;
//   3. chol_update_kernel trailing update C -= P P^T on the lower triangle: 128 x 128 tiles, 8 x 8 fp64 accumulators per
//                         thread, the 128-deep panels streamed through shared memory in 16-column slices. This is where
//                         the n^3 / 6 fused multiply-adds are: DFMA-issue bound (64 lanes per SM and clock).
// A non-positive pivot or a non-finite result sets a status word in the workspace (qtip_block_ldl_status); the
// reference returns false in those cases.
#include "common.cuh"

namespace qb {

constexpr int kNb = 128;   // panel width
constexpr int kTile = 128; // trailing-update tile
constexpr int kKc = 16;    // panel columns per shared-memory slice

struct LdlHeader {
  int status;  // bit 0: a pivot was not positive; bit 1: a non-finite value in the factor
  int pad[63];
};

// A[i][j] = (H[i][j] + H[j][i]) / 2 in fp64, lower triangle (j <= i); the strict upper triangle is never read again.
__global__ void ldl_symmetrise_kernel(const float* __restrict__ H, double* __restrict__ A, long n) {
  __shared__ float t[32][33];
  const long bi = blockIdx.y, bj = blockIdx.x;
  if (bj > bi) return;
  const int tx = threadIdx.x, ty = threadIdx.y;  // 32 x 8
  for (int r = ty; r < 32; r += 8) {
    const long i = bj * 32 + r, j = bi * 32 + tx;  // the transposed block, read along its rows
    t[r][tx] = (i < n && j < n) ? H[i * n + j] : 0.f;
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const long i = bi * 32 + r, j = bj * 32 + tx;
    if (i < n && j < n && j <= i) A[i * n + j] = 0.5 * (double(H[i * n + j]) + double(t[tx][r]));
  }
}

// Unblocked Cholesky of the kb x kb diagonal block at (k, k), one CTA, block held in shared memory (row stride kNb + 1).
__global__ __launch_bounds__(256) void chol_diag_kernel(double* __restrict__ A, long n, long k, int kb, int* status) {
  extern __shared__ double sm[];
  const int ld = kNb + 1;
  for (int idx = threadIdx.x; idx < kb * kb; idx += blockDim.x) {
    const int i = idx / kb, j = idx - i * kb;
    sm[i * ld + j] = j <= i ? A[(k + i) * n + k + j] : 0.0;
  }
  __syncthreads();
  for (int j = 0; j < kb; ++j) {
    // column j: every earlier column has already been subtracted from it (right-looking)
    const double d = sm[j * ld + j];
    __syncthreads();
    const bool ok = d > 0.0;
    if (!ok && threadIdx.x == 0) atomicOr(status, 1);
    const double dj = ok ? sqrt(d) : 1.0;  // a failed pivot is reported; the factor is then meaningless but finite
    for (int i = j + threadIdx.x; i < kb; i += blockDim.x) sm[i * ld + j] = (i == j) ? dj : sm[i * ld + j] / dj;
    __syncthreads();
    // trailing update of the block: a[i][c] -= a[i][j] a[c][j] for j < c <= i
    const int rem = kb - j - 1;
    for (int idx = threadIdx.x; idx < rem * rem; idx += blockDim.x) {
      const int i = j + 1 + idx / rem, c = j + 1 + idx % rem;
      if (c <= i) sm[i * ld + c] = fma(-sm[i * ld + j], sm[c * ld + j], sm[i * ld + c]);
    }
    __syncthreads();
  }
  for (int idx = threadIdx.x; idx < kb * kb; idx += blockDim.x) {
    const int i = idx / kb, j = idx - i * kb;
    if (j <= i) A[(k + i) * n + k + j] = sm[i * ld + j];
  }
}

// Rows r0 + [64 b, 64 b + 64): x L11^T = a, i.e. x[j] = (a[j] - sum_{p < j} x[p] L11[j][p]) / L11[j][j], one thread per
// row. L11 (kb x kb) and the rows sit in shared memory; each thread keeps four running sums so that the fp64 adds of one
// row do not form a single chain.
constexpr int kPanelRows = 64;
__global__ __launch_bounds__(kPanelRows) void chol_panel_kernel(double* __restrict__ A, long n, long k, int kb) {
  extern __shared__ double sm[];
  double* L11 = sm;                   // [kb][kNb + 1]
  double* X = sm + kNb * (kNb + 1);   // [kPanelRows][kNb + 1]
  const int ld = kNb + 1;
  const long r0 = k + kb + long(blockIdx.x) * kPanelRows;
  const int rows = int(min(long(kPanelRows), n - r0));
  for (int idx = threadIdx.x; idx < kb * kb; idx += blockDim.x) {
    const int i = idx / kb, j = idx - i * kb;
    L11[i * ld + j] = j <= i ? A[(k + i) * n + k + j] : 0.0;
  }
  for (int idx = threadIdx.x; idx < rows * kb; idx += blockDim.x) {
    const int i = idx / kb, j = idx - i * kb;
    X[i * ld + j] = A[(r0 + i) * n + k + j];
  }
  __syncthreads();
  if (int(threadIdx.x) < rows) {
    double* x = X + threadIdx.x * ld;
    for (int j = 0; j < kb; ++j) {
      const double* l = L11 + j * ld;
      double s0 = x[j], s1 = 0, s2 = 0, s3 = 0;
      int p = 0;
      for (; p + 4 <= j; p += 4) {
        s0 = fma(-l[p], x[p], s0);
        s1 = fma(-l[p + 1], x[p + 1], s1);
        s2 = fma(-l[p + 2], x[p + 2], s2);
        s3 = fma(-l[p + 3], x[p + 3], s3);
      }
      for (; p < j; ++p) s0 = fma(-l[p], x[p], s0);
      x[j] = ((s0 + s1) + (s2 + s3)) / l[j];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < rows * kb; idx += blockDim.x) {
    const int i = idx / kb, j = idx - i * kb;
    A[(r0 + i) * n + k + j] = X[i * ld + j];
  }
}

// C[i][j] -= sum_p P[i][p] P[j][p] for the tile (ti, tj), tj <= ti, of the trailing matrix that starts at row / column
// r0; P = A[r0.., k .. k + kb). 256 threads as 16 x 16, each 8 x 8 outputs at rows ty + 16 a and columns tx + 16 b.
__global__ __launch_bounds__(256, 1) void chol_update_kernel(double* __restrict__ A, long n, long k, int kb, long r0) {
  __shared__ double Pi[kKc][kTile + 2];
  __shared__ double Pj[kKc][kTile + 2];
  // linear block index -> (ti, tj) of the lower triangle
  const long t = blockIdx.x;
  long ti = long((sqrt(8.0 * double(t) + 1.0) - 1.0) * 0.5);
  while ((ti + 1) * (ti + 2) / 2 <= t) ++ti;
  while (ti * (ti + 1) / 2 > t) --ti;
  const long tj = t - ti * (ti + 1) / 2;
  const long i0 = r0 + ti * kTile, j0 = r0 + tj * kTile;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  double acc[8][8];
#pragma unroll
  for (int a = 0; a < 8; ++a)
#pragma unroll
    for (int b = 0; b < 8; ++b) acc[a][b] = 0.0;
  // staging: thread -> (row = tid / 2, eight consecutive panel columns (tid & 1) * 8 ..)
  const int srow = threadIdx.x >> 1, scol = (threadIdx.x & 1) * 8;
  const bool vi = i0 + srow < n, vj = j0 + srow < n;
  const double* gi = A + (i0 + srow) * n + k + scol;
  const double* gj = A + (j0 + srow) * n + k + scol;
  double ri[8], rj[8];
  auto fetch = [&](int c0) {
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const bool in = c0 + scol + q < kb;
      ri[q] = (vi && in) ? gi[c0 + q] : 0.0;
      rj[q] = (vj && in) ? gj[c0 + q] : 0.0;
    }
  };
  auto stash = [&]() {
#pragma unroll
    for (int q = 0; q < 8; ++q) Pi[scol + q][srow] = ri[q], Pj[scol + q][srow] = rj[q];
  };
  fetch(0);
  stash();
  __syncthreads();
  const int slices = (kb + kKc - 1) / kKc;
  for (int s = 0; s < slices; ++s) {
    if (s + 1 < slices) fetch((s + 1) * kKc);  // the next slice travels to registers under this slice's arithmetic
#pragma unroll
    for (int p = 0; p < kKc; ++p) {
      double a[8], b[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) a[q] = Pi[p][ty + 16 * q], b[q] = Pj[p][tx + 16 * q];
#pragma unroll
      for (int x = 0; x < 8; ++x)
#pragma unroll
        for (int y = 0; y < 8; ++y) acc[x][y] = fma(a[x], b[y], acc[x][y]);
    }
    __syncthreads();
    if (s + 1 < slices) {
      stash();
      __syncthreads();
    }
  }
#pragma unroll
  for (int x = 0; x < 8; ++x) {
    const long i = i0 + ty + 16 * x;
    if (i >= n) continue;
#pragma unroll
    for (int y = 0; y < 8; ++y) {
      const long j = j0 + tx + 16 * y;
      if (j <= i) A[i * n + j] -= acc[x][y];
    }
  }
}

// inv[b] = inverse of the lower-triangular 16 x 16 diagonal block b of C; thread c of a 16-thread group solves column c.
__global__ void ldl_block_inverse_kernel(const double* __restrict__ A, long n, double* __restrict__ inv) {
  const long b = long(blockIdx.x) * (blockDim.x / 16) + threadIdx.x / 16;
  const int c = threadIdx.x & 15;
  if (b * 16 >= n) return;
  const double* D = A + (b * 16) * n + b * 16;
  double col[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    double s = (i == c) ? 1.0 : 0.0;
#pragma unroll
    for (int p = 0; p < 16; ++p)
      if (p < i) s = fma(-D[i * n + p], col[p], s);
    col[i] = s / D[i * n + i];
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) inv[b * 256 + i * 16 + c] = col[i];
}

// L[r][16 bj + j] = sum_{p = j}^{15} C[r][16 bj + p] inv[bj][p][j] for bj < r / 16, zero on and above the diagonal
// block. One thread per (row, column block); fp32 result, optionally the fp64 value beside it.
__global__ __launch_bounds__(128) void ldl_finish_kernel(const double* __restrict__ A, const double* __restrict__ inv,
                                                         long n, float* __restrict__ L, double* __restrict__ L64,
                                                         int* status) {
  const long nb = n / 16;
  const long r = blockIdx.y;
  const long bj = long(blockIdx.x) * blockDim.x + threadIdx.x;
  if (bj >= nb) return;
  float4* out = reinterpret_cast<float4*>(L + r * n + bj * 16);
  double o[16];
  if (bj >= r / 16) {
#pragma unroll
    for (int j = 0; j < 16; ++j) o[j] = 0.0;
  } else {
    const double* a = A + r * n + bj * 16;
    const double* iv = inv + bj * 256;
    double av[16];
#pragma unroll
    for (int p = 0; p < 16; ++p) av[p] = a[p];
    bool finite = true;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      double s = 0.0;
#pragma unroll
      for (int p = 0; p < 16; ++p)
        if (p >= j) s = fma(av[p], iv[p * 16 + j], s);
      o[j] = s;
      finite = finite && isfinite(s);
    }
    if (!finite) atomicOr(status, 2);
  }
#pragma unroll
  for (int q = 0; q < 4; ++q)
    out[q] = make_float4(float(o[4 * q]), float(o[4 * q + 1]), float(o[4 * q + 2]), float(o[4 * q + 3]));
  if (L64) {
#pragma unroll
    for (int j = 0; j < 16; ++j) L64[r * n + bj * 16 + j] = o[j];
  }
}

static size_t align256(size_t x) { return (x + 255) / 256 * 256; }
constexpr size_t kDiagSmem = size_t(kNb) * (kNb + 1) * 8;
constexpr size_t kPanelSmem = size_t(kNb + kPanelRows) * (kNb + 1) * 8;

int block_ldl_device_setup() {
  QB_CUDA(cudaFuncSetAttribute(chol_diag_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kDiagSmem)));
  QB_CUDA(cudaFuncSetAttribute(chol_panel_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kPanelSmem)));
  return QTIP_OK;
}

}  // namespace qb

using namespace qb;

extern "C" size_t qtip_block_ldl_workspace_bytes(long n) {
  if (n <= 0) return 0;
  return sizeof(LdlHeader) + align256(size_t(n) * n * 8) + align256(size_t(n / 16) * 256 * 8);
}

extern "C" int qtip_block_ldl(const float* HR_d, long n, float* L_d, double* L64_d, void* workspace_d,
                              size_t workspace_bytes, void* stream) {
  QB_REQUIRE(HR_d && L_d && workspace_d, QTIP_E_ARG, "qtip_block_ldl: null pointer");
  QB_REQUIRE(n > 0 && n % 16 == 0, QTIP_E_GEOMETRY, "qtip_block_ldl: n = %ld must be a positive multiple of 16", n);
  QB_REQUIRE(workspace_bytes >= qtip_block_ldl_workspace_bytes(n), QTIP_E_WORKSPACE,
             "qtip_block_ldl: workspace of %zu bytes is too small (need %zu)", workspace_bytes,
             qtip_block_ldl_workspace_bytes(n));
  QB_REQUIRE(reinterpret_cast<uintptr_t>(L_d) % 16 == 0, QTIP_E_ARG, "qtip_block_ldl: L_d must be 16-byte aligned");
  if (!device_info()) return QTIP_E_DEVICE;
  cudaStream_t s = as_stream(stream);
  unsigned char* p = static_cast<unsigned char*>(workspace_d);
  int* status = reinterpret_cast<int*>(p);
  double* A = reinterpret_cast<double*>(p + sizeof(LdlHeader));
  double* inv = reinterpret_cast<double*>(p + sizeof(LdlHeader) + align256(size_t(n) * n * 8));
  QB_CUDA(cudaMemsetAsync(status, 0, sizeof(LdlHeader), s));
  {
    const unsigned g = blocks_for(n, 32);
    ldl_symmetrise_kernel<<<dim3(g, g), dim3(32, 8), 0, s>>>(HR_d, A, n);
    QB_LAUNCHED();
  }
  for (long k = 0; k < n; k += kNb) {
    const int kb = int(min(long(kNb), n - k));
    chol_diag_kernel<<<1, 256, kDiagSmem, s>>>(A, n, k, kb, status);
    QB_LAUNCHED();
    const long r0 = k + kb, nr = n - r0;
    if (nr <= 0) break;
    chol_panel_kernel<<<blocks_for(nr, kPanelRows), kPanelRows, kPanelSmem, s>>>(A, n, k, kb);
    QB_LAUNCHED();
    const long tiles = (nr + kTile - 1) / kTile;
    chol_update_kernel<<<unsigned(tiles * (tiles + 1) / 2), 256, 0, s>>>(A, n, k, kb, r0);
    QB_LAUNCHED();
  }
  ldl_block_inverse_kernel<<<blocks_for(n / 16, 8), 128, 0, s>>>(A, n, inv);
  QB_LAUNCHED();
  ldl_finish_kernel<<<dim3(blocks_for(n / 16, 128), unsigned(n)), 128, 0, s>>>(A, inv, n, L_d, L64_d, status);
  QB_LAUNCHED();
  return QTIP_OK;
}

extern "C" int qtip_block_ldl_status(const void* workspace_d, void* stream) {
  QB_REQUIRE(workspace_d, QTIP_E_ARG, "qtip_block_ldl_status: null workspace");
  int st = 0;
  QB_CUDA(cudaMemcpyAsync(&st, workspace_d, 4, cudaMemcpyDeviceToHost, as_stream(stream)));
  QB_CUDA(cudaStreamSynchronize(as_stream(stream)));
  QB_REQUIRE((st & 1) == 0, QTIP_E_NUMERIC, "block LDL: the matrix is not positive definite (a pivot was <= 0)");
  QB_REQUIRE((st & 2) == 0, QTIP_E_NUMERIC, "block LDL: non-finite values in the factor");
  return QTIP_OK;
}
