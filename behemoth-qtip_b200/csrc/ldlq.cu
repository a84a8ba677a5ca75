// LDLQ error feedback around the Viterbi quantiser (128-column buffers, 16-column blocks, right to left).
//
//  * ldlq_prep_kernel: feedback inside the current buffer, fp32 FMA with k ascending exactly as the reference's
//    ldlq_prep_kernel (src/viterbi.hip:241-267), so the sequences handed to the Viterbi are bit-identical given
//    identical inputs. 32 rows x 16 columns per CTA, both operand panels staged in shared memory, two chains per thread.
//  * ldlq_update_kernel: cross-buffer update prod[r][j] += sum_k L[k][r] (WT[k][j] - hatWT[k][j]) over the 128 rows k of
//    the finished buffer, r < c0. The reference does this with a split-bf16 library GEMM (src/quantizer.cpp:64-76); here
//    every element is one thread's fp32 FMA chain over k ascending, which is deterministic and at least as accurate.
//    128 x 128 output tile per CTA, 8 x 8 per thread, the 128-deep operand panels staged through shared memory.
//  * qtip_ldlq: the schedule of ldlq_gpu (src/quantizer.cpp:30-89) on one stream, restricted to a slice of W rows.
#include <cmath>
#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace qb {

int quantize_tiles_impl(const float* X, int B, int b0, const uint32_t* lut, uint16_t* Q, int nblk, int blk, float* hat,
                        float* hatWT, long m, int col0, void* ws, size_t ws_bytes, bool reset_status, cudaStream_t s,
                        bool two_lanes);  // viterbi.cu

// Rows j in [j0, j0 + mj) of W; X is indexed from the slice start: X[(j - j0) >> 4][256].
// A CTA owns 32 rows of W and the block's 16 columns: the (up to 112) rows of L that reach into the block and the
// matching differences WT - hatWT of its 32 rows are staged in shared memory once (coalesced along j), then thread
// (row, column pair) runs its two fused multiply-add chains over k ascending -- the order the reference fixes
// (src/viterbi.hip:241-267), so every element has the reference's bits -- with conflict-free shared reads (a warp is 32
// consecutive rows of one column pair). m / 32 CTAs of 256 threads: 48 CTAs for the 1,536-row shard of an 8-GPU split,
// where one thread per row would leave 142 SMs idle and run 16 chains in each thread.
constexpr int kPrepRows = 32;
__global__ __launch_bounds__(256) void ldlq_prep_kernel(const float* __restrict__ WT, const float* __restrict__ hatWT,
                                                        const float* __restrict__ prod, const float* __restrict__ L,
                                                        long n, long m, long j0, long mj, int col0, int bufend,
                                                        float* __restrict__ X) {
  __shared__ float Ls[112][16];
  __shared__ float Ds[112][kPrepRows];
  const int k0 = col0 + 16, nk = bufend - k0;
  const long jb = j0 + long(blockIdx.x) * kPrepRows;
  const long left = j0 + mj - jb;
  const int rows = left < kPrepRows ? int(left) : kPrepRows;
  for (int idx = threadIdx.x; idx < nk * 16; idx += blockDim.x)
    Ls[idx >> 4][idx & 15] = L[long(k0 + (idx >> 4)) * n + col0 + (idx & 15)];
  for (int idx = threadIdx.x; idx < nk * kPrepRows; idx += blockDim.x) {
    const int k = idx / kPrepRows, jj = idx % kPrepRows;
    const long o = long(k0 + k) * m + jb + jj;
    Ds[k][jj] = jj < rows ? __fsub_rn(WT[o], hatWT[o]) : 0.f;
  }
  __syncthreads();
  const int jj = threadIdx.x % kPrepRows, c = 2 * (threadIdx.x / kPrepRows);
  if (jj >= rows) return;
  const long j = jb + jj;
  float a0 = __fadd_rn(WT[long(col0 + c) * m + j], prod[long(col0 + c) * m + j]);
  float a1 = __fadd_rn(WT[long(col0 + c + 1) * m + j], prod[long(col0 + c + 1) * m + j]);
  for (int kk = 0; kk < nk; ++kk) {
    const float dk = Ds[kk][jj];
    a0 = __fmaf_rn(Ls[kk][c], dk, a0);
    a1 = __fmaf_rn(Ls[kk][c + 1], dk, a1);
  }
  const long jl = j - j0;
  float* xb = X + (jl >> 4) * 256;
  const int r = int(jl & 15);
  xb[perm_inv(r * 16 + c)] = a0;
  xb[perm_inv(r * 16 + c + 1)] = a1;
}

constexpr int kUpTile = 128, kUpK = 128, kUpKc = 16;
// prod[r][j] (r < c0, j in the slice) += sum_{k=c0}^{c0+127} L[k][r] * (WT[k][j] - hatWT[k][j])
__global__ __launch_bounds__(256) void ldlq_update_kernel(const float* __restrict__ WT, const float* __restrict__ hatWT,
                                                          const float* __restrict__ L, float* __restrict__ prod, long n,
                                                          long m, long j0, long mj, int c0) {
  __shared__ float Ls[kUpKc][kUpTile];  // L[c0 + k][r0 + r]
  __shared__ float Ds[kUpKc][kUpTile];  // (WT - hatWT)[c0 + k][jb + j]
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads, 8 x 8 outputs each (strided by 16)
  const long r0 = long(blockIdx.y) * kUpTile, jb = j0 + long(blockIdx.x) * kUpTile;
  float acc[8][8];
#pragma unroll
  for (int a = 0; a < 8; ++a)
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const long r = r0 + ty + 16 * a, j = jb + tx + 16 * b;
      acc[a][b] = (r < c0 && j < j0 + mj) ? prod[r * m + j] : 0.f;
    }
  for (int kc = 0; kc < kUpK; kc += kUpKc) {
    for (int idx = threadIdx.x; idx < kUpKc * kUpTile; idx += 256) {
      const int k = idx / kUpTile, x = idx % kUpTile;
      const long kr = c0 + kc + k;
      Ls[k][x] = (r0 + x < c0) ? L[kr * n + r0 + x] : 0.f;
      const long j = jb + x;
      Ds[k][x] = (j < j0 + mj) ? __fsub_rn(WT[kr * m + j], hatWT[kr * m + j]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kUpKc; ++k) {
      float lv[8], dv[8];
#pragma unroll
      for (int a = 0; a < 8; ++a) lv[a] = Ls[k][ty + 16 * a];
#pragma unroll
      for (int b = 0; b < 8; ++b) dv[b] = Ds[k][tx + 16 * b];
#pragma unroll
      for (int a = 0; a < 8; ++a)
#pragma unroll
        for (int b = 0; b < 8; ++b) acc[a][b] = __fmaf_rn(lv[a], dv[b], acc[a][b]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int a = 0; a < 8; ++a)
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const long r = r0 + ty + 16 * a, j = jb + tx + 16 * b;
      if (r < c0 && j < j0 + mj) prod[r * m + j] = acc[a][b];
    }
}

// Zeroes columns [j0, j0 + mj) of an n x m matrix.
__global__ void zero_cols_kernel(float* A, long n, long m, long j0, long mj) {
  const long total = n * mj;
  for (long i = long(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += long(gridDim.x) * blockDim.x) {
    const long r = i / mj;
    A[r * m + j0 + (i - r * mj)] = 0.f;
  }
}

static size_t align256(size_t x) { return (x + 255) / 256 * 256; }

}  // namespace qb

using namespace qb;

extern "C" int qtip_k_ldlq_prep(const float* WT_d, const float* hatWT_d, const float* prod_d, const float* L_d, long n,
                                long m, int col0, int bufend, float* X_d, void* stream) {
  QB_REQUIRE(WT_d && hatWT_d && prod_d && L_d && X_d && n > 0 && m > 0, QTIP_E_ARG, "qtip_k_ldlq_prep: bad argument");
  QB_REQUIRE(bufend - col0 - 16 <= 112 && bufend - col0 - 16 >= 0 && col0 >= 0 && bufend <= n, QTIP_E_GEOMETRY,
             "qtip_k_ldlq_prep: block [%d, %d) is not inside a 128-column buffer", col0, bufend);
  ldlq_prep_kernel<<<blocks_for(m, kPrepRows), 256, 0, as_stream(stream)>>>(WT_d, hatWT_d, prod_d, L_d, n, m, 0, m, col0,
                                                                      bufend, X_d);
  QB_LAUNCHED();
  return QTIP_OK;
}

// Row slices of one call run as independent chains on side streams (rows of W never interact): while one slice is in
// the last, partly filled round of a Viterbi launch, or in its small prep / backtrace / update kernels, the other
// slices' launches fill the idle clusters.
constexpr int kMaxSlices = 4;
static int ldlq_slices(long ntr) {
  if (const char* e = std::getenv("QTIP_LDLQ_SLICES")) {
    const int v = std::atoi(e);
    if (v >= 1 && v <= kMaxSlices) return ntr >= v ? v : 1;
  }
  return ntr >= 128 ? 2 : 1;  // measured: 192 sequences per step 2.13 s -> 1.64 s, 768: 7.0 -> 5.97 s, 96: no difference
}
static size_t slice_ws_bytes(long ntr, int slices) {  // Viterbi scratch of all slices together
  size_t total = 0;
  for (int i = 0; i < slices; ++i) total += qtip_quantize_workspace_bytes(int(ntr * (i + 1) / slices - ntr * i / slices));
  return total;
}
struct SideStreams {
  cudaStream_t stream[kMaxSlices - 1] = {};
  cudaEvent_t fork = nullptr, join[kMaxSlices - 1] = {};
  bool ready = false;
};
static std::mutex g_side_mu;
static SideStreams g_side[64];
static int side_streams(SideStreams** out) {
  int dev = 0;
  QB_CUDA(cudaGetDevice(&dev));
  QB_REQUIRE(dev >= 0 && dev < 64, QTIP_E_DEVICE, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_side_mu);
  SideStreams& sd = g_side[dev];
  if (!sd.ready) {
    QB_CUDA(cudaEventCreateWithFlags(&sd.fork, cudaEventDisableTiming));
    for (int i = 0; i < kMaxSlices - 1; ++i) {
      QB_CUDA(cudaStreamCreateWithFlags(&sd.stream[i], cudaStreamNonBlocking));
      QB_CUDA(cudaEventCreateWithFlags(&sd.join[i], cudaEventDisableTiming));
    }
    sd.ready = true;
  }
  *out = &sd;
  return QTIP_OK;
}
__global__ void merge_status_kernel(int* dst, const int* src) {
  if (*src) atomicOr(dst, *src);
}

extern "C" size_t qtip_ldlq_workspace_bytes(long n, long m) {
  if (n <= 0 || m <= 0) return 0;
  const long ntr = m / 16;
  return slice_ws_bytes(ntr, kMaxSlices) + align256(size_t(n) * m * 4) + align256(size_t(ntr) * 256 * 4);
}

extern "C" int qtip_ldlq(const float* WT_d, const float* L_d, long n, long m, long j0, long mj, float* hatWT_d,
                         uint16_t* Q_d, const uint32_t* lut_h2_d, void* workspace_d, size_t workspace_bytes,
                         void* stream) {
  QB_REQUIRE(WT_d && L_d && hatWT_d && Q_d && lut_h2_d && workspace_d, QTIP_E_ARG, "qtip_ldlq: null pointer");
  QB_REQUIRE(n > 0 && n % 128 == 0, QTIP_E_GEOMETRY, "LDLQ needs n %% 128 == 0 (n = %ld)", n);
  QB_REQUIRE(m > 0 && m % 16 == 0, QTIP_E_GEOMETRY, "LDLQ needs m %% 16 == 0 (m = %ld)", m);
  QB_REQUIRE(j0 >= 0 && mj > 0 && j0 % 16 == 0 && mj % 16 == 0 && j0 + mj <= m, QTIP_E_GEOMETRY,
             "LDLQ row slice [%ld, %ld) must be whole 16-row blocks inside m = %ld", j0, j0 + mj, m);
  cudaStream_t s = as_stream(stream);
  // Workspace: [Viterbi scratch of every slice, slice 0 (with the status word the caller reads) first][prod, full n x m
  // extent, only the slice's columns are touched][the sequences]. qtip_workspace_status() therefore works on an LDLQ
  // workspace too.
  const int ntr = int(mj / 16), nblk = int(n / 16);
  const int slices = ldlq_slices(ntr);
  const size_t prod_bytes = align256(size_t(n) * m * 4), x_bytes = align256(size_t(ntr) * 256 * 4);
  const size_t vws_bytes = slice_ws_bytes(ntr, slices);
  QB_REQUIRE(workspace_bytes >= vws_bytes + prod_bytes + x_bytes, QTIP_E_WORKSPACE,
             "qtip_ldlq: workspace of %zu bytes is too small (need %zu)", workspace_bytes,
             vws_bytes + prod_bytes + x_bytes);
  unsigned char* p = static_cast<unsigned char*>(workspace_d);
  float* prod = reinterpret_cast<float*>(p + vws_bytes);
  float* X = reinterpret_cast<float*>(p + vws_bytes + prod_bytes);
  struct Slice {
    long j0, mj;
    int ntr;
    float* X;
    void* vws;
    size_t vws_bytes;
    cudaStream_t st;
  } sl[kMaxSlices];
  SideStreams* side = nullptr;
  if (slices > 1) {
    int rc = side_streams(&side);
    if (rc) return rc;
  }
  size_t off = 0;
  for (int i = 0; i < slices; ++i) {
    const long t0 = long(ntr) * i / slices, t1 = long(ntr) * (i + 1) / slices;
    sl[i].j0 = j0 + 16 * t0, sl[i].mj = 16 * (t1 - t0), sl[i].ntr = int(t1 - t0);
    sl[i].X = X + size_t(t0) * 256;
    sl[i].vws = p + off, sl[i].vws_bytes = qtip_quantize_workspace_bytes(sl[i].ntr);
    off += sl[i].vws_bytes;
    sl[i].st = i == 0 ? s : side->stream[i - 1];
    QB_CUDA(cudaMemsetAsync(sl[i].vws, 0, 256, s));  // the slice's status word; it accumulates over all column steps
  }
  zero_cols_kernel<<<148 * 8, 256, 0, s>>>(prod, n, m, j0, mj);
  QB_LAUNCHED();
  zero_cols_kernel<<<148 * 8, 256, 0, s>>>(hatWT_d, n, m, j0, mj);
  QB_LAUNCHED();
  if (slices > 1) {
    QB_CUDA(cudaEventRecord(side->fork, s));
    for (int i = 1; i < slices; ++i) QB_CUDA(cudaStreamWaitEvent(sl[i].st, side->fork, 0));
  }
  // The column loop as a function: a failed launch still passes the join below, so the side streams are never left
  // running (or a stream capture left forked) behind an error return.
  auto columns = [&]() -> int {
    for (long cur = n / 16; cur > 0; cur -= 8) {
      const int bufend = int(16 * cur), c0 = bufend - 128;
      for (int i = 7; i >= 0; --i) {
        const int col0 = c0 + 16 * i;
        for (int q = 0; q < slices; ++q) {  // the same column step of every slice, each on its own stream
          const Slice& a = sl[q];
          ldlq_prep_kernel<<<blocks_for(a.mj, kPrepRows), 256, 0, a.st>>>(WT_d, hatWT_d, prod, L_d, n, m, a.j0, a.mj, col0,
                                                                   bufend, a.X);
          QB_LAUNCHED();
          int rc = quantize_tiles_impl(a.X, a.ntr, int(a.j0 / 16), lut_h2_d, Q_d, nblk, col0 / 16, nullptr, hatWT_d, m,
                                       col0, a.vws, a.vws_bytes, false, a.st, false);
          if (rc) return rc;
        }
      }
      if (c0 > 0) {
        for (int q = 0; q < slices; ++q) {
          const Slice& a = sl[q];
          const dim3 grid(blocks_for(a.mj, kUpTile), blocks_for(c0, kUpTile));
          ldlq_update_kernel<<<grid, 256, 0, a.st>>>(WT_d, hatWT_d, L_d, prod, n, m, a.j0, a.mj, c0);
          QB_LAUNCHED();
        }
      }
    }
    return QTIP_OK;
  };
  const int rc_columns = columns();
  for (int i = 1; i < slices; ++i) {
    QB_CUDA(cudaEventRecord(side->join[i - 1], sl[i].st));
    QB_CUDA(cudaStreamWaitEvent(s, side->join[i - 1], 0));
    if (rc_columns == QTIP_OK) {
      merge_status_kernel<<<1, 1, 0, s>>>(static_cast<int*>(sl[0].vws), static_cast<const int*>(sl[i].vws));
      QB_LAUNCHED();
    }
  }
  return rc_columns;
}

// ---------------------------------------------------------------- one linear of a Hessian group, end to end
// The per-linear body of quantize_group (src/quantizer.cpp:236-320) on one stream: random-Hadamard rotation of W on both
// sides, Wscale from the rotated rms, LDLQ + Viterbi, bit packing and the kernel layout. Workspace:
// [LDLQ workspace][packed words][one double].
static size_t packed_bytes(long m, long n) { return align256(size_t(m / 16) * (n / 16) * 32 * 2); }

extern "C" size_t qtip_quantize_linear_workspace_bytes(long m, long n) {
  if (m <= 0 || n <= 0) return 0;
  return qtip_ldlq_workspace_bytes(n, m) + packed_bytes(m, n) + 256;
}

extern "C" int qtip_quantize_linear(float* W_d, const float* L_d, long m, long n, const float* su_d, const float* sv_d,
                                    const uint32_t* lut_h2_d, double lut_rms, double scale_override, float* WT_d,
                                    float* hatWT_d, uint16_t* Q_d, uint16_t* trellis_d, float* wscale_out,
                                    void* workspace_d, size_t workspace_bytes, void* stream) {
  QB_REQUIRE(W_d && L_d && su_d && sv_d && lut_h2_d && WT_d && hatWT_d && Q_d && trellis_d && wscale_out && workspace_d,
             QTIP_E_ARG, "qtip_quantize_linear: null pointer");
  QB_REQUIRE(m > 0 && n > 0 && m % 32 == 0 && n % 128 == 0, QTIP_E_GEOMETRY,
             "qtip_quantize_linear needs m %% 32 == 0 and n %% 128 == 0 (m = %ld, n = %ld)", m, n);
  QB_REQUIRE(lut_rms > 0 && scale_override > 0, QTIP_E_ARG, "qtip_quantize_linear: lut_rms and scale_override must be > 0");
  const size_t ldlq_bytes = qtip_ldlq_workspace_bytes(n, m), pk_bytes = packed_bytes(m, n);
  QB_REQUIRE(workspace_bytes >= ldlq_bytes + pk_bytes + 256, QTIP_E_WORKSPACE,
             "qtip_quantize_linear: workspace of %zu bytes is too small (need %zu)", workspace_bytes,
             ldlq_bytes + pk_bytes + 256);
  unsigned char* p = static_cast<unsigned char*>(workspace_d);
  uint16_t* packed = reinterpret_cast<uint16_t*>(p + ldlq_bytes);
  double* acc = reinterpret_cast<double*>(p + ldlq_bytes + pk_bytes);
  cudaStream_t s = as_stream(stream);
  int rc;
  // Wr = T_m^T diag(SV) W diag(SU) T_n, kept transposed (n x m) for the column-wise LDLQ
  if ((rc = qtip_k_scale_rows_cols(W_d, m, n, n, sv_d, su_d, stream))) return rc;
  if ((rc = qtip_k_hadamard_rows(W_d, m, int(n), n, 1, stream))) return rc;
  if ((rc = qtip_k_transpose(W_d, m, n, n, WT_d, m, stream))) return rc;
  if ((rc = qtip_k_hadamard_rows(WT_d, n, int(m), m, 1, stream))) return rc;
  QB_CUDA(cudaMemsetAsync(acc, 0, sizeof(double), s));
  if ((rc = qtip_k_sumsq(WT_d, n, m, m, acc, stream))) return rc;
  double sumsq = 0;
  QB_CUDA(cudaMemcpyAsync(&sumsq, acc, sizeof sumsq, cudaMemcpyDeviceToHost, s));
  QB_CUDA(cudaStreamSynchronize(s));  // the reference reads the rms back at the same point
  const double rms = std::sqrt(sumsq / (double(n) * double(m)));
  const float wscale = float(rms / (double(float(lut_rms)) * scale_override));
  QB_REQUIRE(wscale > 0 && std::isfinite(wscale), QTIP_E_ARG, "qtip_quantize_linear: the rotated weights have rms %g", rms);
  *wscale_out = wscale;
  if ((rc = qtip_k_scale(WT_d, n, m, m, float(1.0 / double(wscale)), stream))) return rc;
  if ((rc = qtip_ldlq(WT_d, L_d, n, m, 0, m, hatWT_d, Q_d, lut_h2_d, workspace_d, ldlq_bytes, stream))) return rc;
  const long tiles = (m / 16) * (n / 16);
  if ((rc = qtip_pack_trellis(Q_d, tiles, packed, stream))) return rc;
  return qtip_swizzle_for_kernel(packed, int(m), int(n), trellis_d, stream);
}

// Hessian side of a group (src/quantizer.cpp:124-152): damping by sigma_reg * mean(diag), then the rotation
// HR = T_n^T diag(SU) H diag(SU) T_n with the same row transform applied to both sides through a transpose.
extern "C" int qtip_rotate_hessian(float* H_d, long n, const float* su_d, double sigma_reg, float* HR_d, double* creg_out,
                                   double* scratch_d, void* stream) {
  QB_REQUIRE(H_d && su_d && HR_d && creg_out && scratch_d && n > 0, QTIP_E_ARG, "qtip_rotate_hessian: bad argument");
  cudaStream_t s = as_stream(stream);
  int rc;
  QB_CUDA(cudaMemsetAsync(scratch_d, 0, sizeof(double), s));
  if ((rc = qtip_k_diag_sum(H_d, n, scratch_d, stream))) return rc;
  double tr = 0;
  QB_CUDA(cudaMemcpyAsync(&tr, scratch_d, sizeof tr, cudaMemcpyDeviceToHost, s));
  QB_CUDA(cudaStreamSynchronize(s));  // the reference reads the trace back at the same point
  const double creg = sigma_reg * tr / double(n);
  *creg_out = creg;
  if ((rc = qtip_k_add_diag(H_d, n, float(creg), stream))) return rc;
  if ((rc = qtip_k_scale_rows_cols(H_d, n, n, n, su_d, su_d, stream))) return rc;
  if ((rc = qtip_k_hadamard_rows(H_d, n, int(n), n, 1, stream))) return rc;
  if ((rc = qtip_k_transpose(H_d, n, n, n, HR_d, n, stream))) return rc;
  return qtip_k_hadamard_rows(HR_d, n, int(n), n, 1, stream);
}
