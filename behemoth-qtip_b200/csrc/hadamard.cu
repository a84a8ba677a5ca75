// Random-Hadamard transforms x <- (hadK^(T) (x) H_P) x / sqrt(n), n = K * P, K in {1, 12, 20, 28}, P a power of two.
//
// (hadK (x) H_P) = (I (x) H_P)(hadK (x) I): the order-K mix across the K chunks is done first, then a natural-order
// fast Walsh-Hadamard transform on each chunk of P. Every variant below uses that order and the same summation order,
// so the whole-row kernel and the chunk-per-CTA kernel give identical bits.
//
//  * had_row_kernel: one CTA per row, the whole row (up to 57,344 floats = 224 KiB) in shared memory, read and written
//    once. Used for the quantizer's fp32 matrices and for prefill-sized token batches.
//  * had_chunk_kernel: K CTAs per row, each mixing its own chunk from the full row (served by L2) and transforming it.
//    No inter-CTA step; used for a few tokens where latency, not traffic, decides.
//
// Sources/destinations (Mode): fp32 in place (quantizer); bf16 x times SU -> bf16 (operator input); fp32 partial
// products summed over K-splits, optionally rounded to bf16 -> times SV -> bf16 (operator output); bf16 z -> same.
#include <cmath>

#include <cstdlib>

#include "common.cuh"

namespace qb {

// ---- compile-time signs of the order-12/20 (Paley I) and order-28 (Paley II) factors
__host__ __device__ constexpr int chi_c(int a, int p) {
  a = ((a % p) + p) % p;
  if (a == 0) return 0;
  for (int x = 1; x < p; ++x)
    if ((x * x) % p == a) return 1;
  return -1;
}
template <int K>
__host__ __device__ constexpr int had_sign(int i, int j) {
  if constexpr (K == 1) {
    return 1;
  } else if constexpr (K == 12 || K == 20) {
    constexpr int q = K - 1;
    if (i == 0) return j == 0 ? 1 : -1;
    if (j == 0) return 1;
    const int k = ((j - i) % q + q) % q;
    return k == 0 ? 1 : -chi_c(k, q);
  } else {
    static_assert(K == 28, "unsupported Hadamard order");
    constexpr int q = 13, h = 14;
    const int bi = i / h, bj = j / h, r = i % h, c = j % h;
    const bool core = r >= 1 && c >= 1;
    const int k = ((c - r) % q + q) % q;
    const int x = (core && k != 0) ? chi_c(k, q) : 0;
    if (bi == 0 && bj == 0) return !core ? 1 : (k == 0 ? 1 : x);
    if (bi != bj) return r == 0 ? (c == 0 ? -1 : 1) : (c == 0 ? 1 : (k == 0 ? -1 : x));
    return !core ? -1 : (k == 0 ? -1 : -x);
  }
}
// Sign masks: bit k of kRowMask<K,T>[r] is set where the mixing matrix entry (r, k) is -1 (T: transposed factor).
template <int K, bool T>
struct SignMasks {
  uint32_t m[K];
  constexpr SignMasks() : m{} {
    for (int r = 0; r < K; ++r) {
      uint32_t v = 0;
      for (int k = 0; k < K; ++k)
        if ((T ? had_sign<K>(k, r) : had_sign<K>(r, k)) < 0) v |= 1u << k;
      m[r] = v;
    }
  }
};

enum class Mode { F32Inplace, Prepare, Finish, FinishB16 };

struct HadArgs {
  const void* src;    // fp32 or bf16
  void* dst;          // fp32 (in place) or bf16
  const float* sign;  // SU (Prepare) or SV (Finish*), else null
  long ld;            // row stride of src/dst in elements
  long split_stride;  // Finish: elements between K-split partials
  int n, P;
  int splits, round_z;
  int ranks;  // > 1: the source is gathered rank-major, [rank][row][n / ranks]
  int rows;
  float scale;
};

// Element offset of column element j of `row` relative to the source base: row-major, or [rank][row][n / ranks] when
// the source was gathered from `ranks` ranks.
__device__ __forceinline__ long src_offset(const HadArgs& a, long row, int j) {
  if (a.ranks <= 1) return row * a.ld + j;
  const int part = a.n / a.ranks, r = j / part;
  return (long(r) * a.rows + row) * part + (j - r * part);
}
template <Mode M>
__device__ __forceinline__ float load_one(const void* src, long at) {
  if constexpr (M == Mode::F32Inplace || M == Mode::Finish) return static_cast<const float*>(src)[at];
  else return bf16_to_f32(static_cast<const uint16_t*>(src)[at]);
}
// The K source values of column i (elements k P + i), loaded as one batch: the K loads of a pass are independent
// straight-line code, so they are all in flight together (per-element control flow around each load would serialise
// them on memory latency). K-split partials are added in split order, then optionally rounded to bf16.
template <int K, Mode M>
__device__ __forceinline__ void load_column(const HadArgs& a, long row, int i, int P, float (&v)[K]) {
  if (a.ranks <= 1) {
    const long base = row * a.ld + i;
#pragma unroll
    for (int k = 0; k < K; ++k) v[k] = load_one<M>(a.src, base + k * P);
    if constexpr (M == Mode::Finish) {
      for (int p = 1; p < a.splits; ++p) {
        const float* zp = static_cast<const float*>(a.src) + size_t(p) * a.split_stride + base;
#pragma unroll
        for (int k = 0; k < K; ++k) {
          v[k] += zp[k * P];
          if (k % 8 == 7) asm volatile("" ::: "memory");  // at most 8 partial loads in flight: bounds register use
        }
      }
    }
  } else {
    // gathered source: a chunk never straddles two ranks' parts (n / ranks is a multiple of P), so one offset per chunk
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const long at = src_offset(a, row, k * P + i);
      float x = load_one<M>(a.src, at);
      if constexpr (M == Mode::Finish)
        for (int p = 1; p < a.splits; ++p) x += static_cast<const float*>(a.src)[size_t(p) * a.split_stride + at];
      v[k] = x;
      if (k % 4 == 3) asm volatile("" ::: "memory");
    }
  }
  if constexpr (M == Mode::Prepare) {
#pragma unroll
    for (int k = 0; k < K; ++k) v[k] *= a.sign[k * P + i];
  }
  if constexpr (M == Mode::Finish) {
    if (a.round_z) {
#pragma unroll
      for (int k = 0; k < K; ++k) v[k] = bf16_to_f32(f32_to_bf16(v[k]));
    }
  }
}
template <Mode M>
__device__ __forceinline__ void store_dst(const HadArgs& a, long row, int j, float v) {
  const long at = row * a.ld + j;
  if constexpr (M == Mode::F32Inplace) {
    static_cast<float*>(a.dst)[at] = v * a.scale;
  } else if constexpr (M == Mode::Prepare) {
    static_cast<uint16_t*>(a.dst)[at] = f32_to_bf16(v * a.scale);
  } else {
    static_cast<uint16_t*>(a.dst)[at] = f32_to_bf16(v * a.scale * a.sign[j]);
  }
}

// Natural-order FWHT on `count` contiguous chunks of P floats in shared memory (any power-of-two P). All threads of the
// CTA take part. Used for chunk lengths the register path below does not cover.
__device__ __forceinline__ void fwht_shared(float* a, int P, int count) {
  const int half = (P * count) >> 1;
  int lg = 0;
  for (int h = 1; h < P; h <<= 1, ++lg) {
    for (int t = threadIdx.x; t < half; t += blockDim.x) {
      const int i = ((t >> lg) << (lg + 1)) | (t & (h - 1));  // chunks are multiples of 2h: never straddles two chunks
      const float v = a[i], w = a[i + h];
      a[i] = v + w;
      a[i + h] = v - w;
    }
    __syncthreads();
  }
}

// Natural-order FWHT of one chunk of P = 1024 R floats held in registers by a 1,024-thread CTA: v[r] is element
// tid + 1024 r. Index bits 0..4 are butterflied with warp shuffles; bits 5..9 after an in-place transpose through `buf`
// (1,024 floats of shared memory, XOR-swizzled so that both the row-wise and the column-wise access are
// bank-conflict-free), again with shuffles; bits 10 and up are between the registers of one thread. Same stage order
// (h = 1, 2, 4, ...) and therefore the same bits as fwht_shared.
template <int R>
__device__ __forceinline__ void fwht_regs(float (&v)[R], float* buf) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int h = 1; h < 32; h <<= 1) {
      const float p = __shfl_xor_sync(0xffffffffu, v[r], h);
      v[r] = (lane & h) ? p - v[r] : v[r] + p;
    }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    __syncthreads();  // buf is free: every thread holds its elements in registers
    buf[warp * 32 + (lane ^ warp)] = v[r];
    __syncthreads();
    float t = buf[lane * 32 + (warp ^ lane)];  // element (lane << 5) | warp: lane now indexes bits 5..9
#pragma unroll
    for (int h = 1; h < 32; h <<= 1) {
      const float p = __shfl_xor_sync(0xffffffffu, t, h);
      t = (lane & h) ? p - t : t + p;
    }
    __syncthreads();
    buf[lane * 32 + (warp ^ lane)] = t;
    __syncthreads();
    v[r] = buf[warp * 32 + (lane ^ warp)];
  }
#pragma unroll
  for (int h = 1; h < R; h <<= 1)
#pragma unroll
    for (int r = 0; r < R; ++r)
      if ((r & h) == 0) {
        const float x = v[r], y = v[r + h];
        v[r] = x + y;
        v[r + h] = x - y;
      }
}

// Mixed value of chunk r at column i: sum over k (ascending) of +-v[k].
template <int K>
__device__ __forceinline__ float mix_row(const float (&v)[K], uint32_t mask) {
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < K; ++k) s += __uint_as_float(__float_as_uint(v[k]) ^ (((mask >> k) & 1u) << 31));
  return s;
}

// Natural-order FWHT of 1,024 floats by ONE warp, no block-level synchronisation: v[r] is element 32 r + lane. Index
// bits 0..4 (the lane) are butterflied with shuffles, bits 5..9 (r) between the registers of a thread. Same stage order
// as fwht_shared / fwht_regs, therefore the same bits.
__device__ __forceinline__ void fwht_warp_1024(float (&v)[32]) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int h = 1; h < 32; h <<= 1) {
    const bool upper = lane & h;
#pragma unroll
    for (int r = 0; r < 32; ++r) {
      const float p = __shfl_xor_sync(0xffffffffu, v[r], h);
      v[r] = upper ? p - v[r] : v[r] + p;
    }
  }
#pragma unroll
  for (int h = 1; h < 32; h <<= 1)
#pragma unroll
    for (int r = 0; r < 32; ++r)
      if ((r & h) == 0) {
        const float x = v[r], y = v[r + h];
        v[r] = x + y;
        v[r + h] = x - y;
      }
}

// FWHT of the K chunks (P = 1024 H floats each, H = 1 or 2) of a mixed row in shared memory, one 1,024-float unit per
// warp at a time, results straight to the destination (H = 1) or after one more stage across the two halves (H = 2).
template <int H, Mode M>
__device__ __forceinline__ void row_chunks_warp(const HadArgs& a, long row, float* row_s, int K) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int u = warp; u < K * H; u += nwarps) {
    float* unit = row_s + u * 1024;
    float v[32];
#pragma unroll
    for (int r = 0; r < 32; ++r) v[r] = unit[32 * r + lane];
    fwht_warp_1024(v);
#pragma unroll
    for (int r = 0; r < 32; ++r) {
      if constexpr (H == 1) store_dst<M>(a, row, u * 1024 + 32 * r + lane, v[r]);
      else unit[32 * r + lane] = v[r];
    }
  }
  if constexpr (H == 2) {
    __syncthreads();
    for (int j = threadIdx.x; j < K * 1024; j += blockDim.x) {
      const int c = j >> 10, i = j & 1023;
      const float x = row_s[c * 2048 + i], y = row_s[c * 2048 + 1024 + i];
      store_dst<M>(a, row, c * 2048 + i, x + y);
      store_dst<M>(a, row, c * 2048 + 1024 + i, x - y);
    }
  }
}

template <int K, bool T, Mode M>
__global__ __launch_bounds__(1024, 1) void had_row_kernel(HadArgs a) {
  extern __shared__ float row_s[];
  constexpr SignMasks<K, T> masks{};
  const long row = blockIdx.x;
  const int P = a.P;
  if constexpr (K == 1) {
    for (int i = threadIdx.x; i < P; i += blockDim.x) {
      float v[1];
      load_column<1, M>(a, row, i, P, v);
      row_s[i] = v[0];
    }
  } else {
    for (int i = threadIdx.x; i < P; i += blockDim.x) {
      float v[K];
      load_column<K, M>(a, row, i, P, v);
#pragma unroll
      for (int r = 0; r < K; ++r) row_s[r * P + i] = mix_row<K>(v, masks.m[r]);
    }
  }
  __syncthreads();
  if (P == 1024) return row_chunks_warp<1, M>(a, row, row_s, K);
  if (P == 2048) return row_chunks_warp<2, M>(a, row, row_s, K);
  fwht_shared(row_s, P, K);
  for (int j = threadIdx.x; j < a.n; j += blockDim.x) store_dst<M>(a, row, j, row_s[j]);
}

template <int K, int R, Mode M>
__device__ __forceinline__ void chunk_regs(const HadArgs& a, long row, int r_out, uint32_t mask, float* buf) {
  const int P = 1024 * R;
  float w[R];
#pragma unroll
  for (int q = 0; q < R; ++q) {
    const int i = threadIdx.x + 1024 * q;
    float v[K];
    load_column<K, M>(a, row, i, P, v);
    w[q] = mix_row<K>(v, mask);
  }
  fwht_regs<R>(w, buf);
#pragma unroll
  for (int q = 0; q < R; ++q) store_dst<M>(a, row, r_out * P + threadIdx.x + 1024 * q, w[q]);
}

template <int K, bool T, Mode M>
__global__ __launch_bounds__(1024, 1) void had_chunk_kernel(HadArgs a) {
  extern __shared__ float row_s[];
  constexpr SignMasks<K, T> masks{};
  const int r = blockIdx.x;
  const long row = blockIdx.y;
  const int P = a.P;
  uint32_t mask = 0;
#pragma unroll
  for (int q = 0; q < K; ++q)
    if (q == r) mask = masks.m[q];
  if (P == 1024 && blockDim.x == 1024) return chunk_regs<K, 1, M>(a, row, r, mask, row_s);
  if (P == 2048 && blockDim.x == 1024) return chunk_regs<K, 2, M>(a, row, r, mask, row_s);
  for (int i = threadIdx.x; i < P; i += blockDim.x) {
    float v[K];
    load_column<K, M>(a, row, i, P, v);
    row_s[i] = mix_row<K>(v, mask);
  }
  __syncthreads();
  fwht_shared(row_s, P, 1);
  for (int i = threadIdx.x; i < P; i += blockDim.x) store_dst<M>(a, row, r * P + i, row_s[i]);
}

constexpr int kMaxRowFloats = 57344;  // 224 KiB of the 227 KiB a CTA may hold
#ifndef QB_HAD_CHUNK_ROWS
#define QB_HAD_CHUNK_ROWS 32
#endif
constexpr int kChunkRowsBelow = QB_HAD_CHUNK_ROWS;  // fewer rows than this: K CTAs per row

template <int K, bool T, Mode M>
static int configure() {
  QB_CUDA(cudaFuncSetAttribute(had_row_kernel<K, T, M>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               kMaxRowFloats * 4));
  QB_CUDA(cudaFuncSetAttribute(had_chunk_kernel<K, T, M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8192 * 4));
  return QTIP_OK;
}
template <int K, bool T>
static int configure_modes() {
  int rc;
  if ((rc = configure<K, T, Mode::F32Inplace>())) return rc;
  if ((rc = configure<K, T, Mode::Prepare>())) return rc;
  if ((rc = configure<K, T, Mode::Finish>())) return rc;
  return configure<K, T, Mode::FinishB16>();
}
int hadamard_device_setup() {
  int rc;
  if ((rc = configure_modes<1, false>())) return rc;
  if ((rc = configure_modes<12, false>()) || (rc = configure_modes<12, true>())) return rc;
  if ((rc = configure_modes<20, false>()) || (rc = configure_modes<20, true>())) return rc;
  if ((rc = configure_modes<28, false>()) || (rc = configure_modes<28, true>())) return rc;
  return QTIP_OK;
}

template <int K, bool T, Mode M>
static int launch(const HadArgs& a, long rows, bool force_row, cudaStream_t s) {
  const int threads = a.P >= 1024 ? 1024 : (a.P < 64 ? 64 : a.P);
  if (!force_row && K > 1 && rows < kChunkRowsBelow && a.P <= 8192) {
    QB_REQUIRE(rows <= 65535, QTIP_E_GEOMETRY, "too many rows for the chunk kernel");
    had_chunk_kernel<K, T, M><<<dim3(K, unsigned(rows)), threads, size_t(a.P) * 4, s>>>(a);
  } else {
    QB_REQUIRE(a.n <= kMaxRowFloats, QTIP_E_GEOMETRY, "Hadamard rows longer than %d are not supported (n = %d)",
               kMaxRowFloats, a.n);
    // Rows that leave room for several CTAs per SM run with fewer threads per row once there are rows for every SM:
    // the load, transform and store phases of different rows then overlap on each SM. Measured on 12288-wide fp32 rows:
    // 3.3 TB/s with 1,024 threads (one row per SM), 4.2 with 512 (two), 4.7 with 256 (four); the output transforms
    // (several partial sums per element) and 28,672-wide rows are best with 512.
    static const int forced = [] { const char* e = std::getenv("QTIP_HAD_ROW_THREADS"); return e ? std::atoi(e) : 0; }();
    constexpr bool kLight = M == Mode::F32Inplace || M == Mode::Prepare;
    const size_t row_bytes = size_t(a.n) * 4, room = size_t(224) * 1024;
    int row_threads = 1024;
    if (rows >= 148 && row_bytes * 2 <= room) row_threads = 512;
    if (kLight && rows >= 4 * 148 && row_bytes * 4 <= room) row_threads = 256;
    if (forced == 256 || forced == 512 || forced == 1024) row_threads = forced;
    had_row_kernel<K, T, M><<<unsigned(rows), row_threads, size_t(a.n) * 4, s>>>(a);
  }
  QB_LAUNCHED();
  return QTIP_OK;
}
template <Mode M>
static int dispatch(HadArgs a, long rows, bool transpose, bool force_row, cudaStream_t s) {
  const int K = had_order(a.n);
  QB_REQUIRE(K > 0, QTIP_E_GEOMETRY, "unsupported Hadamard size %d", a.n);
  a.P = a.n / K;
  a.rows = int(rows);
  a.scale = 1.0f / std::sqrt(float(a.n));
  if (a.ranks > 1) QB_REQUIRE(a.n % a.ranks == 0, QTIP_E_GEOMETRY, "n = %d is not divisible by %d ranks", a.n, a.ranks);
  if (rows == 0) return QTIP_OK;
  switch (K) {
    case 1: return launch<1, false, M>(a, rows, true, s);
    case 12: return transpose ? launch<12, true, M>(a, rows, force_row, s) : launch<12, false, M>(a, rows, force_row, s);
    case 20: return transpose ? launch<20, true, M>(a, rows, force_row, s) : launch<20, false, M>(a, rows, force_row, s);
    default: return transpose ? launch<28, true, M>(a, rows, force_row, s) : launch<28, false, M>(a, rows, force_row, s);
  }
}

// Operator-side entry points used by decode.cu. ranks: 0/1 = row-major source, R >= 2 = gathered [rank][row][n/R].
int hadamard_prepare(const uint16_t* x, const float* su, uint16_t* rotated, int n, int tokens, int ranks,
                     cudaStream_t s) {
  HadArgs a{};
  a.src = x, a.dst = rotated, a.sign = su, a.ld = n, a.n = n, a.splits = 1, a.ranks = ranks;
  return dispatch<Mode::Prepare>(a, tokens, true, false, s);
}
int hadamard_finish(const float* z, const float* sv, uint16_t* y, int n, int tokens, int splits, long split_stride,
                    int round_z, int ranks, cudaStream_t s) {
  HadArgs a{};
  a.src = z, a.dst = y, a.sign = sv, a.ld = n, a.n = n, a.splits = splits, a.split_stride = split_stride;
  a.round_z = round_z, a.ranks = ranks;
  return dispatch<Mode::Finish>(a, tokens, false, false, s);
}
int hadamard_finish_b16(const uint16_t* z, const float* sv, uint16_t* y, int n, int tokens, int ranks, cudaStream_t s) {
  HadArgs a{};
  a.src = z, a.dst = y, a.sign = sv, a.ld = n, a.n = n, a.splits = 1, a.ranks = ranks;
  return dispatch<Mode::FinishB16>(a, tokens, false, false, s);
}

}  // namespace qb

using namespace qb;

extern "C" int qtip_k_hadamard_rows(float* X_d, long rows, int n, long ld, int transpose, void* stream) {
  QB_REQUIRE(X_d && rows >= 0 && n > 0 && ld >= n, QTIP_E_ARG, "qtip_k_hadamard_rows: bad argument");
  if (!device_info()) return QTIP_E_DEVICE;
  HadArgs a{};
  a.src = X_d, a.dst = X_d, a.ld = ld, a.n = n, a.splits = 1;
  return dispatch<Mode::F32Inplace>(a, rows, transpose != 0, true, as_stream(stream));
}
