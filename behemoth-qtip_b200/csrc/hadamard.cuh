// Shared templates of the random-Hadamard kernels: modes, loads and stores, the FWHT variants, the whole-row and the
// chunk-per-CTA transforms, launch and dispatch. Included by hadamard.cu (the operator's three stages and the
// quantizer's in-place transform) and by the two epilogue files, each of which instantiates its own modes only, so that
// the three translation units compile side by side.
#pragma once
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

// Prepare / Finish / FinishB16 are the three stages of the operator. The remaining modes are the fused epilogues of a
// decode step (runtime/src/qtip.hip:713-1163 of the reference):
//   PrepareNorm     u = bf16(hadUt(SU (.) x')), x' = bf16(x * rsqrt(mean(x^2) + eps) * w): RMSNorm folded into the input
//                   transform; x' optionally written out (the FP8 K/V projections read it)
//   PrepareSmem     the same from a row that already sits in shared memory as fp32 (second half of the fused
//                   residual + next-input kernel); the norm is optional here
//   FinishResidual  state = bf16(state + bf16(SV (.) hadU(z)))
//   FinishGateUp    the gate/up epilogue in two phases of the same code: phase 0 keeps g = bf16(SVg (.) hadU(zg)) in
//                   shared memory, phase 1 stores h = bf16(silu(g) * bf16(SVu (.) hadU(zu)))
enum class Mode { F32Inplace, Prepare, Finish, FinishB16, PrepareNorm, PrepareSmem, FinishResidual, FinishGateUp };
template <Mode M>
constexpr bool kIsFinish = M == Mode::Finish || M == Mode::FinishResidual || M == Mode::FinishGateUp;
template <Mode M>
constexpr bool kIsPrepare = M == Mode::Prepare || M == Mode::PrepareNorm || M == Mode::PrepareSmem;

struct HadArgs {
  const void* src;    // fp32 or bf16
  void* dst;          // fp32 (in place) or bf16
  const float* sign;  // SU (Prepare*) or SV (Finish*), else null
  long ld;            // row stride of src in elements
  long ld_dst;        // row stride of dst in elements (0: same as ld)
  long split_stride;  // Finish: elements between K-split partials
  int n, P;
  int splits, round_z;
  int ranks;  // > 1: the source is gathered rank-major, [rank][row][n / ranks]
  int rows;
  float scale;
  // fused epilogues
  const uint16_t* norm;  // PrepareNorm / PrepareSmem: RMSNorm weight (bf16) or null
  uint16_t* xn;          // PrepareNorm / PrepareSmem: normalised row out [rows][n] (bf16) or null
  float eps, factor;     // factor = rsqrt(mean(x^2) + eps), computed per row inside the kernel
  float* aux;            // shared-memory row: FinishResidual / FinishGateUp (phase 0) write it, phase 1 / PrepareSmem read it
  int phase;             // FinishGateUp: 0 = gate, 1 = up
  int aux_base;          // element index of aux[0] within the row (chunk kernels hold one chunk)
  bool write_xn;         // this CTA writes xn (one CTA per row does)
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
  if constexpr (M == Mode::F32Inplace || kIsFinish<M> || M == Mode::PrepareSmem) return static_cast<const float*>(src)[at];
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
    if constexpr (kIsFinish<M>) {
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
      if constexpr (kIsFinish<M>)
        for (int p = 1; p < a.splits; ++p) x += static_cast<const float*>(a.src)[size_t(p) * a.split_stride + at];
      v[k] = x;
      if (k % 4 == 3) asm volatile("" ::: "memory");
    }
  }
  if constexpr (M == Mode::PrepareNorm || M == Mode::PrepareSmem) {
    if (a.norm) {  // x' = bf16(x * factor * w), the rounding of the runtime's RMSNorm; one CTA per row writes it out
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const uint16_t xb = f32_to_bf16(v[k] * a.factor * bf16_to_f32(a.norm[k * P + i]));
        v[k] = bf16_to_f32(xb);
        if (a.xn && a.write_xn) a.xn[row * a.n + k * P + i] = xb;
      }
    }
  }
  if constexpr (kIsPrepare<M>) {
#pragma unroll
    for (int k = 0; k < K; ++k) v[k] *= a.sign[k * P + i];
  }
  if constexpr (kIsFinish<M>) {
    if (a.round_z) {
#pragma unroll
      for (int k = 0; k < K; ++k) v[k] = bf16_to_f32(f32_to_bf16(v[k]));
    }
  }
}
template <Mode M>
__device__ __forceinline__ void store_dst(const HadArgs& a, long row, int j, float v) {
  const long at = row * (a.ld_dst ? a.ld_dst : a.ld) + j;
  if constexpr (M == Mode::F32Inplace) {
    static_cast<float*>(a.dst)[at] = v * a.scale;
  } else if constexpr (kIsPrepare<M>) {
    static_cast<uint16_t*>(a.dst)[at] = f32_to_bf16(v * a.scale);
  } else if constexpr (M == Mode::FinishResidual) {
    uint16_t* st = static_cast<uint16_t*>(a.dst) + at;
    const float t = bf16_to_f32(f32_to_bf16(v * a.scale * a.sign[j]));
    const uint16_t nb = f32_to_bf16(bf16_to_f32(*st) + t);
    *st = nb;
    if (a.aux) a.aux[j - a.aux_base] = bf16_to_f32(nb);  // the updated row, for a fused next-input transform
  } else if constexpr (M == Mode::FinishGateUp) {
    const float t = bf16_to_f32(f32_to_bf16(v * a.scale * a.sign[j]));
    if (a.phase == 0) {
      a.aux[j - a.aux_base] = t;
    } else {
      const float g = a.aux[j - a.aux_base];
      static_cast<uint16_t*>(a.dst)[at] = f32_to_bf16(g / (1.f + expf(-g)) * t);
    }
  } else {
    static_cast<uint16_t*>(a.dst)[at] = f32_to_bf16(v * a.scale * a.sign[j]);
  }
}

// rsqrt(mean(x^2) + eps) of one row, the same bits whatever the CTA's thread count: 1,024 slots (slot i adds the
// squares of elements i, i + 1024, ... in ascending order), then one warp adds the slots 32 apart in ascending order
// and folds its 32 lanes with a butterfly. `slots` is shared memory for 1,024 floats. All threads must call it.
template <Mode M>
__device__ __forceinline__ float row_norm_factor(const HadArgs& a, long row, float* slots) {
  const int ns = a.n < 1024 ? a.n : 1024;
  for (int i = threadIdx.x; i < ns; i += blockDim.x) {
    float ss = 0.f;
    for (int e = i; e < a.n; e += 1024) {
      const float x = M == Mode::PrepareSmem ? a.aux[e] : bf16_to_f32(static_cast<const uint16_t*>(a.src)[row * a.ld + e]);
      ss = fmaf(x, x, ss);
    }
    slots[i] = ss;
  }
  __syncthreads();
  float total = 0.f;
  if (threadIdx.x < 32) {
    for (int i = threadIdx.x; i < ns; i += 32) total += slots[i];
#pragma unroll
    for (int h = 16; h > 0; h >>= 1) total += __shfl_xor_sync(0xffffffffu, total, h);
    if (threadIdx.x == 0) slots[0] = total;
  }
  __syncthreads();
  total = slots[0];
  __syncthreads();
  return rsqrtf(total / float(a.n) + a.eps);
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

// One row, whole in shared memory (row_s: n floats): mix, FWHT per chunk, store. Called by every thread of the CTA.
template <int K, bool T, Mode M>
__device__ __forceinline__ void row_transform(const HadArgs& a, long row, float* row_s) {
  constexpr SignMasks<K, T> masks{};
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

template <int K, bool T, Mode M>
__global__ __launch_bounds__(1024, 1) void had_row_kernel(HadArgs a) {
  extern __shared__ float row_s[];
  const long row = blockIdx.x;
  if constexpr (M == Mode::PrepareNorm) {
    __shared__ float slots[1024];
    a.write_xn = true;
    if (a.norm) a.factor = row_norm_factor<M>(a, row, slots);
  }
  row_transform<K, T, M>(a, row, row_s);
}

// Gate/up epilogue of one row: g = bf16(SVg (.) hadU(zg)) into the second half of the shared row, then the up transform
// in the first half with h = bf16(silu(g) * u) as its store. `a` describes the gate half; the up half sits F elements
// further in the source row and uses sign2.
template <int K>
__global__ __launch_bounds__(1024, 1) void had_row_gateup_kernel(HadArgs a, const float* sign_up) {
  extern __shared__ float row_s[];
  const long row = blockIdx.x;
  a.aux = row_s + a.n, a.aux_base = 0;
#pragma unroll 1
  for (int phase = 0; phase < 2; ++phase) {  // one copy of the transform code, run twice
    a.phase = phase;
    row_transform<K, false, Mode::FinishGateUp>(a, row, row_s);
    __syncthreads();
    a.src = static_cast<const float*>(a.src) + a.n;
    a.sign = sign_up;
  }
}

// o / down epilogue fused with the next layer-norm + input transform (same width n): state = bf16(state + bf16(SV (.)
// hadU(z))), kept in shared memory as it is stored, then u = bf16(hadUt(SU (.) rmsnorm(state))) from there.
template <int K>
__global__ __launch_bounds__(1024, 1) void had_row_residual_input_kernel(HadArgs fin, HadArgs prep) {
  extern __shared__ float row_s[];
  __shared__ float slots[1024];
  const long row = blockIdx.x;
  fin.aux = row_s, fin.aux_base = 0;
  row_transform<K, false, Mode::FinishResidual>(fin, row, row_s);
  __syncthreads();
  prep.src = row_s, prep.aux = row_s, prep.ld = 0, prep.write_xn = true;
  if (prep.norm) prep.factor = row_norm_factor<Mode::PrepareSmem>(prep, row, slots);
  row_transform<K, true, Mode::PrepareSmem>(prep, row, row_s);
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

// Output chunk r of one row by one CTA (smem: P floats, or 1,024 as the transpose buffer of the register path).
template <int K, bool T, Mode M>
__device__ __forceinline__ void chunk_transform(const HadArgs& a, long row, int r, float* smem) {
  constexpr SignMasks<K, T> masks{};
  const int P = a.P;
  uint32_t mask = 0;
#pragma unroll
  for (int q = 0; q < K; ++q)
    if (q == r) mask = masks.m[q];
  if (P == 1024 && blockDim.x == 1024) return chunk_regs<K, 1, M>(a, row, r, mask, smem);
  if (P == 2048 && blockDim.x == 1024) return chunk_regs<K, 2, M>(a, row, r, mask, smem);
  for (int i = threadIdx.x; i < P; i += blockDim.x) {
    float v[K];
    load_column<K, M>(a, row, i, P, v);
    smem[i] = mix_row<K>(v, mask);
  }
  __syncthreads();
  fwht_shared(smem, P, 1);
  for (int i = threadIdx.x; i < P; i += blockDim.x) store_dst<M>(a, row, r * P + i, smem[i]);
}

template <int K, bool T, Mode M>
__global__ __launch_bounds__(1024, 1) void had_chunk_kernel(HadArgs a) {
  extern __shared__ float row_s[];
  const int r = blockIdx.x;
  const long row = blockIdx.y;
  chain_release();
  chain_wait();
  if constexpr (M == Mode::PrepareNorm) {
    __shared__ float slots[1024];
    a.write_xn = r == 0;
    if (a.norm) a.factor = row_norm_factor<M>(a, row, slots);
  }
  chunk_transform<K, T, M>(a, row, r, row_s);
}

// Gate/up epilogue, chunk r of one row: g chunk into shared memory behind the work area, then the up chunk.
template <int K>
__global__ __launch_bounds__(1024, 1) void had_chunk_gateup_kernel(HadArgs a, const float* sign_up) {
  extern __shared__ float row_s[];
  const int r = blockIdx.x;
  const long row = blockIdx.y;
  const int work = a.P > 1024 ? a.P : 1024;
  a.aux = row_s + work, a.aux_base = r * a.P;
  chain_release();
  chain_wait();
#pragma unroll 1
  for (int phase = 0; phase < 2; ++phase) {
    a.phase = phase;
    chunk_transform<K, false, Mode::FinishGateUp>(a, row, r, row_s);
    __syncthreads();
    a.src = static_cast<const float*>(a.src) + a.n;
    a.sign = sign_up;
  }
}

constexpr int kMaxRowFloats = 57344;  // 224 KiB of the 227 KiB a CTA may hold
#ifndef QB_HAD_CHUNK_ROWS
#define QB_HAD_CHUNK_ROWS 32
#endif
constexpr int kChunkRowsBelow = QB_HAD_CHUNK_ROWS;  // fewer rows than this: K CTAs per row

template <int K, bool T, Mode M>
static int configure() {
  QB_CUDA(cudaFuncSetAttribute(had_row_kernel<K, T, M>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (M == Mode::PrepareNorm ? kMaxRowFloats - 1024 : kMaxRowFloats) * 4));
  QB_CUDA(cudaFuncSetAttribute(had_chunk_kernel<K, T, M>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8192 * 4));
  return QTIP_OK;
}
template <int K, bool T, Mode M>
static int launch(const HadArgs& a, long rows, bool force_row, cudaStream_t s) {
  const int threads = a.P >= 1024 ? 1024 : (a.P < 64 ? 64 : a.P);
  if (!force_row && K > 1 && rows < kChunkRowsBelow && a.P <= 8192) {
    QB_REQUIRE(rows <= 65535, QTIP_E_GEOMETRY, "too many rows for the chunk kernel");
    // Few rows: a latency-bound link of a decode step's kernel chain, launched so that it can become resident while
    // the kernel before it drains (measured on the layer workload: 295 -> 279 us per layer at one token; the whole-row
    // kernels of larger batches lose 1 % when launched this way and keep the plain launch).
    QB_CUDA(launch_chained(had_chunk_kernel<K, T, M>, dim3(K, unsigned(rows)), dim3(threads), size_t(a.P) * 4, s, a));
  } else {
    constexpr int kRoom = M == Mode::PrepareNorm ? kMaxRowFloats - 1024 : kMaxRowFloats;  // 4 KiB of static slots
    QB_REQUIRE(a.n <= kRoom, QTIP_E_GEOMETRY, "Hadamard rows longer than %d are not supported (n = %d)", kRoom, a.n);
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


// Dispatch of the fused epilogues: the orders the model shapes use (12288 = 12 x 1024, 28672 = 28 x 1024, powers of two).
template <Mode M>
static int dispatch_epilogue(HadArgs a, long rows, bool transpose, cudaStream_t s) {
  const int K = had_order(a.n);
  QB_REQUIRE(K == 1 || K == 12 || K == 28, QTIP_E_GEOMETRY,
             "the fused epilogues carry the Hadamard orders 1, 12 and 28 (n = %d)", a.n);
  a.P = a.n / K;
  a.rows = int(rows);
  a.scale = 1.0f / std::sqrt(float(a.n));
  if (a.ranks > 1) QB_REQUIRE(a.n % a.ranks == 0, QTIP_E_GEOMETRY, "n = %d is not divisible by %d ranks", a.n, a.ranks);
  if (rows == 0) return QTIP_OK;
  if (K == 1) return launch<1, false, M>(a, rows, true, s);
  if (K == 12) return transpose ? launch<12, true, M>(a, rows, false, s) : launch<12, false, M>(a, rows, false, s);
  return transpose ? launch<28, true, M>(a, rows, false, s) : launch<28, false, M>(a, rows, false, s);
}

}  // namespace qb
