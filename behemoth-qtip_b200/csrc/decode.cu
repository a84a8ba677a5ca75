// Trellis-decode linear operator: y = SV (.) hadU_out( hadUt_in(x (.) SU) . What^T ), What decoded on the fly from the
// 2-bit trellis codes (kernel layout: one 32x32 block = 128 uint16 = 256 contiguous bytes; word c of the four 16x16 tiles
// of a block sits at uint16 index 4c + 2 j1 + i1).
//
// trellis_gemm_kernel (1..8 tokens per pass): a warp streams 32x32 blocks of one 32-row block-row. Lane l loads the 8
// bytes holding word l of the four tiles (one fully coalesced 256-byte request per warp), gets word l+1 from its
// neighbour by shuffle, cuts the four 16-bit states of each window and looks their bf16x2 pairs up in shared memory.
// Those four words are exactly the lane's A fragment of an m16n8k16 bf16 MMA for that tile, so the dot products run on
// the tensor cores and the SIMT pipes only decode. The LUT is replicated 32 times (entry e, copy l at byte 128 e + 4 l,
// 128 KiB) so that every lane reads its own bank: the lookup is the co-critical resource (32 lookups per clock per SM),
// and a single-copy table would serialise on bank conflicts. Index arithmetic per state: v = window >> shift,
// X = v * 2v + 2v (= 2 v (v + 1), whose bits 7..16 are the entry), address = (X & 0x1ff80) | 4 l.
// Eight warps share one work item (a block-row, or one K-split of it) and reduce through shared memory in a fixed order,
// so results are deterministic; a CTA runs four items at a time and walks the item list persistently.
#include <mma.h>

#include "common.cuh"

namespace qb {

int hadamard_prepare(const uint16_t* x, const float* su, uint16_t* rotated, int n, int tokens, int ranks, cudaStream_t s);
int hadamard_finish(const float* z, const float* sv, uint16_t* y, int n, int tokens, int splits, long split_stride,
                    int round_z, int ranks, cudaStream_t s);
int hadamard_finish_b16(const uint16_t* z, const float* sv, uint16_t* y, int n, int tokens, int ranks, cudaStream_t s);

constexpr int kGemmThreads = 1024;
constexpr int kWarpsPerItem = 8;
constexpr int kItemsPerCta = kGemmThreads / 32 / kWarpsPerItem;  // 4
constexpr int kLutBytes = 1024 * 32 * 4;                         // 128 KiB, 32 copies
constexpr int kChunk = 4;                                        // blocks loaded ahead per warp

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void group_sync(int group) {
  asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(kWarpsPerItem * 32) : "memory");
}

// Decodes window u (word c << 16 | word c+1) into the four LUT words of states 4c..4c+3 (lane-private LUT copy).
__device__ __forceinline__ void decode_window(uint32_t u, uint32_t lut_lane, uint32_t (&a)[4]) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const uint32_t v = u >> (16 - 4 * k);
    const uint32_t t = v + v;
    const uint32_t x = v * t + t;
    a[k] = lds_u32(lut_lane + (x & 0x1ff80u));
  }
}

// z[(split * tokens_total + token) * stride + row]; x: [tokens_total][in] bf16 (the rotated input). One launch covers
// tokens [t0, t0 + tokens), tokens <= 8 NT: each group of 8 tokens is one MMA column block held in registers.
template <int NT>
__global__ __launch_bounds__(kGemmThreads, 1) void trellis_gemm_kernel(qtip_matrix w, const uint16_t* __restrict__ x,
                                                                       float* __restrict__ z, int stride, int splits,
                                                                       int tokens_total, int t0, int tokens) {
  extern __shared__ __align__(16) unsigned char smem[];
  uint32_t* lut_s = reinterpret_cast<uint32_t*>(smem);
  float* red = reinterpret_cast<float*>(smem + kLutBytes);  // [items][warps][NT*8 tokens][32 rows]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int grp = warp / kWarpsPerItem, wi = warp % kWarpsPerItem;
  for (int i = tid; i < 1024 * 32; i += kGemmThreads) lut_s[i] = w.lut[i >> 5];
  __syncthreads();
  const uint32_t lut_lane = smem_u32(lut_s) + uint32_t(lane) * 4u;
  const int g = lane >> 2, tg = lane & 3;
  const int n2 = w.in / 32, n_items = (w.out / 32) * splits;
  const uint2* codes = reinterpret_cast<const uint2*>(w.trellis);
  const uint32_t* xw = reinterpret_cast<const uint32_t*>(x) + size_t(t0) * (w.in / 2);
  const int in_words = w.in / 2;
  float* my_red = red + size_t(grp) * kWarpsPerItem * (NT * 8) * 32;

  for (int item = blockIdx.x * kItemsPerCta + grp; item < n_items; item += gridDim.x * kItemsPerCta) {
    const int br = item / splits, sp = item - br * splits;
    const int k_lo = int(long(n2) * sp / splits), k_hi = int(long(n2) * (sp + 1) / splits);
    const int span = k_hi - k_lo;
    const int b_lo = k_lo + int(long(span) * wi / kWarpsPerItem), b_hi = k_lo + int(long(span) * (wi + 1) / kWarpsPerItem);
    const uint2* row_codes = codes + size_t(br) * n2 * 32 + lane;
    float acc[NT][2][4];
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int i1 = 0; i1 < 2; ++i1)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[t][i1][q] = 0.f;

    uint2 cur[kChunk], nxt[kChunk];
#pragma unroll
    for (int q = 0; q < kChunk; ++q) nxt[q] = row_codes[size_t(min(b_lo + q, max(b_hi - 1, b_lo))) * 32];
    for (int b0 = b_lo; b0 < b_hi; b0 += kChunk) {
#pragma unroll
      for (int q = 0; q < kChunk; ++q) cur[q] = nxt[q];
      if (b0 + kChunk < b_hi) {
#pragma unroll
        for (int q = 0; q < kChunk; ++q) nxt[q] = row_codes[size_t(min(b0 + kChunk + q, b_hi - 1)) * 32];
      }
#pragma unroll
      for (int q = 0; q < kChunk; ++q) {
        const int blk = b0 + q;
        if (blk >= b_hi) break;
        const uint2 own = cur[q];
        const uint2 peer = make_uint2(__shfl_sync(0xffffffffu, own.x, (lane + 1) & 31),
                                      __shfl_sync(0xffffffffu, own.y, (lane + 1) & 31));
#pragma unroll
        for (int j1 = 0; j1 < 2; ++j1) {
          // B fragments of the 16 input columns of tile column j1: token g, columns 2 tg (+8)
          uint32_t bf[NT][2];
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            const int token = t * 8 + g;
            const uint32_t* xr = xw + size_t(min(token, tokens - 1)) * in_words + blk * 16 + j1 * 8 + tg;
            bf[t][0] = __ldg(xr);
            bf[t][1] = __ldg(xr + 4);
          }
          const uint32_t o = j1 ? own.y : own.x, p = j1 ? peer.y : peer.x;
#pragma unroll
          for (int i1 = 0; i1 < 2; ++i1) {
            uint32_t a[4];
            decode_window(__byte_perm(o, p, i1 ? 0x3276 : 0x1054), lut_lane, a);
#pragma unroll
            for (int t = 0; t < NT; ++t) mma_bf16_16816(acc[t][i1], a, bf[t][0], bf[t][1]);
          }
        }
      }
    }
    // C fragment: c0 (row g, token 2tg), c1 (row g, token 2tg+1), c2 (row g+8, token 2tg), c3 (row g+8, token 2tg+1)
    float* wr = my_red + size_t(wi) * (NT * 8) * 32;
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int i1 = 0; i1 < 2; ++i1) {
        const int tok = t * 8 + 2 * tg, row = i1 * 16 + g;
        wr[tok * 32 + row] = acc[t][i1][0];
        wr[(tok + 1) * 32 + row] = acc[t][i1][1];
        wr[tok * 32 + row + 8] = acc[t][i1][2];
        wr[(tok + 1) * 32 + row + 8] = acc[t][i1][3];
      }
    group_sync(grp);
    for (int o = wi * 32 + lane; o < NT * 8 * 32; o += kWarpsPerItem * 32) {
      const int tok = o >> 5, row = o & 31;
      if (tok < tokens) {
        float s = my_red[o];
#pragma unroll
        for (int q = 1; q < kWarpsPerItem; ++q) s += my_red[size_t(q) * (NT * 8) * 32 + o];
        z[(size_t(sp) * tokens_total + t0 + tok) * stride + br * 32 + row] = s;
      }
    }
    group_sync(grp);
  }
}

// Dense decode to bf16, row-major [out][in]: a CTA decodes a 32-row x 256-column strip through shared memory so that
// global stores are 16-byte and coalesced.
constexpr int kDecCols = 256;
__global__ __launch_bounds__(256) void decode_matrix_kernel(qtip_matrix w, uint16_t* __restrict__ out) {
  __shared__ uint32_t lut_s[1024];
  __shared__ __align__(16) uint32_t tile[32][kDecCols / 2 + 4];  // bf16 pairs; +4 words of padding per row
  for (int i = threadIdx.x; i < 1024; i += 256) lut_s[i] = w.lut[i];
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int br = blockIdx.y, n2 = w.in / 32;
  const int blk0 = blockIdx.x * (kDecCols / 32);
  const int blk = blk0 + warp;
  if (blk < n2) {
    const uint2* codes = reinterpret_cast<const uint2*>(w.trellis) + (size_t(br) * n2 + blk) * 32;
    const uint2 own = codes[lane], peer = codes[(lane + 1) & 31];
    const int A = lane >> 2, B = lane & 3;
#pragma unroll
    for (int j1 = 0; j1 < 2; ++j1)
#pragma unroll
      for (int i1 = 0; i1 < 2; ++i1) {
        const uint32_t u = __byte_perm(j1 ? own.y : own.x, j1 ? peer.y : peer.x, i1 ? 0x3276 : 0x1054);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t pair = lut_s[lut_entry(u >> (16 - 4 * k))];
          const int r = i1 * 16 + (k & 1) * 8 + A, c = warp * 32 + j1 * 16 + (k >> 1) * 8 + B * 2;
          tile[r][c >> 1] = pair;
        }
      }
  }
  __syncthreads();
  const int cols = min(kDecCols, w.in - blk0 * 32);  // multiple of 32
  for (int i = threadIdx.x; i < 32 * (cols / 8); i += 256) {
    const int r = i / (cols / 8), c8 = i % (cols / 8);
    const uint4 v = *reinterpret_cast<const uint4*>(&tile[r][c8 * 4]);
    *reinterpret_cast<uint4*>(out + (size_t(br) * 32 + r) * w.in + blk0 * 32 + c8 * 8) = v;
  }
}

__global__ void reduce_kernel(float* x, size_t n, int splits) {
  const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = x[i];
  for (int p = 1; p < splits; ++p) s += x[size_t(p) * n + i];
  x[i] = s;
}
__global__ void reduce_b16_kernel(const float* x, const float* scale, uint16_t* y, size_t n, int width, int splits) {
  const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = x[i];
  for (int p = 1; p < splits; ++p) s += x[size_t(p) * n + i];
  y[i] = f32_to_bf16(scale ? s * scale[i % width] : s);
}

template <int NT>
static size_t gemm_smem() { return kLutBytes + size_t(kItemsPerCta) * kWarpsPerItem * (NT * 8) * 32 * 4; }

int decode_device_setup(DeviceInfo*) {
  QB_CUDA(cudaFuncSetAttribute(trellis_gemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(gemm_smem<1>())));
  QB_CUDA(cudaFuncSetAttribute(trellis_gemm_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(gemm_smem<2>())));
  return QTIP_OK;
}

static int check_matrix(const qtip_matrix& w, const char* who) {
  QB_REQUIRE(w.trellis && w.lut, QTIP_E_ARG, "%s: null trellis or lut", who);
  QB_REQUIRE(w.in > 0 && w.out > 0 && w.in % 32 == 0 && w.out % 32 == 0, QTIP_E_GEOMETRY,
             "%s: in = %d, out = %d must be positive multiples of 32", who, w.in, w.out);
  return QTIP_OK;
}

static int multiply_impl(qtip_matrix w, const uint16_t* x, float* z, int stride, int splits, int tokens, cudaStream_t s) {
  const DeviceInfo* info = device_info();
  if (!info) return QTIP_E_DEVICE;
  const int n_items = (w.out / 32) * splits;
  const int ctas = min(info->sm_count, (n_items + kItemsPerCta - 1) / kItemsPerCta);
  // Up to 16 tokens per launch (two MMA column blocks in registers); larger batches walk the token axis.
  const int per = tokens <= 8 ? 8 : 16;
  for (int t0 = 0; t0 < tokens; t0 += per) {
    const int nt = min(per, tokens - t0);
    if (per == 8)
      trellis_gemm_kernel<1><<<ctas, kGemmThreads, gemm_smem<1>(), s>>>(w, x, z, stride, splits, tokens, t0, nt);
    else
      trellis_gemm_kernel<2><<<ctas, kGemmThreads, gemm_smem<2>(), s>>>(w, x, z, stride, splits, tokens, t0, nt);
    QB_LAUNCHED();
  }
  return QTIP_OK;
}

}  // namespace qb

using namespace qb;

extern "C" int qtip_prepare(qtip_matrix w, const uint16_t* x_d, float* scratch_d, uint16_t* rotated_d, void* stream,
                            int tokens, int rank_major) {
  (void)scratch_d;  // the transforms keep their intermediate on chip
  int rc = check_matrix(w, "qtip_prepare");
  if (rc) return rc;
  QB_REQUIRE(x_d && rotated_d && w.su && tokens >= 1, QTIP_E_ARG, "qtip_prepare: bad argument");
  if (!device_info()) return QTIP_E_DEVICE;
  const int ranks = (rank_major && tokens > 1) ? (rank_major == 1 ? 2 : rank_major) : 0;
  return hadamard_prepare(x_d, w.su, rotated_d, w.in, tokens, ranks, as_stream(stream));
}
extern "C" int qtip_multiply(qtip_matrix w, const uint16_t* rotated_d, float* z_d, int stride, int splits, void* stream,
                             int tokens) {
  int rc = check_matrix(w, "qtip_multiply");
  if (rc) return rc;
  QB_REQUIRE(rotated_d && z_d && tokens >= 1, QTIP_E_ARG, "qtip_multiply: bad argument");
  QB_REQUIRE(stride >= w.out && splits >= 1 && splits <= 32 && splits <= w.in / 32, QTIP_E_GEOMETRY,
             "qtip_multiply: stride = %d, splits = %d invalid for %d x %d", stride, splits, w.out, w.in);
  return multiply_impl(w, rotated_d, z_d, stride, splits, tokens, as_stream(stream));
}
extern "C" int qtip_finish(qtip_matrix w, const float* z_d, uint16_t* y_d, float* scratch_d, int round_z, int splits,
                           void* stream, int tokens, int rank_major) {
  (void)scratch_d;
  int rc = check_matrix(w, "qtip_finish");
  if (rc) return rc;
  QB_REQUIRE(z_d && y_d && w.sv && tokens >= 1, QTIP_E_ARG, "qtip_finish: bad argument");
  QB_REQUIRE(splits >= 1 && splits <= 32, QTIP_E_GEOMETRY, "qtip_finish: splits = %d", splits);
  if (!device_info()) return QTIP_E_DEVICE;
  const int ranks = (rank_major && tokens > 1) ? (rank_major == 1 ? 2 : rank_major) : 0;
  return hadamard_finish(z_d, w.sv, y_d, w.out, tokens, splits, long(tokens) * w.out, round_z, ranks,
                         as_stream(stream));
}
extern "C" int qtip_finish_b16(qtip_matrix w, const uint16_t* z_d, uint16_t* y_d, float* scratch_d, int tokens,
                               void* stream, int rank_major) {
  (void)scratch_d;
  int rc = check_matrix(w, "qtip_finish_b16");
  if (rc) return rc;
  QB_REQUIRE(z_d && y_d && w.sv && tokens >= 1, QTIP_E_ARG, "qtip_finish_b16: bad argument");
  if (!device_info()) return QTIP_E_DEVICE;
  const int ranks = (rank_major && tokens > 1) ? (rank_major == 1 ? 2 : rank_major) : 0;
  return hadamard_finish_b16(z_d, w.sv, y_d, w.out, tokens, ranks, as_stream(stream));
}
extern "C" int qtip_forward(qtip_matrix w, const uint16_t* x_d, uint16_t* y_d, float* scratch_d, uint16_t* rotated_d,
                            float* z_d, int round_z, void* stream, int splits) {
  int rc = qtip_prepare(w, x_d, scratch_d, rotated_d, stream, 1, 0);
  if (rc) return rc;
  rc = qtip_multiply(w, rotated_d, z_d, w.out, splits, stream, 1);
  if (rc) return rc;
  return qtip_finish(w, z_d, y_d, scratch_d, round_z, splits, stream, 1, 0);
}
extern "C" int qtip_multiply_batch(qtip_matrix w, const uint16_t* x_d, float* z_d, int stride, int splits, int tokens,
                                   void* stream, int implementation) {
  (void)implementation;
  int rc = check_matrix(w, "qtip_multiply_batch");
  if (rc) return rc;
  QB_REQUIRE(x_d && z_d && tokens >= 1, QTIP_E_ARG, "qtip_multiply_batch: bad argument");
  QB_REQUIRE(stride >= w.out && splits >= 1 && splits <= 32 && splits <= w.in / 32, QTIP_E_GEOMETRY,
             "qtip_multiply_batch: stride = %d, splits = %d invalid for %d x %d", stride, splits, w.out, w.in);
  return multiply_impl(w, x_d, z_d, stride, splits, tokens, as_stream(stream));
}
extern "C" int qtip_decode_matrix(qtip_matrix w, uint16_t* out_d, void* stream) {
  int rc = check_matrix(w, "qtip_decode_matrix");
  if (rc) return rc;
  QB_REQUIRE(out_d, QTIP_E_ARG, "qtip_decode_matrix: null output");
  QB_REQUIRE(w.out / 32 <= 65535, QTIP_E_GEOMETRY, "qtip_decode_matrix: out = %d too large", w.out);
  const dim3 grid(blocks_for(w.in, kDecCols), w.out / 32);
  decode_matrix_kernel<<<grid, 256, 0, as_stream(stream)>>>(w, out_d);
  QB_LAUNCHED();
  return QTIP_OK;
}
extern "C" int qtip_reduce_products(float* x_d, size_t elements, int splits, void* stream) {
  QB_REQUIRE(x_d && splits >= 1, QTIP_E_ARG, "qtip_reduce_products: bad argument");
  if (splits == 1 || elements == 0) return QTIP_OK;
  reduce_kernel<<<blocks_for(long(elements), 256), 256, 0, as_stream(stream)>>>(x_d, elements, splits);
  QB_LAUNCHED();
  return QTIP_OK;
}
extern "C" int qtip_reduce_to_b16(const float* x_d, const float* scale_d, uint16_t* y_d, size_t elements, int width,
                                  int splits, void* stream) {
  QB_REQUIRE(x_d && y_d && splits >= 1 && width >= 1, QTIP_E_ARG, "qtip_reduce_to_b16: bad argument");
  if (elements == 0) return QTIP_OK;
  reduce_b16_kernel<<<blocks_for(long(elements), 256), 256, 0, as_stream(stream)>>>(x_d, scale_d, y_d, elements, width,
                                                                                    splits);
  QB_LAUNCHED();
  return QTIP_OK;
}
