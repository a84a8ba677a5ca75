// Prefill-sized products on the 5th-generation tensor cores: z[token][row] = sum_k W[row][k] x[token][k], bf16 operands,
// fp32 accumulation in tensor memory (tcgen05.mma, cta_group::1, M = 128 x N = 256 x K = 16 per instruction). A CTA owns a
// 256 (weight rows) x 256 (tokens) output tile as two 128-row accumulators that share the token tile: 64 KiB of operands
// per 64-deep stage feed 8.4 MFLOP, which keeps the L2-to-SM traffic (the practical limit of this kernel) at
// 131 flop per byte.
//
// Roles inside one 192-thread CTA (one output tile per CTA):
//   warp 0, one lane : TMA producer. cp.async.bulk.tensor.2d loads of the W tile (256 x 64, as two boxes of 128 rows) and
//                      the x tile (256 x 64), K-major with the 128-byte swizzle, into a 3-stage ring; completion by
//                      mbarrier tx bytes.
//   warp 1, one lane : MMA issuer. Eight tcgen05.mma per stage (two row halves x four K = 16 slices) from shared-memory
//                      descriptors, then tcgen05.commit on the stage's "empty" barrier; after the last stage a commit
//                      on "accumulator full".
//   warps 2..5       : epilogue. tcgen05.ld (32 lanes x 32 columns per instruction) of the warp's quarter of the 128
//                      lanes of each accumulator, coalesced fp32 stores of z (32 consecutive rows per token and warp).
// Warp 1 also allocates and frees the 512 TMEM columns. No TMA multicast, no peer memory. Every mbarrier wait is bounded:
// on a time-out the CTA raises a flag in shared memory and in the caller's status word, all roles fall through, TMEM is
// freed and the kernel returns (the result is then invalid and the host reports QTIP_E_KERNEL).
#include "tc_common.cuh"

namespace qb {

constexpr int kTcM = 128, kTcN = 256, kTcK = 64, kTcStages = 3;
constexpr int kTcHalves = 2;  // 128-row accumulators per CTA (out must be a multiple of 128; a last odd half is skipped)
constexpr int kTcThreads = 192;
constexpr uint32_t kTcABytes = kTcHalves * kTcM * kTcK * 2, kTcBBytes = kTcN * kTcK * 2;  // 32 KiB + 32 KiB per stage

struct TcSmem {
  unsigned long long full[kTcStages], empty[kTcStages], acc_full;
  uint32_t tmem_base;
  int abort_flag;
};
constexpr size_t kTcSmemBytes = 1024 /*alignment slack*/ + size_t(kTcStages) * (kTcABytes + kTcBBytes) + sizeof(TcSmem);

__global__ __launch_bounds__(kTcThreads, 1) void gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                const __grid_constant__ CUtensorMap map_x,
                                                                float* __restrict__ z, int stride, int k_total, int tokens,
                                                                int out, int* __restrict__ status) {
  extern __shared__ unsigned char tc_smem_raw[];
  const uint32_t raw = smem_u32(tc_smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;  // swizzled tiles need 1,024-byte alignment
  TcSmem& sm = *reinterpret_cast<TcSmem*>(tc_smem_raw + (tiles - raw) + size_t(kTcStages) * (kTcABytes + kTcBBytes));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.x * (kTcHalves * kTcM), tok0 = blockIdx.y * kTcN;
  const int halves = min(kTcHalves, (out - row0) / kTcM);  // 1 for the last tile when out / 128 is odd
  // K-split blockIdx.z of gridDim.z: its slice of the K steps and its slice [split][token][stride] of z
  const int ks_lo = int(long(k_total) * blockIdx.z / gridDim.z);
  const int k_steps = int(long(k_total) * (blockIdx.z + 1) / gridDim.z) - ks_lo;
  z += size_t(blockIdx.z) * tokens * stride;
  volatile int* abort_flag = &sm.abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kTcStages; ++s) {
      tc_mbar_init(smem_u32(&sm.full[s]), 1);
      tc_mbar_init(smem_u32(&sm.empty[s]), 1);
    }
    tc_mbar_init(smem_u32(&sm.acc_full), 1);
    sm.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // TMEM allocation: whole warp, all 512 columns (two 128 x 256 fp32 accumulators)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(uint32_t(kTcHalves * kTcN))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = sm.tmem_base;

  if (warp == 0 && lane == 0) {
    // ---- TMA producer
    for (int k = 0; k < k_steps; ++k) {
      const int s = k % kTcStages;
      if (k >= kTcStages && !tc_wait(smem_u32(&sm.empty[s]), uint32_t((k / kTcStages - 1) & 1), abort_flag, status)) break;
      const uint32_t bar = smem_u32(&sm.full[s]);
      tc_mbar_expect_tx(bar, uint32_t(halves) * (kTcABytes / kTcHalves) + kTcBBytes);
      const uint32_t a_dst = tiles + uint32_t(s) * (kTcABytes + kTcBBytes);
      for (int h = 0; h < halves; ++h)
        tc_tma_load_2d(a_dst + uint32_t(h) * (kTcABytes / kTcHalves), &map_w, (ks_lo + k) * kTcK, row0 + h * kTcM, bar);
      tc_tma_load_2d(a_dst + kTcABytes, &map_x, (ks_lo + k) * kTcK, tok0, bar);
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer
    bool ok = true;
    for (int k = 0; k < k_steps && ok; ++k) {
      const int s = k % kTcStages;
      ok = tc_wait(smem_u32(&sm.full[s]), uint32_t((k / kTcStages) & 1), abort_flag, status);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a_addr = tiles + uint32_t(s) * (kTcABytes + kTcBBytes);
      const uint64_t b_desc = tc_smem_desc(a_addr + kTcABytes);
      for (int h = 0; h < halves; ++h) {
        const uint64_t a_desc = tc_smem_desc(a_addr + uint32_t(h) * (kTcABytes / kTcHalves));
#pragma unroll
        for (int kk = 0; kk < kTcK / 16; ++kk)  // 16 bf16 = 32 bytes = 2 descriptor units along K inside the swizzled row
          tc_mma(tmem + uint32_t(h * kTcN), a_desc + uint64_t(2 * kk), b_desc + uint64_t(2 * kk), tc_idesc(kTcM, kTcN),
                 k > 0 || kk > 0);
      }
      tc_commit(smem_u32(&sm.empty[s]));  // frees the stage once these MMAs have read it
    }
    if (ok) tc_commit(smem_u32(&sm.acc_full));
  } else if (warp >= 2) {
    // ---- epilogue: TMEM lanes 32 q .. 32 q + 31 belong to the warps with warp % 4 == q
    const int q = warp & 3;
    const bool ok = tc_wait(smem_u32(&sm.acc_full), 0, abort_flag, status);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
#pragma unroll 1
      for (int cc = 0; cc < halves * kTcN; cc += 32) {
        const int h = cc / kTcN, c0 = cc % kTcN;
        const int row = row0 + h * kTcM + q * 32 + lane;
        uint32_t v[32];
        const uint32_t taddr = tmem + (uint32_t(q * 32) << 16) + uint32_t(cc);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
              "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
              "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
              "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
            : "r"(taddr)
            : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int tok = tok0 + c0 + c;
          if (tok < tokens) z[size_t(tok) * stride + row] = __uint_as_float(v[c]);
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(uint32_t(kTcHalves * kTcN)) : "memory");
  }
}

// ---- host side: tensor maps through the driver entry point (no link-time dependency on libcuda)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}
// [rows][k] bf16 row-major, box = box_rows x 64 columns, 128-byte swizzle, zero fill outside the tensor.
int tc_make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t k, uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled();
  QB_REQUIRE(fn, QTIP_E_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {k, rows};
  const cuuint64_t strides[1] = {k * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  QB_REQUIRE(r == CUDA_SUCCESS, QTIP_E_GEOMETRY, "cuTensorMapEncodeTiled failed (%d) for a %llu x %llu bf16 tensor", int(r),
             (unsigned long long)rows, (unsigned long long)k);
  return QTIP_OK;
}

int gemm_tc_device_setup() {
  QB_CUDA(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kTcSmemBytes)));
  return QTIP_OK;
}

}  // namespace qb

using namespace qb;

static int prefill_gemm_impl(const uint16_t* w_dense_d, const uint16_t* x_d, float* z_d, int stride, int in, int out,
                             int tokens, int splits, int* status_d, void* stream, const char* who) {
  QB_REQUIRE(w_dense_d && x_d && z_d && tokens >= 1, QTIP_E_ARG, "%s: bad argument", who);
  QB_REQUIRE(in > 0 && out > 0 && in % kTcK == 0 && out % kTcM == 0 && stride >= out, QTIP_E_GEOMETRY,
             "%s: in = %d must be a multiple of %d, out = %d of %d, stride >= out", who, in, kTcK, out, kTcM);
  QB_REQUIRE(splits >= 1 && splits <= in / kTcK && splits <= 65535, QTIP_E_GEOMETRY,
             "%s: %d K-splits for %d K steps", who, splits, in / kTcK);
  QB_REQUIRE((reinterpret_cast<uintptr_t>(w_dense_d) | reinterpret_cast<uintptr_t>(x_d)) % 16 == 0, QTIP_E_ARG,
             "%s: operands must be 16-byte aligned", who);
  if (!device_info()) return QTIP_E_DEVICE;
  CUtensorMap map_w, map_x;
  int rc = tc_make_map(&map_w, w_dense_d, uint64_t(out), uint64_t(in), kTcM);
  if (rc) return rc;
  rc = tc_make_map(&map_x, x_d, uint64_t(tokens), uint64_t(in), kTcN);
  if (rc) return rc;
  const dim3 grid((out / kTcM + kTcHalves - 1) / kTcHalves, (tokens + kTcN - 1) / kTcN, splits);
  QB_REQUIRE(grid.y <= 65535, QTIP_E_GEOMETRY, "%s: too many tokens (%d)", who, tokens);
  gemm_tc_kernel<<<grid, kTcThreads, kTcSmemBytes, as_stream(stream)>>>(map_w, map_x, z_d, stride, in / kTcK, tokens,
                                                                        out, status_d);
  QB_LAUNCHED();
  return QTIP_OK;
}

extern "C" int qtip_prefill_gemm(const uint16_t* w_dense_d, const uint16_t* x_d, float* z_d, int stride, int in, int out,
                                 int tokens, int* status_d, void* stream) {
  return prefill_gemm_impl(w_dense_d, x_d, z_d, stride, in, out, tokens, 1, status_d, stream, "qtip_prefill_gemm");
}
extern "C" int qtip_prefill_gemm_splitk(const uint16_t* w_dense_d, const uint16_t* x_d, float* z_d, int stride, int in,
                                        int out, int tokens, int splits, int* status_d, void* stream) {
  return prefill_gemm_impl(w_dense_d, x_d, z_d, stride, in, out, tokens, splits, status_d, stream,
                           "qtip_prefill_gemm_splitk");
}
