// Prefill-sized products on the 5th-generation tensor cores: z[token][row] = sum_k W[row][k] x[token][k], bf16 operands,
// fp32 accumulation in tensor memory (tcgen05.mma, cta_group::1, M = 128 x N = 256 x K = 16 per instruction). A work tile
// is 256 (weight rows) x 256 (tokens), held as two 128-row accumulators that share the token tile: 64 KiB of operands per
// 64-deep stage feed 8.4 MFLOP, which keeps the L2-to-SM traffic (the practical limit of this kernel) at 131 flop per byte.
// Two kernels share the roles below: gemm_tc_kernel (one tile, or one K-split of a tile, per CTA: small products and the
// K-split entry point) and gemm_tc_streamk_kernel (one persistent CTA per SM, further down).
//
// Roles inside one 192-thread CTA:
//   warp 0, one lane : TMA producer. cp.async.bulk.tensor.2d loads of the W tile (256 x 64, as two boxes of 128 rows) and
//                      the x tile (256 x 64), K-major with the 128-byte swizzle, into a 3-stage ring; completion by
//                      mbarrier tx bytes.
//   warp 1, one lane : MMA issuer. Eight tcgen05.mma per stage (two row halves x four K = 16 slices) from shared-memory
//                      descriptors, then tcgen05.commit on the stage's "empty" barrier; after the last stage of a tile
//                      (or K range) a commit on "accumulator full".
//   warps 2..5       : epilogue. tcgen05.ld (32 lanes x 32 columns per instruction) of the warp's quarter of the 128
//                      lanes of each accumulator, coalesced fp32 stores of z (32 consecutive rows per token and warp).
// Warp 1 also allocates and frees the 512 TMEM columns. No TMA multicast, no peer memory. Every mbarrier wait is bounded:
// on a time-out the CTA raises a flag in shared memory and in the caller's status word, all roles fall through, TMEM is
// freed and the kernel returns (the result is then invalid and the host reports QTIP_E_KERNEL).
#include <algorithm>
#include <atomic>
#include <cstdlib>

#include "tc_common.cuh"

namespace qb {

#ifndef QB_TC_RASTER
#define QB_TC_RASTER 1
#endif
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

// 32 lanes x 32 consecutive fp32 columns of tensor memory into registers (lane l of the warp reads TMEM lane base + l),
// complete on return.
__device__ __forceinline__ void tc_tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
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
}

__global__ __launch_bounds__(kTcThreads, 1) void gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                const __grid_constant__ CUtensorMap map_x,
                                                                float* __restrict__ z, int stride, int k_total, int tokens,
                                                                int out, int* __restrict__ status) {
  extern __shared__ unsigned char tc_smem_raw[];
  const uint32_t raw = smem_u32(tc_smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;  // swizzled tiles need 1,024-byte alignment
  TcSmem& sm = *reinterpret_cast<TcSmem*>(tc_smem_raw + (tiles - raw) + size_t(kTcStages) * (kTcABytes + kTcBBytes));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Token tiles vary fastest in launch order: the CTAs in flight at any moment (148 of them) then share about 18 row
  // panels of W (each read from HBM once and found in the L2 by the other token tiles) instead of streaming all of W
  // once per wave of token tiles.
#if QB_TC_RASTER
  const int row0 = blockIdx.y * (kTcHalves * kTcM), tok0 = blockIdx.x * kTcN;
#else
  const int row0 = blockIdx.x * (kTcHalves * kTcM), tok0 = blockIdx.y * kTcN;
#endif
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
        tc_tmem_ld32(taddr, v);
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

// ------------------------------------------------------------------------------------------------------------------
// The same product as ONE persistent launch of G CTAs (one per SM) that finish together. With T tiles, the first
// floor(T / G) * G tiles are whole-tile rounds, tile = round * G + c for CTA c, so that the CTAs running at any moment work
// on neighbouring tiles of the token-fastest order and share their W panels in the L2. The remaining R = T mod G tiles,
// which as a round of their own would leave G - R SMs idle, are cut into P equal K ranges each and dealt out as R * P
// units, K range first: unit u = p * R + t goes to CTA u mod G. 384 tiles on 148 SMs are then two whole rounds plus
// 88 x 5 fifths in three short rounds (2.6 tile times instead of 3); a tensor-parallel shard of 48 tiles occupies 144 SMs
// with thirds instead of 48 with whole tiles. K ranges are the same for every tile, so CTAs that share a W panel still
// walk the same K steps at the same time.
//
// A CTA's work is a list of segments (tile, [ka, kb)): its units in rising order, then its whole tiles. The producer and
// the MMA issuer walk the list without regard to segment borders (the operand ring never drains); the accumulator is
// handed to the epilogue at every segment end. A split tile is summed in z itself in K order: part 0 stores, part p > 0
// waits until the tile's counter says "p parts done", adds its accumulator to z, and every part but the last raises the
// counter. The order of the additions is fixed, so results are reproducible. A wait is always for a unit with a lower
// number, every CTA takes its units in rising order, and the launch is cooperative (all G CTAs are resident at once), so
// the lowest unit in flight never waits and the launch always finishes.
//
// The counters live in a small ring of state blocks inside the library (the interface has no workspace argument). A
// launch takes the next block of the ring on the host; inside a block the counter value that means "p parts done" is
// 64 epoch + p and the last CTA to leave advances the epoch, so a block needs no clearing and a captured launch can be
// replayed. Launches that can run at the same time hold different blocks as long as fewer than kSkSets are in flight on
// one GPU.
constexpr int kSkSets = 32, kSkMaxTiles = 512, kSkMaxParts = 8;
struct SkSet {
  unsigned epoch, counter, pad[2];
  unsigned parts_done[kSkMaxTiles];  // per split tile
};
__device__ SkSet g_sk_sets[kSkSets];

struct SkSmem {
  unsigned long long full[kTcStages], empty[kTcStages], acc_full, acc_empty;
  uint32_t tmem_base;
  unsigned epoch;
  int abort_flag;
};
constexpr size_t kSkSmemBytes = 1024 + size_t(kTcStages) * (kTcABytes + kTcBBytes) + sizeof(SkSmem);

struct SkPlan {
  int k_total;      // K steps per tile
  int token_tiles;  // tiles along the token axis (fastest)
  int rounds;       // whole-tile rounds: tiles [0, rounds * G)
  int split_tiles;  // R: tiles [rounds * G, rounds * G + R) are cut into `parts` K ranges
  int parts;        // P
};
struct SkSegment {
  long tile;
  int ka, kb, part, split;  // split: index of the tile among the split ones (its counter), -1 for a whole tile
};
struct SkWork {
  int units, segments, G, c;
  SkPlan p;
  __device__ SkWork(const SkPlan& plan, int G_, int c_) : G(G_), c(c_), p(plan) {
    const int all = p.split_tiles * p.parts;
    units = all > c ? (all - c + G - 1) / G : 0;
    segments = units + p.rounds;
  }
  __device__ SkSegment at(int si) const {
    SkSegment s;
    if (si < units) {
      const int u = c + si * G;
      s.part = u / p.split_tiles, s.split = u - s.part * p.split_tiles;
      s.tile = long(p.rounds) * G + s.split;
      s.ka = int(long(p.k_total) * s.part / p.parts), s.kb = int(long(p.k_total) * (s.part + 1) / p.parts);
    } else {
      s.tile = long(si - units) * G + c, s.ka = 0, s.kb = p.k_total, s.part = 0, s.split = -1;
    }
    return s;
  }
};

// Bounded wait for *flag == target (another CTA's release). Returns false if abandoned.
__device__ __forceinline__ bool sk_wait_flag(const unsigned* flag, unsigned target, volatile int* abort_flag, int* status) {
  const long long start = clock64();
  for (;;) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v == target) return true;
    if (*abort_flag) return false;
    if (clock64() - start > kTcWaitCycles) {
      *abort_flag = 1;
      if (status) atomicExch(status, 2);
      return false;
    }
  }
}
__device__ __forceinline__ void sk_epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__global__ __launch_bounds__(kTcThreads, 1) void gemm_tc_streamk_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                        const __grid_constant__ CUtensorMap map_x,
                                                                        float* __restrict__ z, int stride, int tokens,
                                                                        int out, const SkPlan plan, SkSet* __restrict__ set,
                                                                        int* __restrict__ status) {
  extern __shared__ unsigned char tc_smem_raw[];
  const uint32_t raw = smem_u32(tc_smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  SkSmem& sm = *reinterpret_cast<SkSmem*>(tc_smem_raw + (tiles - raw) + size_t(kTcStages) * (kTcABytes + kTcBBytes));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = gridDim.x;
  const SkWork work(plan, G, int(blockIdx.x));
  volatile int* abort_flag = &sm.abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kTcStages; ++s) {
      tc_mbar_init(smem_u32(&sm.full[s]), 1);
      tc_mbar_init(smem_u32(&sm.empty[s]), 1);
    }
    tc_mbar_init(smem_u32(&sm.acc_full), 1);
    tc_mbar_init(smem_u32(&sm.acc_empty), 128);
    sm.abort_flag = 0;
    sm.epoch = *reinterpret_cast<volatile unsigned*>(&set->epoch);  // cannot change before this CTA has left
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(uint32_t(kTcHalves * kTcN))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = sm.tmem_base;
  const unsigned count_base = sm.epoch * 64u;  // counter value of a split tile with no part done
  // tile -> first row, first token, 128-row halves present
  auto tile_geometry = [&](long t, int& row0, int& tok0, int& halves) {
    row0 = int(t / plan.token_tiles) * (kTcHalves * kTcM), tok0 = int(t % plan.token_tiles) * kTcN;
    halves = min(kTcHalves, (out - row0) / kTcM);
  };

  if (warp == 0 && lane == 0) {
    // ---- TMA producer: every K step of every segment, stage by stage
    long i = 0;
    bool ok = true;
    for (int si = 0; si < work.segments && ok; ++si) {
      const SkSegment g = work.at(si);
      int row0, tok0, halves;
      tile_geometry(g.tile, row0, tok0, halves);
      for (int k = g.ka; k < g.kb; ++k, ++i) {
        const int s = int(i % kTcStages);
        if (i >= kTcStages && !tc_wait(smem_u32(&sm.empty[s]), uint32_t((i / kTcStages - 1) & 1), abort_flag, status)) {
          ok = false;
          break;
        }
        const uint32_t bar = smem_u32(&sm.full[s]);
        tc_mbar_expect_tx(bar, uint32_t(halves) * (kTcABytes / kTcHalves) + kTcBBytes);
        const uint32_t a_dst = tiles + uint32_t(s) * (kTcABytes + kTcBBytes);
        for (int h = 0; h < halves; ++h)
          tc_tma_load_2d(a_dst + uint32_t(h) * (kTcABytes / kTcHalves), &map_w, k * kTcK, row0 + h * kTcM, bar);
        tc_tma_load_2d(a_dst + kTcABytes, &map_x, k * kTcK, tok0, bar);
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer: accumulates a segment, hands the accumulator over, waits until the epilogue has drained it
    long i = 0;
    bool ok = true;
    for (int si = 0; si < work.segments && ok; ++si) {
      const SkSegment g = work.at(si);
      int row0, tok0, halves;
      tile_geometry(g.tile, row0, tok0, halves);
      if (si > 0) {
        ok = tc_wait(smem_u32(&sm.acc_empty), uint32_t((si - 1) & 1), abort_flag, status);
        if (!ok) break;
      }
      for (int k = g.ka; k < g.kb; ++k, ++i) {
        const int s = int(i % kTcStages);
        ok = tc_wait(smem_u32(&sm.full[s]), uint32_t((i / kTcStages) & 1), abort_flag, status);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = tiles + uint32_t(s) * (kTcABytes + kTcBBytes);
        const uint64_t b_desc = tc_smem_desc(a_addr + kTcABytes);
        for (int h = 0; h < halves; ++h) {
          const uint64_t a_desc = tc_smem_desc(a_addr + uint32_t(h) * (kTcABytes / kTcHalves));
#pragma unroll
          for (int kk = 0; kk < kTcK / 16; ++kk)
            tc_mma(tmem + uint32_t(h * kTcN), a_desc + uint64_t(2 * kk), b_desc + uint64_t(2 * kk), tc_idesc(kTcM, kTcN),
                   k > g.ka || kk > 0);
        }
        tc_commit(smem_u32(&sm.empty[s]));
      }
      if (ok) tc_commit(smem_u32(&sm.acc_full));
    }
  } else if (warp >= 2) {
    // ---- epilogue: one pass per segment. TMEM lanes 32 q .. 32 q + 31 belong to the warps with warp % 4 == q.
    const int q = warp & 3;
    const bool leader = threadIdx.x == 64;  // first lane of the first epilogue warp
    for (int si = 0; si < work.segments; ++si) {
      const SkSegment g = work.at(si);
      int row0, tok0, halves;
      tile_geometry(g.tile, row0, tok0, halves);
      const bool add = g.part > 0;  // the earlier K ranges of this tile are already in z
      const bool publish = g.split >= 0 && g.part + 1 < plan.parts;  // a later K range will add itself to what this one leaves
      if (add) {
        if (leader) sk_wait_flag(&set->parts_done[g.split], count_base + unsigned(g.part), abort_flag, status);
        sk_epilogue_sync();
        if (*abort_flag) break;
      }
      if (!tc_wait(smem_u32(&sm.acc_full), uint32_t(si & 1), abort_flag, status)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (int cc = 0; cc < halves * kTcN; cc += 32) {
        const int h = cc / kTcN, c0 = cc % kTcN;
        const int row = row0 + h * kTcM + q * 32 + lane;
        uint32_t v[32];
        float* at = z + size_t(tok0 + c0) * stride + row;
        const int live = min(32, tokens - tok0 - c0);  // token columns of this chunk that exist
        float sum[32];
        if (add) {  // all 32 loads in flight before the first store (a load behind a store to z would wait for it)
#pragma unroll
          for (int c = 0; c < 32; ++c) sum[c] = c < live ? __ldcg(at + size_t(c) * stride) : 0.f;
        }
        tc_tmem_ld32(tmem + (uint32_t(q * 32) << 16) + uint32_t(cc), v);
#pragma unroll
        for (int c = 0; c < 32; ++c) sum[c] = add ? sum[c] + __uint_as_float(v[c]) : __uint_as_float(v[c]);
#pragma unroll
        for (int c = 0; c < 32; ++c)
          if (c < live) at[size_t(c) * stride] = sum[c];
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      tc_mbar_arrive(smem_u32(&sm.acc_empty));  // 128 arrivals: the accumulator may be overwritten
      if (publish) {
        __threadfence();  // this thread's stores to z, before the flag
        sk_epilogue_sync();
        if (leader)
          asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(&set->parts_done[g.split]),
                       "r"(count_base + unsigned(g.part) + 1u)
                       : "memory");
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(uint32_t(kTcHalves * kTcN)) : "memory");
  }
  if (threadIdx.x == 0) {
    // The last CTA to leave advances the epoch: every flag of this launch then reads as "not done" to the next one.
    __threadfence();
    if (atomicAdd(&set->counter, 1u) == unsigned(G - 1)) {
      *reinterpret_cast<volatile unsigned*>(&set->counter) = 0u;
      __threadfence();
      atomicAdd(&set->epoch, 1u);
    }
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

static SkSet* g_sk_ptr[64];                 // device address of the state ring on each device
static std::atomic<unsigned> g_sk_next[64];  // launches so far on each device: picks the block of the ring
int gemm_tc_device_setup() {
  QB_CUDA(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kTcSmemBytes)));
  QB_CUDA(cudaFuncSetAttribute(gemm_tc_streamk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSkSmemBytes)));
  int dev = 0;
  QB_CUDA(cudaGetDevice(&dev));
  QB_REQUIRE(dev >= 0 && dev < 64, QTIP_E_DEVICE, "device index %d out of range", dev);
  void* at = nullptr;
  QB_CUDA(cudaGetSymbolAddress(&at, g_sk_sets));
  QB_CUDA(cudaMemset(at, 0, sizeof(SkSet) * kSkSets));
  g_sk_ptr[dev] = static_cast<SkSet*>(at);
  return QTIP_OK;
}
// QTIP_GEMM_STREAMK=0 keeps the tile-per-CTA launch for every shape (A/B timing).
static bool streamk_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("QTIP_GEMM_STREAMK");
    return !(e && e[0] == '0');
  }();
  return on;
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
  const unsigned row_tiles = (out / kTcM + kTcHalves - 1) / kTcHalves, token_tiles = (tokens + kTcN - 1) / kTcN;
  const DeviceInfo* info = device_info();
  if (splits == 1 && streamk_enabled()) {
    // Whole-tile rounds for as many tiles as divide evenly among the SMs; the rest is cut into the number of K ranges
    // that minimises rounds x (1 / P + the cost of one more epilogue, about 1/16 of a tile).
    const long n_tiles = long(row_tiles) * token_tiles;
    const int k_total = in / kTcK;
    const int G = info->sm_count;
    const long rounds = n_tiles / G, rest = n_tiles - rounds * G;
    int parts = 1;
    double best = 1e30;
    for (int p = 1; p <= kSkMaxParts && p <= k_total / 8; ++p) {
      const double cost = double((rest * p + G - 1) / G) * (1.0 / p + 1.0 / 16);
      if (cost < best - 1e-9) best = cost, parts = p;
    }
    if (rest < kSkMaxTiles && (rounds > 0 || rest > 0) && !(rounds == 0 && parts == 1)) {
      int dev = 0;
      QB_CUDA(cudaGetDevice(&dev));
      QB_REQUIRE(dev >= 0 && dev < 64 && g_sk_ptr[dev], QTIP_E_DEVICE, "%s: device %d is not initialised", who, dev);
      SkSet* set = g_sk_ptr[dev] + g_sk_next[dev].fetch_add(1u, std::memory_order_relaxed) % kSkSets;
      SkPlan plan;
      plan.k_total = k_total, plan.token_tiles = int(token_tiles), plan.rounds = int(rounds);
      plan.split_tiles = int(rest), plan.parts = parts;
      const long busy = rounds > 0 ? G : std::min<long>(G, rest * parts);
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3(unsigned(busy)), cfg.blockDim = dim3(kTcThreads);
      cfg.dynamicSmemBytes = kSkSmemBytes, cfg.stream = as_stream(stream);
      cudaLaunchAttribute attr{};
      attr.id = cudaLaunchAttributeCooperative;  // all CTAs resident at once: a wait is never for a CTA still to be launched
      attr.val.cooperative = 1;
      cfg.attrs = &attr, cfg.numAttrs = 1;
      QB_CUDA(cudaLaunchKernelEx(&cfg, gemm_tc_streamk_kernel, map_w, map_x, z_d, stride, tokens, out, plan, set, status_d));
      return QTIP_OK;
    }
  }
#if QB_TC_RASTER
  const dim3 grid(token_tiles, row_tiles, splits);
#else
  const dim3 grid(row_tiles, token_tiles, splits);
#endif
  QB_REQUIRE(grid.y <= 65535, QTIP_E_GEOMETRY, "%s: %d tokens x %d rows exceed the launch grid", who, tokens, out);
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
