// Mid-size batches (17 .. a few hundred tokens): z[token][row] = sum_k What[row][k] x[token][k] with What decoded from the
// 2-bit trellis codes INSIDE the kernel, straight into the shared-memory A operand of tcgen05.mma. No dense copy of the
// weights is ever written: the codes are read once per 256-token tile, which is what keeps this regime on the HBM
// roofline of the codes instead of that of bf16 weights.
//
// Work item = 128 output rows (four 32-row block-rows) x one token tile (N = 64, 128 or 256 tokens) x one K-split.
// The kernel is persistent: one CTA per SM walks its items (item = CTA, CTA + grid, ...) and every role keeps a running
// K-step index, so the stage ring, the table in shared memory and the TMEM allocation live across items and the
// pipeline never drains between them. Per K step (64 input columns = two 32-column blocks per block-row):
//   warps 0..15 (decoders), in G groups (4, or 2 with 128/256-token tiles); group g owns the steps gk = g (mod G) and
//       stage g of the ring, so G steps are being decoded at once and a warp meets a barrier only once per whole
//       32 x 32 block or two. Per block: 8 bytes of codes per lane (requested 4 G steps ahead), the neighbour's words
//       by shuffle, four windows of four states, sixteen look-ups in the 32-copy table (as the GEMV kernel), and four
//       stmatrix.x4: the four look-ups of a window are exactly an m16n8k16 A fragment, i.e. four 8 x 8 bf16 matrices,
//       and stmatrix writes them as 16-byte rows to the addresses the lanes name -- here the K-major, 128-byte-swizzled
//       positions tcgen05 expects (row r, 16-byte chunk c at r * 128 + ((c ^ (r & 7)) << 4)). Eight consecutive rows
//       hit eight different chunk positions: no bank conflicts. Then fence.proxy.async (the MMA reads through the
//       async proxy) and one arrive per warp on the stage's "full" barrier.
//   warp 16, one lane : TMA load of the step's activation tile (N tokens x 64 columns, K-major, 128-byte swizzle, zero
//       fill beyond the last token) into the same stage; its transaction bytes complete the same "full" barrier.
//   warp 17, one lane : ONE wait, four tcgen05.mma (M128 x N x K16) and ONE tcgen05.commit (on the stage's "empty"
//       barrier) per step -- with few tokens an MMA is short, and the waits and commits of this single thread set the
//       pace, so there is exactly one of each. Item i accumulates in TMEM buffer i & 1; after an item's last step a
//       commit on "accumulator full". Warp 17 also allocates and frees the 2 N TMEM columns.
//   warps 18..21      : epilogue of item i (tcgen05.ld of their 32 TMEM lanes, coalesced fp32 stores of z) under the
//       main loop of item i + 1, then an arrive on "accumulator empty".
// Every mbarrier wait is bounded (tc_wait): on a time-out the CTA's abort flag and the status word are raised, all
// roles fall through, TMEM is freed and the kernel returns.
#include "tc_common.cuh"

namespace qb {

constexpr int kFtRows = 128, kFtDecoders = 16, kFtEpilogueWarps = 4;
constexpr int kFtThreads = (kFtDecoders + 2 + kFtEpilogueWarps) * 32;
constexpr int kFtLutBytes = 1024 * 32 * 4;         // 32 copies of the table
constexpr int kFtMaxStages = 8;

struct FtSmem {
  unsigned long long full[kFtMaxStages], empty[kFtMaxStages], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};
// One ring: a stage holds the decoded A tile and the activation tile of a K step, filled behind ONE barrier (the arrivals
// of the group's decoder warps plus the TMA's transaction bytes) and released by ONE tcgen05.commit, so the single MMA
// thread runs one wait and one commit per step. A K step is KB blocks of 32 columns; stages = decoder groups = G.
// 64-token tiles: 128-column steps, two stages (fewer, larger steps: 229 us against 264 us with 64-column steps and
// four stages on 57344 x 12288); 128- and 256-token tiles: 64-column steps, two stages (96 KiB of stages in all cases).
struct FtConfig {
  int groups, kblk;
};
static FtConfig ft_config(int n_tile, int n_in) {
  if (n_tile <= 64) return n_in % 128 == 0 ? FtConfig{2, 4} : FtConfig{4, 2};
  return FtConfig{2, 2};
}
static size_t ft_smem(int n_tile, FtConfig c) {
  return 1024 + kFtLutBytes + size_t(c.groups) * (size_t(kFtRows) * 32 * c.kblk * 2 + size_t(n_tile) * 32 * c.kblk * 2) +
         sizeof(FtSmem);
}

__device__ int g_ft_status;  // used when the caller passes no status word

extern __shared__ __align__(16) unsigned char ft_smem_raw[];

// No "memory" clobber: the stores go to the A ring only, and the compiler must stay free to issue the table look-ups of
// the following windows before this store (a clobber would serialise look-up latency window by window). The fence and
// the barrier arrive that follow the last store of a step are volatile with a clobber, which keeps the order that matters.
__device__ __forceinline__ void stmatrix_x4(uint32_t addr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
  asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(r0), "r"(r1), "r"(r2),
               "r"(r3));
}

// One work item = 128 output rows x one token tile x one K-split.
struct FtItem {
  int row0, tok0, split, ks_lo, steps;
};
__device__ __forceinline__ FtItem ft_item(int item, int tok_tiles, int splits, int k_total, int n_tile) {
  FtItem it;
  it.split = item % splits;
  const int t = item / splits;
  it.tok0 = (t % tok_tiles) * n_tile;
  it.row0 = (t / tok_tiles) * kFtRows;
  it.ks_lo = int(long(k_total) * it.split / splits);
  it.steps = int(long(k_total) * (it.split + 1) / splits) - it.ks_lo;  // >= 1: the host keeps splits <= k_total
  return it;
}
// Walks the K steps of this CTA's items (item = first + i * stride) as one long sequence with a running index `gk`:
// stage and barrier parity of a step depend on gk alone, so the ring keeps turning across item boundaries.
struct FtWalk {
  int item, n_items, stride, tok_tiles, splits, k_total, n_tile;
  int gk, base;  // global step index of the cursor, and of the first step of the current item
  FtItem cur;
  __device__ __forceinline__ void start(int first, int n_items_, int stride_, int tok_tiles_, int splits_, int k_total_,
                                        int n_tile_, int gk0) {
    item = first, n_items = n_items_, stride = stride_, tok_tiles = tok_tiles_, splits = splits_, k_total = k_total_;
    n_tile = n_tile_, gk = gk0, base = 0;
    if (item < n_items) cur = ft_item(item, tok_tiles, splits, k_total, n_tile);
    settle();
  }
  __device__ __forceinline__ void settle() {
    while (item < n_items && gk >= base + cur.steps) {
      base += cur.steps;
      item += stride;
      if (item < n_items) cur = ft_item(item, tok_tiles, splits, k_total, n_tile);
    }
  }
  __device__ __forceinline__ bool done() const { return item >= n_items; }
  __device__ __forceinline__ int k() const { return gk - base; }  // step inside the current item
  __device__ __forceinline__ void advance(int by) {
    gk += by;
    settle();
  }
};

// Persistent: grid = min(SMs, items); CTA c takes items c, c + grid, ... z[(split * tokens + token) * stride + row].
// G = decoder groups = stages of the ring, KB = 32-column blocks per K step.
template <int G, int KB>
__global__ __launch_bounds__(kFtThreads, 1) void trellis_tc_kernel(qtip_matrix w, const __grid_constant__ CUtensorMap map_x,
                                                                   float* __restrict__ z, int stride, int tokens, int n_tile,
                                                                   int splits, int n_items, int* __restrict__ status) {
  constexpr int kFtKblk = KB, kFtK = 32 * KB;
  constexpr uint32_t kFtABytes = kFtRows * kFtK * 2;  // 16 or 32 KiB per stage
  const uint32_t raw = smem_u32(ft_smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // swizzled tiles need 1,024-byte alignment
  unsigned char* smem = ft_smem_raw + (base - raw);
  uint32_t* lut_s = reinterpret_cast<uint32_t*>(smem);
  const uint32_t a_ring = base + kFtLutBytes, b_ring = a_ring + uint32_t(G) * kFtABytes;
  const uint32_t b_bytes = uint32_t(n_tile) * kFtK * 2;
  FtSmem& sm = *reinterpret_cast<FtSmem*>(smem + kFtLutBytes + size_t(G) * (kFtABytes + b_bytes));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_total = w.in / kFtK, tok_tiles = (tokens + n_tile - 1) / n_tile;
  volatile int* abort_flag = &sm.abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kFtMaxStages; ++s) {
      tc_mbar_init(smem_u32(&sm.full[s]), kFtDecoders / G + 1);  // the group's warps + the TMA lane (with its bytes)
      tc_mbar_init(smem_u32(&sm.empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc_mbar_init(smem_u32(&sm.acc_full[b]), 1);
      tc_mbar_init(smem_u32(&sm.acc_empty[b]), kFtEpilogueWarps);
    }
    sm.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kFtDecoders + 1) {  // TMEM allocation: whole warp, two accumulators of n_tile columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                 "r"(uint32_t(2 * n_tile))
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (warp < kFtDecoders) {
    // 32 copies of the table: each decoder thread reads two entries, the warp spreads them with shuffles so that every
    // store instruction writes 32 consecutive words.
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int e0 = (warp * 2 + h) * 32;
      const uint32_t mine = w.lut[e0 + lane];
#pragma unroll
      for (int e = 0; e < 32; ++e) lut_s[(e0 + e) * 32 + lane] = __shfl_sync(0xffffffffu, mine, e);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = sm.tmem_base;

  if (warp < kFtDecoders) {
    // ---- decoders: G groups of 16 / G warps; group g decodes the steps gk = g (mod G) into stage g, so G steps are in
    // the making at any time and a warp meets a barrier once per G / 2 whole 32 x 32 blocks.
    constexpr int kWpg = kFtDecoders / G, kBpw = 4 * kFtKblk / kWpg;  // warps per group, blocks per warp and step
    const int grp = warp / kWpg, mem = warp % kWpg;
    const int n2 = w.in / 32;
    const uint32_t a_tile = a_ring + uint32_t(grp) * kFtABytes;
    // stmatrix row addresses of this lane inside a 16 x 16 tile: matrix q = lane >> 3 (q & 1: rows + 8, q >> 1:
    // columns + 8), row lane & 7
    const int lrow = (lane & 7) + ((lane >> 3) & 1) * 8, lchunk = lane >> 4;
    int brl[kBpw], kbl[kBpw];
#pragma unroll
    for (int i = 0; i < kBpw; ++i) {
      const int blk = mem * kBpw + i;  // block of the step: block-row blk / kFtKblk, column block blk % kFtKblk
      brl[i] = blk / kFtKblk, kbl[i] = blk % kFtKblk;
    }
    const uint2* codes = reinterpret_cast<const uint2*>(w.trellis) + lane;
    auto fetch = [&](const FtWalk& wk, uint2(&dst)[kBpw]) {
      // block (block-row, column block) of K step ks: 8-byte unit ((br * n2 + 2 ks + kbl) * 32 + lane)
      const FtWalk& x = wk;
      const bool live = !x.done();
      const int ks = live ? x.cur.ks_lo + x.k() : 0, r0 = live ? x.cur.row0 / 32 : 0;
#pragma unroll
      for (int i = 0; i < kBpw; ++i) dst[i] = codes[(size_t(r0 + brl[i]) * n2 + kFtKblk * ks + kbl[i]) * 32];
    };
    constexpr int kAhead = 4;  // group steps of codes in flight per lane (= 4 G K steps)
    uint2 next[kAhead][kBpw];
    FtWalk use, pre;  // the step being decoded, and the step whose codes are being requested (kAhead group steps later)
    use.start(blockIdx.x, n_items, gridDim.x, tok_tiles, splits, k_total, n_tile, grp);
    pre = use;
#pragma unroll
    for (int q = 0; q < kAhead; ++q) {
      fetch(pre, next[q]);
      pre.advance(G);
    }
    bool ok = true;
    while (!use.done() && ok) {
#pragma unroll
      for (int q = 0; q < kAhead; ++q) {
        if (use.done()) break;
        uint2 own[kBpw];
#pragma unroll
        for (int i = 0; i < kBpw; ++i) own[i] = next[q][i];
        fetch(pre, next[q]);
        pre.advance(G);
        const int uses = use.gk / G;  // earlier uses of stage `grp`
        if (uses >= 1 && !tc_wait(smem_u32(&sm.empty[grp]), uint32_t((uses - 1) & 1), abort_flag, status)) {
          ok = false;
          break;
        }
#pragma unroll
        for (int i = 0; i < kBpw; ++i) {
          const uint2 peer = make_uint2(__shfl_sync(0xffffffffu, own[i].x, (lane + 1) & 31),
                                        __shfl_sync(0xffffffffu, own[i].y, (lane + 1) & 31));
#pragma unroll
          for (int j1 = 0; j1 < 2; ++j1) {
            const uint32_t o = j1 ? own[i].y : own[i].x, pw = j1 ? peer.y : peer.x;
#pragma unroll
            for (int i1 = 0; i1 < 2; ++i1) {
              const uint32_t u = __byte_perm(o, pw, i1 ? 0x3276 : 0x1054);  // word c << 16 | word c + 1
              uint32_t a[4];
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                const uint32_t v = u >> (16 - 4 * t);
                const uint32_t y = v * v + v;
                a[t] = lut_s[((y >> 6) & 1023u) * 32u + lane];
              }
              const int r = brl[i] * 32 + i1 * 16 + lrow, ch = kbl[i] * 4 + j1 * 2 + lchunk;
              stmatrix_x4(a_tile + uint32_t(ch >> 3) * 16384u + uint32_t(r) * 128u + (uint32_t((ch & 7) ^ (r & 7)) << 4),
                          a[0], a[1], a[2], a[3]);
            }
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) tc_mbar_arrive(smem_u32(&sm.full[grp]));
        use.advance(G);
      }
    }
  } else if (warp == kFtDecoders) {
    // ---- TMA producer of the activation tiles
    if (lane == 0) {
      FtWalk wk;
      wk.start(blockIdx.x, n_items, gridDim.x, tok_tiles, splits, k_total, n_tile, 0);
      for (; !wk.done(); wk.advance(1)) {
        const int s = wk.gk % G, uses = wk.gk / G;
        if (uses >= 1 && !tc_wait(smem_u32(&sm.empty[s]), uint32_t((uses - 1) & 1), abort_flag, status)) break;
        const uint32_t bar = smem_u32(&sm.full[s]);
        tc_mbar_expect_tx(bar, b_bytes);
        for (int sub = 0; sub < kFtKblk / 2; ++sub)  // one 64-column box per 128-byte-swizzled sub-tile
          tc_tma_load_2d(b_ring + uint32_t(s) * b_bytes + uint32_t(sub) * uint32_t(n_tile) * 128u, &map_x,
                         (wk.cur.ks_lo + wk.k()) * kFtK + 64 * sub, wk.cur.tok0, bar);
      }
    }
  } else if (warp == kFtDecoders + 1) {
    // ---- MMA issuer: item i of this CTA accumulates in TMEM buffer i & 1, so the epilogue of one item runs under the
    // main loop of the next
    if (lane == 0) {
      const uint32_t idesc = tc_idesc(kFtRows, n_tile);
      FtWalk wk;
      wk.start(blockIdx.x, n_items, gridDim.x, tok_tiles, splits, k_total, n_tile, 0);
      bool ok = true;
      for (int i = 0; !wk.done() && ok; ++i) {
        const int buf = i & 1, steps = wk.cur.steps;
        if (i >= 2) ok = tc_wait(smem_u32(&sm.acc_empty[buf]), uint32_t(((i >> 1) - 1) & 1), abort_flag, status);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int k = 0; k < steps; ++k) {
          const int s = wk.gk % G;
          ok = tc_wait(smem_u32(&sm.full[s]), uint32_t((wk.gk / G) & 1), abort_flag, status);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
          for (int sub = 0; sub < kFtKblk / 2; ++sub) {
            const uint64_t a_desc = tc_smem_desc(a_ring + uint32_t(s) * kFtABytes + uint32_t(sub) * 16384u);
            const uint64_t b_desc = tc_smem_desc(b_ring + uint32_t(s) * b_bytes + uint32_t(sub) * uint32_t(n_tile) * 128u);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              tc_mma(tmem + uint32_t(buf * n_tile), a_desc + uint64_t(2 * kk), b_desc + uint64_t(2 * kk), idesc,
                     k > 0 || kk > 0 || sub > 0);
          }
          tc_commit(smem_u32(&sm.empty[s]));
          wk.advance(1);
        }
        if (ok) tc_commit(smem_u32(&sm.acc_full[buf]));
      }
    }
  } else {
    // ---- epilogue warps: warp e reads TMEM lanes 32 (e % 4) .. + 31 (rows), columns = tokens of the tile
    const int quarter = warp & 3;
    int i = 0;
    for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++i) {
      const FtItem it = ft_item(item, tok_tiles, splits, k_total, n_tile);
      const int buf = i & 1;
      if (!tc_wait(smem_u32(&sm.acc_full[buf]), uint32_t((i >> 1) & 1), abort_flag, status)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float* zs = z + size_t(it.split) * tokens * stride + it.row0 + quarter * 32 + lane;
#pragma unroll 1
      for (int cc = 0; cc < n_tile; cc += 32) {
        if (it.tok0 + cc >= tokens) break;
        uint32_t v[32];
        const uint32_t taddr = tmem + (uint32_t(quarter * 32) << 16) + uint32_t(buf * n_tile + cc);
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
          const int tok = it.tok0 + cc + c;
          if (tok < tokens) zs[size_t(tok) * stride] = __uint_as_float(v[c]);
        }
      }
      // the accumulator has been read: hand the buffer back to the MMA thread
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) tc_mbar_arrive(smem_u32(&sm.acc_empty[buf]));
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == kFtDecoders + 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(uint32_t(2 * n_tile)) : "memory");
  }
}

int trellis_tc_device_setup() {
  const int big = int(ft_smem(256, FtConfig{2, 2}));  // every configuration stays within this size
  QB_CUDA(cudaFuncSetAttribute(trellis_tc_kernel<2, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
  QB_CUDA(cudaFuncSetAttribute(trellis_tc_kernel<4, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
  QB_CUDA(cudaFuncSetAttribute(trellis_tc_kernel<2, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, big));
  return QTIP_OK;
}

// Token tile of the fused kernel for a batch: the smallest of 64 / 128 / 256 that holds it, else 256.
static int ft_token_tile(int tokens) { return tokens <= 64 ? 64 : (tokens <= 128 ? 128 : 256); }

int trellis_tc_multiply(qtip_matrix w, const uint16_t* x, float* z, int stride, int splits, int tokens, int* status,
                        cudaStream_t s) {
  QB_REQUIRE(w.in % 64 == 0 && w.out % kFtRows == 0, QTIP_E_GEOMETRY,
             "the fused tensor-core product needs in %% 64 == 0 and out %% 128 == 0 (in = %d, out = %d)", w.in, w.out);
  QB_REQUIRE(reinterpret_cast<uintptr_t>(x) % 16 == 0, QTIP_E_ARG, "activations must be 16-byte aligned");
  const int n_tile = ft_token_tile(tokens);
  CUtensorMap map_x;
  int rc = tc_make_map(&map_x, x, uint64_t(tokens), uint64_t(w.in), uint32_t(n_tile));
  if (rc) return rc;
  if (!status) {
    void* p = nullptr;
    QB_CUDA(cudaGetSymbolAddress(&p, g_ft_status));
    status = static_cast<int*>(p);
  }
  const DeviceInfo* info = device_info();
  if (!info) return QTIP_E_DEVICE;
  // More K-splits than K steps: the surplus slices of z hold zeros, the kernel runs with one step per split.
  const FtConfig cfg = ft_config(n_tile, w.in);
  const int k_total = w.in / (32 * cfg.kblk), eff = splits < k_total ? splits : k_total;
  if (eff < splits)
    QB_CUDA(cudaMemsetAsync(z + size_t(eff) * tokens * stride, 0, size_t(splits - eff) * tokens * stride * sizeof(float), s));
  const long items = long(w.out / kFtRows) * ((tokens + n_tile - 1) / n_tile) * eff;
  QB_REQUIRE(items < (1l << 30), QTIP_E_GEOMETRY, "too many work items (%ld)", items);
  const int grid = int(items < info->sm_count ? items : info->sm_count);
  const size_t smem = ft_smem(n_tile, cfg);
  if (cfg.groups == 2 && cfg.kblk == 4)
    trellis_tc_kernel<2, 4><<<grid, kFtThreads, smem, s>>>(w, map_x, z, stride, tokens, n_tile, eff, int(items), status);
  else if (cfg.groups == 4)
    trellis_tc_kernel<4, 2><<<grid, kFtThreads, smem, s>>>(w, map_x, z, stride, tokens, n_tile, eff, int(items), status);
  else
    trellis_tc_kernel<2, 2><<<grid, kFtThreads, smem, s>>>(w, map_x, z, stride, tokens, n_tile, eff, int(items), status);
  QB_LAUNCHED();
  return QTIP_OK;
}

}  // namespace qb

using namespace qb;

extern "C" int qtip_multiply_tc(qtip_matrix w, const uint16_t* rotated_d, float* z_d, int stride, int splits, int tokens,
                                int* status_d, void* stream) {
  QB_REQUIRE(w.trellis && w.lut && rotated_d && z_d && tokens >= 1, QTIP_E_ARG, "qtip_multiply_tc: bad argument");
  QB_REQUIRE(w.in > 0 && w.out > 0 && stride >= w.out && splits >= 1 && splits <= 32, QTIP_E_GEOMETRY,
             "qtip_multiply_tc: stride = %d, splits = %d invalid for %d x %d", stride, splits, w.out, w.in);
  if (!device_info()) return QTIP_E_DEVICE;
  return trellis_tc_multiply(w, rotated_d, z_d, stride, splits, tokens, status_d, as_stream(stream));
}
extern "C" int qtip_kernel_status(void* stream) {
  int h = 0, v = 0, na = 0;
  void* ft = nullptr;
  QB_CUDA(cudaGetSymbolAddress(&ft, g_ft_status));
  QB_CUDA(cudaMemcpyAsync(&h, ft, sizeof h, cudaMemcpyDeviceToHost, as_stream(stream)));
  QB_CUDA(cudaMemsetAsync(ft, 0, sizeof h, as_stream(stream)));  // clear on read
  int rc = viterbi_read_status(&v, &na, as_stream(stream));
  if (rc) return rc;
  QB_CUDA(cudaStreamSynchronize(as_stream(stream)));
  QB_REQUIRE(h == 0, QTIP_E_KERNEL, "a bounded pipeline wait of a tensor-core kernel ran out (status %d)", h);
  QB_REQUIRE(v == 0, QTIP_E_KERNEL, "a bounded wait of the cluster Viterbi kernel ran out (status %d)", v);
  QB_REQUIRE(na == 0, QTIP_E_KERNEL,
             "a bounded wait of the cluster Viterbi kernel ran out inside qtip_quantize_tiles_noalloc (status %d)", na);
  return QTIP_OK;
}
extern "C" int qtip_debug_set_status(int which, int value, void* stream) {
  QB_REQUIRE(which >= 0 && which <= 2, QTIP_E_ARG, "qtip_debug_set_status: which = %d", which);
  if (which != 0) return viterbi_set_status(which, value, as_stream(stream));
  void* ft = nullptr;
  QB_CUDA(cudaGetSymbolAddress(&ft, g_ft_status));
  QB_CUDA(cudaMemcpyAsync(ft, &value, sizeof value, cudaMemcpyHostToDevice, as_stream(stream)));
  QB_CUDA(cudaStreamSynchronize(as_stream(stream)));
  return QTIP_OK;
}
