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
// y = v v + v (bits 6..15 are the entry), word index = 32 entry + l.
// Eight warps share one work item (a block-row, or one K-split of it) and reduce through shared memory in a fixed order,
// so results are deterministic; a CTA runs four items at a time and walks the item list persistently.
#include <mma.h>

#include <cstring>

#include "common.cuh"

namespace qb {

int hadamard_prepare(const uint16_t* x, const float* su, uint16_t* rotated, int n, int tokens, int ranks, cudaStream_t s);
int hadamard_finish(const float* z, const float* sv, uint16_t* y, int n, int tokens, int splits, long split_stride,
                    int round_z, int ranks, cudaStream_t s);
int hadamard_finish_b16(const uint16_t* z, const float* sv, uint16_t* y, int n, int tokens, int ranks, cudaStream_t s);
int trellis_tc_multiply(qtip_matrix w, const uint16_t* x, float* z, int stride, int splits, int tokens, int* status,
                        cudaStream_t s);  // trellis_tc.cu

#ifndef QB_GEMV_THREADS
#define QB_GEMV_THREADS 1024
#endif
constexpr int kGemmThreads = QB_GEMV_THREADS;  // 1024 (64 registers per thread) or 512 (128)
constexpr int kMaxItemsPerCta = kGemmThreads / 32 / 8;  // 4 concurrent work items of 8 warps each, or 2 x 16, or 1 x 32
constexpr int kLutBytes = 1024 * 32 * 4;                         // 128 KiB, 32 copies
#ifndef QB_GEMV_CHUNK
#define QB_GEMV_CHUNK 2
#endif
constexpr int kChunk = QB_GEMV_CHUNK;  // blocks per register set; two sets alternate, so up to 2 kChunk loads are in flight per warp

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void warps_sync(int id, int warps) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(warps * 32) : "memory");
}

// Dynamic shared memory of the GEMM kernel, named at namespace scope so that every access is known to be a
// shared-memory access at a constant base (a pointer carried through a struct is not): words [0, 32768) hold the
// replicated LUT.
extern __shared__ __align__(16) uint32_t gemm_smem_words[];

// Decodes the two windows that one 32-bit word pair holds: o = word c of tiles (i1 = 1 : i1 = 0) of one tile column,
// p = word c + 1 of the same tiles. State t of a window is its 16 bits starting at bit 4 t; bits above 15 of a state
// register never reach the table index, so a state is cut with ONE funnel shift from the two source registers (the first
// state of the low tile is `o` itself), doubled, hashed with one multiply-add (2 v (v + 1), entry in bits 7..16) and
// turned into the byte address of the lane's own copy (entry e, copy l at byte 128 e + 4 l) with one three-input logic
// operation: shift, add, multiply-add, and-or, load per state.
#ifndef QB_GEMV_DECODE
#define QB_GEMV_DECODE 1
#endif
__device__ __forceinline__ uint32_t lut_word(uint32_t v, uint32_t lane4) {
#if QB_GEMV_DECODE == 1
  const uint32_t v2 = v + v;
  uint32_t y2;
  asm("mad.lo.u32 %0, %1, %2, %2;" : "=r"(y2) : "r"(v), "r"(v2));
  const uint32_t at = (y2 & 0x1ff80u) | lane4;
#elif QB_GEMV_DECODE == 2
  const uint32_t y = v * v + v;
  const uint32_t at = ((y << 1) & 0x1ff80u) | lane4;
#else
  const uint32_t y = v * v + v;
  const uint32_t at = (((y >> 6) & 1023u) << 7) + lane4;
#endif
  return *reinterpret_cast<const uint32_t*>(reinterpret_cast<const unsigned char*>(gemm_smem_words) + at);
}
__device__ __forceinline__ void decode_pair(uint32_t o, uint32_t p, uint32_t lane4, uint32_t (&lo)[4],
                                            uint32_t (&hi)[4]) {
#if QB_GEMV_DECODE == 0
  const uint32_t u0 = __byte_perm(o, p, 0x1054), u1 = __byte_perm(o, p, 0x3276);
#pragma unroll
  for (int k = 0; k < 4; ++k) lo[k] = lut_word(u0 >> (16 - 4 * k), lane4), hi[k] = lut_word(u1 >> (16 - 4 * k), lane4);
#else
  const uint32_t pl = p << 16, oh = o >> 16;
  lo[0] = lut_word(o, lane4);
  hi[0] = lut_word(oh, lane4);
#pragma unroll
  for (int k = 1; k < 4; ++k) {
    lo[k] = lut_word(__funnelshift_l(pl, o, 4 * k), lane4);
    hi[k] = lut_word(__funnelshift_l(p, oh, 4 * k), lane4);
  }
#endif
}

// Tensor-parallel push: the products of this rank's rows go straight into every rank's gathered buffer (plain stores
// to peer memory) instead of a local z, and the last CTA of the launch raises this rank's flag on every rank.
constexpr int kTpMaxRanks = QTIP_TP_MAX_RANKS;
struct TpPush {
  float* z[kTpMaxRanks];        // rank p's gathered buffer of the slot, already offset to this rank's first row
  unsigned* flag[kTpMaxRanks];  // rank p's flag word of (slot, this rank)
  unsigned* ctl;                // this rank's control block (TpControl)
  int ranks, slot, signal;
  int wait;  // the last CTA also waits for the peers' flags (only when every rank runs on a GPU of its own)
};
// Control block at the start of every exchange buffer. flags are written by the peers, the rest is local.
struct TpControl {
  unsigned flags[2][kTpMaxRanks];  // [slot][source rank]: epoch of the last complete push
  unsigned done[2];                // [slot]: epoch of the last completed wait
  unsigned counter;                // CTAs of the running push launch that have finished storing
  unsigned status;                 // non-zero: a bounded wait ran out
};

struct ItemCtx {
  const uint2* codes;     // kernel-layout words as 8-byte units (word c of the four tiles of a block)
  const uint32_t* xw;     // rotated input, bf16 pairs, first token of this launch
  int xs_word;            // XS: word offset in shared memory of the single token's B fragments (16 B per block and lane quarter)
  float* z;
  int n2, in_words, stride, splits, tokens_total, t0, tokens;
};

// This warp's run of 32x32 blocks inside a work item (block-row br, K-split sp): [b_lo, b_hi).
__device__ __forceinline__ void item_run(const ItemCtx& c, int item, int nw, int wi, int& br, int& sp, int& b_lo, int& b_hi) {
  br = item / c.splits, sp = item - br * c.splits;
  const int k_lo = int(long(c.n2) * sp / c.splits), k_hi = int(long(c.n2) * (sp + 1) / c.splits);
  const int span = k_hi - k_lo;
  b_lo = k_lo + int(long(span) * wi / nw), b_hi = k_lo + int(long(span) * (wi + 1) / nw);
}
// Optional (off): asks the memory system to bring a warp's run of code blocks (256 bytes each, contiguous) into the L2
// ahead of the loads that will read it: one bulk prefetch issued by one lane, no destination, no completion to wait
// for. Measured on 57344 x 12288: same duration with and without, but 30 % more DRAM reads with it (229.8 MB against
// the 176.4 MB of codes: a whole round of next items is 58 MB, part of it is evicted before its turn), so it stays off.
#ifndef QB_GEMV_PREFETCH
#define QB_GEMV_PREFETCH 0
#endif
__device__ __forceinline__ void prefetch_run(const ItemCtx& c, int item, int n_items, int nw, int wi) {
#if QB_GEMV_PREFETCH
  if (item >= n_items || (threadIdx.x & 31) != 0) return;
  int br, sp, b_lo, b_hi;
  item_run(c, item, nw, wi, br, sp, b_lo, b_hi);
  if (b_hi <= b_lo) return;
  const uint2* at = c.codes + (size_t(br) * size_t(c.n2) + size_t(b_lo)) * 32u;
  const uint32_t bytes = uint32_t(b_hi - b_lo) * 256u;
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(at), "r"(bytes) : "memory");
#endif
}

// One work item = one 32-row block-row x one K-split, shared by `nw` warps (this is warp `wi` of them): each warp takes
// a contiguous run of 32x32 blocks, then the partial sums are added in warp order through `red` and written to z.
template <int NT, bool XS, bool PUSH>
__device__ __forceinline__ void run_item(const ItemCtx& c, const TpPush& push, int item, int nw, int wi, int bar_id,
                                         float* red) {
  constexpr int RT = XS ? 1 : NT * 8;  // tokens kept per warp in the reduction buffer
  const int lane = threadIdx.x & 31, g = lane >> 2, tg = lane & 3;
  const uint32_t lane4 = uint32_t(lane) * 4u;
  int br, sp, b_lo, b_hi;
  item_run(c, item, nw, wi, br, sp, b_lo, b_hi);
  float acc[NT][2][4];
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int i1 = 0; i1 < 2; ++i1)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[t][i1][q] = 0.f;

  // One 32x32 block: the lane's word of the four tiles, its neighbour's word, four windows, four MMAs per token group.
  auto process = [&](uint2 own, uint2 peer, int blk) {
    // B fragments of the block: for tile column j1 a lane needs bf16 pairs tg and tg + 4 of token g's eight pairs, i.e.
    // words tg, tg + 4, tg + 8, tg + 12 of the block's 16 words. XS: staged in that order in shared memory. Otherwise one
    // 16-byte load of words 4 tg .. 4 tg + 3 per token group and a 4 x 4 word transpose inside the quad (four shuffles).
    uint32_t bw[NT][4];
    if constexpr (XS) {
      // One token is column 0 of the MMA's B operand, which lanes 0..3 supply; the other lanes' registers feed columns
      // whose results are never read, so only the first quad loads (one 64-byte shared-memory wavefront, not four).
      uint4 xb = make_uint4(0u, 0u, 0u, 0u);
      if (lane < 4) xb = reinterpret_cast<const uint4*>(gemm_smem_words + c.xs_word)[blk * 4 + tg];
      bw[0][0] = xb.x, bw[0][1] = xb.y, bw[0][2] = xb.z, bw[0][3] = xb.w;
    } else {
      const bool odd = tg & 1, hi = tg & 2;
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(c.xw + size_t(min(t * 8 + g, c.tokens - 1)) * c.in_words +
                                                             blk * 16 + 4 * tg));
        uint32_t r0 = v.x, r1 = v.y, r2 = v.z, r3 = v.w;
        uint32_t s0 = __shfl_xor_sync(0xffffffffu, odd ? r0 : r1, 1), s1 = __shfl_xor_sync(0xffffffffu, odd ? r2 : r3, 1);
        if (odd) r0 = s0, r2 = s1;
        else r1 = s0, r3 = s1;
        s0 = __shfl_xor_sync(0xffffffffu, hi ? r0 : r2, 2), s1 = __shfl_xor_sync(0xffffffffu, hi ? r1 : r3, 2);
        if (hi) r0 = s0, r1 = s1;
        else r2 = s0, r3 = s1;
        bw[t][0] = r0, bw[t][1] = r1, bw[t][2] = r2, bw[t][3] = r3;
      }
    }
#pragma unroll
    for (int j1 = 0; j1 < 2; ++j1) {
      uint32_t a[2][4];
      decode_pair(j1 ? own.y : own.x, j1 ? peer.y : peer.x, lane4, a[0], a[1]);
#pragma unroll
      for (int i1 = 0; i1 < 2; ++i1)
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          mma_bf16_16816(acc[t][i1], a[i1], bw[t][2 * j1], bw[t][2 * j1 + 1]);
        }
    }
  };
  // Two register sets of CH blocks alternate: one is consumed while the loads of the other are in flight. The main
  // loop takes whole double chunks without per-block tests; what is left of the run (fewer than 2 CH blocks) goes
  // block by block. Measured on 57344 x 12288: CH = 2 (four blocks per loop body) 100 us, CH = 1 111 us, CH = 3 106 us,
  // CH = 4 118 us; a rolled loop of one block with the loads kept four or eight blocks ahead in a shifting register ring
  // 136 us -- the kernel lives on the instruction-level parallelism between neighbouring blocks, within 64 registers.
  constexpr int CH = NT == 2 ? 2 : kChunk;  // 16 tokens keep twice the accumulators: shorter register sets
  const uint2* mine = c.codes + (size_t(br) * size_t(c.n2) * 32u + unsigned(lane));
  auto fetch = [&](uint2(&dst)[CH], int first) {
#pragma unroll
    for (int q = 0; q < CH; ++q) dst[q] = mine[unsigned(first + q) * 32u];
  };
  auto one = [&](uint2 own, int blk) {
    process(own, make_uint2(__shfl_sync(0xffffffffu, own.x, (lane + 1) & 31),
                            __shfl_sync(0xffffffffu, own.y, (lane + 1) & 31)), blk);
  };
  auto consume = [&](const uint2(&src)[CH], int first) {
#pragma unroll
    for (int q = 0; q < CH; ++q) one(src[q], first + q);
  };
  int b = b_lo;
  const int rounds = (b_hi - b) / (2 * CH);
  if (rounds > 0) {
    uint2 bufA[CH], bufB[CH];
    fetch(bufA, b);
    for (int it = 0; it < rounds; ++it, b += 2 * CH) {
      fetch(bufB, b + CH);
      consume(bufA, b);
      if (it + 1 < rounds) fetch(bufA, b + 2 * CH);
      consume(bufB, b + CH);
    }
  }
#pragma unroll 1
  for (; b < b_hi; ++b) one(mine[unsigned(b) * 32u], b);
  // C fragment: c0 (row g, token 2tg), c1 (row g, token 2tg+1), c2 (row g+8, token 2tg), c3 (row g+8, token 2tg+1)
  float* wr = red + size_t(wi) * RT * 32;
  if constexpr (XS) {
    if (tg == 0) {
#pragma unroll
      for (int i1 = 0; i1 < 2; ++i1) {
        wr[i1 * 16 + g] = acc[0][i1][0];
        wr[i1 * 16 + g + 8] = acc[0][i1][2];
      }
    }
  } else {
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
  }
  warps_sync(bar_id, nw);
  for (int o = wi * 32 + lane; o < RT * 32; o += nw * 32) {
    const int tok = o >> 5, row = o & 31;
    if (tok < c.tokens) {
      float s = red[o];
      for (int q = 1; q < nw; ++q) s += red[size_t(q) * RT * 32 + o];
      const size_t at = (size_t(sp) * c.tokens_total + c.t0 + tok) * c.stride + br * 32 + row;
      if constexpr (PUSH) {
#pragma unroll
        for (int p = 0; p < kTpMaxRanks; ++p)
          if (p < push.ranks) push.z[p][at] = s;
      } else {
        c.z[at] = s;
      }
    }
  }
  warps_sync(bar_id, nw);
}

// One warp: lane r waits (bounded) until rank r's push of the slot's next epoch has landed in this rank's buffer, then
// lane 0 records the epoch as done. A wait that runs out leaves the epoch untouched and raises the status word.
__device__ __forceinline__ void tp_wait_warp(TpControl* ctl, int slot, int ranks) {
  const int lane = threadIdx.x & 31;
  const unsigned epoch = *reinterpret_cast<volatile unsigned*>(&ctl->done[slot]) + 1u;
  bool ok = true;
  if (lane < ranks) {
    const unsigned* f = &ctl->flags[slot][lane];
    const long long start = clock64();
    for (;;) {
      if (*reinterpret_cast<const volatile unsigned*>(f) == epoch) break;
      if (clock64() - start > 2000000000LL) {
        ok = false;
        break;
      }
    }
  }
  ok = __all_sync(0xffffffffu, ok);
  __threadfence_system();  // the flags were read before, the gathered products are read after (by the next kernel)
  if (lane == 0) {
    if (ok) *reinterpret_cast<volatile unsigned*>(&ctl->done[slot]) = epoch;
    else atomicExch(&ctl->status, 3u);
  }
}

// z[(split * tokens_total + token) * stride + row]; x: [tokens_total][in] bf16 (the rotated input). One launch covers
// tokens [t0, t0 + tokens), tokens <= 8 NT: each group of 8 tokens is one MMA column block held in registers. XS (one
// token): the activations are staged in shared memory in fragment order, one 16-byte read per block and lane.
// Work items are dealt round-robin to groups of 32 / IPC warps (IPC = 4, 2 or 1 items at a time per CTA; the host
// picks it for the one-token kernel so that a launch with few items still puts a CTA on every SM) for as many full
// rounds as there are; the remainder is done by whole CTAs (32 warps per item) so that the tail of the launch is short.
template <int NT, bool XS, bool PUSH, int IPC>
__global__ __launch_bounds__(kGemmThreads, 1) void trellis_gemm_kernel(qtip_matrix w, const uint16_t* __restrict__ x,
                                                                       float* __restrict__ z, int stride, int splits,
                                                                       int tokens_total, int t0, int tokens,
                                                                       const __grid_constant__ TpPush push) {
  unsigned char* smem = reinterpret_cast<unsigned char*>(gemm_smem_words);
  constexpr int RT = XS ? 1 : NT * 8;
  uint32_t* lut_s = gemm_smem_words;
  float* red = reinterpret_cast<float*>(smem + kLutBytes);  // [32 warps][RT tokens][32 rows]
  uint32_t* xs = reinterpret_cast<uint32_t*>(smem + kLutBytes + 32 * RT * 32 * 4);
  const int tid = threadIdx.x, warp = tid >> 5;
  chain_release();  // the output transform behind this launch may be scheduled as SMs free up
  {
    // 32 copies of the table: each thread reads ONE entry from global memory, a warp then spreads its 32 entries with
    // shuffles so that every store instruction writes 32 consecutive words (no bank conflicts, one load latency).
    const int lane = tid & 31;
#pragma unroll
    for (int h = 0; h < 1024 / kGemmThreads; ++h) {
      const int e0 = (h * (kGemmThreads / 32) + warp) << 5;
      const uint32_t mine = w.lut[e0 + lane];
#pragma unroll
      for (int e = 0; e < 32; ++e) lut_s[(e0 + e) * 32 + lane] = __shfl_sync(0xffffffffu, mine, e);
    }
  }
  chain_wait();  // the table above does not depend on the kernel before this one; the activations and z do
  const uint32_t* xw = reinterpret_cast<const uint32_t*>(x) + size_t(t0) * (w.in / 2);
  if constexpr (XS) {
    for (int i = tid; i < w.in / 2; i += kGemmThreads) {
      const int q = i & 15;  // word j1 * 8 + hi * 4 + tg of its block -> slot tg * 4 + j1 * 2 + hi
      xs[(i & ~15) + (q & 3) * 4 + (q >> 3) * 2 + ((q >> 2) & 1)] = xw[i];
    }
  }
  __syncthreads();
  ItemCtx c;
  c.codes = reinterpret_cast<const uint2*>(w.trellis);
  c.xw = xw;
  c.xs_word = (kLutBytes + 32 * RT * 32 * 4) / 4;
  c.z = z;
  c.n2 = w.in / 32, c.in_words = w.in / 2, c.stride = stride, c.splits = splits;
  c.tokens_total = tokens_total, c.t0 = t0, c.tokens = tokens;
  const int n_items = (w.out / 32) * splits;
  constexpr int ipc = IPC, wpi = (kGemmThreads / 32) / IPC;  // items per CTA at a time, warps per work item
  const int slots = gridDim.x * ipc;
  const int n_grouped = n_items / slots * slots;
  const int grp = warp / wpi, wi = warp % wpi;
  prefetch_run(c, blockIdx.x * ipc + grp, n_grouped, wpi, wi);  // the first item's codes
  for (int item = blockIdx.x * ipc + grp; item < n_grouped; item += slots) {
    prefetch_run(c, item + slots, n_grouped, wpi, wi);  // the next item's codes travel while this one is decoded
    run_item<NT, XS, PUSH>(c, push, item, wpi, wi, grp + 1, red + size_t(grp) * wpi * RT * 32);
  }
  prefetch_run(c, n_grouped + blockIdx.x, n_items, kGemmThreads / 32, warp);
  __syncthreads();
  for (int item = n_grouped + blockIdx.x; item < n_items; item += gridDim.x)
    run_item<NT, XS, PUSH>(c, push, item, kGemmThreads / 32, warp, 0, red);
  if constexpr (PUSH) {
    // The barrier orders every thread's peer stores before thread 0's fence (fences are cumulative), the fence orders
    // them before the CTA's arrival on the local counter; the CTA that arrives last fences once more (observing all
    // arrivals, releasing all stores) and raises this rank's flag on every rank. With push.wait its first warp then
    // waits for the peers' flags itself, which saves the separate wait kernel.
    volatile uint32_t& wait_here = gemm_smem_words[0];  // the table is no longer needed once every warp is past the barrier
    __syncthreads();
    if (tid == 0) {
      TpControl* ctl = reinterpret_cast<TpControl*>(push.ctl);
      bool last = false;
      __threadfence_system();
      if (atomicAdd(&ctl->counter, 1u) == gridDim.x - 1) {
        *reinterpret_cast<volatile unsigned*>(&ctl->counter) = 0;
        if (push.signal) {
          const unsigned epoch = *reinterpret_cast<volatile unsigned*>(&ctl->done[push.slot]) + 1u;
          __threadfence_system();
#pragma unroll
          for (int p = 0; p < kTpMaxRanks; ++p)
            if (p < push.ranks) *reinterpret_cast<volatile unsigned*>(push.flag[p]) = epoch;
          last = true;
        }
      }
      wait_here = (last && push.wait) ? 1u : 0u;
    }
    __syncthreads();
    if (wait_here && warp == 0) tp_wait_warp(reinterpret_cast<TpControl*>(push.ctl), push.slot, push.ranks);
  }
}

__global__ void tp_wait_kernel(unsigned* ctl_words, int slot, int ranks) {
  tp_wait_warp(reinterpret_cast<TpControl*>(ctl_words), slot, ranks);
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

// Items a CTA works on at a time: a full round of ipc items per CTA costs about ipc units (32 warps on ipc items at
// once), what is left after the full rounds runs one item per CTA (1 unit per round); ties go to the larger ipc
// (longer runs of blocks per warp).
static int gemm_items_per_cta(int n_items, int sms) {
  int best = kMaxItemsPerCta;
  long best_cost = 0;
  for (int ipc = kMaxItemsPerCta; ipc >= 1; ipc >>= 1) {
    const long ctas = min(long(sms), (long(n_items) + ipc - 1) / ipc);
    const long full = n_items / (ctas * ipc), rest = n_items - full * ctas * ipc;  // the rest runs one item per CTA
    const long cost = full * ipc + (rest + ctas - 1) / ctas;
    if (ipc == kMaxItemsPerCta || cost < best_cost) best = ipc, best_cost = cost;
  }
  return best;
}

constexpr size_t kMaxSmem = 227 * 1024;
static size_t gemm_smem(int nt, bool xs, int n_in) {
  return kLutBytes + size_t(32) * (xs ? 1 : nt * 8) * 32 * 4 + (xs ? size_t(n_in) * 2 : 0);
}
template <int NT, bool XS, bool PUSH, int IPC>
static int gemm_attr(size_t bytes) {
  QB_CUDA(cudaFuncSetAttribute(trellis_gemm_kernel<NT, XS, PUSH, IPC>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes)));
  return QTIP_OK;
}
template <bool PUSH>
static int gemm_attrs() {
  int rc;
  if ((rc = gemm_attr<1, true, PUSH, 4>(kMaxSmem)) || (rc = gemm_attr<1, true, PUSH, 2>(kMaxSmem)) ||
      (rc = gemm_attr<1, true, PUSH, 1>(kMaxSmem)))
    return rc;
  if ((rc = gemm_attr<1, false, PUSH, 4>(gemm_smem(1, false, 0)))) return rc;
  return gemm_attr<2, false, PUSH, 4>(gemm_smem(2, false, 0));
}
int decode_device_setup(DeviceInfo*) {
  int rc = gemm_attrs<false>();
  return rc ? rc : gemm_attrs<true>();
}

// need_codes: the multiply and decode entry points read the trellis and the LUT; the two transforms only need the
// geometry and SU / SV (a tensor-parallel rank runs the output transform on the full width but holds a shard of codes).
static int check_matrix(const qtip_matrix& w, const char* who, bool need_codes = true) {
  QB_REQUIRE(!need_codes || (w.trellis && w.lut), QTIP_E_ARG, "%s: null trellis or lut", who);
  QB_REQUIRE(w.in > 0 && w.out > 0 && w.in % 32 == 0 && w.out % 32 == 0, QTIP_E_GEOMETRY,
             "%s: in = %d, out = %d must be positive multiples of 32", who, w.in, w.out);
  return QTIP_OK;
}

template <bool PUSH>
static int multiply_impl(qtip_matrix w, const uint16_t* x, float* z, int stride, int splits, int tokens, cudaStream_t s,
                         TpPush push = TpPush{}) {
  const DeviceInfo* info = device_info();
  if (!info) return QTIP_E_DEVICE;
  const int n_items = (w.out / 32) * splits;
  // Up to 16 tokens per launch (two MMA column blocks in registers); larger batches walk the token axis.
  const int per = tokens <= 8 ? 8 : 16;
  const bool one = tokens == 1 && gemm_smem(1, true, w.in) <= kMaxSmem;
  const int ipc = one ? gemm_items_per_cta(n_items, info->sm_count) : kMaxItemsPerCta;
  const int ctas = min(info->sm_count, (n_items + ipc - 1) / ipc);
  for (int t0 = 0; t0 < tokens; t0 += per) {
    const int nt = min(per, tokens - t0);
    push.signal = t0 + per >= tokens;  // the flags go up after the last launch of the token walk
#define QB_GEMM_LAUNCH(NT_, XS_, IPC_, BYTES_)                                                                      \
  QB_CUDA(launch_chained(trellis_gemm_kernel<NT_, XS_, PUSH, IPC_>, dim3(ctas), dim3(kGemmThreads), BYTES_, s, w, x, z, \
                         stride, splits, tokens, t0, nt, push))
    if (one && ipc == 4) QB_GEMM_LAUNCH(1, true, 4, gemm_smem(1, true, w.in));
    else if (one && ipc == 2) QB_GEMM_LAUNCH(1, true, 2, gemm_smem(1, true, w.in));
    else if (one) QB_GEMM_LAUNCH(1, true, 1, gemm_smem(1, true, w.in));
    else if (per == 8) QB_GEMM_LAUNCH(1, false, 4, gemm_smem(1, false, 0));
    else QB_GEMM_LAUNCH(2, false, 4, gemm_smem(2, false, 0));
#undef QB_GEMM_LAUNCH
    QB_LAUNCHED();
  }
  return QTIP_OK;
}

}  // namespace qb

using namespace qb;

extern "C" int qtip_prepare(qtip_matrix w, const uint16_t* x_d, float* scratch_d, uint16_t* rotated_d, void* stream,
                            int tokens, int rank_major) {
  (void)scratch_d;  // the transforms keep their intermediate on chip
  int rc = check_matrix(w, "qtip_prepare", false);
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
  return multiply_impl<false>(w, rotated_d, z_d, stride, splits, tokens, as_stream(stream));
}
extern "C" int qtip_finish(qtip_matrix w, const float* z_d, uint16_t* y_d, float* scratch_d, int round_z, int splits,
                           void* stream, int tokens, int rank_major) {
  (void)scratch_d;
  int rc = check_matrix(w, "qtip_finish", false);
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
  int rc = check_matrix(w, "qtip_finish_b16", false);
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
  int rc = check_matrix(w, "qtip_multiply_batch");
  if (rc) return rc;
  QB_REQUIRE(x_d && z_d && tokens >= 1, QTIP_E_ARG, "qtip_multiply_batch: bad argument");
  QB_REQUIRE(stride >= w.out && splits >= 1 && splits <= 32 && splits <= w.in / 32, QTIP_E_GEOMETRY,
             "qtip_multiply_batch: stride = %d, splits = %d invalid for %d x %d", stride, splits, w.out, w.in);
  // implementation: 0 = MMA-fragment kernel (16 tokens per pass), 2 = decode fused into the tcgen05 product, other
  // values = by batch size and shape (below).
  const bool fused_ok = w.in % 64 == 0 && w.out % 128 == 0 && reinterpret_cast<uintptr_t>(x_d) % 16 == 0;
  // By batch size: above 16 tokens always; from 9 tokens for matrices of up to 16,384 rows, where the fused kernel's
  // K-splits fill the SMs better than 32-row work items do (12288 x 12288 at 16 tokens: 53 us against 63 us; 57344 rows:
  // 221 us against 196 us).
  const bool fused_pays = tokens > 16 || (tokens > 8 && w.out <= 16384);
  if (implementation == 2 || (implementation != 0 && fused_pays && fused_ok)) {
    if (!device_info()) return QTIP_E_DEVICE;
    return trellis_tc_multiply(w, x_d, z_d, stride, splits, tokens, nullptr, as_stream(stream));
  }
  return multiply_impl<false>(w, x_d, z_d, stride, splits, tokens, as_stream(stream));
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

// ---------------------------------------------------------------- tensor-parallel exchange (rotated-row sharding)
// Exchange buffer of one rank: [TpControl, 256 bytes][gathered z, slot 0][gathered z, slot 1]; a slot holds
// [split][token][out_full] fp32. Consecutive uses of an exchange alternate the two slots, so a rank that is already
// pushing the next product never overwrites a buffer a slower rank is still transforming: rank r's push k + 2 follows
// its wait k + 1, which saw rank p's push k + 1, which p's stream ordered after its output transform of step k.
static_assert(sizeof(TpControl) <= 256, "control block");
static size_t tp_slot_bytes(size_t exchange_bytes) { return (exchange_bytes - 256) / 2 / 256 * 256; }

extern "C" size_t qtip_tp_exchange_bytes(int out_full, int max_tokens, int max_splits) {
  if (out_full <= 0 || max_tokens <= 0 || max_splits <= 0) return 0;
  const size_t slot = (size_t(out_full) * max_tokens * max_splits * 4 + 255) / 256 * 256;
  return 256 + 2 * slot;
}
extern "C" int qtip_tp_alloc(size_t bytes, void** buf_d) {
  QB_REQUIRE(buf_d && bytes >= 256 + 512, QTIP_E_ARG, "qtip_tp_alloc: bad argument");
  QB_CUDA(cudaMalloc(buf_d, bytes));
  QB_CUDA(cudaMemset(*buf_d, 0, bytes));
  return QTIP_OK;
}
extern "C" int qtip_tp_free(void* buf_d) {
  if (buf_d) QB_CUDA(cudaFree(buf_d));
  return QTIP_OK;
}
extern "C" int qtip_tp_export(void* buf_d, unsigned char handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  QB_REQUIRE(buf_d && handle, QTIP_E_ARG, "qtip_tp_export: null pointer");
  cudaIpcMemHandle_t h;
  QB_CUDA(cudaIpcGetMemHandle(&h, buf_d));
  std::memcpy(handle, &h, 64);
  return QTIP_OK;
}
extern "C" int qtip_tp_import(const unsigned char handle[64], void** peer_d) {
  QB_REQUIRE(handle && peer_d, QTIP_E_ARG, "qtip_tp_import: null pointer");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, 64);
  QB_CUDA(cudaIpcOpenMemHandle(peer_d, h, cudaIpcMemLazyEnablePeerAccess));
  return QTIP_OK;
}
extern "C" int qtip_tp_close(void* peer_d) {
  if (peer_d) QB_CUDA(cudaIpcCloseMemHandle(peer_d));
  return QTIP_OK;
}
static int check_exchange(const qtip_tp_exchange* ex, int slot, const char* who) {
  QB_REQUIRE(ex && ex->ranks >= 1 && ex->ranks <= kTpMaxRanks && ex->rank >= 0 && ex->rank < ex->ranks, QTIP_E_ARG,
             "%s: bad exchange (ranks 1..%d)", who, kTpMaxRanks);
  QB_REQUIRE(slot == 0 || slot == 1, QTIP_E_ARG, "%s: slot must be 0 or 1", who);
  QB_REQUIRE(ex->bytes >= 256 + 512, QTIP_E_WORKSPACE, "%s: exchange buffer too small", who);
  for (int p = 0; p < ex->ranks; ++p)
    QB_REQUIRE(ex->base[p] && reinterpret_cast<uintptr_t>(ex->base[p]) % 256 == 0, QTIP_E_ARG,
               "%s: exchange base %d is null or not 256-byte aligned", who, p);
  return QTIP_OK;
}
extern "C" int qtip_tp_reset(const qtip_tp_exchange* ex, void* stream) {
  int rc = check_exchange(ex, 0, "qtip_tp_reset");
  if (rc) return rc;
  QB_CUDA(cudaMemsetAsync(ex->base[ex->rank], 0, 256, as_stream(stream)));
  return QTIP_OK;
}
extern "C" int qtip_multiply_push(qtip_matrix w_shard, const uint16_t* rotated_d, const qtip_tp_exchange* ex, int slot,
                                  int out_full, int row0, int splits, void* stream, int tokens, int wait) {
  int rc = check_matrix(w_shard, "qtip_multiply_push");
  if (rc) return rc;
  if ((rc = check_exchange(ex, slot, "qtip_multiply_push"))) return rc;
  QB_REQUIRE(rotated_d && tokens >= 1, QTIP_E_ARG, "qtip_multiply_push: bad argument");
  QB_REQUIRE(splits >= 1 && splits <= 32 && splits <= w_shard.in / 32 && row0 >= 0 && row0 % 32 == 0 &&
                 row0 + w_shard.out <= out_full,
             QTIP_E_GEOMETRY, "qtip_multiply_push: rows [%d, %d) of %d, splits = %d", row0, row0 + w_shard.out, out_full,
             splits);
  const size_t slot_bytes = tp_slot_bytes(ex->bytes);
  QB_REQUIRE(size_t(out_full) * tokens * splits * 4 <= slot_bytes, QTIP_E_WORKSPACE,
             "qtip_multiply_push: %d x %d tokens x %d splits does not fit a slot of %zu bytes", out_full, tokens, splits,
             slot_bytes);
  TpPush push{};
  for (int p = 0; p < ex->ranks; ++p) {
    unsigned char* b = static_cast<unsigned char*>(ex->base[p]);
    push.z[p] = reinterpret_cast<float*>(b + 256 + size_t(slot) * slot_bytes) + row0;
    push.flag[p] = &reinterpret_cast<TpControl*>(b)->flags[slot][ex->rank];
  }
  push.ctl = static_cast<unsigned*>(ex->base[ex->rank]);
  push.ranks = ex->ranks, push.slot = slot, push.wait = wait != 0;
  return multiply_impl<true>(w_shard, rotated_d, nullptr, out_full, splits, tokens, as_stream(stream), push);
}
extern "C" int qtip_gather_wait(const qtip_tp_exchange* ex, int slot, const float** z_gathered_d, void* stream) {
  int rc = check_exchange(ex, slot, "qtip_gather_wait");
  if (rc) return rc;
  unsigned char* b = static_cast<unsigned char*>(ex->base[ex->rank]);
  tp_wait_kernel<<<1, 32, 0, as_stream(stream)>>>(reinterpret_cast<unsigned*>(b), slot, ex->ranks);
  QB_LAUNCHED();
  if (z_gathered_d) *z_gathered_d = reinterpret_cast<const float*>(b + 256 + size_t(slot) * tp_slot_bytes(ex->bytes));
  return QTIP_OK;
}
extern "C" int qtip_gathered_products(const qtip_tp_exchange* ex, int slot, const float** z_gathered_d) {
  int rc = check_exchange(ex, slot, "qtip_gathered_products");
  if (rc) return rc;
  QB_REQUIRE(z_gathered_d, QTIP_E_ARG, "qtip_gathered_products: null pointer");
  const unsigned char* b = static_cast<const unsigned char*>(ex->base[ex->rank]);
  *z_gathered_d = reinterpret_cast<const float*>(b + 256 + size_t(slot) * tp_slot_bytes(ex->bytes));
  return QTIP_OK;
}
extern "C" int qtip_tp_status(const qtip_tp_exchange* ex, void* stream) {
  int rc = check_exchange(ex, 0, "qtip_tp_status");
  if (rc) return rc;
  TpControl h;
  QB_CUDA(cudaMemcpyAsync(&h, ex->base[ex->rank], sizeof h, cudaMemcpyDeviceToHost, as_stream(stream)));
  QB_CUDA(cudaStreamSynchronize(as_stream(stream)));
  QB_REQUIRE(h.status == 0, QTIP_E_KERNEL, "tensor-parallel exchange: a wait for a peer's push ran out (status %u)", h.status);
  return QTIP_OK;
}
