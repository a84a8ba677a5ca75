// Bitshift-trellis Viterbi (L = 16 state bits, 4 new bits and 2 weights per step, 256-weight sequences) for sm_100a.
//
// Arithmetic contract (bit-exact with the reference kernel, src/viterbi.hip:106-140,145-187 of the reference):
//   inputs are rounded to fp16 first; per step (x0, x1): m0 = fp16(-2 x0), m1 = fp16(-2 x1), xx = x0^2 + x1^2;
//   for state s = (d << 12) | j with LUT pair (l0, l1):  c = fma(l1, m1, fma(l0, m0, (l0^2 + l1^2) + (M[s >> 4] + xx)));
//   new minimum of group j = min over d of float((bits(c) & ~15) | d); back-pointer = low 4 bits of that minimum,
//   stored minimum = the same with the low 4 bits cleared. The last step takes the untagged argmin, lowest state on ties.
//
// vit_fwd_cluster_kernel: an 8-CTA thread-block cluster owns the 65,536 states of the trellis
//    (8,192 per SM, one group index j and its 16 predecessors d per thread), keeps each state's LUT pair and norm in
//    registers for the whole launch, and runs 8 sequences at a time through them. The 4,096 group minima of a step are
//    exchanged between the 8 SMs through distributed shared memory (each minimum is pushed with st.async to the one CTA
//    that reads it next step and counted on that CTA's mbarrier); the two 4-sequence halves of a batch alternate so that one half computes while
//    the other half's minima are in flight. Back-pointers go to global memory as one 32-bit word per (8 steps, group).
#include <cooperative_groups.h>

#include <mutex>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace qb {

// ------------------------------------------------------------------------------------------------- shared device code

__device__ __forceinline__ float state_cost(float l0, float l1, float nrm, float mp, float m0, float m1) {
  return __fmaf_rn(l1, m1, __fmaf_rn(l0, m0, __fadd_rn(nrm, mp)));
}
__device__ __forceinline__ float min3(float a, float b, float c) {
  float r;
  asm("min.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// (bits & mask) | d in one LOP3. With the mask as an immediate the compiler needs two instructions (an immediate AND and
// an immediate OR) on the half-rate integer pipe, which is the busiest pipe of the inner loop; the kernels therefore
// take the mask (0xfffffff0) as a run-time argument so that it lives in a register and only d is an immediate.
__device__ __forceinline__ float tag_cost(float c, uint32_t mask, int d) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(__float_as_uint(c)), "r"(mask), "r"(uint32_t(d)));
  return __uint_as_float(r);
}
constexpr uint32_t kTagMask = 0xfffffff0u;

// (cost, state) candidates of the last step order by cost, then by state.
__device__ __forceinline__ void take_better(float& bv, uint32_t& bs, float ov, uint32_t os) {
  if (ov < bv || (ov == bv && os < bs)) bv = ov, bs = os;
}

// ------------------------------------------------------------------------------------------------- backtraces

// Back-pointer lookup in the [127][1024] uint16 layout.
__device__ __forceinline__ uint32_t prev_state_u16(const uint16_t* Ab, int i, uint32_t s) {
  const uint32_t j = s >> 4;
  const uint32_t d = (uint32_t(Ab[i * 1024 + (j >> 2)]) >> (4 * (j & 3))) & 15u;
  return j | (d << 12);
}
__global__ void vit_overlap_u16_kernel(const uint16_t* __restrict__ A, const uint16_t* __restrict__ final_state, int B,
                                       int* __restrict__ overlap) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const uint16_t* Ab = A + size_t(b) * 127 * 1024;
  uint32_t s = final_state[b];
  for (int i = 126; i >= 64; --i) s = prev_state_u16(Ab, i, s);
  overlap[b] = int(s >> 4);
}
__device__ __forceinline__ void emit_state(int i, uint32_t s, uint16_t* q, float* hatWT, long m, long row0, int col0,
                                           float* hat, const uint32_t* lut_h2) {
  if (q) q[i] = uint16_t(s);
  if (hatWT || hat) {
    const uint32_t u = lut_h2[s];
    const float v0 = half_lo(u), v1 = half_hi(u);
    if (hat) hat[2 * i] = v0, hat[2 * i + 1] = v1;
    if (hatWT) {
      const int t0 = perm_fwd(2 * i), t1 = perm_fwd(2 * i + 1);
      hatWT[long(col0 + (t0 & 15)) * m + row0 + (t0 >> 4)] = v0;
      hatWT[long(col0 + (t1 & 15)) * m + row0 + (t1 >> 4)] = v1;
    }
  }
}
__global__ void vit_finish_u16_kernel(const uint16_t* __restrict__ A, const uint16_t* __restrict__ final_state, int B,
                                      int b0, uint16_t* __restrict__ Q, int nblk, int blk, float* __restrict__ hatWT,
                                      long m, int col0, const uint32_t* __restrict__ lut_h2) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const uint16_t* Ab = A + size_t(b) * 127 * 1024;
  uint16_t* q = Q ? Q + (size_t(b0 + b) * nblk + blk) * 128 : nullptr;
  uint32_t s = final_state[b];
  for (int i = 127; i >= 0; --i) {
    if (i < 127) s = prev_state_u16(Ab, i, s);
    emit_state(i, s, q, hatWT, m, long(b0 + b) * 16, col0, nullptr, lut_h2);
  }
}
__global__ void decode_states_kernel(const uint16_t* __restrict__ st, long n, float* __restrict__ hat,
                                     const uint32_t* __restrict__ lut_h2) {
  const long i = long(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const uint32_t u = lut_h2[st[i]];
  reinterpret_cast<float2*>(hat)[i] = make_float2(half_lo(u), half_hi(u));
}

// ------------------------------------------------------------------------------------------------- 8-CTA cluster kernel

constexpr int kCl = 8;          // CTAs per cluster; each owns 512 group indices j (8,192 states)
constexpr int kClThreads = 512; // one j per thread
constexpr int kTG = 4;          // sequences per half-batch (one float4 of minima per predecessor)
#ifndef QB_VIT_GROUPS
#define QB_VIT_GROUPS 2
#endif
constexpr int kNG = QB_VIT_GROUPS;  // groups of kTG sequences in flight: one computes while the others' minima travel
constexpr int kTB = kTG * kNG;  // sequences per cluster batch
constexpr int kBufs = 3;        // exchange buffers per half-batch (see the hazard note in the kernel)
constexpr long long kWaitCycles = 2000000000LL;  // give up a hand-shake after about a second
constexpr uint32_t kBufBytes = 16 * 32 * kTG * 4;  // one exchange buffer

struct __align__(16) ClusterSmem {
  // M[g][buf][d][gl][t]: minimum (+ next step's xx) of predecessor group (d << 8) | (32 * rank + gl) for sequence t of
  // half-batch g. Written by remote CTAs (and locally for step 0), read as float4 over t.
  float M[kNG][kBufs][16][32][kTG];
  float m01[128][kNG][2][kTG];  // fp16(-2 x0), fp16(-2 x1) per step
  float xx[128][kNG][kTG];      // x0^2 + x1^2 per step
  unsigned long long full[kNG][kBufs];
  float red_c[kClThreads / 32][kTB];
  uint32_t red_s[kClThreads / 32][kTB];
  float fin_c[kCl][kTB];  // used in CTA 0 only: one candidate per CTA
  uint32_t fin_s[kCl][kTB];
  int ov[kTB];
  int abort_flag;
};

__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
// 16-byte store into a peer CTA's shared memory that, on delivery, counts 16 bytes on that CTA's mbarrier: data and
// signal travel together, no fence on the sending side.
__device__ __forceinline__ void st_async_v4(uint32_t addr, float a, float b, float c, float d, uint32_t bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(addr),
               "f"(a), "f"(b), "f"(c), "f"(d), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float a) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(a) : "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t addr, uint32_t a) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(a) : "memory");
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
// Arms the next phase of a local mbarrier: one arrival (this one) plus `bytes` of incoming st.async traffic.
__device__ __forceinline__ void mbar_arm(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Waits for phase `parity` of a local mbarrier. Never spins forever: after kWaitCycles it raises the CTA's abort flag and
// the launch's status word, after which every wait in the CTA falls through (results are then garbage and the host
// reports QTIP_E_KERNEL).
__device__ __forceinline__ void wait_full(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status) {
  if (mbar_try_wait(bar, parity)) return;
  const long long start = clock64();
  for (;;) {
#pragma unroll 1
    for (int spin = 0; spin < 256; ++spin)
      if (mbar_try_wait(bar, parity)) return;
    if (*abort_flag) return;
    if (clock64() - start > kWaitCycles) {
      *abort_flag = 1;
      atomicExch(status, 1);
      return;
    }
  }
}

// Back-pointers of eight steps (one 32-bit word per thread, oldest step in the top nibble) written in the layout of the
// reference's k_viterbi_fwd: A[step][j >> 2] uint16, nibble j & 3. The four lanes of a quad own j & 3 = 0..3; lane q
// collects byte 3 - q (steps 2 q, 2 q + 1) of all four words and squeezes the nibbles of each step into one uint16.
__device__ __forceinline__ void store_ref_layout(uint16_t* __restrict__ Ab, int blk, int j, uint32_t h, int last_step) {
  const int q = threadIdx.x & 3;
  uint32_t w = 0;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const uint32_t other = __shfl_sync(0xffffffffu, h, (threadIdx.x & 28) | r, 32);  // word of the lane with j & 3 == r
    w |= ((other >> (8 * (3 - q))) & 0xffu) << (8 * r);
  }
  uint32_t hi = (w >> 4) & 0x0f0f0f0fu, lo = w & 0x0f0f0f0fu;  // nibbles of step 2 q and of step 2 q + 1, one per byte
  hi = (hi | (hi >> 4)) & 0x00ff00ffu, hi = (hi | (hi >> 8)) & 0xffffu;
  lo = (lo | (lo >> 4)) & 0x00ff00ffu, lo = (lo | (lo >> 8)) & 0xffffu;
  const int s0 = blk * 8 + 2 * q;
  if (s0 <= last_step) Ab[size_t(s0) * 1024 + (j >> 2)] = uint16_t(hi);
  if (s0 + 1 <= last_step) Ab[size_t(s0 + 1) * 1024 + (j >> 2)] = uint16_t(lo);
}

// X [B][256]; overlap [B] or null; final_state [B]. Back-pointers, kRefOut = false: bp [B][16][4096] uint32, word
// (b, i >> 3, j) holds the back-pointer of step i of group j in bits [4 (7 - (i & 7)), +4); blocks below first_blk are
// not stored. kRefOut = true: the reference's [B][127][1024] uint16 table (see store_ref_layout).
template <bool kRefOut>
__global__ __cluster_dims__(kCl, 1, 1) __launch_bounds__(kClThreads, 1) void vit_fwd_cluster_kernel(
    const float* __restrict__ X, const int* __restrict__ overlap, int roll, int B, uint32_t* __restrict__ bp,
    int first_blk, uint16_t* __restrict__ final_state, const uint32_t* __restrict__ lut_h2, int* __restrict__ status,
    uint32_t tag_mask) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  ClusterSmem& sm = *reinterpret_cast<ClusterSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cg::this_cluster().block_rank();
  const int cluster_id = blockIdx.x / kCl, n_clusters = gridDim.x / kCl;
  const int j = int(rank) * kClThreads + tid;  // this thread's group index
  const int gl = tid >> 4;                     // local index of the predecessor groups it reads

  // The 16 states (d << 12) | j of this thread: LUT pair and squared norm stay in registers for the whole launch.
  float l0[16], l1[16], nr[16];
#pragma unroll
  for (int d = 0; d < 16; ++d) {
    const uint32_t u = lut_h2[(d << 12) | j];
    l0[d] = half_lo(u);
    l1[d] = half_hi(u);
    nr[d] = __fadd_rn(__fmul_rn(l0[d], l0[d]), __fmul_rn(l1[d], l1[d]));
  }

  if (tid == 0) {
    for (int g = 0; g < kNG; ++g)
      for (int b = 0; b < kBufs; ++b) mbar_init(smem_u32(&sm.full[g][b]), 1);
    sm.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // Every phase of every barrier receives one full buffer: 16 x 32 rows of kTG floats from the 8 CTAs.
    for (int g = 0; g < kNG; ++g)
      for (int b = 0; b < kBufs; ++b) mbar_arm(smem_u32(&sm.full[g][b]), kBufBytes);
  }
  cluster_sync_all();

  // Minimum of group j is read next step as predecessor (d' << 8) | g' with d' = j >> 8, g' = j & 255, i.e. by CTA
  // g' >> 5 at row (d', g' & 31). A warp covers 32 consecutive j, so all its lanes push to the same CTA.
  const uint32_t dst = uint32_t(warp & 7);
  const int dprime = int(rank) * 2 + (warp >> 3);
  const uint32_t push_base = map_to_cta(smem_u32(&sm.M[0][0][dprime][lane][0]), dst);
  const uint32_t bar_base = map_to_cta(smem_u32(&sm.full[0][0]), dst);
  constexpr uint32_t kGrpBytes = kBufs * kBufBytes;
  volatile int* abort_flag = &sm.abort_flag;
  uint32_t phase_bits = 0;  // bit g * kBufs + buf: parity of the next wait on full[g][buf]

  for (int batch = cluster_id; batch * kTB < B; batch += n_clusters) {
    const int t_first = batch * kTB;
    // Per-step input terms of the kTB sequences (sequences past B repeat the last one and are not stored).
    for (int idx = tid; idx < 128 * kTB; idx += kClThreads) {
      const int tl = idx % kTB, step = idx / kTB;
      const float* src = X + size_t(min(t_first + tl, B - 1)) * 256;
      const int p0 = roll ? ((2 * step + 128) & 255) : 2 * step;
      const float x0 = round_half(src[p0]), x1 = round_half(src[p0 + 1]);
      sm.m01[step][tl / kTG][0][tl % kTG] = round_half(-2.f * x0);
      sm.m01[step][tl / kTG][1][tl % kTG] = round_half(-2.f * x1);
      sm.xx[step][tl / kTG][tl % kTG] = __fadd_rn(__fmul_rn(x0, x0), __fmul_rn(x1, x1));
    }
    if (tid < kTB) sm.ov[tid] = overlap ? overlap[min(t_first + tid, B - 1)] : -1;
    __syncthreads();
    {  // step-0 predecessors: 0 where the start constraint allows, 1e30 elsewhere, plus xx of step 0
      const int d = tid >> 5, g0 = tid & 31;
      const int k = (d << 8) | (int(rank) * 32 + g0);
#pragma unroll
      for (int g = 0; g < kNG; ++g)
#pragma unroll
        for (int t = 0; t < kTG; ++t) {
          const int ov = sm.ov[g * kTG + t];
          sm.M[g][0][d][g0][t] = __fadd_rn((ov < 0 || k == ov) ? 0.f : 1e30f, sm.xx[0][g][t]);
        }
    }
    __syncthreads();

    uint32_t hist[kTB];
#pragma unroll
    for (int t = 0; t < kTB; ++t) hist[t] = 0;

    // Hazard note: a warp reads buffer i % 3 at step i; that buffer is rewritten by pushes of step i + 2. A CTA can only
    // compute step i + 2 after receiving every CTA's step-(i + 1) minima, and those in turn needed this warp's step-i
    // arrival at the CTA it feeds, so the reads are done by then. With two buffers that chain is one link short.
#pragma unroll 1
    for (int i = 0; i < 127; ++i) {
      const int buf = i % kBufs, nbuf = (i + 1) % kBufs;
#pragma unroll
      for (int g = 0; g < kNG; ++g) {
        if (i > 0) {
          const uint32_t bit = uint32_t(g * kBufs + buf);
          wait_full(smem_u32(&sm.full[g][buf]), (phase_bits >> bit) & 1u, abort_flag, status);
          phase_bits ^= 1u << bit;
          if (tid == 0) mbar_arm(smem_u32(&sm.full[g][buf]), kBufBytes);  // for this buffer's next use
        }
        const float4 m0 = *reinterpret_cast<const float4*>(&sm.m01[i][g][0][0]);
        const float4 m1 = *reinterpret_cast<const float4*>(&sm.m01[i][g][1][0]);
        const float m0a[4] = {m0.x, m0.y, m0.z, m0.w}, m1a[4] = {m1.x, m1.y, m1.z, m1.w};
        float best[4] = {3e30f, 3e30f, 3e30f, 3e30f};
        const float4* Mrow = reinterpret_cast<const float4*>(&sm.M[g][buf][0][gl][0]);
#pragma unroll
        for (int d = 0; d < 16; d += 2) {
          const float4 pa = Mrow[d * 32], pb = Mrow[(d + 1) * 32];
          const float paa[4] = {pa.x, pa.y, pa.z, pa.w}, pba[4] = {pb.x, pb.y, pb.z, pb.w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float ca = state_cost(l0[d], l1[d], nr[d], paa[t], m0a[t], m1a[t]);
            const float cb = state_cost(l0[d + 1], l1[d + 1], nr[d + 1], pba[t], m0a[t], m1a[t]);
            best[t] = min3(best[t], tag_cost(ca, tag_mask, d), tag_cost(cb, tag_mask, d + 1));
          }
        }
        const float4 xn = *reinterpret_cast<const float4*>(&sm.xx[i + 1][g][0]);
        const float xna[4] = {xn.x, xn.y, xn.z, xn.w};
        float out[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const uint32_t bb = __float_as_uint(best[t]);
          hist[g * kTG + t] = hist[g * kTG + t] * 16u + (bb & 15u);  // multiply-add: keeps the shift off the integer pipe
          out[t] = __fadd_rn(__uint_as_float(bb & ~15u), xna[t]);
        }
        st_async_v4(push_base + uint32_t(g) * kGrpBytes + uint32_t(nbuf) * kBufBytes, out[0], out[1], out[2], out[3],
                    bar_base + uint32_t(g * kBufs + nbuf) * 8u);
      }
      if ((i & 7) == 7 || i == 126) {
        const int blk = i >> 3;
        if (blk >= first_blk) {
#pragma unroll
          for (int t = 0; t < kTB; ++t)
            if (t_first + t < B) {  // uniform over the CTA: the quad shuffles of the reference layout are safe
              const uint32_t h = (i == 126) ? (hist[t] << 4) : hist[t];
              if constexpr (kRefOut)
                store_ref_layout(reinterpret_cast<uint16_t*>(bp) + size_t(t_first + t) * 127 * 1024, blk, j, h, 126);
              else
                bp[(size_t(t_first + t) * 16 + blk) * 4096 + j] = h;
            }
        }
      }
    }

    // Last step: untagged costs over the allowed states, lowest state on ties.
    {
      const int buf = 127 % kBufs;
#pragma unroll
      for (int g = 0; g < kNG; ++g) {
        const uint32_t bit = uint32_t(g * kBufs + buf);
        wait_full(smem_u32(&sm.full[g][buf]), (phase_bits >> bit) & 1u, abort_flag, status);
        phase_bits ^= 1u << bit;
        if (tid == 0) mbar_arm(smem_u32(&sm.full[g][buf]), kBufBytes);
        const float4 m0 = *reinterpret_cast<const float4*>(&sm.m01[127][g][0][0]);
        const float4 m1 = *reinterpret_cast<const float4*>(&sm.m01[127][g][1][0]);
        const float m0a[4] = {m0.x, m0.y, m0.z, m0.w}, m1a[4] = {m1.x, m1.y, m1.z, m1.w};
        float bv[4] = {3e30f, 3e30f, 3e30f, 3e30f};
        uint32_t bs[4] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0xffffffffu};
        const float4* Mrow = reinterpret_cast<const float4*>(&sm.M[g][buf][0][gl][0]);
#pragma unroll
        for (int d = 0; d < 16; ++d) {
          const float4 pa = Mrow[d * 32];
          const float paa[4] = {pa.x, pa.y, pa.z, pa.w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float c = state_cost(l0[d], l1[d], nr[d], paa[t], m0a[t], m1a[t]);
            if (c < bv[t]) bv[t] = c, bs[t] = (uint32_t(d) << 12) | uint32_t(j);  // d ascending: lowest state wins ties
          }
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int ov = sm.ov[g * kTG + t];
          if (ov >= 0 && j != ov) bv[t] = 3e30f, bs[t] = 0xffffffffu;
#pragma unroll
          for (int off = 16; off > 0; off >>= 1)
            take_better(bv[t], bs[t], __shfl_xor_sync(0xffffffffu, bv[t], off),
                        __shfl_xor_sync(0xffffffffu, bs[t], off));
          if (lane == 0) sm.red_c[warp][g * kTG + t] = bv[t], sm.red_s[warp][g * kTG + t] = bs[t];
        }
      }
      __syncthreads();
      if (tid < kTB) {
        float bv = sm.red_c[0][tid];
        uint32_t bs = sm.red_s[0][tid];
        for (int w = 1; w < kClThreads / 32; ++w) take_better(bv, bs, sm.red_c[w][tid], sm.red_s[w][tid]);
        st_cluster_f32(map_to_cta(smem_u32(&sm.fin_c[rank][tid]), 0), bv);
        st_cluster_u32(map_to_cta(smem_u32(&sm.fin_s[rank][tid]), 0), bs);
      }
      cluster_sync_all();  // also keeps a fast CTA from pushing the next batch into buffers still being read
      if (rank == 0 && tid < kTB && t_first + tid < B) {
        float bv = sm.fin_c[0][tid];
        uint32_t bs = sm.fin_s[0][tid];
        for (int c = 1; c < kCl; ++c) take_better(bv, bs, sm.fin_c[c][tid], sm.fin_s[c][tid]);
        final_state[t_first + tid] = uint16_t(bs);
      }
    }
  }
  cluster_sync_all();  // no CTA leaves while a peer may still write into its shared memory
}

// Back-pointer lookup in the cluster kernel's word layout.
__device__ __forceinline__ uint32_t prev_state_w(const uint32_t* bpb, int i, uint32_t s) {
  const uint32_t j = s >> 4;
  const uint32_t d = (bpb[size_t(i >> 3) * 4096 + j] >> (4 * (7 - (i & 7)))) & 15u;
  return j | (d << 12);
}
__global__ void vit_overlap_w_kernel(const uint32_t* __restrict__ bp, const uint16_t* __restrict__ final_state, int B,
                                     int* __restrict__ overlap) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const uint32_t* bpb = bp + size_t(b) * 16 * 4096;
  uint32_t s = final_state[b];
  for (int i = 126; i >= 64; --i) s = prev_state_w(bpb, i, s);
  overlap[b] = int(s >> 4);
}
// states -> Q[(b0+b)*nblk+blk][128]; decoded values -> hat[b][256] (sequence order) and/or hatWT (tile scatter).
__global__ void vit_finish_w_kernel(const uint32_t* __restrict__ bp, const uint16_t* __restrict__ final_state, int B,
                                    int b0, uint16_t* __restrict__ Q, int nblk, int blk, float* __restrict__ hat,
                                    float* __restrict__ hatWT, long m, int col0, const uint32_t* __restrict__ lut_h2) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const uint32_t* bpb = bp + size_t(b) * 16 * 4096;
  uint16_t* q = Q ? Q + (size_t(b0 + b) * nblk + blk) * 128 : nullptr;
  float* h = hat ? hat + size_t(b) * 256 : nullptr;
  uint32_t s = final_state[b];
  for (int i = 127; i >= 0; --i) {
    if (i < 127) s = prev_state_w(bpb, i, s);
    emit_state(i, s, q, hatWT, m, long(b0 + b) * 16, col0, h, lut_h2);
  }
}

// The same two backtraces for launches of few sequences, where the 63 / 127 dependent global loads of the
// one-thread-per-sequence kernels (about 0.5 us each) are the whole duration and sit on the critical path of an LDLQ
// column step. One CTA per sequence: the 4,096 words of an 8-step block (16 KB) are staged in shared memory through a
// ring of cp.async copies, thread 0 walks the 8 steps there, and the next blocks are in flight meanwhile; the states are
// then emitted by 128 threads at once. Reads 128 / 256 KB per sequence instead of 63 / 127 words, which is why the
// one-thread kernels stay for large batches. Same integer arithmetic, same outputs.
constexpr int kBtStages = 4;
constexpr int kBtThreads = 256;
constexpr size_t kBtSmem = size_t(kBtStages) * 4096 * 4;
__device__ __forceinline__ void bt_stage_block(uint32_t* dst, const uint32_t* src, int tid) {
  const uint32_t d = smem_u32(dst) + tid * 16;
  const char* g = reinterpret_cast<const char*>(src) + tid * 16;
#pragma unroll
  for (int k = 0; k < 4096 * 4 / (kBtThreads * 16); ++k)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d + k * kBtThreads * 16), "l"(g + k * kBtThreads * 16));
}
template <bool kFinish>
__global__ __launch_bounds__(kBtThreads) void vit_backtrace_staged_kernel(
    const uint32_t* __restrict__ bp, const uint16_t* __restrict__ final_state, int* __restrict__ overlap, int b0,
    uint16_t* __restrict__ Q, int nblk, int blk, float* __restrict__ hat, float* __restrict__ hatWT, long m, int col0,
    const uint32_t* __restrict__ lut_h2) {
  extern __shared__ __align__(16) uint32_t bt_ring[];  // kBtStages x 4096 words
  __shared__ uint32_t states[128];
  const int b = blockIdx.x, tid = threadIdx.x;
  const uint32_t* bpb = bp + size_t(b) * 16 * 4096;
  constexpr int kLast = kFinish ? 0 : 8;  // the overlap walk ends at step 64
  for (int k = 0; k < kBtStages - 1; ++k) {
    if (15 - k >= kLast) bt_stage_block(bt_ring + (k % kBtStages) * 4096, bpb + size_t(15 - k) * 4096, tid);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  uint32_t s = 0;
  if (tid == 0) states[127] = s = final_state[b];
  for (int q = 15; q >= kLast; --q) {
    const int ahead = q - (kBtStages - 1);
    if (ahead >= kLast) bt_stage_block(bt_ring + ((15 - ahead) % kBtStages) * 4096, bpb + size_t(ahead) * 4096, tid);
    asm volatile("cp.async.commit_group;" ::: "memory");  // one group per iteration, empty at the end
    asm volatile("cp.async.wait_group %0;" ::"n"(kBtStages - 1) : "memory");
    __syncthreads();  // block q has landed, for every thread's copies
    if (tid == 0) {
      const uint32_t* w = bt_ring + ((15 - q) % kBtStages) * 4096;
      for (int i = q == 15 ? 126 : 8 * q + 7; i >= 8 * q; --i) {
        const uint32_t j = s >> 4;
        s = j | (((w[j] >> (4 * (7 - (i & 7)))) & 15u) << 12);
        states[i] = s;
      }
    }
    __syncthreads();  // the buffer of block q is re-used by the copy issued in the next iteration
  }
  if (!kFinish) {
    if (tid == 0) overlap[b] = int(s >> 4);
    return;
  }
  if (tid < 128)
    emit_state(tid, states[tid], Q ? Q + (size_t(b0 + b) * nblk + blk) * 128 : nullptr, hatWT, m, long(b0 + b) * 16, col0,
               hat ? hat + size_t(b) * 256 : nullptr, lut_h2);
}
constexpr int kBtMaxBatch = 1024;  // launches of up to this many sequences take the staged kernels

// ------------------------------------------------------------------------------------------------- host side

__device__ int g_vit_status;  // time-outs of cluster launches made through the kernel-level entry point

// ---- scratch of the allocation-free entry point (qtip_quantize_tiles_noalloc, at the end of this file)
constexpr int kNoAllocMaxTiles = 64;
constexpr size_t kNoAllocHeader = 256;  // status word; the same header a caller-owned workspace starts with
constexpr size_t kNoAllocBytes = kNoAllocHeader + 256 + 256 + size_t(kNoAllocMaxTiles) * 16 * 4096 * 4;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];
static std::mutex g_noalloc_mu;
static void* g_noalloc_ptr[64];  // device address of the array on each device, resolved on first use

// Status words that live inside the library (no caller-owned workspace to carry them): the kernel-level cluster
// launches and the built-in scratch of the allocation-free entry point. Queues the copies on `s` and, behind them,
// the clearing of both words, so that one reported time-out does not stay set for the rest of the process.
int viterbi_read_status(int* kernel_level, int* noalloc, cudaStream_t s) {
  *kernel_level = 0, *noalloc = 0;
  void* kv = nullptr;
  QB_CUDA(cudaGetSymbolAddress(&kv, g_vit_status));
  QB_CUDA(cudaMemcpyAsync(kernel_level, kv, sizeof(int), cudaMemcpyDeviceToHost, s));
  QB_CUDA(cudaMemsetAsync(kv, 0, sizeof(int), s));
  int dev = -1;
  QB_CUDA(cudaGetDevice(&dev));
  void* na = nullptr;
  if (dev >= 0 && dev < 64) {
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    na = g_noalloc_ptr[dev];
  }
  if (na) {  // the entry point has run on this device
    QB_CUDA(cudaMemcpyAsync(noalloc, na, sizeof(int), cudaMemcpyDeviceToHost, s));
    QB_CUDA(cudaMemsetAsync(na, 0, sizeof(int), s));
  }
  return QTIP_OK;
}

int viterbi_set_status(int which, int value, cudaStream_t s) {
  void* at = nullptr;
  if (which == 1) {
    QB_CUDA(cudaGetSymbolAddress(&at, g_vit_status));
  } else {
    int dev = -1;
    QB_CUDA(cudaGetDevice(&dev));
    QB_REQUIRE(dev >= 0 && dev < 64, QTIP_E_DEVICE, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    at = g_noalloc_ptr[dev];
    QB_REQUIRE(at, QTIP_E_ARG, "qtip_quantize_tiles_noalloc has not run on device %d yet", dev);
  }
  QB_CUDA(cudaMemcpyAsync(at, &value, sizeof(int), cudaMemcpyHostToDevice, s));
  QB_CUDA(cudaStreamSynchronize(s));  // `value` is on this function's stack
  return QTIP_OK;
}

int viterbi_device_setup(DeviceInfo* info) {
  QB_CUDA(cudaFuncSetAttribute(vit_fwd_cluster_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               int(sizeof(ClusterSmem))));
  QB_CUDA(cudaFuncSetAttribute(vit_fwd_cluster_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               int(sizeof(ClusterSmem))));
  QB_CUDA(cudaFuncSetAttribute(vit_backtrace_staged_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kBtSmem)));
  QB_CUDA(cudaFuncSetAttribute(vit_backtrace_staged_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kBtSmem)));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(kCl * 64);
  cfg.blockDim = dim3(kClThreads);
  cfg.dynamicSmemBytes = sizeof(ClusterSmem);
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = kCl;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int n = 0;
  QB_CUDA(cudaOccupancyMaxActiveClusters(&n, vit_fwd_cluster_kernel<false>, &cfg));
  QB_REQUIRE(n > 0, QTIP_E_DEVICE, "the device cannot co-schedule an %d-CTA cluster of the Viterbi kernel", kCl);
  info->max_clusters = n;
  return QTIP_OK;
}

// Workspace of the fused path: [status (256 B)] [final_state u16 x cap] [overlap i32 x cap] [bp 256 KiB x cap].
struct QuantWorkspace {
  int* status;
  uint16_t* fs;
  int* ov;
  uint32_t* bp;
  int cap;
};
constexpr size_t kWsHeader = 256, kBpBytes = size_t(16) * 4096 * 4;
static size_t ws_bytes_for(size_t cap) {
  size_t o = kWsHeader + ((cap * 2 + 255) / 256) * 256 + ((cap * 4 + 255) / 256) * 256;
  return o + cap * kBpBytes;
}
static bool carve_workspace(void* ws, size_t bytes, QuantWorkspace* out) {
  if (!ws || bytes < ws_bytes_for(kTB)) return false;
  size_t cap = (bytes - kWsHeader) / kBpBytes;
  while (cap > 0 && ws_bytes_for(cap) > bytes) --cap;
  if (cap < size_t(kTB)) return false;
  cap = cap / kTB * kTB;
  if (cap > (1u << 20)) cap = 1u << 20;
  unsigned char* p = static_cast<unsigned char*>(ws);
  out->status = reinterpret_cast<int*>(p);
  p += kWsHeader;
  out->fs = reinterpret_cast<uint16_t*>(p);
  p += ((cap * 2 + 255) / 256) * 256;
  out->ov = reinterpret_cast<int*>(p);
  p += ((cap * 4 + 255) / 256) * 256;
  out->bp = reinterpret_cast<uint32_t*>(p);
  out->cap = int(cap);
  return true;
}

template <bool kRefOut = false>
static int launch_cluster_fwd(const DeviceInfo* info, const float* X, const int* overlap, int roll, int B, uint32_t* bp,
                              int first_blk, uint16_t* fs, const uint32_t* lut, int* status, cudaStream_t s) {
  const int batches = (B + kTB - 1) / kTB;
  const int clusters = batches < info->max_clusters ? batches : info->max_clusters;
  vit_fwd_cluster_kernel<kRefOut><<<dim3(clusters * kCl), dim3(kClThreads), sizeof(ClusterSmem), s>>>(
      X, overlap, roll, B, bp, first_blk, fs, lut, status, kTagMask);
  QB_LAUNCHED();
  return QTIP_OK;
}

// One side stream and two events per device for the two-lane schedule below (created on first use, never destroyed).
struct LaneStreams {
  cudaStream_t side = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
  bool ready = false;
};
static std::mutex g_lane_mu;
static LaneStreams g_lane[64];
static int lane_streams(LaneStreams** out) {
  int dev = 0;
  QB_CUDA(cudaGetDevice(&dev));
  QB_REQUIRE(dev >= 0 && dev < 64, QTIP_E_DEVICE, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_lane_mu);
  LaneStreams& l = g_lane[dev];
  if (!l.ready) {
    QB_CUDA(cudaStreamCreateWithFlags(&l.side, cudaStreamNonBlocking));
    QB_CUDA(cudaEventCreateWithFlags(&l.fork, cudaEventDisableTiming));
    QB_CUDA(cudaEventCreateWithFlags(&l.join, cudaEventDisableTiming));
    l.ready = true;
  }
  *out = &l;
  return QTIP_OK;
}

// Shared body of the fused entry points. The sequences are processed in chunks that fit the workspace: forward (rolled),
// overlap, forward (constrained), finish. two_lanes: the workspace is halved and consecutive chunks alternate between
// the caller's stream and a side stream, so that one chunk's backtrace kernels (one thread per sequence) and the partly
// filled last round of its forward launches run under the other chunk's forward pass.
int quantize_tiles_impl(const float* X, int B, int b0, const uint32_t* lut, uint16_t* Q, int nblk, int blk, float* hat,
                        float* hatWT, long m, int col0, void* ws, size_t ws_bytes, bool reset_status, cudaStream_t s,
                        bool two_lanes) {
  const DeviceInfo* info = device_info();
  if (!info) return QTIP_E_DEVICE;
  QuantWorkspace w;
  QB_REQUIRE(carve_workspace(ws, ws_bytes, &w), QTIP_E_WORKSPACE,
             "workspace of %zu bytes is too small (need at least %zu)", ws_bytes, ws_bytes_for(kTB));
  if (reset_status) QB_CUDA(cudaMemsetAsync(w.status, 0, kWsHeader, s));
  const int half = w.cap / 2 / kTB * kTB;
  two_lanes = two_lanes && half >= 16 * kTB && B > half;  // worth it only with several chunks of a useful size
  LaneStreams* ls = nullptr;
  if (two_lanes) {
    int rc = lane_streams(&ls);
    if (rc) return rc;
    QB_CUDA(cudaEventRecord(ls->fork, s));
    QB_CUDA(cudaStreamWaitEvent(ls->side, ls->fork, 0));
  }
  const int cap = two_lanes ? half : w.cap;
  // The chunk loop as a function, so that every way out of it passes the join below: a failed launch must not leave the
  // side stream un-joined (it may still be writing the outputs, and an open fork would invalidate a stream capture).
  auto chunks = [&]() -> int {
    int lane = 0;
    for (int c0 = 0; c0 < B; c0 += cap, lane ^= 1) {
      const int nb = B - c0 < cap ? B - c0 : cap;
      const float* xc = X + size_t(c0) * 256;
      const int o = (two_lanes && lane) ? half : 0;  // this lane's part of the scratch arrays
      cudaStream_t st = (two_lanes && lane) ? ls->side : s;
      uint32_t* bp = w.bp + size_t(o) * (kBpBytes / 4);
      int rc = launch_cluster_fwd(info, xc, nullptr, 1, nb, bp, 8, w.fs + o, lut, w.status, st);
      if (rc) return rc;
      if (nb <= kBtMaxBatch)
        vit_backtrace_staged_kernel<false><<<nb, kBtThreads, kBtSmem, st>>>(bp, w.fs + o, w.ov + o, 0, nullptr, 0, 0, nullptr,
                                                                           nullptr, 0, 0, nullptr);
      else
        vit_overlap_w_kernel<<<blocks_for(nb, 64), 64, 0, st>>>(bp, w.fs + o, nb, w.ov + o);
      QB_LAUNCHED();
      rc = launch_cluster_fwd(info, xc, w.ov + o, 0, nb, bp, 0, w.fs + o, lut, w.status, st);
      if (rc) return rc;
      float* hc = hat ? hat + size_t(c0) * 256 : nullptr;
      if (nb <= kBtMaxBatch)
        vit_backtrace_staged_kernel<true><<<nb, kBtThreads, kBtSmem, st>>>(bp, w.fs + o, nullptr, b0 + c0, Q, nblk, blk, hc,
                                                                          hatWT, m, col0, lut);
      else
        vit_finish_w_kernel<<<blocks_for(nb, 64), 64, 0, st>>>(bp, w.fs + o, nb, b0 + c0, Q, nblk, blk, hc, hatWT, m, col0,
                                                               lut);
      QB_LAUNCHED();
    }
    return QTIP_OK;
  };
  const int rc = chunks();
  if (two_lanes) {
    QB_CUDA(cudaEventRecord(ls->join, ls->side));
    QB_CUDA(cudaStreamWaitEvent(s, ls->join, 0));
  }
  return rc;
}

}  // namespace qb

using namespace qb;

extern "C" int qtip_k_viterbi_fwd(const float* X_d, const int* overlap_d, int roll, int B, uint16_t* A_d,
                                  uint16_t* final_state_d, const uint32_t* lut_h2_d, void* stream) {
  QB_REQUIRE(X_d && A_d && final_state_d && lut_h2_d && B >= 0, QTIP_E_ARG, "qtip_k_viterbi_fwd: bad argument");
  if (B == 0) return QTIP_OK;
  // The cluster kernel with the reference's back-pointer layout as its output; its bounded waits report through a word
  // inside the library (qtip_kernel_status), since this entry point has no status argument.
  const DeviceInfo* info = device_info();
  if (!info) return QTIP_E_DEVICE;
  void* st = nullptr;
  QB_CUDA(cudaGetSymbolAddress(&st, g_vit_status));
  return launch_cluster_fwd<true>(info, X_d, overlap_d, roll, B, reinterpret_cast<uint32_t*>(A_d), 0, final_state_d,
                                  lut_h2_d, static_cast<int*>(st), as_stream(stream));
}
extern "C" int qtip_k_viterbi_overlap(const uint16_t* A_d, const uint16_t* final_state_d, int B, int* overlap_d,
                                      void* stream) {
  QB_REQUIRE(A_d && final_state_d && overlap_d && B >= 0, QTIP_E_ARG, "qtip_k_viterbi_overlap: bad argument");
  if (B == 0) return QTIP_OK;
  vit_overlap_u16_kernel<<<blocks_for(B, 64), 64, 0, as_stream(stream)>>>(A_d, final_state_d, B, overlap_d);
  QB_LAUNCHED();
  return QTIP_OK;
}
extern "C" int qtip_k_viterbi_finish(const uint16_t* A_d, const uint16_t* final_state_d, int B, int b0, uint16_t* Q_d,
                                     int nblk, int blk, float* hatWT_d, long m, int col0, const uint32_t* lut_h2_d,
                                     void* stream) {
  QB_REQUIRE(A_d && final_state_d && lut_h2_d && B >= 0, QTIP_E_ARG, "qtip_k_viterbi_finish: bad argument");
  if (B == 0) return QTIP_OK;
  vit_finish_u16_kernel<<<blocks_for(B, 64), 64, 0, as_stream(stream)>>>(A_d, final_state_d, B, b0, Q_d, nblk, blk,
                                                                         hatWT_d, m, col0, lut_h2_d);
  QB_LAUNCHED();
  return QTIP_OK;
}
extern "C" int qtip_k_decode_states(const uint16_t* states_d, int B, float* hat_d, const uint32_t* lut_h2_d,
                                    void* stream) {
  QB_REQUIRE(states_d && hat_d && lut_h2_d && B >= 0, QTIP_E_ARG, "qtip_k_decode_states: bad argument");
  if (B == 0) return QTIP_OK;
  const long n = long(B) * 128;
  decode_states_kernel<<<blocks_for(n, 256), 256, 0, as_stream(stream)>>>(states_d, n, hat_d, lut_h2_d);
  QB_LAUNCHED();
  return QTIP_OK;
}

extern "C" int qtip_k_viterbi_fwd_words(const float* X_d, const int* overlap_d, int roll, int B, uint32_t* bp_d,
                                        int first_block, uint16_t* final_state_d, const uint32_t* lut_h2_d,
                                        int* status_d, void* stream) {
  QB_REQUIRE(X_d && bp_d && final_state_d && lut_h2_d && status_d && B >= 0 && first_block >= 0 && first_block < 16,
             QTIP_E_ARG, "qtip_k_viterbi_fwd_words: bad argument");
  const DeviceInfo* info = device_info();
  if (!info) return QTIP_E_DEVICE;
  if (B == 0) return QTIP_OK;
  return launch_cluster_fwd(info, X_d, overlap_d, roll, B, bp_d, first_block, final_state_d, lut_h2_d, status_d,
                            as_stream(stream));
}
extern "C" int qtip_k_viterbi_overlap_words(const uint32_t* bp_d, const uint16_t* final_state_d, int B, int* overlap_d,
                                            void* stream) {
  QB_REQUIRE(bp_d && final_state_d && overlap_d && B >= 0, QTIP_E_ARG, "qtip_k_viterbi_overlap_words: bad argument");
  if (B == 0) return QTIP_OK;
  vit_overlap_w_kernel<<<blocks_for(B, 64), 64, 0, as_stream(stream)>>>(bp_d, final_state_d, B, overlap_d);
  QB_LAUNCHED();
  return QTIP_OK;
}
extern "C" int qtip_k_viterbi_finish_words(const uint32_t* bp_d, const uint16_t* final_state_d, int B, int b0,
                                           uint16_t* Q_d, int nblk, int blk, float* hat_d, float* hatWT_d, long m,
                                           int col0, const uint32_t* lut_h2_d, void* stream) {
  QB_REQUIRE(bp_d && final_state_d && lut_h2_d && B >= 0, QTIP_E_ARG, "qtip_k_viterbi_finish_words: bad argument");
  if (B == 0) return QTIP_OK;
  vit_finish_w_kernel<<<blocks_for(B, 64), 64, 0, as_stream(stream)>>>(bp_d, final_state_d, B, b0, Q_d, nblk, blk,
                                                                       hat_d, hatWT_d, m, col0, lut_h2_d);
  QB_LAUNCHED();
  return QTIP_OK;
}

extern "C" size_t qtip_quantize_workspace_bytes(int max_tiles) {
  size_t cap = max_tiles < kTB ? size_t(kTB) : size_t((max_tiles + kTB - 1) / kTB * kTB);
  return ws_bytes_for(cap);
}
extern "C" int qtip_quantize_tiles(const float* X_d, int B, const uint32_t* lut_h2_d, uint16_t* states_d, float* hat_d,
                                   void* workspace_d, size_t workspace_bytes, void* stream) {
  if (B == 0) return QTIP_OK;
  QB_REQUIRE(X_d && lut_h2_d && B > 0, QTIP_E_ARG, "qtip_quantize_tiles: bad argument");
  return quantize_tiles_impl(X_d, B, 0, lut_h2_d, states_d, 1, 0, hat_d, nullptr, 0, 0, workspace_d, workspace_bytes,
                             true, as_stream(stream), true);
}
extern "C" int qtip_quantize_tiles_scatter(const float* X_d, int B, int b0, const uint32_t* lut_h2_d, uint16_t* Q_d,
                                           int nblk, int blk, float* hatWT_d, long m, int col0, void* workspace_d,
                                           size_t workspace_bytes, void* stream) {
  QB_REQUIRE(X_d && lut_h2_d && B >= 0 && b0 >= 0 && nblk >= 1 && blk >= 0 && blk < nblk, QTIP_E_ARG,
             "qtip_quantize_tiles_scatter: bad argument");
  QB_REQUIRE(!hatWT_d || m >= long(b0 + B) * 16, QTIP_E_GEOMETRY,
             "qtip_quantize_tiles_scatter: m = %ld does not cover %d row blocks", m, b0 + B);
  if (B == 0) return QTIP_OK;
  return quantize_tiles_impl(X_d, B, b0, lut_h2_d, Q_d, nblk, blk, nullptr, hatWT_d, m, col0, workspace_d,
                             workspace_bytes, true, as_stream(stream), true);
}
// ---- allocation-free variant of qtip_quantize_tiles
// Some hosts of this library may not allocate device memory at all: a serving process whose memory pool is sized once at
// start-up and frozen, a plugin that is handed a fixed arena by its framework, or a latency-critical loop in which
// cudaMalloc is banned because it synchronises the whole device and can fail once memory is fragmented. For them the
// Viterbi scratch (status word, final states, overlaps, back-pointer words) lives in the array below, which is part of
// the loaded module: every GPU that loads the library holds these 16 MiB until the process exits.
static_assert(kNoAllocHeader == kWsHeader && kNoAllocBytes == kWsHeader + 256 + 256 + size_t(kNoAllocMaxTiles) * kBpBytes,
              "the built-in scratch is laid out like a workspace of 64 sequences");

extern "C" int qtip_quantize_tiles_noalloc(const float* X_d, int B, const uint32_t* lut_h2_d, uint16_t* states_d,
                                           float* hat_d, void* stream) {
  if (B == 0) return QTIP_OK;
  QB_REQUIRE(X_d && lut_h2_d && B > 0, QTIP_E_ARG, "qtip_quantize_tiles_noalloc: bad argument");
  QB_REQUIRE(B <= kNoAllocMaxTiles, QTIP_E_WORKSPACE,
             "qtip_quantize_tiles_noalloc: %d sequences exceed the built-in scratch of %d; split the batch or use "
             "qtip_quantize_tiles with a caller-owned workspace", B, kNoAllocMaxTiles);
  if (!device_info()) return QTIP_E_DEVICE;
  int dev = 0;
  QB_CUDA(cudaGetDevice(&dev));
  QB_REQUIRE(dev >= 0 && dev < 64, QTIP_E_DEVICE, "device index %d out of range", dev);
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (!g_noalloc_ptr[dev]) {
      // In host code the array's name is only a handle; the kernels need its address on the current device.
      void* p = nullptr;
      QB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
      g_noalloc_ptr[dev] = p;
    }
    scratch = g_noalloc_ptr[dev];
  }
  // The array keeps whatever the previous call left. Every field but the status word is written before it is read; the
  // status word is NOT cleared here, so that a time-out of any call since the last qtip_kernel_status (which reads and
  // clears it) is still reported.
  return quantize_tiles_impl(X_d, B, 0, lut_h2_d, states_d, 1, 0, hat_d, nullptr, 0, 0, scratch, kNoAllocBytes, false,
                             as_stream(stream), false);  // one lane: this entry point creates no streams or events
}

extern "C" int qtip_workspace_status(const void* workspace_d, void* stream) {
  QB_REQUIRE(workspace_d, QTIP_E_ARG, "qtip_workspace_status: null workspace");
  int st = 0;
  QB_CUDA(cudaMemcpyAsync(&st, workspace_d, 4, cudaMemcpyDeviceToHost, as_stream(stream)));
  QB_CUDA(cudaStreamSynchronize(as_stream(stream)));
  QB_REQUIRE(st == 0, QTIP_E_KERNEL, "a Viterbi hand-shake between thread blocks timed out (status %d)", st);
  return QTIP_OK;
}
