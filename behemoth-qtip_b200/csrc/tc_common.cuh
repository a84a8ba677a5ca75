// Shared pieces of the tcgen05 kernels: mbarrier and TMA wrappers, bounded waits, shared-memory and instruction
// descriptors, the tensor-map encoder. Every wait gives up after kTcWaitCycles and raises the CTA's abort flag and the
// caller's status word, so that a broken pipeline ends as an error code and not as a hung GPU.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace qb {

constexpr long long kTcWaitCycles = 2000000000LL;

__device__ __forceinline__ void tc_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void tc_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool tc_mbar_try(uint32_t bar, uint32_t parity) {
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
// Returns false if the wait was abandoned (time-out here or elsewhere in the CTA).
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status) {
  if (tc_mbar_try(bar, parity)) return true;
  const long long start = clock64();
  for (;;) {
#pragma unroll 1
    for (int spin = 0; spin < 128; ++spin)
      if (tc_mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - start > kTcWaitCycles) {
      *abort_flag = 1;
      if (status) atomicExch(status, 2);
      return false;
    }
  }
}
__device__ __forceinline__ void tc_tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bf16) with the 128-byte swizzle:
// 8-row groups 1,024 bytes apart (stride byte offset), descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= uint64_t((addr & 0x3ffffu) >> 4);       // start address, 16-byte units
  d |= uint64_t(1) << 16;                      // leading byte offset: unused for swizzled K-major tiles
  d |= uint64_t(1024 >> 4) << 32;              // stride byte offset
  d |= uint64_t(1) << 46;                      // descriptor version (Blackwell)
  d |= uint64_t(2) << 61;                      // SWIZZLE_128B
  return d;
}
// Instruction descriptor: D fp32, A and B bf16, both K-major, M x N per instruction (K = 16).
constexpr uint32_t tc_idesc(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(uint32_t(accumulate))
      : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tc_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// [rows][k] bf16 row-major, box = box_rows x 64 columns, 128-byte swizzle, zero fill outside the tensor.
int tc_make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t k, uint32_t box_rows);

}  // namespace qb
