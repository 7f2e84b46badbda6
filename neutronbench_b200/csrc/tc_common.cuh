// Helpers shared by the tensor-core GEMM kernels (dense_tc.cu: operands staged by cp.async; dense_tma.cu: operands
// staged by TMA tensor loads): mbarrier, tcgen05 descriptors and MMA issue, the hi/lo split.
#pragma once
#include "common.cuh"

namespace nb {

constexpr int kBM = 128;           // rows of a C tile = TMEM lanes
constexpr int kBK = 16;            // cp.async kernel: K elements per shared-memory chunk (2 MMA K-steps of 8)
constexpr int kCtasPerSM = 2;      // cp.async kernel with three stages: 108 KB of shared memory per CTA
constexpr uint32_t kTcWaitLimit = 1u << 20;


struct TcGemmArgs {
  const float *a, *b;
  float *c;                 // output, or split-K partials [splits][M][N]
  int64_t M, N, K;
  int64_t a_row, a_k;       // element strides of op(A)(i,k): address = a + i*a_row + k*a_k
  int64_t b_row, b_k;       // element strides of op(B)^T(j,k): address = b + j*b_row + k*b_k
  int64_t k_per_split;
  int a_vec, b_vec;         // widest aligned vector (floats) along the unit-stride dimension
  int mode;                 // 1: 3xTF32, 2: 1xTF32
};

__device__ __forceinline__ uint32_t tc_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void tc_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ bool tc_mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: false when the limit ran out (the caller records the error and winds down).
__device__ __forceinline__ bool tc_mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < kTcWaitLimit; i++)
    if (tc_mbar_try_wait(bar, parity)) return true;
  return false;
}

// Shared-memory matrix descriptor: start address, the two strides (see the tile layouts below), bit 46 =
// descriptor version 1, bits 61-63 = layout type.
__device__ __forceinline__ uint64_t tc_make_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo, uint32_t layout = 0) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)(layout & 7) << 61;   // 0: no swizzle, 1: 128-byte swizzle with 32-byte atoms
  return d;
}

__device__ __forceinline__ void tc_mma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_split(float x, float &hi, float &lo) {
  hi = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
  lo = x - hi;
}


}  // namespace nb
