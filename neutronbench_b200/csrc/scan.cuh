// Block-level exclusive scan and the one-block scan kernel, shared by the scan entry points and by the
// kernels that fuse the production of the scanned values into the scan (hop counts, bitmap popcounts).
#pragma once
#include "common.cuh"

namespace nb {

constexpr int kScanThreads = 256;
constexpr int kScanItems = 8;
constexpr int kScanTile = kScanThreads * kScanItems;

template <typename T>
__device__ __forceinline__ T block_exclusive_scan(T val, T *total, T *smem /* 32 entries */) {
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  T incl = val;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    T n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= (unsigned)o) incl += n;
  }
  if (lane == 31) smem[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    T w = (lane < (blockDim.x >> 5)) ? smem[lane] : (T)0;
    T wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      T n = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= (unsigned)o) wi += n;
    }
    smem[lane] = wi - w;  // exclusive prefix of the warp totals
    if (lane == 31) smem[32] = wi;
  }
  __syncthreads();
  T res = smem[warp] + incl - val;
  *total = smem[32];
  __syncthreads();
  return res;
}

// Reads element i of the sequence to scan.  ScanLoadArray is the plain case; fused producers define
// their own functor with the same call operator.
struct ScanLoadArray {
  const uint32_t *in;
  __device__ __forceinline__ uint32_t operator()(uint64_t i) const { return in[i]; }
};

// Small inputs (the per-hop arrays of a sampled block): one block walks the sequence in chunks of
// 1024 x 8 with a running carry.  One launch instead of three; every element is produced once.
template <typename TOut, typename Load>
__global__ void __launch_bounds__(1024) scan_single_block(Load load, TOut *out, uint64_t n, bool write_total) {
  __shared__ TOut smem[33];
  TOut carry = 0;
  for (uint64_t start = 0; start < n; start += 1024 * kScanItems) {
    const uint64_t base = start + (uint64_t)threadIdx.x * kScanItems;
    uint32_t v[kScanItems];
    TOut sum = 0;
#pragma unroll
    for (int k = 0; k < kScanItems; k++) {
      v[k] = (base + k < n) ? load(base + k) : 0u;
      sum += v[k];
    }
    TOut total;
    TOut ex = block_exclusive_scan<TOut>(sum, &total, smem) + carry;
#pragma unroll
    for (int k = 0; k < kScanItems; k++) {
      if (base + k < n) out[base + k] = ex;
      ex += v[k];
    }
    carry += total;
  }
  if (write_total && threadIdx.x == 0) out[n] = carry;
}

// One block walks 8192 elements per round trip through its barrier: beyond a few rounds the three-launch
// scan (all SMs) is faster.  Fused producers that read scattered memory per element get a lower limit.
constexpr uint64_t kSingleBlockScanMax = 1u << 13;
constexpr uint64_t kSingleBlockGatherScanMax = 1u << 12;

}  // namespace nb
