// Block construction on the device: bitmap dedup -> ordered reindex -> CSR transpose -> degree
// factors and edge weights.  Integer / byte work, HBM- and L2-bound; no sort of the vertex set.
//
// Ordering contract (what makes the result bit-identical to the reference):
//   source[]        ascending global id  (the reference scans its bitmap low bit first,
//                   core/coocsc.hpp:372-391); here rank(g) = prefix[g>>5] + popc(word & below(g)).
//   column_indices  ascending local destination inside every source row (stable counting sort in
//                   core/coocsc.hpp:293-298); here rows are filled with atomic cursors and then each
//                   row is sorted — equal keys are indistinguishable, so the result is unique.
#include "common.cuh"
#include "scan.cuh"

namespace nb {

constexpr int kThreads = 256;

// ------------------------------------------------------------------------------------ dedup / reindex
__global__ void mark_bitmap_kernel(const uint32_t *__restrict__ row_indices, uint32_t e, uint32_t num_vertices,
                                   uint32_t *bitmap, uint32_t *err) {
  for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < e; j += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t g = row_indices[j];
    if (g >= num_vertices) {  // corrupt input: record it, touch nothing
      atomicExch(err, 1u);
      continue;
    }
    const uint32_t bit = 1u << (g & 31);
    if ((bitmap[g >> 5] & bit) == 0) atomicOr(&bitmap[g >> 5], bit);
  }
}

__global__ void popc_words_kernel(const uint32_t *__restrict__ bitmap, uint32_t *__restrict__ counts, uint64_t words) {
  for (uint64_t w = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; w < words; w += (uint64_t)gridDim.x * blockDim.x)
    counts[w] = __popc(bitmap[w]);
}

// Scan input produced on the fly: the population count of bitmap word i.
struct ScanLoadPopc {
  const uint32_t *bitmap;
  __device__ __forceinline__ uint32_t operator()(uint64_t i) const { return __popc(bitmap[i]); }
};

// Also clears the CSR row counters (zero_n entries) that the next kernel accumulates into.
__global__ void emit_source_kernel(const uint32_t *__restrict__ bitmap, const uint32_t *__restrict__ prefix,
                                   uint64_t words, uint32_t *__restrict__ source, uint32_t *__restrict__ zero,
                                   uint64_t zero_n) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < zero_n; i += (uint64_t)gridDim.x * blockDim.x)
    zero[i] = 0u;
  for (uint64_t w = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; w < words; w += (uint64_t)gridDim.x * blockDim.x) {
    uint32_t word = bitmap[w];
    uint32_t p = prefix[w];
    while (word) {
      const int b = __ffs(word) - 1;
      source[p++] = (uint32_t)(w << 5) + b;
      word &= word - 1;
    }
  }
}

// row_indices: global id -> local rank; also counts the length of every CSR row.
__global__ void remap_count_kernel(uint32_t *row_indices, uint32_t e, const uint32_t *__restrict__ bitmap,
                                   const uint32_t *__restrict__ prefix, uint32_t num_vertices,
                                   uint32_t *row_count) {
  for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < e; j += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t g = row_indices[j];
    if (g >= num_vertices) continue;
    const uint32_t below = (1u << (g & 31)) - 1u;
    const uint32_t local = prefix[g >> 5] + __popc(bitmap[g >> 5] & below);
    row_indices[j] = local;
    atomicAdd(&row_count[local], 1u);
  }
}

// ------------------------------------------------------------------------------------ norms
// Both degree factors of a block and the fill cursors (a copy of the row offsets) in one pass.
__global__ void degree_norms_kernel(const uint32_t *__restrict__ row_offset, uint32_t s, float *__restrict__ src_norm,
                                    uint32_t *__restrict__ cursor, const uint32_t *__restrict__ column_offset,
                                    uint32_t v, float *__restrict__ dst_norm) {
  const uint64_t n = s > v ? s : v;
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
    if (i < s) {
      const uint32_t lo = row_offset[i];
      src_norm[i] = (float)sqrt((double)(row_offset[i + 1] - lo));
      if (cursor) cursor[i] = lo;
    }
    if (i < v) dst_norm[i] = (float)sqrt((double)(column_offset[i + 1] - column_offset[i]));
  }
}

// Index of the segment that holds position j: largest i with offsets[i] <= j (offsets ascending, n+1 entries).
__device__ __forceinline__ uint32_t find_segment(const uint32_t *__restrict__ offsets, uint32_t n, uint32_t j) {
  uint32_t lo = 0, hi = n;  // answer in [lo, hi)
  while (hi - lo > 1) {
    const uint32_t mid = (lo + hi) >> 1;
    if (offsets[mid] <= j) lo = mid; else hi = mid;
  }
  return lo;
}

// ------------------------------------------------------------------------------------ CSR fill
// One thread per CSC edge: append the edge's destination to its source row, emit the forward weight.
__global__ void csr_fill_kernel(const uint32_t *__restrict__ column_offset, const uint32_t *__restrict__ row_indices,
                                uint32_t v, uint32_t e, uint32_t *cursor, uint32_t *__restrict__ column_indices,
                                const float *__restrict__ src_norm, const float *__restrict__ dst_norm,
                                float *__restrict__ w_fwd) {
  for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < e; j += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t d = find_segment(column_offset, v, (uint32_t)j);
    const uint32_t ls = row_indices[j];
    const uint32_t pos = atomicAdd(&cursor[ls], 1u);
    column_indices[pos] = d;
    if (w_fwd) w_fwd[j] = __fdiv_rn(1.0f, __fmul_rn(src_norm[ls], dst_norm[d]));
  }
}

__global__ void csr_weight_kernel(const uint32_t *__restrict__ row_offset, const uint32_t *__restrict__ column_indices,
                                  uint32_t s, uint32_t e, const float *__restrict__ src_norm,
                                  const float *__restrict__ dst_norm, float *__restrict__ w_bwd) {
  for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < e; j += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t r = find_segment(row_offset, s, (uint32_t)j);
    w_bwd[j] = __fdiv_rn(1.0f, __fmul_rn(src_norm[r], dst_norm[column_indices[j]]));
  }
}

// Lean path (no explicit weight arrays): source emission, reindex + row counting and cursor clearing in one
// launch.  The three jobs are independent of one another; the row counters were cleared by an earlier launch.
__global__ void emit_remap_kernel(const uint32_t *__restrict__ bitmap, const uint32_t *__restrict__ prefix,
                                  uint64_t words, uint32_t *__restrict__ source, uint32_t *row_indices, uint32_t e,
                                  uint32_t num_vertices, uint32_t *row_count, uint32_t *__restrict__ cursor, uint32_t s) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, t0 = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (uint64_t i = t0; i < s; i += stride) cursor[i] = 0u;
  for (uint64_t w = t0; w < words; w += stride) {
    uint32_t word = bitmap[w];
    uint32_t p = prefix[w];
    while (word) {
      const int b = __ffs(word) - 1;
      source[p++] = (uint32_t)(w << 5) + b;
      word &= word - 1;
    }
  }
  for (uint64_t j = t0; j < e; j += stride) {
    const uint32_t g = row_indices[j];
    if (g >= num_vertices) continue;
    const uint32_t below = (1u << (g & 31)) - 1u;
    const uint32_t local = prefix[g >> 5] + __popc(bitmap[g >> 5] & below);
    row_indices[j] = local;
    atomicAdd(&row_count[local], 1u);
  }
}

// Lean path: CSR fill (cursor counts from zero on top of the row offsets) and both degree factors in one launch.
__global__ void fill_norms_kernel(const uint32_t *__restrict__ column_offset, const uint32_t *__restrict__ row_indices,
                                  uint32_t v, uint32_t e, const uint32_t *__restrict__ row_offset, uint32_t *cursor,
                                  uint32_t *__restrict__ column_indices, uint32_t s, float *__restrict__ src_norm,
                                  float *__restrict__ dst_norm) {
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, t0 = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (uint64_t i = t0; i < s; i += stride) src_norm[i] = (float)sqrt((double)(row_offset[i + 1] - row_offset[i]));
  for (uint64_t i = t0; i < v; i += stride) dst_norm[i] = (float)sqrt((double)(column_offset[i + 1] - column_offset[i]));
  for (uint64_t j = t0; j < e; j += stride) {
    const uint32_t d = find_segment(column_offset, v, (uint32_t)j);
    const uint32_t ls = row_indices[j];
    column_indices[row_offset[ls] + atomicAdd(&cursor[ls], 1u)] = d;
  }
}

// ------------------------------------------------------------------------------------ per-row sort
// Rows of length <= 32: one warp, rank by counting (stable for equal keys, which are identical anyway).
// Longer rows go to a worklist handled by whole CTAs.
__global__ void sort_short_rows_kernel(const uint32_t *__restrict__ row_offset, uint32_t s, uint32_t *column_indices,
                                       uint32_t *long_rows, uint32_t *long_count) {
  const unsigned lane = threadIdx.x & 31;
  const uint64_t warps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
  for (uint64_t r = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < s; r += warps) {
    const uint32_t start = row_offset[r], len = row_offset[r + 1] - start;
    if (len <= 1) continue;
    if (len > 32) {
      if (lane == 0) long_rows[atomicAdd(long_count, 1u)] = (uint32_t)r;
      continue;
    }
    const uint32_t mine = lane < len ? column_indices[start + lane] : 0xFFFFFFFFu;
    uint32_t rank = 0;
    for (uint32_t k = 0; k < len; k++) {
      const uint32_t other = __shfl_sync(0xffffffffu, mine, k);
      rank += (other < mine) || (other == mine && k < lane);
    }
    __syncwarp();
    if (lane < len) column_indices[start + rank] = mine;
  }
}

constexpr int kSortSmem = 4096;   // keys sorted in shared memory by one CTA
constexpr int kWindow = 8192;     // counters per pass of the windowed counting sort

__device__ __forceinline__ uint32_t block_scan_excl(uint32_t val, uint32_t *total, uint32_t *smem33) {
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t incl = val;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= (unsigned)o) incl += n;
  }
  if (lane == 31) smem33[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const uint32_t w = (lane < (blockDim.x >> 5)) ? smem33[lane] : 0u;
    uint32_t wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t n = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= (unsigned)o) wi += n;
    }
    smem33[lane] = wi - w;
    if (lane == 31) smem33[32] = wi;
  }
  __syncthreads();
  const uint32_t res = smem33[warp] + incl - val;
  *total = smem33[32];
  __syncthreads();
  return res;
}

// One CTA per long row.  len <= kSortSmem: bitonic sort in shared memory.  Longer: counting sort over
// the destination range in windows of kWindow values, reading the row from a scratch copy.
__global__ void __launch_bounds__(kThreads) sort_long_rows_kernel(const uint32_t *__restrict__ row_offset,
                                                                  uint32_t *column_indices, uint32_t v,
                                                                  const uint32_t *__restrict__ long_rows,
                                                                  const uint32_t *__restrict__ long_count,
                                                                  uint32_t *scratch) {
  __shared__ uint32_t keys[kWindow];  // 32 KB: sort buffer (first kSortSmem) or counters
  __shared__ uint32_t scan_smem[33];
  const uint32_t n_long = *long_count;
  for (uint32_t item = blockIdx.x; item < n_long; item += gridDim.x) {
    const uint32_t r = long_rows[item];
    const uint32_t start = row_offset[r], len = row_offset[r + 1] - start;
    uint32_t *row = column_indices + start;
    if (len <= kSortSmem) {
      uint32_t p2 = 64;
      while (p2 < len) p2 <<= 1;
      for (uint32_t i = threadIdx.x; i < p2; i += blockDim.x) keys[i] = i < len ? row[i] : 0xFFFFFFFFu;
      __syncthreads();
      for (uint32_t k = 2; k <= p2; k <<= 1) {
        for (uint32_t j = k >> 1; j > 0; j >>= 1) {
          for (uint32_t i = threadIdx.x; i < p2; i += blockDim.x) {
            const uint32_t partner = i ^ j;
            if (partner > i) {
              const uint32_t a = keys[i], b = keys[partner];
              const bool up = (i & k) == 0;
              if ((a > b) == up) { keys[i] = b; keys[partner] = a; }
            }
          }
          __syncthreads();
        }
      }
      for (uint32_t i = threadIdx.x; i < len; i += blockDim.x) row[i] = keys[i];
      __syncthreads();
    } else {
      uint32_t *copy = scratch + start;
      for (uint32_t i = threadIdx.x; i < len; i += blockDim.x) copy[i] = row[i];
      __syncthreads();
      uint32_t out_base = 0;
      for (uint32_t lo = 0; lo < v; lo += kWindow) {
        for (uint32_t i = threadIdx.x; i < kWindow; i += blockDim.x) keys[i] = 0;
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < len; i += blockDim.x) {
          const uint32_t x = copy[i] - lo;  // wraps to a huge value when copy[i] < lo
          if (x < (uint32_t)kWindow) atomicAdd(&keys[x], 1u);
        }
        __syncthreads();
        // each thread owns kWindow/kThreads consecutive counters
        constexpr int kPer = kWindow / kThreads;
        uint32_t local = 0;
#pragma unroll 4
        for (int k = 0; k < kPer; k++) local += keys[threadIdx.x * kPer + k];
        uint32_t total;
        uint32_t pos = out_base + block_scan_excl(local, &total, scan_smem);
        for (int k = 0; k < kPer; k++) {
          const uint32_t c = keys[threadIdx.x * kPer + k];
          const uint32_t val = lo + threadIdx.x * kPer + k;
          for (uint32_t q = 0; q < c; q++) row[pos++] = val;
        }
        out_base += total;
        __syncthreads();
        if (out_base >= len) break;
      }
    }
  }
}

}  // namespace nb

using namespace nb;

namespace nb {
// nb_block_build; `marked` (nullable) is a bitmap of |V| bits plus 4 flag words that the sampler has already
// cleared and marked (the native step fuses the marking into its sampling kernel), and zero_cap, when not 0,
// tells how many row counters of d_row_offset this call may clear inside its first launch.
int block_build_impl(nb_ws *ws, uint32_t num_vertices, uint32_t *d_row_indices, const uint32_t *d_column_offset,
                     uint32_t v, uint32_t e, uint32_t *d_source, uint32_t *src_size, uint32_t *d_row_offset,
                     uint32_t *d_column_indices, float *d_src_norm, float *d_dst_norm, float *d_w_fwd, float *d_w_bwd,
                     uint32_t *marked, void *stream_) {
  NB_REQUIRE(ws && src_size, "nb_block_build: null workspace or src_size");
  NB_REQUIRE(d_column_offset && d_source && d_row_offset && d_src_norm && d_dst_norm,
             "nb_block_build: null output pointer");
  NB_REQUIRE(e == 0 || (d_row_indices && d_column_indices), "nb_block_build: null edge arrays");
  NB_REQUIRE(num_vertices > 0, "nb_block_build: empty graph");
  cudaStream_t stream = as_stream(stream_);
  WsScope scope(ws);

  const uint64_t words = ((uint64_t)num_vertices + 31) / 32;
  uint32_t *bitmap = marked ? marked : ws->alloc_n<uint32_t>(words + 4);   // + flags, cleared by the same memset
  uint32_t *prefix = ws->alloc_n<uint32_t>(words + 1);
  if (!bitmap || !prefix) return fail(NB_ERR_NOMEM, "nb_block_build: workspace arena exhausted");
  uint32_t *flags = bitmap + words;  // [0] error, [1] long-row count
  if (!marked) {
    NB_CUDA(cudaMemsetAsync(bitmap, 0, (words + 4) * sizeof(uint32_t), stream));
    if (e > 0) {
      mark_bitmap_kernel<<<grid_for(e, kThreads), kThreads, 0, stream>>>(d_row_indices, e, num_vertices, bitmap, flags);
      NB_LAUNCH_CHECK();
    }
  }
  // Without explicit weight arrays the rest runs in fewer, merged launches; their first one needs the row
  // counters cleared.
  const bool lean = d_w_fwd == nullptr && d_w_bwd == nullptr && e > 0;
  if (lean) {   // at most min(|V|, e) + 1 row counters exist; cleared before the size is known, off the critical path
    const uint64_t zero_cap = (uint64_t)(e < num_vertices ? e : num_vertices) + 1;
    NB_CUDA(cudaMemsetAsync(d_row_offset, 0, zero_cap * sizeof(uint32_t), stream));
  }
  if (words <= kSingleBlockScanMax) {   // popcount and scan in one launch
    scan_single_block<uint32_t, ScanLoadPopc><<<1, 1024, 0, stream>>>(ScanLoadPopc{bitmap}, prefix, words, true);
    NB_LAUNCH_CHECK();
  } else {
    popc_words_kernel<<<grid_for(words, kThreads), kThreads, 0, stream>>>(bitmap, prefix, words);
    NB_LAUNCH_CHECK();
    NB_TRY(exclusive_scan_u32(ws, prefix, prefix, words, true, stream));
  }
  NB_CUDA(cudaMemcpyAsync(ws->mailbox, prefix + words, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream));
  NB_CUDA(cudaMemcpyAsync(ws->mailbox + 1, flags, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream));
  NB_CUDA(wait_stream_host(stream));
  const uint32_t s = ws->mailbox[0];
  if (ws->mailbox[1] != 0) return fail(NB_ERR_INVALID, "nb_block_build: a source id is >= num_vertices");
  *src_size = s;

  if (lean) {
    uint32_t *cursor = ws->alloc_n<uint32_t>((size_t)s + 1);
    uint32_t *long_rows = ws->alloc_n<uint32_t>((size_t)e / 32 + 1);
    uint32_t *scratch = ws->alloc_n<uint32_t>(e);
    if (!cursor || !long_rows || !scratch) return fail(NB_ERR_NOMEM, "nb_block_build: workspace arena exhausted");
    emit_remap_kernel<<<grid_for(words > e ? words : e, kThreads), kThreads, 0, stream>>>(
        bitmap, prefix, words, d_source, d_row_indices, e, num_vertices, d_row_offset, cursor, s);
    NB_LAUNCH_CHECK();
    NB_TRY(exclusive_scan_u32(ws, d_row_offset, d_row_offset, s, true, stream));
    fill_norms_kernel<<<grid_for(e, kThreads), kThreads, 0, stream>>>(d_column_offset, d_row_indices, v, e, d_row_offset,
                                                                      cursor, d_column_indices, s, d_src_norm, d_dst_norm);
    NB_LAUNCH_CHECK();
    sort_short_rows_kernel<<<grid_for((uint64_t)s * 32, kThreads), kThreads, 0, stream>>>(
        d_row_offset, s, d_column_indices, long_rows, flags + 1);
    NB_LAUNCH_CHECK();
    sort_long_rows_kernel<<<num_sms() * 4, kThreads, 0, stream>>>(d_row_offset, d_column_indices, v, long_rows,
                                                                flags + 1, scratch);
    NB_LAUNCH_CHECK();
    return 0;
  }

  // CSR: count -> scan -> fill -> sort rows
  emit_source_kernel<<<grid_for(words > s ? words : s + 1, kThreads), kThreads, 0, stream>>>(
      bitmap, prefix, words, d_source, d_row_offset, (uint64_t)s + 1);
  NB_LAUNCH_CHECK();
  if (e > 0) {
    remap_count_kernel<<<grid_for(e, kThreads), kThreads, 0, stream>>>(d_row_indices, e, bitmap, prefix,
                                                                       num_vertices, d_row_offset);
    NB_LAUNCH_CHECK();
  }
  NB_TRY(exclusive_scan_u32(ws, d_row_offset, d_row_offset, s, true, stream));
  uint32_t *cursor = nullptr;
  if (e > 0) {
    cursor = ws->alloc_n<uint32_t>((size_t)s + 1);
    if (!cursor) return fail(NB_ERR_NOMEM, "nb_block_build: workspace arena exhausted");
  }
  if (s > 0 || v > 0) {
    degree_norms_kernel<<<grid_for(s > v ? s : v, kThreads), kThreads, 0, stream>>>(d_row_offset, s, d_src_norm, cursor,
                                                                                d_column_offset, v, d_dst_norm);
    NB_LAUNCH_CHECK();
  }
  if (e > 0) {
    uint32_t *long_rows = ws->alloc_n<uint32_t>((size_t)e / 32 + 1);
    uint32_t *scratch = ws->alloc_n<uint32_t>(e);
    if (!long_rows || !scratch) return fail(NB_ERR_NOMEM, "nb_block_build: workspace arena exhausted");
    csr_fill_kernel<<<grid_for(e, kThreads), kThreads, 0, stream>>>(d_column_offset, d_row_indices, v, e, cursor,
                                                                    d_column_indices, d_src_norm, d_dst_norm, d_w_fwd);
    NB_LAUNCH_CHECK();
    sort_short_rows_kernel<<<grid_for((uint64_t)s * 32, kThreads), kThreads, 0, stream>>>(
        d_row_offset, s, d_column_indices, long_rows, flags + 1);
    NB_LAUNCH_CHECK();
    sort_long_rows_kernel<<<num_sms() * 4, kThreads, 0, stream>>>(d_row_offset, d_column_indices, v, long_rows,
                                                                flags + 1, scratch);
    NB_LAUNCH_CHECK();
    if (d_w_bwd) {
      csr_weight_kernel<<<grid_for(e, kThreads), kThreads, 0, stream>>>(d_row_offset, d_column_indices, s, e,
                                                                        d_src_norm, d_dst_norm, d_w_bwd);
      NB_LAUNCH_CHECK();
    }
  }
  return 0;
}
}  // namespace nb

NB_API int nb_block_build(nb_ws *ws, uint32_t num_vertices, uint32_t *d_row_indices,
                          const uint32_t *d_column_offset, uint32_t v, uint32_t e, uint32_t *d_source,
                          uint32_t *src_size, uint32_t *d_row_offset, uint32_t *d_column_indices,
                          float *d_src_norm, float *d_dst_norm, float *d_w_fwd, float *d_w_bwd, void *stream) {
  return nb::block_build_impl(ws, num_vertices, d_row_indices, d_column_offset, v, e, d_source, src_size, d_row_offset,
                              d_column_indices, d_src_norm, d_dst_norm, d_w_fwd, d_w_bwd, nullptr, stream);
}
