// Fan-out neighbour sampling of one hop and the whole-graph CSC build.
#include "common.cuh"
#include "scan.cuh"
#include "philox.cuh"

namespace nb {

constexpr int kThreads = 256;

// count[i] = min(deg(dst[i]), fanout)  (deg when fanout < 0) — core/ntsSampler.hpp:914-923
__global__ void hop_counts_kernel(const uint64_t *__restrict__ g_co, const uint32_t *__restrict__ dst, uint32_t v,
                                  int fanout, uint32_t *__restrict__ counts) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < v; i += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t d = dst[i];
    const uint64_t deg = g_co[d + 1] - g_co[d];
    counts[i] = (uint32_t)((fanout < 0 || deg < (uint64_t)fanout) ? deg : (uint64_t)fanout);
  }
}

// The same count as a scan input, so that small hops need one launch for counts and offsets.
struct ScanLoadHopCount {
  const uint64_t *g_co;
  const uint32_t *dst;
  int fanout;
  __device__ __forceinline__ uint32_t operator()(uint64_t i) const {
    const uint32_t d = dst[i];
    const uint64_t deg = g_co[d + 1] - g_co[d];
    return (uint32_t)((fanout < 0 || deg < (uint64_t)fanout) ? deg : (uint64_t)fanout);
  }
};

// Marks a sampled source in the dedup bitmap of the hop (the block builder's first step, done here while the id is
// in a register).
__device__ __forceinline__ void mark_source(uint32_t *bitmap, uint32_t g) {
  if (bitmap == nullptr) return;
  const uint32_t bit = 1u << (g & 31);
  if ((bitmap[g >> 5] & bit) == 0) atomicOr(&bitmap[g >> 5], bit);
}

constexpr uint32_t kFloydMax = 128;   // Floyd's duplicate test is quadratic in the subset size

// count[i] = max(int(deg * rate), min(lower, deg))  — SAMPLE_RATE mode, core/ntsSampler.hpp:901-912
__device__ __forceinline__ uint32_t rate_count(uint64_t deg64, float rate, int lower) {
  const int deg = (int)deg64;
  const int lo = lower < deg ? lower : deg;
  const int by_rate = (int)__fmul_rn((float)deg, rate);
  int k = by_rate > lo ? by_rate : lo;
  k = k > deg ? deg : k;
  return (uint32_t)(k < 0 ? 0 : k);
}
__global__ void hop_counts_rate_kernel(const uint64_t *__restrict__ g_co, const uint32_t *__restrict__ dst, uint32_t v,
                                       float rate, int lower, uint32_t *__restrict__ counts) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < v; i += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t d = dst[i];
    counts[i] = rate_count(g_co[d + 1] - g_co[d], rate, lower);
  }
}

// One thread per destination.  deg <= fanout: copy the column.  Otherwise Floyd's algorithm picks
// `fanout` distinct positions; the chosen positions are parked in the output slots (read back by the
// same thread for the membership test) and then replaced by the neighbour ids.
__global__ void sample_hop_kernel(const uint64_t *__restrict__ g_co, const uint32_t *__restrict__ g_ri,
                                  const uint32_t *__restrict__ dst, uint32_t v, int fanout,
                                  const uint32_t *__restrict__ column_offset, uint32_t seed_lo, uint32_t seed_hi,
                                  uint32_t hop, uint32_t *row_indices, uint32_t *bitmap) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < v; i += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t d = dst[i];
    const uint64_t base = g_co[d];
    const uint32_t deg = (uint32_t)(g_co[d + 1] - base);
    const uint32_t pos = column_offset[i];
    const uint32_t k = column_offset[i + 1] - pos;
    if (k >= deg) {   // the counts already carry the fan-out rule: nothing to choose
      for (uint32_t j = 0; j < deg; j++) {
        const uint32_t g = g_ri[base + j];
        row_indices[pos + j] = g;
        mark_source(bitmap, g);
      }
      continue;
    }
    uint32_t r[4];
    if (k > kFloydMax) {
      // Large subsets (SAMPLE_RATE on hub vertices): selection sampling, one draw per neighbour in column
      // order (stream tag 2 in the fourth counter word); picks exactly k, in ascending position.
      uint32_t m = 0;
      for (uint32_t j = 0; j < deg && m < k; j++) {
        if ((j & 3) == 0) philox4x32_10(j >> 2, (uint32_t)i, hop, 2u, seed_lo, seed_hi, r);
        if (__umulhi(r[j & 3], deg - j) < k - m) {
          const uint32_t g = g_ri[base + j];
          row_indices[pos + m++] = g;
          mark_source(bitmap, g);
        }
      }
      continue;
    }
    for (uint32_t t = 0; t < k; t++) {
      if ((t & 3) == 0) philox4x32_10(t >> 2, (uint32_t)i, hop, 0u, seed_lo, seed_hi, r);
      const uint32_t j = deg - k + t;
      uint32_t c = __umulhi(r[t & 3], j + 1);  // uniform in [0, j]
      for (uint32_t q = 0; q < t; q++)
        if (row_indices[pos + q] == c) { c = j; break; }
      row_indices[pos + t] = c;
    }
    for (uint32_t t = 0; t < k; t++) {
      const uint32_t g = g_ri[base + row_indices[pos + t]];
      row_indices[pos + t] = g;
      mark_source(bitmap, g);
    }
  }
}

// Warp per destination for fanouts up to 32: lane t makes draw t of the destination's Philox stream,
// the Floyd duplicate rule is resolved in draw order with ballots, and the lanes fetch the chosen
// neighbours together.  Produces exactly what sample_hop_kernel produces.
__global__ void sample_hop_warp_kernel(const uint64_t *__restrict__ g_co, const uint32_t *__restrict__ g_ri,
                                       const uint32_t *__restrict__ dst, uint32_t v, int fanout,
                                       const uint32_t *__restrict__ column_offset, uint32_t seed_lo,
                                       uint32_t seed_hi, uint32_t hop, uint32_t *__restrict__ row_indices,
                                       uint32_t *bitmap) {
  const unsigned lane = threadIdx.x & 31;
  const uint64_t warps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
  for (uint64_t i = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < v; i += warps) {
    const uint32_t d = dst[i];
    const uint64_t base = g_co[d];
    const uint32_t deg = (uint32_t)(g_co[d + 1] - base);
    const uint32_t pos = column_offset[i];
    if (deg <= (uint32_t)fanout) {
      for (uint32_t j = lane; j < deg; j += 32) {
        const uint32_t g = g_ri[base + j];
        row_indices[pos + j] = g;
        mark_source(bitmap, g);
      }
      continue;
    }
    const uint32_t k = (uint32_t)fanout;      // <= 32
    uint32_t chosen = 0xFFFFFFFFu;
    if (lane < k) {
      uint32_t r[4];
      philox4x32_10(lane >> 2, (uint32_t)i, hop, 0u, seed_lo, seed_hi, r);
      chosen = __umulhi(r[lane & 3], deg - k + lane + 1);   // candidate of draw `lane`: uniform in [0, j]
    }
    for (uint32_t t = 1; t < k; t++) {
      const uint32_t c = __shfl_sync(0xffffffffu, chosen, t);
      const unsigned dup = __ballot_sync(0xffffffffu, lane < t && chosen == c);
      if (dup && lane == t) chosen = deg - k + t;           // Floyd: a repeated candidate yields j itself
    }
    if (lane < k) {
      const uint32_t g = g_ri[base + chosen];
      row_indices[pos + lane] = g;
      mark_source(bitmap, g);
    }
  }
}

// ------------------------------------------------------------------------------------ graph CSC
__global__ void edge_degree_kernel(const uint32_t *__restrict__ edges, uint64_t E, uint32_t V, uint32_t *in_deg,
                                   uint32_t *out_deg, uint32_t *err) {
  for (uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; e < E; e += (uint64_t)gridDim.x * blockDim.x) {
    const uint2 sd = reinterpret_cast<const uint2 *>(edges)[e];
    if (sd.x >= V || sd.y >= V) { atomicExch(err, 1u); continue; }
    atomicAdd(&in_deg[sd.y], 1u);
    if (out_deg) atomicAdd(&out_deg[sd.x], 1u);
  }
}

// Each edge is tagged with its position in the file so that a column can be put back in file order.
__global__ void csc_scatter_kernel(const uint32_t *__restrict__ edges, uint64_t E, uint32_t V,
                                   const uint64_t *__restrict__ column_offset, uint32_t *cursor,
                                   uint32_t *__restrict__ row_indices, uint64_t *__restrict__ tags) {
  for (uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; e < E; e += (uint64_t)gridDim.x * blockDim.x) {
    const uint2 sd = reinterpret_cast<const uint2 *>(edges)[e];
    if (sd.x >= V || sd.y >= V) continue;
    const uint64_t p = column_offset[sd.y] + atomicAdd(&cursor[sd.y], 1u);
    tags[p] = e;
    row_indices[p] = sd.x;
  }
}

// Restore file order inside every column.  Columns of up to 32 entries: one warp ranks the file tags
// by counting.  Longer columns go to a worklist sorted by whole CTAs (below).
__global__ void csc_order_short_columns_kernel(const uint64_t *__restrict__ column_offset, uint32_t V,
                                               const uint64_t *__restrict__ tags, uint32_t *row_indices,
                                               uint32_t *long_cols, uint32_t *long_count) {
  const unsigned lane = threadIdx.x & 31;
  const uint64_t warps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
  for (uint64_t c = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; c < V; c += warps) {
    const uint64_t start = column_offset[c];
    const uint64_t len = column_offset[c + 1] - start;
    if (len <= 1) continue;
    if (len > 32) {
      if (lane == 0) long_cols[atomicAdd(long_count, 1u)] = (uint32_t)c;
      continue;
    }
    const uint64_t tag = lane < len ? tags[start + lane] : ~0ull;
    const uint32_t val = lane < len ? row_indices[start + lane] : 0u;
    uint32_t rank = 0;
    for (uint32_t k = 0; k < (uint32_t)len; k++) {
      const uint64_t other = __shfl_sync(0xffffffffu, tag, k);
      rank += other < tag;
    }
    __syncwarp();
    if (lane < len) row_indices[start + rank] = val;
  }
}

// One CTA per long column: bitonic network in its normalised form (every comparator moves the smaller
// tag to the lower index), run in place in global memory.  Positions >= len act as +infinity, so
// comparators that reach past the end are skipped.  Tags are distinct, hence the order is unique.
__global__ void __launch_bounds__(kThreads) csc_order_long_columns_kernel(const uint64_t *__restrict__ column_offset,
                                                                          uint64_t *tags, uint32_t *row_indices,
                                                                          const uint32_t *__restrict__ long_cols,
                                                                          const uint32_t *__restrict__ long_count) {
  const uint32_t n_long = *long_count;
  for (uint32_t item = blockIdx.x; item < n_long; item += gridDim.x) {
    const uint32_t c = long_cols[item];
    const uint64_t start = column_offset[c];
    const uint64_t len = column_offset[c + 1] - start;
    uint64_t *t = tags + start;
    uint32_t *r = row_indices + start;
    uint64_t p2 = 64;
    while (p2 < len) p2 <<= 1;
    for (uint64_t k = 2; k <= p2; k <<= 1) {
      for (uint64_t j = k >> 1; j > 0; j >>= 1) {
        const uint64_t mask = (j == (k >> 1)) ? (k - 1) : j;
        for (uint64_t i = threadIdx.x; i < len; i += blockDim.x) {
          const uint64_t partner = i ^ mask;
          if (partner > i && partner < len) {
            const uint64_t a = t[i], b = t[partner];
            if (a > b) {
              t[i] = b; t[partner] = a;
              const uint32_t x = r[i]; r[i] = r[partner]; r[partner] = x;
            }
          }
        }
        __syncthreads();
      }
    }
  }
}

}  // namespace nb

using namespace nb;

NB_API int nb_sample_hop_offsets(nb_ws *ws, const uint64_t *d_graph_column_offset, const uint32_t *d_dst,
                                 uint32_t v, int fanout, uint32_t *d_column_offset, uint32_t *e_size,
                                 void *stream_) {
  NB_REQUIRE(ws && d_graph_column_offset && d_column_offset && e_size, "nb_sample_hop_offsets: null pointer");
  NB_REQUIRE(v == 0 || d_dst, "nb_sample_hop_offsets: null destination list");
  NB_REQUIRE(fanout != 0, "nb_sample_hop_offsets: fanout must be positive, or negative for all neighbours");
  cudaStream_t stream = as_stream(stream_);
  if (v > 0 && v <= kSingleBlockGatherScanMax) {
    scan_single_block<uint32_t, ScanLoadHopCount><<<1, 1024, 0, stream>>>(
        ScanLoadHopCount{d_graph_column_offset, d_dst, fanout}, d_column_offset, v, true);
    NB_LAUNCH_CHECK();
  } else {
    if (v > 0) {
      hop_counts_kernel<<<grid_for(v, kThreads), kThreads, 0, stream>>>(d_graph_column_offset, d_dst, v, fanout,
                                                                       d_column_offset);
      NB_LAUNCH_CHECK();
    }
    NB_TRY(exclusive_scan_u32(ws, d_column_offset, d_column_offset, v, true, stream));
  }
  NB_CUDA(cudaMemcpyAsync(ws->mailbox + 2, d_column_offset + v, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream));
  NB_CUDA(wait_stream_host(stream));
  *e_size = ws->mailbox[2];
  return 0;
}

NB_API int nb_sample_hop_offsets_rate(nb_ws *ws, const uint64_t *d_graph_column_offset, const uint32_t *d_dst, uint32_t v,
                                      float sample_rate, int lower_fanout, uint32_t *d_column_offset, uint32_t *e_size,
                                      void *stream_) {
  NB_REQUIRE(ws && d_graph_column_offset && d_column_offset && e_size, "nb_sample_hop_offsets_rate: null pointer");
  NB_REQUIRE(v == 0 || d_dst, "nb_sample_hop_offsets_rate: null destination list");
  NB_REQUIRE(sample_rate > 0.0f && sample_rate <= 1.0f, "nb_sample_hop_offsets_rate: sample rate must be in (0, 1]");
  NB_REQUIRE(lower_fanout >= 0, "nb_sample_hop_offsets_rate: negative lower fan-out");
  cudaStream_t stream = as_stream(stream_);
  if (v > 0) {
    hop_counts_rate_kernel<<<grid_for(v, kThreads), kThreads, 0, stream>>>(d_graph_column_offset, d_dst, v, sample_rate,
                                                                          lower_fanout, d_column_offset);
    NB_LAUNCH_CHECK();
  }
  NB_TRY(exclusive_scan_u32(ws, d_column_offset, d_column_offset, v, true, stream));
  NB_CUDA(cudaMemcpyAsync(ws->mailbox + 2, d_column_offset + v, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream));
  NB_CUDA(wait_stream_host(stream));
  *e_size = ws->mailbox[2];
  return 0;
}

namespace nb {
// nb_sample_hop that also marks every sampled source in `bitmap` (nullable; |V| bits, cleared by the caller).
int sample_hop_impl(const uint64_t *d_graph_column_offset, const uint32_t *d_graph_row_indices, const uint32_t *d_dst,
                    uint32_t v, int fanout, const uint32_t *d_column_offset, uint64_t seed, uint32_t hop,
                    uint32_t *d_row_indices, uint32_t *bitmap, void *stream_) {
  if (v == 0) return 0;
  NB_REQUIRE(d_graph_column_offset && d_graph_row_indices && d_dst && d_column_offset && d_row_indices,
             "nb_sample_hop: null pointer");
  NB_REQUIRE(fanout != 0, "nb_sample_hop: fanout must be positive, or negative for all neighbours");
  if (fanout > 0 && fanout <= 32) {
    sample_hop_warp_kernel<<<grid_for((uint64_t)v * 32, 256), 256, 0, as_stream(stream_)>>>(
        d_graph_column_offset, d_graph_row_indices, d_dst, v, fanout, d_column_offset, (uint32_t)seed,
        (uint32_t)(seed >> 32), hop, d_row_indices, bitmap);
  } else {
    sample_hop_kernel<<<grid_for(v, 128), 128, 0, as_stream(stream_)>>>(
        d_graph_column_offset, d_graph_row_indices, d_dst, v, fanout, d_column_offset, (uint32_t)seed,
        (uint32_t)(seed >> 32), hop, d_row_indices, bitmap);
  }
  NB_LAUNCH_CHECK();
  return 0;
}
}  // namespace nb

NB_API int nb_sample_hop(const uint64_t *d_graph_column_offset, const uint32_t *d_graph_row_indices,
                         const uint32_t *d_dst, uint32_t v, int fanout, const uint32_t *d_column_offset,
                         uint64_t seed, uint32_t hop, uint32_t *d_row_indices, void *stream) {
  return nb::sample_hop_impl(d_graph_column_offset, d_graph_row_indices, d_dst, v, fanout, d_column_offset, seed, hop,
                             d_row_indices, nullptr, stream);
}

NB_API int nb_graph_build_csc(nb_ws *ws, const uint32_t *d_edges, uint64_t num_edges, uint32_t num_vertices,
                              uint64_t *d_column_offset, uint32_t *d_row_indices, uint32_t *d_out_degree,
                              uint32_t *d_in_degree, void *stream_) {
  NB_REQUIRE(ws && d_column_offset, "nb_graph_build_csc: null pointer");
  NB_REQUIRE(num_edges == 0 || (d_edges && d_row_indices), "nb_graph_build_csc: null edge arrays");
  NB_REQUIRE(num_vertices > 0, "nb_graph_build_csc: empty graph");
  NB_REQUIRE((reinterpret_cast<uintptr_t>(d_edges) & 7) == 0, "nb_graph_build_csc: edge list must be 8-byte aligned");
  cudaStream_t stream = as_stream(stream_);
  WsScope scope(ws);
  uint32_t *in_deg = d_in_degree ? d_in_degree : ws->alloc_n<uint32_t>(num_vertices);
  uint32_t *cursor = ws->alloc_n<uint32_t>(num_vertices);
  uint64_t *tags = ws->alloc_n<uint64_t>(num_edges ? num_edges : 1);
  uint32_t *err = ws->alloc_n<uint32_t>(1);
  if (!in_deg || !cursor || !tags || !err) return fail(NB_ERR_NOMEM, "nb_graph_build_csc: workspace arena exhausted");
  NB_CUDA(cudaMemsetAsync(in_deg, 0, (size_t)num_vertices * sizeof(uint32_t), stream));
  NB_CUDA(cudaMemsetAsync(cursor, 0, (size_t)num_vertices * sizeof(uint32_t), stream));
  NB_CUDA(cudaMemsetAsync(err, 0, sizeof(uint32_t), stream));
  if (d_out_degree) NB_CUDA(cudaMemsetAsync(d_out_degree, 0, (size_t)num_vertices * sizeof(uint32_t), stream));
  if (num_edges > 0) {
    edge_degree_kernel<<<grid_for(num_edges, kThreads), kThreads, 0, stream>>>(d_edges, num_edges, num_vertices,
                                                                                in_deg, d_out_degree, err);
    NB_LAUNCH_CHECK();
  }
  NB_TRY(exclusive_scan_u32_to_u64(ws, in_deg, d_column_offset, num_vertices, true, stream));
  if (num_edges > 0) {
    csc_scatter_kernel<<<grid_for(num_edges, kThreads), kThreads, 0, stream>>>(d_edges, num_edges, num_vertices,
                                                                                d_column_offset, cursor,
                                                                                d_row_indices, tags);
    NB_LAUNCH_CHECK();
    uint32_t *long_cols = ws->alloc_n<uint32_t>(num_edges / 32 + 1);
    uint32_t *long_count = ws->alloc_n<uint32_t>(1);
    if (!long_cols || !long_count) return fail(NB_ERR_NOMEM, "nb_graph_build_csc: workspace arena exhausted");
    NB_CUDA(cudaMemsetAsync(long_count, 0, sizeof(uint32_t), stream));
    csc_order_short_columns_kernel<<<grid_for((uint64_t)num_vertices * 32, kThreads), kThreads, 0, stream>>>(
        d_column_offset, num_vertices, tags, d_row_indices, long_cols, long_count);
    NB_LAUNCH_CHECK();
    csc_order_long_columns_kernel<<<num_sms() * 4, kThreads, 0, stream>>>(d_column_offset, tags, d_row_indices,
                                                                       long_cols, long_count);
    NB_LAUNCH_CHECK();
  }
  NB_CUDA(cudaMemcpyAsync(ws->mailbox + 3, err, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream));
  NB_CUDA(wait_stream_host(stream));
  if (ws->mailbox[3] != 0) return fail(NB_ERR_INVALID, "nb_graph_build_csc: an edge endpoint is >= num_vertices");
  return 0;
}
