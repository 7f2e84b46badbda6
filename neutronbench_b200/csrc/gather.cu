// Feature and label movement: one fused gather that resolves cache hits (HBM-resident cache),
// misses (device table, mapped pinned host memory, or a node-id-sharded table on peer GPUs) on the
// device, plus the cache fill.
#include <initializer_list>

#include "common.cuh"

namespace nb {

constexpr int kWarps = 8;

// Set (never cleared by the kernels) when an id named a row outside every table it could come from: beyond the last
// shard of a sharded table, or not cached while there is no table to read it from.  The row is skipped, not read.
__device__ unsigned int g_gather_error = 0;

struct GatherArgs {
  float *x0;
  size_t x0_ld;            // pitch of x0 in floats
  int misses_only;         // 1: rows with a cache slot are left untouched (the caller reads them from the cache)
  const float *feat;
  size_t feat_ld;
  const float *const *shards;
  uint32_t num_shards;
  uint32_t shard_rows;
  const float *cache;
  size_t cache_ld;
  const uint32_t *hashmap;
  const uint32_t *source;
  uint32_t n;
  uint32_t F;
  uint32_t tiles;
};

template <int VEC>
__device__ __forceinline__ void copy_vec(float *dst, const float *src) {
  if constexpr (VEC == 4) {
    *reinterpret_cast<float4 *>(dst) = __ldg(reinterpret_cast<const float4 *>(src));
  } else if constexpr (VEC == 2) {
    *reinterpret_cast<float2 *>(dst) = __ldg(reinterpret_cast<const float2 *>(src));
  } else {
    *dst = __ldg(src);
  }
}

// A warp copies kRows rows per pass so that several independent row reads are in flight per lane.
template <int VEC>
__global__ void __launch_bounds__(kWarps * 32) feature_gather_kernel(const GatherArgs a) {
  constexpr int kRows = 4;
  const unsigned lane = threadIdx.x & 31;
  const uint64_t groups = ((uint64_t)a.n + kRows - 1) / kRows;
  const uint64_t total_warps = (uint64_t)gridDim.x * kWarps;
  // grid-stride over (group of kRows rows, column tile) items: the launch may be much smaller than the work, which
  // is how a copy that is bound by a slow link (host memory) leaves the SMs to the kernels that run beside it
  for (uint64_t item = (uint64_t)blockIdx.x * kWarps + (threadIdx.x >> 5); item < groups * a.tiles; item += total_warps) {
  const uint64_t grp = item / a.tiles;
  const uint32_t tile = (uint32_t)(item - grp * a.tiles);
  const uint32_t col = tile * (32 * VEC) + lane * VEC;
  const float *src[kRows];
#pragma unroll
  for (int k = 0; k < kRows; k++) {
    const uint64_t i = grp * kRows + k;
    src[k] = nullptr;
    if (i < a.n) {
      const uint32_t g = a.source[i];
      const uint32_t slot = a.hashmap ? a.hashmap[g] : 0xFFFFFFFFu;
      if (slot != 0xFFFFFFFFu) {
        if (!a.misses_only) src[k] = a.cache + (size_t)slot * a.cache_ld;
      } else if (a.shards) {
        const uint32_t owner = g / a.shard_rows;
        if (owner < a.num_shards) src[k] = a.shards[owner] + (size_t)(g - owner * a.shard_rows) * a.feat_ld;
        else if (lane == 0) atomicOr(&g_gather_error, 1u);
      } else if (a.feat) {
        src[k] = a.feat + (size_t)g * a.feat_ld;
      } else if (lane == 0) {
        atomicOr(&g_gather_error, 1u);
      }
    }
  }
  if (col >= a.F) continue;
  // all kRows reads first, then the writes: over a link of a few microseconds (a peer GPU, host memory) a lane must
  // have its reads in flight together, and a store between two loads would keep the second one back
  float v[kRows][VEC];
#pragma unroll
  for (int k = 0; k < kRows; k++) {
    if (src[k]) {
      if constexpr (VEC == 4) {
        const float4 t = __ldg(reinterpret_cast<const float4 *>(src[k] + col));
        v[k][0] = t.x; v[k][1] = t.y; v[k][2] = t.z; v[k][3] = t.w;
      } else if constexpr (VEC == 2) {
        const float2 t = __ldg(reinterpret_cast<const float2 *>(src[k] + col));
        v[k][0] = t.x; v[k][1] = t.y;
      } else {
        v[k][0] = __ldg(src[k] + col);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < kRows; k++) {
    if (src[k]) {
      float *dst = a.x0 + (grp * kRows + k) * a.x0_ld + col;
      if constexpr (VEC == 4) *reinterpret_cast<float4 *>(dst) = make_float4(v[k][0], v[k][1], v[k][2], v[k][3]);
      else if constexpr (VEC == 2) *reinterpret_cast<float2 *>(dst) = make_float2(v[k][0], v[k][1]);
      else *dst = v[k][0];
    }
  }
  }
}

// x0[lid,:] = table[map(src[lid]),:] for lid = local_idx[i], i < n: the index-list form of the reference's two cache
// kernels (misses: map = identity over the host table; hits: map = the slot map over the cache).
template <int VEC>
__global__ void __launch_bounds__(kWarps * 32) gather_indexed_kernel(float *x0, size_t x0_ld, const float *table,
                                                                     size_t table_ld, const uint32_t *__restrict__ src,
                                                                     const uint32_t *__restrict__ local_idx,
                                                                     const uint32_t *__restrict__ slot_map, uint32_t n,
                                                                     uint32_t F, uint32_t tiles) {
  const unsigned lane = threadIdx.x & 31;
  const uint64_t warps = (uint64_t)gridDim.x * kWarps;
  for (uint64_t w = (uint64_t)blockIdx.x * kWarps + (threadIdx.x >> 5); w < (uint64_t)n * tiles; w += warps) {
    const uint32_t i = (uint32_t)(w / tiles);
    const uint32_t col = (uint32_t)(w - (uint64_t)i * tiles) * (32 * VEC) + lane * VEC;
    if (col >= F) continue;
    const uint32_t lid = local_idx[i];
    uint32_t row = src[lid];
    if (slot_map) {
      row = slot_map[row];
      if (row == 0xFFFFFFFFu) {   // listed as cached but has no slot: skipped, reported
        if (lane == 0) atomicOr(&g_gather_error, 1u);
        continue;
      }
    }
    copy_vec<VEC>(x0 + (size_t)lid * x0_ld + col, table + (size_t)row * table_ld + col);
  }
}

__global__ void label_gather_kernel(int64_t *__restrict__ lab, const int64_t *__restrict__ label,
                                    const uint32_t *__restrict__ dst, uint32_t n, uint32_t label_size) {
  const uint64_t total = (uint64_t)n * label_size;
  for (uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (uint64_t)gridDim.x * blockDim.x) {
    const uint64_t i = t / label_size, k = t - i * label_size;
    lab[t] = label[(uint64_t)dst[i] * label_size + k];
  }
}

template <int VEC>
__global__ void __launch_bounds__(kWarps * 32) cache_fill_kernel(float *cache, size_t cache_ld, const float *feat,
                                                                 size_t feat_ld, const uint32_t *__restrict__ hashmap,
                                                                 uint32_t V, uint32_t F, uint32_t tiles) {
  const unsigned lane = threadIdx.x & 31;
  const uint64_t warps = (uint64_t)gridDim.x * kWarps;
  for (uint64_t w = (uint64_t)blockIdx.x * kWarps + (threadIdx.x >> 5); w < (uint64_t)V * tiles; w += warps) {
    const uint32_t g = (uint32_t)(w / tiles);
    const uint32_t col = (uint32_t)(w - (uint64_t)g * tiles) * (32 * VEC) + lane * VEC;
    const uint32_t slot = hashmap[g];
    if (slot == 0xFFFFFFFFu || col >= F) continue;
    copy_vec<VEC>(cache + (size_t)slot * cache_ld + col, feat + (size_t)g * feat_ld + col);
  }
}

// counts[id] += 1 for every id of the list (ids outside the graph are skipped)
__global__ void count_ids_kernel(const uint32_t *__restrict__ ids, uint64_t n, uint32_t V, uint32_t *counts) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t g = ids[i];
    if (g < V) atomicAdd(&counts[g], 1u);
  }
}

static inline bool aligned_to(const void *p, size_t bytes) {
  return p == nullptr || (reinterpret_cast<uintptr_t>(p) % bytes) == 0;
}
static int pick_vec(uint32_t F, std::initializer_list<size_t> pitches, std::initializer_list<const void *> ptrs) {
  for (int vec = 4; vec >= 2; vec >>= 1) {
    bool ok = (F % vec) == 0;
    for (size_t ld : pitches) ok = ok && (ld % vec) == 0;
    for (const void *p : ptrs) ok = ok && aligned_to(p, vec * sizeof(float));
    if (ok) return vec;
  }
  return 1;
}

int read_gather_error_flag(unsigned int *value) {
  NB_CUDA(cudaMemcpyFromSymbol(value, g_gather_error, sizeof(unsigned int)));
  return 0;
}

int reset_gather_error_flag() {
  const unsigned int zero = 0;
  NB_CUDA(cudaMemcpyToSymbol(g_gather_error, &zero, sizeof(unsigned int)));
  return 0;
}
}  // namespace nb

using namespace nb;

NB_API int nb_feature_gather(float *d_x0, const float *feat, size_t feat_ld, const float *const *feat_shards,
                             uint32_t num_shards, uint32_t shard_rows, const float *d_cache, size_t cache_ld,
                             const uint32_t *d_hashmap, const uint32_t *d_source, uint32_t n, uint32_t F,
                             void *stream) {
  return feature_gather_impl(d_x0, F, 0, feat, feat_ld, feat_shards, num_shards, shard_rows, d_cache, cache_ld, d_hashmap,
                             d_source, n, F, stream, 0);
}

int nb::feature_gather_impl(float *d_x0, size_t x0_ld, int misses_only, const float *feat, size_t feat_ld,
                            const float *const *feat_shards, uint32_t num_shards, uint32_t shard_rows,
                            const float *d_cache, size_t cache_ld, const uint32_t *d_hashmap, const uint32_t *d_source,
                            uint32_t n, uint32_t F, void *stream, uint32_t max_ctas) {
  if (n == 0) return 0;
  NB_REQUIRE(x0_ld >= F, "nb_feature_gather: output pitch smaller than width");
  NB_REQUIRE(d_x0 && d_source, "nb_feature_gather: null pointer");
  NB_REQUIRE(F > 0, "nb_feature_gather: feature width is zero");
  NB_REQUIRE(feat || feat_shards || (d_cache && d_hashmap), "nb_feature_gather: no feature store");
  NB_REQUIRE(d_hashmap == nullptr || d_cache != nullptr, "nb_feature_gather: hashmap without cache");
  NB_REQUIRE(feat_shards == nullptr || (num_shards > 0 && shard_rows > 0), "nb_feature_gather: bad shard geometry");
  NB_REQUIRE((!feat && !feat_shards) || feat_ld >= F, "nb_feature_gather: feature pitch smaller than width");
  NB_REQUIRE(d_cache == nullptr || cache_ld >= F, "nb_feature_gather: cache pitch smaller than width");
  GatherArgs a{};
  a.x0 = d_x0; a.x0_ld = x0_ld; a.misses_only = misses_only; a.feat = feat; a.feat_ld = feat_ld; a.shards = feat_shards; a.num_shards = num_shards;
  a.shard_rows = shard_rows; a.cache = d_cache; a.cache_ld = cache_ld; a.hashmap = d_hashmap;
  a.source = d_source; a.n = n; a.F = F;
  // Shard base pointers live in device memory; they are cudaMalloc'ed, hence at least 256-byte aligned.
  const int vec = pick_vec(F, {(feat || feat_shards) ? feat_ld : (size_t)4, d_cache ? cache_ld : (size_t)4, x0_ld},
                           {d_x0, feat, d_cache});
  a.tiles = (F + 32 * vec - 1) / (32 * vec);
  const uint64_t warps = (((uint64_t)n + 3) / 4) * a.tiles;
  uint64_t blocks = (warps + kWarps - 1) / kWarps;
  if (max_ctas > 0 && blocks > max_ctas) blocks = max_ctas;
  NB_REQUIRE(blocks <= 0x7fffffffull, "nb_feature_gather: too many rows for one launch");
  cudaStream_t st = as_stream(stream);
  switch (vec) {
    case 4: feature_gather_kernel<4><<<(unsigned)blocks, kWarps * 32, 0, st>>>(a); break;
    case 2: feature_gather_kernel<2><<<(unsigned)blocks, kWarps * 32, 0, st>>>(a); break;
    default: feature_gather_kernel<1><<<(unsigned)blocks, kWarps * 32, 0, st>>>(a); break;
  }
  NB_LAUNCH_CHECK();
  return 0;
}

NB_API int nb_feature_gather_indexed(float *d_x0, size_t x0_ld, const float *table, size_t table_ld,
                                     const uint32_t *d_source, const uint32_t *d_local_idx, const uint32_t *d_slot_map,
                                     uint32_t n, uint32_t F, void *stream) {
  if (n == 0) return 0;
  NB_REQUIRE(d_x0 && table && d_source && d_local_idx, "nb_feature_gather_indexed: null pointer");
  NB_REQUIRE(F > 0 && x0_ld >= F && table_ld >= F, "nb_feature_gather_indexed: bad width or pitch");
  const int vec = pick_vec(F, {x0_ld, table_ld}, {d_x0, table});
  const uint32_t tiles = (F + 32 * vec - 1) / (32 * vec);
  const unsigned grid = grid_for((uint64_t)n * tiles * 32, kWarps * 32, 8, 8);
  cudaStream_t st = as_stream(stream);
  switch (vec) {
    case 4: gather_indexed_kernel<4><<<grid, kWarps * 32, 0, st>>>(d_x0, x0_ld, table, table_ld, d_source, d_local_idx, d_slot_map, n, F, tiles); break;
    case 2: gather_indexed_kernel<2><<<grid, kWarps * 32, 0, st>>>(d_x0, x0_ld, table, table_ld, d_source, d_local_idx, d_slot_map, n, F, tiles); break;
    default: gather_indexed_kernel<1><<<grid, kWarps * 32, 0, st>>>(d_x0, x0_ld, table, table_ld, d_source, d_local_idx, d_slot_map, n, F, tiles); break;
  }
  NB_LAUNCH_CHECK();
  return 0;
}

NB_API int nb_label_gather(int64_t *d_lab, const int64_t *d_label, const uint32_t *d_dst, uint32_t n,
                           uint32_t label_size, void *stream) {
  if (n == 0) return 0;
  NB_REQUIRE(d_lab && d_label && d_dst, "nb_label_gather: null pointer");
  NB_REQUIRE(label_size > 0, "nb_label_gather: label_size is zero");
  label_gather_kernel<<<grid_for((uint64_t)n * label_size, 256), 256, 0, as_stream(stream)>>>(d_lab, d_label, d_dst,
                                                                                             n, label_size);
  NB_LAUNCH_CHECK();
  return 0;
}

NB_API int nb_count_ids(const uint32_t *d_ids, uint64_t n, uint32_t num_vertices, uint32_t *d_counts, void *stream) {
  if (n == 0) return 0;
  NB_REQUIRE(d_ids && d_counts, "nb_count_ids: null pointer");
  nb::count_ids_kernel<<<nb::grid_for(n, 256), 256, 0, nb::as_stream(stream)>>>(d_ids, n, num_vertices, d_counts);
  NB_LAUNCH_CHECK();
  return 0;
}

NB_API int nb_cache_fill(float *d_cache, size_t cache_ld, const float *feat, size_t feat_ld,
                         const uint32_t *d_hashmap, uint32_t num_vertices, uint32_t F, void *stream) {
  if (num_vertices == 0) return 0;
  NB_REQUIRE(d_cache && feat && d_hashmap, "nb_cache_fill: null pointer");
  NB_REQUIRE(F > 0 && cache_ld >= F && feat_ld >= F, "nb_cache_fill: bad width or pitch");
  const int vec = pick_vec(F, {feat_ld, cache_ld}, {d_cache, feat});
  const uint32_t tiles = (F + 32 * vec - 1) / (32 * vec);
  const unsigned grid = grid_for((uint64_t)num_vertices * tiles * 32, kWarps * 32, 8, 8);
  cudaStream_t st = as_stream(stream);
  switch (vec) {
    case 4: cache_fill_kernel<4><<<grid, kWarps * 32, 0, st>>>(d_cache, cache_ld, feat, feat_ld, d_hashmap, num_vertices, F, tiles); break;
    case 2: cache_fill_kernel<2><<<grid, kWarps * 32, 0, st>>>(d_cache, cache_ld, feat, feat_ld, d_hashmap, num_vertices, F, tiles); break;
    default: cache_fill_kernel<1><<<grid, kWarps * 32, 0, st>>>(d_cache, cache_ld, feat, feat_ld, d_hashmap, num_vertices, F, tiles); break;
  }
  NB_LAUNCH_CHECK();
  return 0;
}
