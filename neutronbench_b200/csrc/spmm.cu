// Aggregation kernels: forward CSC SpMM, backward transposed-CSR SpMM, fused-weight and
// gather-fused variants.  HBM-bound: every lane issues 8- or 16-byte coalesced loads, a warp owns one
// (output row, 32*VEC-float tile) and keeps UNROLL source rows in flight.
//
// Arithmetic contract: out[k] = (((0 + x0[k]*w0) + x1[k]*w1) + ...) with one IEEE multiply and one
// IEEE add per edge, in edge order.  __fmul_rn/__fadd_rn are never contracted into an FMA, so the
// result equals the reference kernel's atomicAdd(out, in*w) sequence
// (cuda/ntsCUDAFuseKernel.cuh:272-290, 450-468) bit for bit and is independent of the launch shape.
#include "common.cuh"

namespace nb {

constexpr int kSpmmWarps = 8;    // warps per CTA
constexpr int kSpmmUnroll = 8;   // source rows in flight per warp

template <int VEC>
struct Vec;
template <>
struct Vec<1> {
  using T = float;
};
template <>
struct Vec<2> {
  using T = float2;
};
template <>
struct Vec<4> {
  using T = float4;
};

template <int VEC>
__device__ __forceinline__ void load_vec(float (&v)[VEC], const float *p) {
  if constexpr (VEC == 1) {
    v[0] = __ldg(p);
  } else if constexpr (VEC == 2) {
    float2 t = __ldg(reinterpret_cast<const float2 *>(p));
    v[0] = t.x; v[1] = t.y;
  } else {
    float4 t = __ldg(reinterpret_cast<const float4 *>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
}
template <int VEC>
__device__ __forceinline__ void store_vec(float *p, const float (&v)[VEC]) {
  if constexpr (VEC == 1) {
    *p = v[0];
  } else if constexpr (VEC == 2) {
    *reinterpret_cast<float2 *>(p) = make_float2(v[0], v[1]);
  } else {
    *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
}

enum SpmmMode { kExplicitW = 0, kFusedW = 1, kFusedGather = 2 };

struct SpmmArgs {
  const float *x;          // input rows (explicit / fused modes)
  size_t x_ld;             // pitch of x in floats
  float *y;                // n x F output
  const uint32_t *offs;    // n+1 offsets (column_offset fwd, row_offset bwd)
  const uint32_t *idx;     // e indices into x rows
  const float *w;          // explicit per-edge weights
  const float *norm_row;   // fused: sqrt-degree factor of the output row side  [n]
  const float *norm_idx;   // fused: sqrt-degree factor of the indexed side      [rows of x]
  const float *act;        // nullable n x F activation for the relu/dropout gradient mask
  float act_scale;
  // gather-fused mode: x row of local index i is row(source[i]) of the feature store
  const float *feat;
  size_t feat_ld;
  const float *cache;
  size_t cache_ld;
  const uint32_t *hashmap;
  const uint32_t *source;
  uint32_t n;
  uint32_t F;
  uint32_t tiles;          // ceil(F / (32*VEC))
};

template <int VEC, int MODE, bool MASK>
__global__ void __launch_bounds__(kSpmmWarps * 32) spmm_rows_kernel(const SpmmArgs a) {
  const unsigned lane = threadIdx.x & 31;
  const uint64_t warp_global = (uint64_t)blockIdx.x * kSpmmWarps + (threadIdx.x >> 5);
  const uint32_t r = (uint32_t)(warp_global / a.tiles);
  if (r >= a.n) return;
  const uint32_t tile = (uint32_t)(warp_global - (uint64_t)r * a.tiles);
  const uint32_t col = tile * (32 * VEC) + lane * VEC;
  const bool active = col < a.F;

  const uint32_t start = a.offs[r], end = a.offs[r + 1];
  float acc[VEC];
#pragma unroll
  for (int k = 0; k < VEC; k++) acc[k] = 0.0f;

  float nr = 0.0f;
  if constexpr (MODE != kExplicitW) nr = a.norm_row[r];

  for (uint32_t base = start; base < end; base += 32) {
    const uint32_t j = base + lane;
    const float *my_ptr = nullptr;
    float my_w = 0.0f;
    if (j < end) {
      const uint32_t li = a.idx[j];
      if constexpr (MODE == kExplicitW) {
        my_w = __ldg(a.w + j);
      } else {
        // 1 / ((float)sqrt(out_deg[src]) * (float)sqrt(in_deg[dst])): float multiply, IEEE divide.
        my_w = __fdiv_rn(1.0f, __fmul_rn(a.norm_idx[li], nr));
      }
      if constexpr (MODE == kFusedGather) {
        const uint32_t g = a.source[li];
        const uint32_t slot = a.hashmap ? a.hashmap[g] : 0xFFFFFFFFu;
        my_ptr = (slot != 0xFFFFFFFFu) ? a.cache + (size_t)slot * a.cache_ld : a.feat + (size_t)g * a.feat_ld;
      } else {
        my_ptr = a.x + (size_t)li * a.x_ld;
      }
    }
    const uint32_t cnt = min(32u, end - base);
    for (uint32_t jj = 0; jj < cnt; jj += kSpmmUnroll) {
      float vals[kSpmmUnroll][VEC];
      float ws[kSpmmUnroll];
#pragma unroll
      for (int u = 0; u < kSpmmUnroll; u++) {
        const unsigned src_lane = (jj + u) & 31;  // lanes >= cnt hold nullptr / 0 weights
        const uintptr_t p = __shfl_sync(0xffffffffu, (unsigned long long)(uintptr_t)my_ptr, src_lane);
        ws[u] = __shfl_sync(0xffffffffu, my_w, src_lane);
        if (active && (jj + u) < cnt) {
          load_vec<VEC>(vals[u], reinterpret_cast<const float *>(p) + col);
        } else {
#pragma unroll
          for (int k = 0; k < VEC; k++) vals[u][k] = 0.0f;
        }
      }
#pragma unroll
      for (int u = 0; u < kSpmmUnroll; u++) {
        if ((jj + u) < cnt) {
#pragma unroll
          for (int k = 0; k < VEC; k++) acc[k] = __fadd_rn(acc[k], __fmul_rn(vals[u][k], ws[u]));
        }
      }
    }
  }
  if (!active) return;
  if constexpr (MASK) {
    float av[VEC];
    load_vec<VEC>(av, a.act + (size_t)r * a.F + col);
#pragma unroll
    for (int k = 0; k < VEC; k++) acc[k] = av[k] > 0.0f ? __fmul_rn(acc[k], a.act_scale) : 0.0f;
  }
  store_vec<VEC>(a.y + (size_t)r * a.F + col, acc);
}

static inline bool aligned_to(const void *p, size_t bytes) {
  return p == nullptr || (reinterpret_cast<uintptr_t>(p) % bytes) == 0;
}

// Widest vector (in floats) usable for rows of width F with the given pitches and base pointers.
static int pick_vec(uint32_t F, std::initializer_list<size_t> pitches, std::initializer_list<const void *> ptrs) {
  for (int vec = 4; vec >= 2; vec >>= 1) {
    bool ok = (F % vec) == 0;
    for (size_t ld : pitches) ok = ok && (ld % vec) == 0;
    for (const void *p : ptrs) ok = ok && aligned_to(p, vec * sizeof(float));
    if (ok) return vec;
  }
  return 1;
}

template <int MODE, bool MASK>
static int launch_spmm(SpmmArgs a, int vec, cudaStream_t stream) {
  if (a.n == 0) return 0;
  a.tiles = (a.F + 32 * vec - 1) / (32 * vec);
  const uint64_t warps = (uint64_t)a.n * a.tiles;
  const uint64_t blocks = (warps + kSpmmWarps - 1) / kSpmmWarps;
  if (blocks > 0x7fffffffull) return fail(NB_ERR_INVALID, "spmm: too many rows for one launch");
  switch (vec) {
    case 4: spmm_rows_kernel<4, MODE, MASK><<<(unsigned)blocks, kSpmmWarps * 32, 0, stream>>>(a); break;
    case 2: spmm_rows_kernel<2, MODE, MASK><<<(unsigned)blocks, kSpmmWarps * 32, 0, stream>>>(a); break;
    default: spmm_rows_kernel<1, MODE, MASK><<<(unsigned)blocks, kSpmmWarps * 32, 0, stream>>>(a); break;
  }
  NB_LAUNCH_CHECK();
  return 0;
}

}  // namespace nb

using namespace nb;

NB_API int nb_spmm_csc_fwd(const float *d_x, float *d_y, const float *d_w, const uint32_t *d_row_indices,
                           const uint32_t *d_column_offset, uint32_t v, uint32_t F, void *stream) {
  if (v == 0) return 0;
  NB_REQUIRE(d_x && d_y && d_w && d_row_indices && d_column_offset, "nb_spmm_csc_fwd: null pointer");
  NB_REQUIRE(F > 0, "nb_spmm_csc_fwd: feature width is zero");
  SpmmArgs a{};
  a.x = d_x; a.x_ld = F; a.y = d_y; a.offs = d_column_offset; a.idx = d_row_indices; a.w = d_w;
  a.n = v; a.F = F;
  return launch_spmm<kExplicitW, false>(a, pick_vec(F, {}, {d_x, d_y}), as_stream(stream));
}

NB_API int nb_spmm_csr_bwd(const float *d_gy, float *d_gx, const float *d_w, const uint32_t *d_row_offset,
                           const uint32_t *d_column_indices, uint32_t s, uint32_t F, void *stream) {
  if (s == 0) return 0;
  NB_REQUIRE(d_gy && d_gx && d_w && d_row_offset && d_column_indices, "nb_spmm_csr_bwd: null pointer");
  NB_REQUIRE(F > 0, "nb_spmm_csr_bwd: feature width is zero");
  SpmmArgs a{};
  a.x = d_gy; a.x_ld = F; a.y = d_gx; a.offs = d_row_offset; a.idx = d_column_indices; a.w = d_w;
  a.n = s; a.F = F;
  return launch_spmm<kExplicitW, false>(a, pick_vec(F, {}, {d_gy, d_gx}), as_stream(stream));
}

NB_API int nb_spmm_csc_fwd_fused(const float *d_x, float *d_y, const uint32_t *d_row_indices,
                                 const uint32_t *d_column_offset, const float *d_src_norm,
                                 const float *d_dst_norm, uint32_t v, uint32_t F, void *stream) {
  if (v == 0) return 0;
  NB_REQUIRE(d_x && d_y && d_row_indices && d_column_offset && d_src_norm && d_dst_norm,
             "nb_spmm_csc_fwd_fused: null pointer");
  NB_REQUIRE(F > 0, "nb_spmm_csc_fwd_fused: feature width is zero");
  SpmmArgs a{};
  a.x = d_x; a.x_ld = F; a.y = d_y; a.offs = d_column_offset; a.idx = d_row_indices;
  a.norm_row = d_dst_norm; a.norm_idx = d_src_norm; a.n = v; a.F = F;
  return launch_spmm<kFusedW, false>(a, pick_vec(F, {}, {d_x, d_y}), as_stream(stream));
}

NB_API int nb_spmm_csr_bwd_fused(const float *d_gy, float *d_gx, const uint32_t *d_row_offset,
                                 const uint32_t *d_column_indices, const float *d_src_norm,
                                 const float *d_dst_norm, const float *d_act, float act_scale, uint32_t s,
                                 uint32_t F, void *stream) {
  if (s == 0) return 0;
  NB_REQUIRE(d_gy && d_gx && d_row_offset && d_column_indices && d_src_norm && d_dst_norm,
             "nb_spmm_csr_bwd_fused: null pointer");
  NB_REQUIRE(F > 0, "nb_spmm_csr_bwd_fused: feature width is zero");
  SpmmArgs a{};
  a.x = d_gy; a.x_ld = F; a.y = d_gx; a.offs = d_row_offset; a.idx = d_column_indices;
  a.norm_row = d_src_norm; a.norm_idx = d_dst_norm; a.act = d_act; a.act_scale = act_scale;
  a.n = s; a.F = F;
  const int vec = pick_vec(F, {}, {d_gy, d_gx, d_act});
  if (d_act) return launch_spmm<kFusedW, true>(a, vec, as_stream(stream));
  return launch_spmm<kFusedW, false>(a, vec, as_stream(stream));
}

NB_API int nb_spmm_csc_fwd_gather_fused(const float *feat, size_t feat_ld, const float *d_cache,
                                        size_t cache_ld, const uint32_t *d_hashmap,
                                        const uint32_t *d_source, float *d_y,
                                        const uint32_t *d_row_indices, const uint32_t *d_column_offset,
                                        const float *d_src_norm, const float *d_dst_norm, uint32_t v,
                                        uint32_t F, void *stream) {
  if (v == 0) return 0;
  NB_REQUIRE(d_source && d_y && d_row_indices && d_column_offset && d_src_norm && d_dst_norm,
             "nb_spmm_csc_fwd_gather_fused: null pointer");
  NB_REQUIRE(feat != nullptr || (d_cache != nullptr && d_hashmap != nullptr),
             "nb_spmm_csc_fwd_gather_fused: no feature store");
  NB_REQUIRE(d_hashmap == nullptr || d_cache != nullptr, "nb_spmm_csc_fwd_gather_fused: hashmap without cache");
  NB_REQUIRE(F > 0 && (feat == nullptr || feat_ld >= F) && (d_cache == nullptr || cache_ld >= F),
             "nb_spmm_csc_fwd_gather_fused: bad width or pitch");
  SpmmArgs a{};
  a.feat = feat; a.feat_ld = feat_ld; a.cache = d_cache; a.cache_ld = cache_ld; a.hashmap = d_hashmap;
  a.source = d_source; a.y = d_y; a.offs = d_column_offset; a.idx = d_row_indices;
  a.norm_row = d_dst_norm; a.norm_idx = d_src_norm; a.n = v; a.F = F;
  std::initializer_list<size_t> pitches = {feat ? feat_ld : (size_t)4, d_cache ? cache_ld : (size_t)4};
  return launch_spmm<kFusedGather, false>(a, pick_vec(F, pitches, {feat, d_cache, d_y}), as_stream(stream));
}
