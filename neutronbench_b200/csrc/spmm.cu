// Aggregation kernels: forward CSC SpMM, backward transposed-CSR SpMM, fused-weight and
// gather-fused variants.  HBM-bound: every lane issues 8- or 16-byte coalesced loads; a warp owns one
// (output row, chunk of CT tiles of 32*VEC floats) and keeps U source rows x CT tiles in flight.
//
// Arithmetic contract: out[k] = fma(x_n[k], w_n, ... fma(x1[k], w1, fma(x0[k], w0, 0))) — one IEEE fused multiply-add per
// edge and element, in edge order.  That is what the reference's CPU operator executes (nts_comp, core/ntsBaseOp.hpp:
// 76-97: _mm256_add_ps(_mm256_mul_ps(source, w), destination), which its -O3 -march=native build contracts into
// vfmadd), so results equal MiniBatchFuseOp's bit for bit and do not depend on the launch shape.  The reference's CUDA
// kernel rounds the product before its atomicAdd (cuda/ntsCUDAFuseKernel.cuh:272-290, 450-468) and therefore differs
// from its own CPU operator, and from this code, in the last bit of some sums.
#include <initializer_list>

#include "common.cuh"

namespace nb {

constexpr int kSpmmWarps = 8;    // warps per CTA

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

// Set (never cleared by the kernels) when the gather-fused aggregation met a source that is not cached while there is
// no table to read it from; the edge is skipped.
__device__ unsigned int g_spmm_error = 0;

struct SpmmArgs {
  const float *x;          // input rows (explicit / fused modes)
  size_t x_ld;             // pitch of x in floats
  float *y;                // n x F output
  size_t y_ld;             // pitch of y in floats (0 = F)
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
  int feat_by_local;       // 1: `feat` holds one row per source of the block (row li), not one per vertex (row g)
  const float *cache;
  size_t cache_ld;
  const uint32_t *hashmap;
  const uint32_t *source;
  uint32_t n;
  uint32_t F;
  uint32_t tiles;          // chunks per row: ceil(F / (CT*32*VEC))
  // Long rows: rows of at least hub_min edges (0 = no such treatment) are left out by the one-warp-per-row part of
  // the launch and taken by its first hub_ctas CTAs, where a team of ceil(F/32) warps walks one such row with one
  // column per lane and 32 row reads in flight per lane.
  uint32_t hub_min, hub_ctas;
};

template <int MODE, bool MASK>
__device__ __forceinline__ void hub_one_row(const SpmmArgs &a, uint32_t r, uint32_t col, unsigned lane) {
  const uint32_t start = __ldg(a.offs + r), end = __ldg(a.offs + r + 1);
  float nr = 0.0f;
  if constexpr (MODE != kExplicitW) nr = __ldg(a.norm_row + r);
  const bool live = col < a.F;
  // reference (row start) and weight of edge base + lane; lanes past the end hold a null row and weight 0
  auto refs = [&](uint32_t base, const float *&ptr, float &w) {
    const uint32_t j = base + lane;
    ptr = nullptr; w = 0.0f;
    if (j < end) {
      const uint32_t li = __ldg(a.idx + j);
      if constexpr (MODE == kExplicitW) w = __ldg(a.w + j);
      else w = __fdiv_rn(1.0f, __fmul_rn(__ldg(a.norm_idx + li), nr));
      ptr = a.x + (size_t)li * a.x_ld;
    }
  };
  const float *p_cur, *p_nxt;
  float w_cur, w_nxt;
  refs(start, p_cur, w_cur);
  float acc = 0.0f;
  for (uint32_t base = start; base < end; base += 32) {
    refs(base + 32, p_nxt, w_nxt);                // in flight while the 32 rows below are read
    const uint32_t cnt = min(32u, end - base);
    float v[32];
#pragma unroll
    for (int u = 0; u < 32; u++) {
      const uintptr_t p = __shfl_sync(0xffffffffu, (unsigned long long)(uintptr_t)p_cur, u);
      v[u] = (live && (uint32_t)u < cnt) ? __ldg(reinterpret_cast<const float *>(p) + col) : 0.0f;
    }
#pragma unroll
    for (int u = 0; u < 32; u++) {
      const float wu = __shfl_sync(0xffffffffu, w_cur, u);
      if ((uint32_t)u < cnt) acc = __fmaf_rn(v[u], wu, acc);
    }
    p_cur = p_nxt;
    w_cur = w_nxt;
  }
  if (live) {
    if constexpr (MASK) acc = __ldg(a.act + (size_t)r * a.F + col) > 0.0f ? __fmul_rn(acc, a.act_scale) : 0.0f;
    a.y[(size_t)r * a.y_ld + col] = acc;
  }
}

// Long rows of a launch (a source that hundreds or thousands of sampled destinations share, in the transposed
// aggregation of the backward pass).  One warp per row keeps 8 row reads in flight, so a row of 2,000 edges alone takes
// longer than all other rows of the block together.  Here the first CTAs of the launch look for such rows, each in its
// own slice of the row range, and a team of ceil(F/32) warps walks one row: a lane owns ONE column and keeps 32 reads of
// it in flight, and the references of the next 32 edges are requested before the current 32 are consumed.  Every
// element is still one fused multiply-add per edge in edge order, so results do not depend on which path took a row.
template <int MODE, bool MASK>
__device__ __forceinline__ void hub_rows_part(const SpmmArgs &a) {
  constexpr uint32_t kThreads = kSpmmWarps * 32;
  __shared__ uint32_t s_list[kThreads];                        // long rows of one stretch of kThreads rows
  __shared__ uint32_t s_count;
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t team_warps = (a.F + 31) / 32;                 // <= kSpmmWarps (the launcher checks)
  const uint32_t teams = kSpmmWarps / team_warps;
  const uint32_t team = warp / team_warps, col = (warp % team_warps) * 32 + lane;
  const uint32_t slice = (a.n + a.hub_ctas - 1) / a.hub_ctas;
  const uint32_t r0 = blockIdx.x * slice, r1 = min(a.n, r0 + slice);
  for (uint32_t from = r0; from < r1; from += kThreads) {     // one row per thread and stretch
    if (threadIdx.x == 0) s_count = 0;
    __syncthreads();
    const uint32_t r = from + threadIdx.x;
    if (r < r1 && __ldg(a.offs + r + 1) - __ldg(a.offs + r) >= a.hub_min) s_list[atomicAdd(&s_count, 1u)] = r;
    __syncthreads();
    const uint32_t found = s_count;
    if (team < teams)                                          // uniform over the warp
      for (uint32_t k = team; k < found; k += teams) hub_one_row<MODE, MASK>(a, s_list[k], col, lane);
    __syncthreads();
  }
}

// A warp owns one (output row, chunk) where a chunk is CT consecutive tiles of 32*VEC floats.  Per
// edge a lane issues CT independent vector loads, and U edges are in flight, so CT*U loads per lane
// hide the latency of the index chain (offsets -> indices -> [ids -> cache slots] -> rows), which is
// paid once per chunk.  Wide rows (F = 602: VEC 2, CT 5 -> 2 chunks) need it most.
template <int VEC, int CT, int U, int MODE, bool MASK>
__global__ void __launch_bounds__(kSpmmWarps * 32) spmm_rows_kernel(const SpmmArgs a) {
  pdl_enter();
  const unsigned lane = threadIdx.x & 31;
  if constexpr (MODE != kFusedGather) {
    if (blockIdx.x < a.hub_ctas) {   // uniform over the CTA
      hub_rows_part<MODE, MASK>(a);
      return;
    }
  }
  const uint64_t warp_global = (uint64_t)(blockIdx.x - (MODE != kFusedGather ? a.hub_ctas : 0u)) * kSpmmWarps +
                               (threadIdx.x >> 5);
  const uint32_t r = (uint32_t)(warp_global / a.tiles);   // a.tiles = chunks per row
  if (r >= a.n) return;
  const uint32_t chunk = (uint32_t)(warp_global - (uint64_t)r * a.tiles);
  const uint32_t col0 = chunk * (CT * 32 * VEC) + lane * VEC;

  const uint32_t start = a.offs[r], end = a.offs[r + 1];
  if constexpr (MODE != kFusedGather) {
    if (a.hub_ctas && end - start >= a.hub_min) return;   // a long row: the hub CTAs of this launch take it
  }
  float acc[CT][VEC];
#pragma unroll
  for (int t = 0; t < CT; t++)
#pragma unroll
    for (int k = 0; k < VEC; k++) acc[t][k] = 0.0f;

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
        if (slot != 0xFFFFFFFFu) my_ptr = a.cache + (size_t)slot * a.cache_ld;
        else if (a.feat) my_ptr = a.feat + (size_t)(a.feat_by_local ? li : g) * a.feat_ld;
        else atomicOr(&g_spmm_error, 1u);   // my_ptr stays null: the edge contributes nothing
      } else {
        my_ptr = a.x + (size_t)li * a.x_ld;
      }
    }
    const uint32_t cnt = min(32u, end - base);
    for (uint32_t jj = 0; jj < cnt; jj += U) {
      float vals[U][CT][VEC];
      float ws[U];
#pragma unroll
      for (int u = 0; u < U; u++) {
        const unsigned src_lane = (jj + u) & 31;  // lanes >= cnt hold nullptr / 0 weights
        const uintptr_t p = __shfl_sync(0xffffffffu, (unsigned long long)(uintptr_t)my_ptr, src_lane);
        ws[u] = __shfl_sync(0xffffffffu, my_w, src_lane);
        const bool valid = (jj + u) < cnt && p != 0;
#pragma unroll
        for (int t = 0; t < CT; t++) {
          const uint32_t col = col0 + t * (32 * VEC);
          if (valid && col < a.F) {
            load_vec<VEC>(vals[u][t], reinterpret_cast<const float *>(p) + col);
          } else {
#pragma unroll
            for (int k = 0; k < VEC; k++) vals[u][t][k] = 0.0f;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
        if ((jj + u) < cnt) {
#pragma unroll
          for (int t = 0; t < CT; t++) {
            if constexpr (VEC == 1) {
              acc[t][0] = __fmaf_rn(vals[u][t][0], ws[u], acc[t][0]);
            } else {   // packed pairs: one fused multiply-add instruction per two elements
#pragma unroll
              for (int k = 0; k < VEC; k += 2) {
                const float2 s = fma2_rn(make_float2(vals[u][t][k], vals[u][t][k + 1]), make_float2(ws[u], ws[u]),
                                         make_float2(acc[t][k], acc[t][k + 1]));
                acc[t][k] = s.x;
                acc[t][k + 1] = s.y;
              }
            }
          }
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < CT; t++) {
    const uint32_t col = col0 + t * (32 * VEC);
    if (col >= a.F) continue;
    if constexpr (MASK) {
      float av[VEC];
      load_vec<VEC>(av, a.act + (size_t)r * a.F + col);
#pragma unroll
      for (int k = 0; k < VEC; k++) acc[t][k] = av[k] > 0.0f ? __fmul_rn(acc[t][k], a.act_scale) : 0.0f;
    }
    store_vec<VEC>(a.y + (size_t)r * a.y_ld + col, acc[t]);
  }
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

template <int VEC, int CT, int U, int MODE, bool MASK>
static int launch_one(SpmmArgs a, cudaStream_t stream) {
  a.tiles = (a.F + CT * 32 * VEC - 1) / (CT * 32 * VEC);  // chunks per row
  if (a.y_ld == 0) a.y_ld = a.F;
  const uint64_t warps = (uint64_t)a.n * a.tiles;
  // long rows: only where a team of warps fits a CTA and the rows are plain tables (not the gather-fused forward,
  // whose rows are as long as the fanout at most)
  a.hub_min = 0; a.hub_ctas = 0;
  if (MODE != kFusedGather && tuning().hub_min_edges > 0 && (a.F + 31) / 32 <= (uint32_t)kSpmmWarps &&
      a.n >= 4u * (uint32_t)num_sms()) {
    a.hub_min = (uint32_t)tuning().hub_min_edges;
    a.hub_ctas = (uint32_t)num_sms();
  }
  const uint64_t blocks = (warps + kSpmmWarps - 1) / kSpmmWarps + a.hub_ctas;
  if (blocks > 0x7fffffffull) return fail(NB_ERR_INVALID, "spmm: too many rows for one launch");
  NB_CUDA(launch_chained(spmm_rows_kernel<VEC, CT, U, MODE, MASK>, dim3((unsigned)blocks), dim3(kSpmmWarps * 32), 0, stream, a));
  NB_LAUNCH_CHECK();
  return 0;
}

template <int VEC, int MODE, bool MASK>
static int launch_vec(const SpmmArgs &a, cudaStream_t stream) {
  const uint32_t tiles = (a.F + 32 * VEC - 1) / (32 * VEC);
  if (tiles >= 5) return launch_one<VEC, 5, (VEC == 4 ? 2 : 4), MODE, MASK>(a, stream);
  if (tiles >= 2) return launch_one<VEC, 2, (VEC == 4 ? 4 : 8), MODE, MASK>(a, stream);
  return launch_one<VEC, 1, 8, MODE, MASK>(a, stream);
}

template <int MODE, bool MASK>
static int launch_spmm(const SpmmArgs &a, int vec, cudaStream_t stream) {
  if (a.n == 0) return 0;
  switch (vec) {
    case 4: return launch_vec<4, MODE, MASK>(a, stream);
    case 2: return launch_vec<2, MODE, MASK>(a, stream);
    default: return launch_vec<1, MODE, MASK>(a, stream);
  }
}


// ---------------------------------------------------------------------------------------------
// Wide rows (hundreds of floats) with plain 16-byte loads: one warp per output row, every lane owns TILES float4
// columns of the row, U source rows are in flight per warp, and the per-edge references of the NEXT row of the warp
// (index -> source id -> cache slot -> row address, weight) are requested before the current row is accumulated, so
// that the index chain is off the critical path.  Many resident warps (the kernel holds no shared memory) keep far
// more row reads in flight than the shared-memory ring can, which is what random 2.4 KB row reads from DRAM need:
// measured on B200, 140 K such rows stream at 5.9 TB/s with plain loads.
// Needs the cache (or, without one, the plain input) 16-byte aligned with a pitch that is a multiple of 4 floats and
// at least ceil(F/4)*4 (the cache and the staging table are laid out like that; columns from F up to the pitch are
// never stored).  Rows without a cache slot may come from a table of any pitch and alignment (mapped host memory):
// those are read element by element.
// Same arithmetic and order as every other aggregation path.
// ---------------------------------------------------------------------------------------------
struct WideArgs {
  const float *x;          // rows named by a plain index (no cache): row(li) = x + li * x_ld   (gather == 0)
  size_t x_ld;
  // gather form: row of edge j = cache[hashmap[source[idx[j]]]] if it has a slot, else miss row
  const float *cache; size_t cache_ld;
  const uint32_t *hashmap, *source;
  const float *miss; size_t miss_ld;   // table for rows without a slot: by vertex id, or (miss_local) by source index
  int miss_local;
  int miss_aligned;        // rows of `miss` can be read with float4 loads like cache rows
  int gather;
  float *y; size_t y_ld;
  const uint32_t *offs, *idx;
  const float *norm_row, *norm_idx;
  uint32_t n, F;
  int out_vec;             // 4: whole float4 stores (the row's padding takes the tail), else 2 or 1
  int stream_stores;
  uint32_t split;          // warps per output row: each takes part_f4 consecutive float4 columns
  uint32_t part_f4;
};

constexpr int kWideThreads = 128;

template <int TILES, int U>
__global__ void __launch_bounds__(kWideThreads) spmm_wide_kernel(const WideArgs a) {
  pdl_enter();
  const unsigned lane = threadIdx.x & 31;
  // work items are (row, part) pairs, a.split parts per row; a warp walks items item, item + stride, ...
  const uint32_t items = a.n * a.split;
  const uint32_t total_warps = ((gridDim.x * blockDim.x) >> 5) / a.split * a.split;   // keeps a warp on one part
  uint32_t item = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (item >= total_warps || item >= items) return;
  const uint32_t part = item % a.split;
  uint32_t r = item / a.split;
  const uint32_t row_stride = total_warps / a.split;
  const uint32_t q0 = part * a.part_f4;                                       // first float4 column of this part
  const uint32_t fpad4 = min((a.F + 3) >> 2, q0 + a.part_f4);                 // one past its last float4 column

  // Reference and weight of edge `j` of a row whose degree factor is nr (lanes past the row's end get a null row).
  auto resolve = [&](uint32_t j, uint32_t end, float nr, const float4 *&ptr, float &w) {
    ptr = nullptr; w = 0.0f;
    if (j >= end) return;
    const uint32_t li = __ldg(a.idx + j);
    w = __fdiv_rn(1.0f, __fmul_rn(__ldg(a.norm_idx + li), nr));
    if (a.gather) {
      const uint32_t g = __ldg(a.source + li);
      const uint32_t slot = a.hashmap ? __ldg(a.hashmap + g) : 0xFFFFFFFFu;
      if (slot != 0xFFFFFFFFu) ptr = reinterpret_cast<const float4 *>(a.cache + (size_t)slot * a.cache_ld);
      else if (a.miss) {
        // bit 0 of the address marks a row that has to be read element by element
        const uintptr_t p = reinterpret_cast<uintptr_t>(a.miss + (size_t)(a.miss_local ? li : g) * a.miss_ld);
        ptr = reinterpret_cast<const float4 *>(a.miss_aligned ? p : (p | 1u));
      } else atomicOr(&g_spmm_error, 1u);
    } else {
      ptr = reinterpret_cast<const float4 *>(a.x + (size_t)li * a.x_ld);
    }
  };

  uint32_t start = __ldg(a.offs + r), end = __ldg(a.offs + r + 1);
  float nr = __ldg(a.norm_row + r);
  const float4 *my_ptr; float my_w;
  resolve(start + lane, end, nr, my_ptr, my_w);
  while (true) {
    // request the first window of this warp's next row now; it is consumed after the current row
    const uint32_t r_next = r + row_stride;
    uint32_t n_start = 0, n_end = 0; float n_nr = 0.0f;
    const float4 *n_ptr = nullptr; float n_w = 0.0f;
    if (r_next < a.n) {
      n_start = __ldg(a.offs + r_next); n_end = __ldg(a.offs + r_next + 1); n_nr = __ldg(a.norm_row + r_next);
      resolve(n_start + lane, n_end, n_nr, n_ptr, n_w);
    }
    float acc[TILES][4];
#pragma unroll
    for (int t = 0; t < TILES; t++) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f;
    for (uint32_t base = start; base < end; base += 32) {
      if (base != start) resolve(base + lane, end, nr, my_ptr, my_w);   // rows of more than 32 edges: further windows
      const uint32_t cnt = min(32u, end - base);
      for (uint32_t jj = 0; jj < cnt; jj += U) {
        float4 v[U][TILES];
        float ws[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
          const unsigned src_lane = (jj + u) & 31;
          const unsigned long long praw = __shfl_sync(0xffffffffu, (unsigned long long)(uintptr_t)my_ptr, src_lane);
          ws[u] = __shfl_sync(0xffffffffu, my_w, src_lane);
          const bool valid = (jj + u) < cnt && praw != 0;
          if (praw & 1ull) {      // a row of a table without 16-byte alignment
            const float *fp = reinterpret_cast<const float *>(praw & ~1ull);
#pragma unroll
            for (int t = 0; t < TILES; t++) {
              const uint32_t c = (q0 + lane + 32 * t) * 4;
              float4 x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
              if (valid && q0 + lane + 32 * t < fpad4) {
                if (c < a.F) x.x = __ldg(fp + c);
                if (c + 1 < a.F) x.y = __ldg(fp + c + 1);
                if (c + 2 < a.F) x.z = __ldg(fp + c + 2);
                if (c + 3 < a.F) x.w = __ldg(fp + c + 3);
              }
              v[u][t] = x;
            }
          } else {
            const float4 *p = reinterpret_cast<const float4 *>(praw);
#pragma unroll
            for (int t = 0; t < TILES; t++) {
              const uint32_t q = q0 + lane + 32 * t;
              v[u][t] = (valid && q < fpad4) ? __ldg(p + q) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
          if ((jj + u) < cnt) {
#pragma unroll
            for (int t = 0; t < TILES; t++) {
              const float2 w2 = make_float2(ws[u], ws[u]);
              const float2 lo = fma2_rn(make_float2(v[u][t].x, v[u][t].y), w2, make_float2(acc[t][0], acc[t][1]));
              const float2 hi = fma2_rn(make_float2(v[u][t].z, v[u][t].w), w2, make_float2(acc[t][2], acc[t][3]));
              acc[t][0] = lo.x; acc[t][1] = lo.y; acc[t][2] = hi.x; acc[t][3] = hi.y;
            }
          }
        }
      }
    }
    float *out = a.y + (size_t)r * a.y_ld;
#pragma unroll
    for (int t = 0; t < TILES; t++) {
      const uint32_t col = (q0 + lane + 32 * t) * 4;
      if (q0 + lane + 32 * t >= fpad4) continue;
      if (a.out_vec == 4) {
        const float4 o = make_float4(acc[t][0], acc[t][1], acc[t][2], acc[t][3]);
        if (a.stream_stores) __stcs(reinterpret_cast<float4 *>(out + col), o);
        else *reinterpret_cast<float4 *>(out + col) = o;
      } else if (a.out_vec == 2) {
        if (col + 1 < a.F) __stcs(reinterpret_cast<float2 *>(out + col), make_float2(acc[t][0], acc[t][1]));
        if (col + 3 < a.F) __stcs(reinterpret_cast<float2 *>(out + col + 2), make_float2(acc[t][2], acc[t][3]));
      } else {
#pragma unroll
        for (int c = 0; c < 4; c++)
          if (col + c < a.F) __stcs(out + col + c, acc[t][c]);
      }
    }
    if (r_next >= a.n) break;
    r = r_next; start = n_start; end = n_end; nr = n_nr; my_ptr = n_ptr; my_w = n_w;
  }
}

template <int TILES, int U>
static int launch_wide_tiles(const WideArgs &a, cudaStream_t stream) {
  int per_sm = 0;   // resident CTAs per SM of this instantiation: the grid is exactly one wave of them
  NB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, spmm_wide_kernel<TILES, U>, kWideThreads, 0));
  if (per_sm < 1) per_sm = 1;
  const int reserve = tuning().reserve_sms > 0 ? tuning().reserve_sms : 0;
  const unsigned sms = (unsigned)(num_sms() > reserve + 1 ? num_sms() - reserve : 1);
  const unsigned warps_per_cta = kWideThreads / 32;
  const unsigned need = (unsigned)(((uint64_t)a.n * a.split + warps_per_cta - 1) / warps_per_cta);
  const unsigned grid = need < sms * per_sm ? need : sms * per_sm;
  if ((uint64_t)grid * warps_per_cta < a.split) return fail(NB_ERR_INVALID, "spmm (wide rows): grid smaller than a row's parts");
  NB_CUDA(launch_chained(spmm_wide_kernel<TILES, U>, dim3(grid), dim3(kWideThreads), 0, stream, a));
  NB_LAUNCH_CHECK();
  return 0;
}

template <int U>
static int launch_wide_u(const WideArgs &a, cudaStream_t stream) {
  switch ((a.part_f4 + 31) / 32) {
    case 1: return launch_wide_tiles<1, U>(a, stream);
    case 2: return launch_wide_tiles<2, U>(a, stream);
    case 3: return launch_wide_tiles<3, U>(a, stream);
    case 4: return launch_wide_tiles<4, U>(a, stream);
    case 5: return launch_wide_tiles<5, U>(a, stream);
    case 6: return launch_wide_tiles<6, U>(a, stream);
    case 7: return launch_wide_tiles<7, U>(a, stream);
    case 8: return launch_wide_tiles<8, U>(a, stream);
    default: return fail(NB_ERR_INVALID, "spmm (wide rows): feature width above 1024");
  }
}

static int launch_wide(WideArgs a, cudaStream_t stream) {
  if (a.n == 0) return 0;
  const uint32_t f4 = (a.F + 3) / 4;
  a.split = tuning().wide_col_split > 1 && f4 >= 64 ? (uint32_t)tuning().wide_col_split : 1u;
  a.part_f4 = (f4 + a.split - 1) / a.split;
  switch (tuning().wide_rows_in_flight) {
    case 1: return launch_wide_u<1>(a, stream);
    case 4: return launch_wide_u<4>(a, stream);
    default: return launch_wide_u<2>(a, stream);
  }
}

// A row source can be read with aligned float4 loads over ceil(F/4) columns.
static bool wide_rows_ok(const float *p, size_t ld, uint32_t F) {
  return p == nullptr || (aligned_to(p, 16) && ld % 4 == 0 && ld >= (size_t)(F + 3) / 4 * 4);
}

// Staged (TMA) path for the plain forms: references are the block-local indices themselves.
static int try_staged(const float *x, float *y, const uint32_t *offs, const uint32_t *idx, const float *w,
                      const float *norm_row, const float *norm_idx, const float *act, float act_scale, uint32_t n,
                      uint32_t F, cudaStream_t stream, bool *done) {
  *done = false;
  if (!tuning().staged_spmm || !tma_spmm_applicable(x, F, F)) return 0;
  TmaSpmmArgs t{};
  t.x = x; t.x_ld = F; t.y = y; t.offs = offs; t.ref = idx; t.w = w; t.norm_row = norm_row; t.norm_idx = norm_idx;
  t.act = act; t.act_scale = act_scale; t.n = n; t.F = F;
  t.out_vec = pick_vec(F, {}, {y, act});
  *done = true;
  return launch_spmm_tma(t, stream);
}

}  // namespace nb

using namespace nb;

NB_API int nb_set_staged_spmm(int enabled) {
  Tuning &t = default_tuning();
  const int old = t.staged_spmm;
  t.staged_spmm = enabled ? 1 : 0;
  t.staged_min_width = (enabled == 2 || enabled == 4) ? 1 : 256;   // 2, 4: stage every allowed width
  t.spmm_ring = (enabled == 3 || enabled == 4) ? 0 : 1;            // 3, 4: two-stage segment kernel, no ring
  t.ring_group_shift = enabled == 5 ? 0 : 1;                       // 5: ring with one barrier per row, not per pair
  return old;
}

NB_API uint64_t nb_set_l2_panel_bytes(uint64_t bytes) {
  const uint64_t old = default_tuning().l2_panel_bytes;
  default_tuning().l2_panel_bytes = bytes;
  return old;
}

NB_API int nb_device_error_flags(uint32_t *flags) {
  NB_REQUIRE(flags != nullptr, "nb_device_error_flags: null pointer");
  unsigned int v = 0, t = 0, g = 0, s = 0, l = 0;
  NB_TRY(read_tma_error_flag(&v));
  NB_TRY(read_tc_error_flag(&t));
  NB_TRY(read_gather_error_flag(&g));
  NB_CUDA(cudaMemcpyFromSymbol(&s, g_spmm_error, sizeof(unsigned int)));
  NB_TRY(read_loss_error_flag(&l));
  *flags = ((v & 1u) ? 1u : 0u) | (t ? 2u : 0u) | ((g || s || (v & 2u)) ? 4u : 0u) | (l ? 8u : 0u);
  return 0;
}

NB_API int nb_device_error_reset(void) {
  NB_TRY(reset_tma_error_flag());
  NB_TRY(reset_tc_error_flag());
  NB_TRY(reset_gather_error_flag());
  NB_TRY(reset_loss_error_flag());
  const unsigned int zero = 0;
  NB_CUDA(cudaMemcpyToSymbol(g_spmm_error, &zero, sizeof(unsigned int)));
  return 0;
}

NB_API int nb_spmm_csc_fwd(const float *d_x, float *d_y, const float *d_w, const uint32_t *d_row_indices,
                           const uint32_t *d_column_offset, uint32_t v, uint32_t F, void *stream) {
  if (v == 0) return 0;
  NB_REQUIRE(d_x && d_y && d_w && d_row_indices && d_column_offset, "nb_spmm_csc_fwd: null pointer");
  NB_REQUIRE(F > 0, "nb_spmm_csc_fwd: feature width is zero");
  bool done;
  NB_TRY(try_staged(d_x, d_y, d_column_offset, d_row_indices, d_w, nullptr, nullptr, nullptr, 1.0f, v, F,
                    as_stream(stream), &done));
  if (done) return 0;
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
  bool done;
  NB_TRY(try_staged(d_gy, d_gx, d_row_offset, d_column_indices, d_w, nullptr, nullptr, nullptr, 1.0f, s, F,
                    as_stream(stream), &done));
  if (done) return 0;
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
  bool done;
  NB_TRY(try_staged(d_x, d_y, d_column_offset, d_row_indices, nullptr, d_dst_norm, d_src_norm, nullptr, 1.0f, v, F,
                    as_stream(stream), &done));
  if (done) return 0;
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
  bool done;
  NB_TRY(try_staged(d_gy, d_gx, d_row_offset, d_column_indices, nullptr, d_src_norm, d_dst_norm, d_act, act_scale, s,
                    F, as_stream(stream), &done));
  if (done) return 0;
  SpmmArgs a{};
  a.x = d_gy; a.x_ld = F; a.y = d_gx; a.offs = d_row_offset; a.idx = d_column_indices;
  a.norm_row = d_src_norm; a.norm_idx = d_dst_norm; a.act = d_act; a.act_scale = act_scale;
  a.n = s; a.F = F;
  const int vec = pick_vec(F, {}, {d_gy, d_gx, d_act});
  if (d_act) return launch_spmm<kFusedW, true>(a, vec, as_stream(stream));
  return launch_spmm<kFusedW, false>(a, vec, as_stream(stream));
}

namespace nb {
// nb_spmm_csc_fwd_gather_fused with an output pitch (floats, >= F): the native step pads the rows of the
// layer-0 aggregate to 16 bytes so that the dense layers can read them with TMA tensor loads.
//
// d_stage (nullable): a staging table with one row per source of the block (row li, pitch stage_ld floats) that holds
// the rows of the sources without a cache slot (every source's row when there is no cache).  Rows that are not cached
// are then read from it instead of from `feat`: the table a batch's sampling half fills from host or peer memory, so
// that each distinct row crosses that link once and the aggregation reads device memory only.
int spmm_csc_fwd_gather_fused_ld(nb_ws *ws, const float *feat, size_t feat_ld, const float *d_cache, size_t cache_ld,
                                 const uint32_t *d_hashmap, const uint32_t *d_source, float *d_y, size_t y_ld,
                                 const uint32_t *d_row_indices, const uint32_t *d_column_offset,
                                 const float *d_src_norm, const float *d_dst_norm, uint32_t v, uint32_t s, uint32_t e,
                                 uint32_t F, void *stream, const float *d_stage, size_t stage_ld) {
  if (v == 0) return 0;
  if (d_stage != nullptr) {
    NB_REQUIRE(stage_ld >= F, "nb_spmm_csc_fwd_gather_fused: staging pitch smaller than width");
    if (d_hashmap == nullptr) {   // no cache: the staging table is the gathered input itself
      NB_REQUIRE(d_y && d_row_indices && d_column_offset && d_src_norm && d_dst_norm && y_ld >= F,
                 "nb_spmm_csc_fwd_gather_fused: null pointer or bad pitch");
      if (tuning().staged_spmm && tuning().spmm_ring && tuning().l2_panel_bytes == 0 && e > 0 &&
          tma_spmm_applicable(d_stage, stage_ld, F)) {
        TmaSpmmArgs t{};
        t.x = d_stage; t.x_ld = stage_ld; t.y = d_y; t.y_ld = y_ld; t.offs = d_column_offset; t.ref = d_row_indices;
        t.norm_row = d_dst_norm; t.norm_idx = d_src_norm; t.n = v; t.F = F; t.act_scale = 1.0f; t.src_rows_hint = s;
        t.out_vec = pick_vec(F, {y_ld}, {d_y});
        return launch_spmm_tma(t, as_stream(stream));
      }
      SpmmArgs a{};
      a.x = d_stage; a.x_ld = stage_ld; a.y = d_y; a.y_ld = y_ld; a.offs = d_column_offset; a.idx = d_row_indices;
      a.norm_row = d_dst_norm; a.norm_idx = d_src_norm; a.n = v; a.F = F;
      return launch_spmm<kFusedW, false>(a, pick_vec(F, {stage_ld, y_ld}, {d_stage, d_y}), as_stream(stream));
    }
    feat = d_stage;               // rows without a slot: row li of the staging table
    feat_ld = stage_ld;
  }
  const int by_local = d_stage != nullptr ? 1 : 0;
  NB_REQUIRE(d_source && d_y && d_row_indices && d_column_offset && d_src_norm && d_dst_norm,
             "nb_spmm_csc_fwd_gather_fused: null pointer");
  NB_REQUIRE(feat != nullptr || (d_cache != nullptr && d_hashmap != nullptr),
             "nb_spmm_csc_fwd_gather_fused: no feature store");
  NB_REQUIRE(d_hashmap == nullptr || d_cache != nullptr, "nb_spmm_csc_fwd_gather_fused: hashmap without cache");
  NB_REQUIRE(F > 0 && (feat == nullptr || feat_ld >= F) && (d_cache == nullptr || cache_ld >= F) && y_ld >= F,
             "nb_spmm_csc_fwd_gather_fused: bad width or pitch");
  // Staged path: hits (cache rows, or the table itself when there is no cache) go through the TMA
  // unit; misses are rows of `feat` that the lanes copy.  Needs scratch for per-edge references.
  // Wide rows with plain loads (tuning().wide_direct), when every row source is aligned for float4 loads.
  if (tuning().wide_direct && F >= (uint32_t)tuning().staged_min_width && F <= 1024 && e > 0 &&
      wide_rows_ok(d_cache, cache_ld, F) && (d_hashmap != nullptr || wide_rows_ok(feat, feat_ld, F))) {
    WideArgs w{};
    w.gather = 1; w.cache = d_cache; w.cache_ld = cache_ld; w.hashmap = d_hashmap; w.source = d_source;
    w.miss = feat; w.miss_ld = feat_ld; w.miss_local = by_local;
    w.miss_aligned = feat != nullptr && wide_rows_ok(feat, feat_ld, F);
    w.y = d_y; w.y_ld = y_ld; w.offs = d_column_offset; w.idx = d_row_indices; w.norm_row = d_dst_norm;
    w.norm_idx = d_src_norm; w.n = v; w.F = F; w.stream_stores = tuning().y_stream_stores;
    w.out_vec = pick_vec(F, {y_ld}, {d_y});
    if (y_ld % 4 == 0 && y_ld >= (size_t)(F + 3) / 4 * 4 && aligned_to(d_y, 16)) w.out_vec = 4;
    return launch_wide(w, as_stream(stream));
  }
  {
    const float *hit_base = d_hashmap ? d_cache : feat;
    const size_t hit_ld = d_hashmap ? cache_ld : feat_ld;
    if (tuning().staged_spmm && tuning().spmm_ring && tuning().l2_panel_bytes == 0 && e > 0 && tma_spmm_applicable(hit_base, hit_ld, F)) {
      // ring kernel: references and weights are formed inside the kernel, one window of 32 edges ahead
      TmaSpmmArgs t{};
      t.x = hit_base; t.x_ld = hit_ld; t.miss = feat; t.miss_ld = feat_ld; t.y = d_y; t.y_ld = y_ld; t.offs = d_column_offset;
      t.miss_local = by_local;
      t.miss_bulk = by_local && aligned_to(feat, 16) && feat_ld % 4 == 0 && feat_ld >= (size_t)(F + 3) / 4 * 4;
      t.gidx = d_row_indices; t.gsource = d_source; t.ghashmap = d_hashmap;
      t.norm_row = d_dst_norm; t.norm_idx = d_src_norm;
      t.n = v; t.F = F; t.act = nullptr; t.act_scale = 1.0f; t.src_rows_hint = s;
      t.out_vec = pick_vec(F, {}, {d_y});
      // rows padded to 16 bytes take whole float4 stores even when F is not a multiple of 4 (the tail lands in the
      // padding)
      if (y_ld % 4 == 0 && y_ld >= (size_t)(F + 3) / 4 * 4 && aligned_to(d_y, 16)) t.out_vec = 4;
      return launch_spmm_tma(t, as_stream(stream));
    }
    if (!by_local && tuning().staged_spmm && ws != nullptr && e > 0 && tma_spmm_applicable(hit_base, hit_ld, F)) {
      cudaStream_t st = as_stream(stream);
      WsScope scope(ws);
      uint32_t *ref = ws->alloc_n<uint32_t>(e);
      float *w = ws->alloc_n<float>(e);
      if (!ref || !w) return fail(NB_ERR_NOMEM, "nb_spmm_csc_fwd_gather_fused: workspace arena exhausted");
      NB_TRY(launch_gather_refs(d_column_offset, d_row_indices, v, e, d_source, d_hashmap, d_hashmap == nullptr,
                                d_src_norm, d_dst_norm, ref, w, st));
      TmaSpmmArgs t{};
      t.x = hit_base; t.x_ld = hit_ld; t.miss = feat; t.miss_ld = feat_ld; t.y = d_y; t.y_ld = y_ld; t.offs = d_column_offset;
      t.ref = ref; t.w = w; t.n = v; t.F = F; t.act = nullptr; t.act_scale = 1.0f; t.src_rows_hint = s;
      t.out_vec = pick_vec(F, {}, {d_y});
      return launch_spmm_tma(t, st);
    }
  }
  SpmmArgs a{};
  a.feat = feat; a.feat_ld = feat_ld; a.feat_by_local = by_local; a.cache = d_cache; a.cache_ld = cache_ld; a.hashmap = d_hashmap;
  a.source = d_source; a.y = d_y; a.y_ld = y_ld; a.offs = d_column_offset; a.idx = d_row_indices;
  a.norm_row = d_dst_norm; a.norm_idx = d_src_norm; a.n = v; a.F = F;
  std::initializer_list<size_t> pitches = {feat ? feat_ld : (size_t)4, d_cache ? cache_ld : (size_t)4};
  return launch_spmm<kFusedGather, false>(a, pick_vec(F, pitches, {feat, d_cache, d_y}), as_stream(stream));
}
}  // namespace nb

NB_API int nb_spmm_csc_fwd_gather_fused(nb_ws *ws, const float *feat, size_t feat_ld, const float *d_cache,
                                        size_t cache_ld, const uint32_t *d_hashmap,
                                        const uint32_t *d_source, float *d_y,
                                        const uint32_t *d_row_indices, const uint32_t *d_column_offset,
                                        const float *d_src_norm, const float *d_dst_norm, uint32_t v,
                                        uint32_t s, uint32_t e, uint32_t F, void *stream) {
  return nb::spmm_csc_fwd_gather_fused_ld(ws, feat, feat_ld, d_cache, cache_ld, d_hashmap, d_source, d_y, F,
                                          d_row_indices, d_column_offset, d_src_norm, d_dst_norm, v, s, e, F, stream,
                                          nullptr, 0);
}
