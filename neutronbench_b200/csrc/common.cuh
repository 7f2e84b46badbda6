// Shared helpers of libnb_b200: status / error string, launch checks, workspace arena, warp utilities.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "nb_b200.h"

#define NB_API extern "C" __attribute__((visibility("default")))

namespace nb {

// Number of SMs of the current device (148 on B200: 2 dies x 74), asked from the driver once per device.
int num_sms();
// Host wait for everything enqueued on `stream` so far.  With Tuning::blocking_sync the calling thread sleeps on an
// event created with cudaEventBlockingSync instead of spinning in cudaStreamSynchronize: the sampler threads of
// several ranks (and several batches in flight per rank) then leave the cores to the threads that launch kernels
// when a node has fewer cores than such threads.
cudaError_t wait_stream_host(cudaStream_t stream);

// Flag per device for set-up that CUDA keeps per device (function attributes such as the dynamic shared-memory
// limit): need() is true until done() has been called with that device current.
constexpr int kMaxDevices = 64;
struct PerDeviceOnce {
  bool flag[kMaxDevices] = {};
  static int dev() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= kMaxDevices) return -1;
    return d;
  }
  bool need() const { const int d = dev(); return d < 0 || !flag[d]; }
  void done() { const int d = dev(); if (d >= 0) flag[d] = true; }
};

// Tuning switches.  Stand-alone entry points read the process defaults (changed by the nb_set_* calls);
// an nb_gcn handle copies the defaults when it is created, keeps its own copy (nb_gcn_set_option) and makes it
// current for the calling thread while one of its entry points runs, so that two handles, or two threads,
// never see each other's settings.
struct Tuning {
  int gemm_mode = 1;             // 0: CUDA cores (fp32 FMA), 1: tcgen05 3xTF32 (fp32-level accuracy), 2: tcgen05 TF32
  int gemm_force_tc = 0;         // tensor cores for every product size
  int use_pdl = 1;               // programmatic dependent launch for the training half's kernels
  int fuse_output_layer = 1;     // last layer + loss + its gradients in two launches
  int staged_spmm = 1;           // TMA-staged aggregation where its alignment rules hold
  int spmm_ring = 1;             // per-edge ring variant when rows are not cut into panels
  int staged_min_width = 256;    // narrowest row (floats) that takes the staged path
  int l2_prefetch = 0;           // segment kernel: prefetch rows into L2 two segments ahead
  int l2_hint = 3;               // ring kernel, fused weights: rows used by one edge only are copied with the
                                 // L2 evict-first policy (1); 2: rows with more uses evict-last as well; 3: only
                                 // rows with at least l2_keep_min_uses uses evict-last; 0: off
  int l2_keep_min_uses = 4;
  int ring_wait_ns = 0;          // ring kernel: a warp waiting for its copies may sleep this long per try (0: plain spin)
  int ring_prefetch = 0;         // ring kernel: groups of rows whose L2 prefetch is issued ahead of the ring's copies
  int hub_min_edges = 256;       // aggregation of plain tables: rows of at least this many edges go to warp teams (0: off)
  // ReLU + dropout of a hidden layer applied in the GEMM's epilogue where the kernel can.  Off: measured no faster.
  // The row-balanced kernel holds one column per thread, so its four-column Philox words cost a round of shuffles per
  // row (Reddit-shaped step 0.230 -> 0.238 ms); the 128-row-tile kernel saves two launches per Products-shaped step
  // and the step time stays at 0.697 ms.
  int fuse_relu = 0;
  int blocking_sync = 0;         // host waits of the sampling half sleep on a blocking event instead of spinning
  int ring_warps = 24;           // ring kernel: warps per CTA (20, 22 or 24), i.e. row slots in flight per SM
  int fuse_last_aggregation = 1; // the fused output layer aggregates the last block itself (one launch fewer)
  int ring_balance = 0;          // ring kernel: warps take shares of equal edge count (1) or of equal row count (0)
  int y_stream_stores = 1;       // ring kernel: output rows written with streaming stores (1) or default stores (0)
  int wide_direct = 0;           // wide rows: plain-load kernel (one warp per row, many warps resident) instead of the ring
  int wide_rows_in_flight = 2;   // source rows in flight per warp of that kernel: 1, 2 or 4
  int wide_col_split = 1;        // warps that share one output row of that kernel, each taking a range of columns
  int stage_ctas = 0;            // CTAs of the staging gather (0: 32 for a table in host memory, 2 per SM for shards)
  int reserve_sms = 0;           // SMs the one-CTA-per-SM aggregation kernel leaves to kernels that run beside it
  uint32_t ring_group_shift = 1; // ring kernel: 1 << shift row slots share one barrier
  uint64_t l2_panel_bytes = 0;   // working-set target of one column panel (0: no panels)
};
Tuning &default_tuning();
Tuning &tuning();                // the calling thread's current settings
struct TuningScope {
  Tuning *prev;
  explicit TuningScope(Tuning *t);
  ~TuningScope();
};

void set_error(const char *fmt, ...);

inline int fail(nb_status st, const char *what) {
  set_error("%s", what);
  return (int)st;
}

#define NB_CUDA(call)                                                                         \
  do {                                                                                        \
    cudaError_t err__ = (call);                                                               \
    if (err__ != cudaSuccess) {                                                               \
      nb::set_error("%s:%d %s -> %s", __FILE__, __LINE__, #call, cudaGetErrorString(err__));  \
      return (int)NB_ERR_CUDA;                                                                \
    }                                                                                         \
  } while (0)

// Every kernel launch in the library is followed by NB_LAUNCH_CHECK, which also counts it
// (nb_launch_count reports the total, so that callers can state how many kernels a step ran).
extern unsigned long long g_launches;

#define NB_LAUNCH_CHECK()                                                                     \
  do {                                                                                        \
    __atomic_fetch_add(&nb::g_launches, 1ull, __ATOMIC_RELAXED);                              \
    cudaError_t err__ = cudaGetLastError();                                                   \
    if (err__ != cudaSuccess) {                                                               \
      nb::set_error("%s:%d kernel launch -> %s", __FILE__, __LINE__, cudaGetErrorString(err__)); \
      return (int)NB_ERR_CUDA;                                                                \
    }                                                                                         \
  } while (0)

#define NB_REQUIRE(cond, msg)                                  \
  do {                                                         \
    if (!(cond)) return nb::fail(NB_ERR_INVALID, msg);         \
  } while (0)

#define NB_TRY(expr)            \
  do {                          \
    int st__ = (expr);          \
    if (st__ != 0) return st__; \
  } while (0)

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

inline unsigned div_up(uint64_t a, uint64_t b) { return (unsigned)((a + b - 1) / b); }

// Grid for a grid-stride kernel: enough blocks to cover `items`, capped at `waves` full waves of the
// device's SMs at `blocks_per_sm` resident blocks each.
inline unsigned grid_for(uint64_t items, unsigned block, unsigned blocks_per_sm = 8, unsigned waves = 4) {
  uint64_t need = (items + block - 1) / block;
  uint64_t cap = (uint64_t)num_sms() * blocks_per_sm * waves;
  if (need < 1) need = 1;
  return (unsigned)(need < cap ? need : cap);
}

}  // namespace nb

// The workspace: bump allocator over one device arena + a pinned mailbox for size read-backs.
struct nb_ws {
  char *base = nullptr;
  size_t bytes = 0;
  size_t used = 0;
  size_t high = 0;
  bool owns = false;
  uint32_t *mailbox = nullptr;  // pinned host, 64 words

  // 256-byte aligned sub-allocation; returns nullptr when the arena is exhausted.
  void *alloc(size_t n) {
    size_t start = (used + 255) & ~(size_t)255;
    if (start + n > bytes) return nullptr;
    used = start + n;
    if (used > high) high = used;
    return base + start;
  }
  template <typename T>
  T *alloc_n(size_t count) {
    return reinterpret_cast<T *>(alloc(count * sizeof(T)));
  }
};

namespace nb {
// Arguments of the shared-memory-staged aggregation kernel (spmm_tma.cu).
struct TmaSpmmArgs {
  const float *x;          // base of the rows that the TMA unit copies: row(ref) = x + ref * x_ld
  size_t x_ld;             // pitch in floats, a multiple of 4; x is 16-byte aligned
  const float *miss;       // base of rows whose reference has bit 31 set, or null
  size_t miss_ld;
  int miss_local;          // 1: `miss` holds one row per source of the block (row li), not one per vertex (row g)
  int miss_bulk;           // 1: rows of `miss` are 16-byte aligned device memory: the TMA unit copies them too
  float *y;                // n x F output
  size_t y_ld;             // pitch of y in floats (0 = F)
  const uint32_t *offs;    // n + 1 offsets
  const uint32_t *ref;     // per edge: row reference (null in the gather form below)
  // gather form (ring kernel only): the reference of edge j is formed on the fly from idx[j] -> source -> hashmap
  const uint32_t *gidx, *gsource, *ghashmap;   // ghashmap null = no cache: rows come from x by global id
  const float *w;          // per edge weight, or null to form it from the two factors below
  const float *norm_row;   // [n]
  const float *norm_idx;   // indexed by ref (only valid when references are plain local indices)
  const float *act;        // nullable n x F activation for the relu/dropout gradient mask
  float act_scale;
  uint32_t n, F;
  uint32_t src_rows_hint;  // number of distinct rows the references can name (0 = unknown): sizes the panels
  uint32_t slot_bytes, copy_bytes, seg, grp_shift, fpad, panels, panel_floats;   // filled by launch_spmm_tma
  int l2_prefetch;
  uint32_t ring_prefetch;  // ring kernel: groups of rows prefetched into L2 beyond the ring
  uint32_t wait_ns;        // ring kernel: suspend-time hint of the copy-barrier wait (0: plain try_wait)
  int l2_hint;             // ring kernel: L2 eviction policy per copied row (Tuning::l2_hint)
  float keep_uses;         // rows read by at least this many edges of the launch are copied with evict-last
  int y_stream;            // ring kernel: streaming stores for y
  int balance;             // ring kernel: warps take shares of equal edge count (1) or equal row count (0)
  int out_vec;             // widest vector (floats) usable for y and act rows: 4, 2 or 1
};
bool tma_spmm_applicable(const float *x, size_t x_ld, uint32_t F);
int launch_spmm_tma(TmaSpmmArgs a, cudaStream_t stream);
int launch_gather_refs(const uint32_t *offs, const uint32_t *idx, uint32_t v, uint32_t e, const uint32_t *source,
                       const uint32_t *hashmap, bool feat_is_hit, const float *norm_idx, const float *norm_row,
                       uint32_t *ref, float *w, cudaStream_t stream);
int read_tma_error_flag(unsigned int *value);
int read_gather_error_flag(unsigned int *value);
int read_spmm_error_flag(unsigned int *value);
int read_loss_error_flag(unsigned int *value);
int reset_tma_error_flag();
int reset_tc_error_flag();
int reset_gather_error_flag();
int reset_loss_error_flag();
// nb_feature_gather with an output pitch; misses_only = 1 copies only the rows that have no cache slot (row i of the
// output belongs to source[i] either way); max_ctas > 0 caps the launch (the kernel strides over the rows).
int feature_gather_impl(float *d_x0, size_t x0_ld, int misses_only, const float *feat, size_t feat_ld,
                        const float *const *feat_shards, uint32_t num_shards, uint32_t shard_rows, const float *d_cache,
                        size_t cache_ld, const uint32_t *d_hashmap, const uint32_t *d_source, uint32_t n, uint32_t F,
                        void *stream, uint32_t max_ctas);
int read_tc_error_flag(unsigned int *value);
// ReLU followed by inverted dropout applied to a product C as it leaves the GEMM (what nb_relu_dropout does to C
// afterwards: element i takes word i & 3 of Philox4x32-10 at counter (i >> 2, layer, step, 1) under the seed).
// on == 0: nothing is applied.
struct ReluEpi {
  int on;
  float p, scale;
  uint32_t seed_lo, seed_hi, layer, step;
};
// `epi` (nullable) asks for ReLU + dropout in the epilogue; *applied says whether the kernel that ran could do it
// (tensor-core kernels with TMA operands, no split-K, N a multiple of 4) - if not, the caller runs nb_relu_dropout.
int gemm_tensor_core(nb_ws *ws, const float *d_a, int64_t lda, const float *d_b, int64_t ldb, float *d_c, int64_t M,
                     int64_t N, int64_t K, int trans_a, int trans_b, int mode, cudaStream_t stream,
                     const ReluEpi *epi = nullptr, bool *applied = nullptr);
int gemm_ld(nb_ws *ws, const float *d_a, int64_t lda, const float *d_b, int64_t ldb, float *d_c, int64_t M, int64_t N,
            int64_t K, int trans_a, int trans_b, cudaStream_t stream, const ReluEpi *epi = nullptr,
            bool *applied = nullptr);
bool gemm_uses_tensor_cores(int64_t M, int64_t N, int64_t K);
// nb_output_layer that forms the aggregate of the last block itself (dense.cu)
bool output_layer_can_aggregate(const float *d_x, size_t x_ld, uint32_t H, uint32_t C);
int output_layer_aggregating(nb_ws *ws, const float *d_x, size_t x_ld, const uint32_t *d_row_indices,
                             const uint32_t *d_column_offset, const float *d_src_norm, const float *d_dst_norm,
                             const float *d_w, const int64_t *d_label, const uint32_t *d_dst, uint32_t B, uint32_t H,
                             uint32_t C, int train, float *d_dw, float *d_dy, float *d_stats, void *stream);
bool tma_gemm_applicable(const float *d_a, int64_t lda, const float *d_b, int64_t ldb);
int gemm_tma_launch(const float *d_a, int64_t lda, const float *d_b, int64_t ldb, float *c, int64_t M, int64_t N,
                    int64_t K, int trans_a, int trans_b, int bn, int splits, int64_t k_per_split, int mode,
                    cudaStream_t stream, const ReluEpi *epi = nullptr);
int read_tma_gemm_error_flag(unsigned int *value);
int reset_tma_gemm_error_flag();
int sample_hop_impl(const uint64_t *d_graph_column_offset, const uint32_t *d_graph_row_indices, const uint32_t *d_dst,
                    uint32_t v, int fanout, const uint32_t *d_column_offset, uint64_t seed, uint32_t hop,
                    uint32_t *d_row_indices, uint32_t *bitmap, void *stream);
int block_build_impl(nb_ws *ws, uint32_t num_vertices, uint32_t *d_row_indices, const uint32_t *d_column_offset,
                     uint32_t v, uint32_t e, uint32_t *d_source, uint32_t *src_size, uint32_t *d_row_offset,
                     uint32_t *d_column_indices, float *d_src_norm, float *d_dst_norm, float *d_w_fwd, float *d_w_bwd,
                     uint32_t *marked, void *stream);
bool tma_rows_form_applicable(int64_t M, int64_t N, int64_t K);
int gemm_tma_rows_launch(const float *d_y, int64_t ldy, const float *d_w, int64_t ldw, float *c, int64_t M, int64_t N,
                         int64_t K, int mode, cudaStream_t stream, const ReluEpi *epi = nullptr);
int spmm_csc_fwd_gather_fused_ld(nb_ws *ws, const float *feat, size_t feat_ld, const float *d_cache, size_t cache_ld,
                                 const uint32_t *d_hashmap, const uint32_t *d_source, float *d_y, size_t y_ld,
                                 const uint32_t *d_row_indices, const uint32_t *d_column_offset,
                                 const float *d_src_norm, const float *d_dst_norm, uint32_t v, uint32_t s, uint32_t e,
                                 uint32_t F, void *stream, const float *d_stage, size_t stage_ld);

// Scoped mark/release so that a call's scratch is returned to the arena when it ends.
struct WsScope {
  nb_ws *ws;
  size_t mark;
  explicit WsScope(nb_ws *w) : ws(w), mark(w ? w->used : 0) {}
  ~WsScope() {
    if (ws) ws->used = mark;
  }
};

// Exclusive prefix sum of n uint32 values (d_in may equal d_out).  d_out has n+1 entries when
// write_total is true (d_out[n] = total).  Scratch from ws.
int exclusive_scan_u32(nb_ws *ws, const uint32_t *d_in, uint32_t *d_out, uint64_t n, bool write_total,
                       cudaStream_t stream);
// Same for 64-bit outputs from 32-bit inputs.
int exclusive_scan_u32_to_u64(nb_ws *ws, const uint32_t *d_in, uint64_t *d_out, uint64_t n,
                              bool write_total, cudaStream_t stream);
}  // namespace nb

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch (PDL) for the kernels of the training half of a step, which follow one another
// on one stream: a dependent kernel may be scheduled while its predecessor drains, and waits at
// griddepcontrol.wait — its first statement here, so nothing of the predecessor's output is read and none of its
// inputs overwritten before the predecessor has completed and flushed.  Every such kernel lets its own dependents
// go right afterwards.  Kernels launched without the attribute execute the two instructions as no-ops.
// ---------------------------------------------------------------------------------------------
namespace nb {

#if defined(__CUDACC__)
// Two IEEE fused multiply-adds in one instruction (sm_100 packed f32x2 arithmetic): d = a * b + c per element with
// a single rounding, exactly what __fmaf_rn gives for each element.
__device__ __forceinline__ float2 fma2_rn(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rb, {%4, %5};\n\t"
      "mov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}

__device__ __forceinline__ void pdl_enter() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  Args &&...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  unsigned n = 0;
  if (tuning().use_pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    n++;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif
}  // namespace nb
