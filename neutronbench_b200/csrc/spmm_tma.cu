// Aggregation with source rows staged through shared memory by the TMA unit (non-multicast
// cp.async.bulk global -> shared, completion on an mbarrier).
//
// Why: the gather side of the SpMM is a latency problem — a destination has only `fanout` source rows
// and the address of each row comes out of an index chain.  Loading rows into registers limits the
// bytes in flight per warp to what the register file can hold.  Here each warp owns a two-stage ring of
// SEG row slots in shared memory; the lanes issue one bulk copy per source row of the NEXT segment
// (no registers, no LSU instructions per element), then the warp accumulates the CURRENT segment from
// shared memory, edge after edge, in the same multiply-then-add order as every other path, so results
// stay bit-identical.  Per warp up to 2*SEG rows (about 24 KB) are in flight.
//
// Requirements checked by the host: row starts 16-byte aligned (base aligned, pitch a multiple of 4
// floats) and ceil(F/4)*16 bytes readable per row.  Rows flagged as misses (bit 31 of the row
// reference: features that live in pinned host memory with an arbitrary pitch) are copied by the lanes
// with ordinary loads into the same slot.
#include "common.cuh"

namespace nb {

constexpr int kTmaWarps = 8;
constexpr int kTmaStages = 2;
constexpr uint32_t kWaitLimit = 1u << 18;   // bounded spin on the mbarrier; then the error flag is set

__device__ unsigned int g_tma_spmm_error = 0;   // 1: an mbarrier wait gave up

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
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
// The same test with a suspend-time hint: the thread may sleep up to `ns` nanoseconds waiting for the phase instead of
// returning at once, so a waiting warp takes no issue slots from the warps that have rows to accumulate.
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// Non-multicast bulk copy, global -> this CTA's shared memory.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
// The same copy with an L2 eviction policy for the lines it brings in.
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
// Ask L2 to fetch a row ahead of the copy that will stage it (no shared memory is held meanwhile).
__device__ __forceinline__ void prefetch_l2(const void *src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// One warp's walk over its work items, cut into segments of at most `seg` edges.  An item is an
// (output row, column panel) pair; items are ordered panel-major and dealt round-robin to the warps.
// The offsets of the item after the current one are loaded when the current item is opened, so
// opening an item never waits.
struct SegIter {
  uint32_t row, panel;             // current item
  uint32_t ahead_row, ahead_panel; // the item after it
  uint32_t stride, n, panels;
  uint32_t pos, end;               // edge range still to emit for the current item
  uint32_t ahead_pos, ahead_end;   // offsets of the item after it, already requested
  bool fresh;                      // next segment is the first of its item
  __device__ void step(uint32_t &r, uint32_t &p) const {
    r += stride;
    while (r >= n && p < panels) { r -= n; p++; }
  }
  __device__ void prefetch(const uint32_t *__restrict__ offs) {
    if (ahead_panel < panels) { ahead_pos = __ldg(offs + ahead_row); ahead_end = __ldg(offs + ahead_row + 1); }
  }
  __device__ void start(const uint32_t *__restrict__ offs, uint32_t first, uint32_t stride_, uint32_t rows,
                        uint32_t panels_) {
    stride = stride_; n = rows; panels = panels_;
    ahead_row = first; ahead_panel = 0;
    while (ahead_row >= n && ahead_panel < panels) { ahead_row -= n; ahead_panel++; }
    ahead_pos = ahead_end = 0;
    prefetch(offs);
    advance(offs);
  }
  __device__ void advance(const uint32_t *__restrict__ offs) {
    row = ahead_row; panel = ahead_panel; pos = ahead_pos; end = ahead_end; fresh = true;
    step(ahead_row, ahead_panel);
    prefetch(offs);
  }
  __device__ bool done() const { return panel >= panels; }
};
struct Seg {
  uint32_t row, panel, begin, cnt;
  bool first, last, valid;
};
// Per-lane operands of one segment: the row reference and what is needed to form the edge weight.
struct Operands {
  uint32_t ref;
  float w_or_nidx;   // explicit weight, or the sqrt-degree factor of the indexed side
  float nrow;        // sqrt-degree factor of the output row (fused form)
};

template <int TILES, bool MASK>
__global__ void __launch_bounds__(kTmaWarps * 32, 1) spmm_tma_kernel(const TmaSpmmArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t stage_bytes = a.seg * a.slot_bytes;
  unsigned char *my_smem = smem_raw + (size_t)warp * kTmaStages * stage_bytes;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw + (size_t)kTmaWarps * kTmaStages * stage_bytes) +
                   warp * kTmaStages;
  const uint32_t bar0 = smem_u32(bars);
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < kTmaStages; s++) mbar_init(bar0 + 8 * s, 1);
  }
  fence_proxy_async();   // make the initialised barriers visible to the async proxy
  __syncwarp();

  // Work items are (panel, row) pairs, panel-major: all rows of column panel 0 come before panel 1,
  // so that the source rows touched by one panel stay resident in L2 between their uses.
  SegIter it;
  it.start(a.offs, blockIdx.x * kTmaWarps + warp, gridDim.x * kTmaWarps, a.n, a.panels);


  auto next_seg = [&]() -> Seg {
    Seg s{};
    s.valid = !it.done();
    if (!s.valid) return s;
    s.row = it.row;
    s.panel = it.panel;
    s.begin = it.pos;
    s.cnt = min(a.seg, it.end - it.pos);
    s.first = it.fresh;
    it.pos += s.cnt;
    it.fresh = false;
    s.last = it.pos >= it.end;
    if (s.last) it.advance(a.offs);
    return s;
  };

  // Request a segment's per-edge operands.  Nothing here waits: the values are first used when the
  // segment's copies are issued, one loop iteration later.
  auto load_operands = [&](const Seg &s) -> Operands {
    Operands o{0u, 0.0f, 0.0f};
    if (s.valid && lane < s.cnt) {
      const uint32_t j = s.begin + lane;
      o.ref = __ldg(a.ref + j);
      if (a.w) o.w_or_nidx = __ldg(a.w + j); else o.nrow = __ldg(a.norm_row + s.row);
    }
    return o;
  };

  // Issue the copies of one segment into `stage`.
  auto issue = [&](const Seg &s, uint32_t stage, Operands &o) {
    __syncwarp();   // every lane is done reading the slots that are about to be refilled
    const bool mine = lane < s.cnt;
    const bool miss = mine && (o.ref & 0x80000000u);
    const unsigned hit_mask = __ballot_sync(0xffffffffu, mine && !miss);
    const unsigned miss_mask = __ballot_sync(0xffffffffu, miss);
    const uint32_t bar = bar0 + 8 * stage;
    unsigned char *stage_base = my_smem + (size_t)stage * stage_bytes;
    const uint32_t col0 = s.panel * a.panel_floats;                       // first column of this panel
    const uint32_t pbytes = min(a.copy_bytes, (a.fpad - col0) * 4u);    // bytes of one row inside the panel
    // Slots of this stage were read with ordinary loads (and possibly written by the miss path) two
    // segments ago; order those accesses before the async-proxy writes that follow.
    fence_proxy_async();
    if (lane == 0) mbar_arrive_expect_tx(bar, __popc(hit_mask) * pbytes);
    __syncwarp();
    if (mine && !miss)
      bulk_g2s(smem_u32(stage_base + (size_t)lane * a.slot_bytes), a.x + (size_t)o.ref * a.x_ld + col0, pbytes, bar);
    if (mine && !a.w) o.w_or_nidx = __ldg(a.norm_idx + o.ref);   // consumed one iteration later
    // misses: the whole warp copies each flagged row with plain loads (any pitch, any alignment)
    unsigned mm = miss_mask;
    while (mm) {
      const int u = __ffs(mm) - 1;
      mm &= mm - 1;
      const uint32_t id = __shfl_sync(0xffffffffu, o.ref, u) & 0x7FFFFFFFu;
      float *dst = reinterpret_cast<float *>(stage_base + (size_t)u * a.slot_bytes);
      const uint32_t width = min(a.panel_floats, a.F - col0);
      if (a.miss) {
        const float *src = a.miss + (size_t)id * a.miss_ld + col0;
        for (uint32_t c = lane; c < width; c += 32) dst[c] = __ldg(src + c);
      } else {                      // no table to read the row from: zeros, reported through the error word
        for (uint32_t c = lane; c < width; c += 32) dst[c] = 0.0f;
        if (lane == 0) atomicOr(&g_tma_spmm_error, 2u);
      }
    }
  };

  // L2 prefetch of a segment's rows: issued two iterations before the rows are staged, so that the
  // DRAM latency is paid while the rows do not yet occupy a shared-memory slot.
  auto prefetch = [&](const Seg &s, const Operands &o) {
    if (!s.valid || lane >= s.cnt || (o.ref & 0x80000000u)) return;
    const uint32_t col0 = s.panel * a.panel_floats;
    prefetch_l2(a.x + (size_t)o.ref * a.x_ld + col0, min(a.copy_bytes, (a.fpad - col0) * 4u));
  };

  // Software pipeline over this warp's segments:
  //   cur  copies in flight into shared memory, consumed in this iteration
  //   nxt  operands arrived an iteration ago, copies issued now
  //   far  operands requested now
  Seg cur = next_seg();
  Operands o_cur = load_operands(cur);
  Seg nxt = next_seg();
  Operands o_nxt = load_operands(nxt);
  if (cur.valid) issue(cur, 0, o_cur);
  float acc[TILES][4];
  uint32_t k = 0;
  while (cur.valid) {
    const uint32_t stage = k & 1;
    if (nxt.valid) issue(nxt, stage ^ 1, o_nxt);
    Seg far = next_seg();
    Operands o_far = load_operands(far);
    if (a.l2_prefetch) prefetch(far, o_far);

    // wait for the current segment's rows (bounded)
    {
      const uint32_t bar = bar0 + 8 * stage, parity = (k >> 1) & 1;
      uint32_t spins = 0;
      while (!mbar_try_wait(bar, parity)) {
        if (++spins > kWaitLimit) {
          if (lane == 0) atomicOr(&g_tma_spmm_error, 1u);
          // give copies that may still be in flight a second, equally bounded, chance to land
          for (uint32_t t = 0; t < kWaitLimit && !mbar_try_wait(bar, parity); t++) {}
          return;
        }
      }
    }
    __syncwarp();   // also orders the miss path's shared-memory writes before the reads below

    if (cur.first) {
#pragma unroll
      for (int t = 0; t < TILES; t++)
#pragma unroll
        for (int c = 0; c < 4; c++) acc[t][c] = 0.0f;
    }
    // 1 / ((float)sqrt(out_deg[src]) * (float)sqrt(in_deg[dst])) in the fused form
    const float w_cur = a.w ? o_cur.w_or_nidx : __fdiv_rn(1.0f, __fmul_rn(o_cur.w_or_nidx, o_cur.nrow));
    const unsigned char *stage_base = my_smem + (size_t)stage * stage_bytes;
    const uint32_t pcol0 = cur.panel * a.panel_floats;
    const uint32_t pwidth = min(a.panel_floats, a.F - pcol0);           // valid floats of this panel
    for (uint32_t u = 0; u < cur.cnt; u++) {
      const float wu = __shfl_sync(0xffffffffu, w_cur, u);
      const float4 *row = reinterpret_cast<const float4 *>(stage_base + (size_t)u * a.slot_bytes);
#pragma unroll
      for (int t = 0; t < TILES; t++) {
        const uint32_t q = lane + 32 * t;           // float4 index inside the row
        if (q * 4 < pwidth) {
          const float4 v = row[q];
          acc[t][0] = __fmaf_rn(v.x, wu, acc[t][0]);
          acc[t][1] = __fmaf_rn(v.y, wu, acc[t][1]);
          acc[t][2] = __fmaf_rn(v.z, wu, acc[t][2]);
          acc[t][3] = __fmaf_rn(v.w, wu, acc[t][3]);
        }
      }
    }
    if (cur.last) {
      const uint32_t out_row = cur.row;
      float *out = a.y + (size_t)out_row * a.y_ld + pcol0;
      const float *act = MASK ? a.act + (size_t)out_row * a.F + pcol0 : nullptr;
#pragma unroll
      for (int t = 0; t < TILES; t++) {
        const uint32_t col = (lane + 32 * t) * 4;
        if (col >= pwidth) continue;
        float r[4] = {acc[t][0], acc[t][1], acc[t][2], acc[t][3]};
        if (a.out_vec == 4) {
          if constexpr (MASK) {
            const float4 m = __ldg(reinterpret_cast<const float4 *>(act + col));
            r[0] = m.x > 0.0f ? __fmul_rn(r[0], a.act_scale) : 0.0f;
            r[1] = m.y > 0.0f ? __fmul_rn(r[1], a.act_scale) : 0.0f;
            r[2] = m.z > 0.0f ? __fmul_rn(r[2], a.act_scale) : 0.0f;
            r[3] = m.w > 0.0f ? __fmul_rn(r[3], a.act_scale) : 0.0f;
          }
          *reinterpret_cast<float4 *>(out + col) = make_float4(r[0], r[1], r[2], r[3]);
        } else {
#pragma unroll
          for (int c = 0; c < 4; c++) {
            if (col + c < pwidth) {
              float val = r[c];
              if constexpr (MASK) val = __ldg(act + col + c) > 0.0f ? __fmul_rn(val, a.act_scale) : 0.0f;
              if (a.out_vec != 2) out[col + c] = val;
              r[c] = val;
            }
          }
          if (a.out_vec == 2) {   // F is even and rows are 8-byte aligned
            if (col + 1 < pwidth) *reinterpret_cast<float2 *>(out + col) = make_float2(r[0], r[1]);
            if (col + 3 < pwidth) *reinterpret_cast<float2 *>(out + col + 2) = make_float2(r[2], r[3]);
          }
        }
      }
    }
    cur = nxt;
    o_cur = o_nxt;
    nxt = far;
    o_nxt = o_far;
    k++;
  }
}

// ---------------------------------------------------------------------------------------------
// Ring variant: a warp owns a CONTIGUOUS range of output rows, hence a contiguous range of edges,
// and streams those edges through a ring of row slots in shared memory.  The slots form R groups of G
// (1 or 2) rows with one mbarrier per group: the warp waits once per group, accumulates its rows in edge
// order and refills the group with the edges R groups ahead (lane u issues the u-th copy), so R - 1
// groups are in flight at any time.  Measured on the 2.4 KB rows of the Reddit-shaped layer-0 block:
// the time per row and warp is set by this wait-accumulate-refill chain, not by the depth of the ring,
// so pairs of rows per wait and 20 warps per CTA (about 10.8 KB of slots each) beat deeper rings.
// Arithmetic and order are those of every other path.
// ---------------------------------------------------------------------------------------------
constexpr int kRingWarps = 20;      // default warps per CTA; 22 and 24 are built as well (Tuning::ring_warps)
constexpr uint32_t kRingSmemMax = 227 * 1024;   // dynamic shared memory one CTA can have

template <int TILES, bool MASK, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 1) spmm_ring_kernel(const TmaSpmmArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  pdl_enter();
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t R = a.seg;                                   // groups per warp, one barrier each
  const uint32_t Gs = a.grp_shift, G = 1u << Gs;              // row slots per group
  unsigned char *my_smem = smem_raw + (size_t)warp * R * G * a.slot_bytes;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw + (size_t)WARPS * R * G * a.slot_bytes) + warp * R;
  const uint32_t bar0 = smem_u32(bars);
  if (lane < R) mbar_init(bar0 + 8 * lane, 1);
  fence_proxy_async();
  __syncwarp();

  // rows of this warp: a contiguous share; shares differ by at most one row and the longer ones are spread over all
  // CTAs, so that every SM has the same amount of work
  const uint32_t total_warps = gridDim.x * WARPS;
  const uint32_t gw = blockIdx.x * WARPS + warp;
  uint32_t r_begin, r_end, j0, j1;
  if (a.balance) {
    // Option: shares of equal EDGE count, cut at row boundaries: share p starts at the first row whose offset reaches
    // p * E / total_warps (rows differ in length, 1 .. fanout edges, so equal row counts give warps unequal byte
    // counts); a row still belongs to one warp, which adds its edges in order.  Both ends are found together by a
    // 32-ary search over the offsets (3 rounds for 20 K rows).  Measured on the Reddit-shaped layer-0 block it is
    // 1-1.5 us SLOWER than equal row counts (67.7 vs 66.0 us in the training step): the kernel runs at the DRAM
    // throughput this access pattern allows, which all SMs share, so a warp that ends early leaves its bandwidth to
    // the others, while the search delays every warp's first copy.  Hence off by default.
    const uint32_t E = __ldg(a.offs + a.n);
    const uint32_t tgt0 = (uint32_t)((uint64_t)gw * E / total_warps);
    const uint32_t tgt1 = (uint32_t)((uint64_t)(gw + 1) * E / total_warps);
    // smallest r in [0, n] with offs[r] >= target; lo = last row known to be below (-1: none), hi = known at/above
    int lo0 = -1, lo1 = -1;
    uint32_t hi0 = a.n, hi1 = a.n, v0 = E, v1 = E;              // v = offs[hi]
    while ((int)hi0 - lo0 > 1 || (int)hi1 - lo1 > 1) {
      const uint32_t st0 = ((uint32_t)((int)hi0 - lo0) + 31u) / 32u, st1 = ((uint32_t)((int)hi1 - lo1) + 31u) / 32u;
      const uint32_t p0 = min((uint32_t)(lo0 + (int)((lane + 1) * st0)), hi0);
      const uint32_t p1 = min((uint32_t)(lo1 + (int)((lane + 1) * st1)), hi1);
      const uint32_t o0 = __ldg(a.offs + p0), o1 = __ldg(a.offs + p1);
      const int f0 = __ffs(__ballot_sync(0xffffffffu, o0 >= tgt0)) - 1;   // lane 31 probes hi: always set
      const int f1 = __ffs(__ballot_sync(0xffffffffu, o1 >= tgt1)) - 1;
      const uint32_t nh0 = __shfl_sync(0xffffffffu, p0, f0), nh1 = __shfl_sync(0xffffffffu, p1, f1);
      const uint32_t nv0 = __shfl_sync(0xffffffffu, o0, f0), nv1 = __shfl_sync(0xffffffffu, o1, f1);
      const uint32_t pl0 = __shfl_sync(0xffffffffu, p0, f0 > 0 ? f0 - 1 : 0);
      const uint32_t pl1 = __shfl_sync(0xffffffffu, p1, f1 > 0 ? f1 - 1 : 0);
      if (f0 > 0) lo0 = (int)pl0;
      if (f1 > 0) lo1 = (int)pl1;
      hi0 = nh0; v0 = nv0; hi1 = nh1; v1 = nv1;
    }
    r_begin = gw == 0 ? 0u : hi0;                               // target 0 is reached by row 0
    r_end = gw + 1 == total_warps ? a.n : hi1;                  // trailing rows without edges go to the last share
    if (r_begin >= r_end) return;
    j0 = gw == 0 ? 0u : v0;
    j1 = gw + 1 == total_warps ? E : v1;
  } else {
    r_begin = (uint32_t)((uint64_t)gw * a.n / total_warps);
    r_end = (uint32_t)((uint64_t)(gw + 1) * a.n / total_warps);
    if (r_begin >= r_end) return;
    j0 = __ldg(a.offs + r_begin);
    j1 = __ldg(a.offs + r_end);
  }

  // operand windows of 32 edges aligned to j0: `cur` holds the window being consumed, `nxt` the next
  // Reference and weight (or, without explicit weights, the degree factor of the indexed side) of edge wbase + lane.
  // In the gather form the reference is the cache slot of the edge's source (bit 31 set + global id when the source
  // is not cached and rows come from `miss`; the plain global id when there is no cache at all).
  // row bookkeeping: lane holds the end offset of row rw_base + lane
  uint32_t rw_base = r_begin;
  uint32_t rend = (rw_base + lane < r_end) ? __ldg(a.offs + rw_base + lane + 1) : j1;

  // Operands of edge wbase + lane, requested one window (32 edges) ahead of their use; nothing here waits for a load.
  // `f` receives the degree factor of the indexed side (its square is the number of edges of this launch that read
  // the row) and, with fused weights, `nr` the factor of the edge's output row; with explicit weights `nr` is the
  // weight itself.  The output row of an edge is found without touching memory: it is rw_base + the number of held
  // row ends at or before the edge (a search over the offsets only for an edge beyond the 32 rows a warp holds).
  // finish_weight() then forms 1 / (f * nr) once per edge, when the window becomes the current one, instead of every
  // lane of the warp repeating that division when the edge is consumed.
  auto load_edge = [&](uint32_t wbase, uint32_t &ref, float &f, float &nr) {
    const uint32_t j = wbase + lane;
    const bool valid = j < j1;
    ref = 0u; nr = 0.0f; f = 0.0f;
    uint32_t li = 0;
    if (valid) {
      if (a.gidx) {
        li = __ldg(a.gidx + j);
        const uint32_t g = __ldg(a.gsource + li);
        const uint32_t slot = a.ghashmap ? __ldg(a.ghashmap + g) : 0xFFFFFFFFu;
        // not cached: row g of the table `miss`, or row li of a staging table that holds one row per source
        ref = slot != 0xFFFFFFFFu ? slot : (a.ghashmap ? ((a.miss_local ? li : g) | 0x80000000u) : g);
        f = __ldg(a.norm_idx + li);
      } else {
        ref = __ldg(a.ref + j);
        if (a.w) nr = __ldg(a.w + j);
        else f = __ldg(a.norm_idx + ref);                      // fused form: factor of the indexed side
      }
    }
    if (a.w) return;                                           // uniform over the warp
    uint32_t cnt = 0;
#pragma unroll
    for (int k = 0; k < 32; k++) cnt += __shfl_sync(0xffffffffu, rend, k) <= j ? 1u : 0u;
    uint32_t rr = rw_base + cnt;
    if (valid && cnt >= 32) {                                  // beyond the rows held in `rend`: search the offsets
      uint32_t lo = rw_base + 31, hi = r_end;                  // the last row of this warp that starts at or before j
      while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (__ldg(a.offs + mid) <= j) lo = mid; else hi = mid;
      }
      rr = lo;
    }
    if (valid) nr = __ldg(a.norm_row + rr);
  };
  auto finish_weight = [&](float f, float nr) -> float {       // 1 / (sqrt(deg_src) * sqrt(deg_dst)); 0 past the end
    if (a.w) return nr;
    return (f != 0.0f) ? __fdiv_rn(1.0f, __fmul_rn(f, nr)) : 0.0f;
  };
  uint32_t win = j0;                                          // base of the consume window
  uint32_t ref_cur, ref_nxt;
  float w_cur, f_cur, f_nxt, nr_nxt;
  {
    float nr_cur;
    load_edge(win, ref_cur, f_cur, nr_cur);
    w_cur = finish_weight(f_cur, nr_cur);
  }
  load_edge(win + 32, ref_nxt, f_nxt, nr_nxt);
  // L2 policy per copied row.  With fused weights the lane's factor is (float)sqrt(number of edges that use the
  // row in this block), so a factor of exactly 1 marks a row that no other edge of the launch will read: it is
  // copied with the evict-first policy and leaves L2 to the rows that are read again.
  // Rows that at least keep_uses edges read (factor^2 = number of uses) are kept with the evict-last policy.  The
  // factor is looked at when the copy is issued, not when it is loaded, so that nothing waits for the window's loads.
  const bool hints = a.l2_hint != 0 && a.w == nullptr;
  const uint64_t pol_first = policy_evict_first(), pol_last = policy_evict_last();

  // Issue the copies of group `gi` (edges j0 + gi*G .. of this warp) into the group's slots `gs`; executed by the
  // whole warp.  Lane u takes the group's u-th edge.  The references come from the two operand windows, which cover
  // every edge up to R*G ahead of the one being consumed (R*G <= 32).
  const uint32_t n_edges = j1 - j0;
  auto issue_group = [&](uint32_t gi, uint32_t gs) {
    const uint32_t t = (gi << Gs) + lane;                     // this lane's edge, relative to j0
    const uint32_t cnt = min(G, n_edges - (gi << Gs));
    const uint32_t rc = __shfl_sync(0xffffffffu, ref_cur, t & 31), rn = __shfl_sync(0xffffffffu, ref_nxt, t & 31);
    const bool in_cur = j0 + t < win + 32;
    const uint32_t ref = in_cur ? rc : rn;
    const float fc = __shfl_sync(0xffffffffu, f_cur, t & 31), fn = __shfl_sync(0xffffffffu, f_nxt, t & 31);
    const float fe = in_cur ? fc : fn;
    const bool once = hints && fe == 1.0f;
    const bool keep = hints && __fmul_rn(fe, fe) >= a.keep_uses;
    const bool mine = lane < cnt;
    const uint32_t bar = bar0 + 8 * gs;
    unsigned char *dst0 = my_smem + (size_t)(gs << Gs) * a.slot_bytes;
    const bool is_miss = (ref & 0x80000000u) != 0;
    // Rows that are not cached: copied by the TMA unit like the hits when they sit in an aligned staging table
    // (miss_bulk), else by the lanes (any pitch, any alignment: a table in mapped host memory).
    const unsigned miss_mask = a.miss_bulk ? 0u : __ballot_sync(0xffffffffu, mine && is_miss);
    unsigned mm = miss_mask;
    while (mm) {
      const int u = __ffs(mm) - 1;
      mm &= mm - 1;
      const uint32_t id = __shfl_sync(0xffffffffu, ref, u) & 0x7FFFFFFFu;
      float *dst = reinterpret_cast<float *>(dst0 + (size_t)u * a.slot_bytes);
      if (a.miss) {
        const float *src = a.miss + (size_t)id * a.miss_ld;
        for (uint32_t c = lane; c < a.F; c += 32) dst[c] = __ldg(src + c);
      } else {                      // no table to read the row from: contributes zeros, reported through the error word
        for (uint32_t c = lane; c < a.F; c += 32) dst[c] = 0.0f;
        if (lane == 0) atomicOr(&g_tma_spmm_error, 2u);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive_expect_tx(bar, a.copy_bytes * (cnt - __popc(miss_mask)));   // the group's one arrival
    __syncwarp();
    if (mine && (a.miss_bulk || !is_miss)) {
      const uint32_t dst = smem_u32(dst0 + (size_t)lane * a.slot_bytes);
      const float *src = is_miss ? a.miss + (size_t)(ref & 0x7FFFFFFFu) * a.miss_ld : a.x + (size_t)ref * a.x_ld;
      if (once) bulk_g2s_hint(dst, src, a.copy_bytes, bar, pol_first);
      else if (keep) bulk_g2s_hint(dst, src, a.copy_bytes, bar, pol_last);
      else bulk_g2s(dst, src, a.copy_bytes, bar);
    }
  };

  // L2 prefetch of group `gi` (a.ring_prefetch groups beyond the ring): the rows start their way from DRAM while they
  // hold no shared-memory slot yet, so a warp has ring + prefetch rows in flight instead of the ring's few.  Needs the
  // group's references in the two operand windows: callers keep (R + ring_prefetch + 1) * G <= 32.
  auto prefetch_group = [&](uint32_t gi) {
    if ((gi << Gs) >= n_edges) return;                         // uniform over the warp
    const uint32_t t = (gi << Gs) + lane;
    const uint32_t cnt = min(G, n_edges - (gi << Gs));
    const uint32_t rc = __shfl_sync(0xffffffffu, ref_cur, t & 31), rn = __shfl_sync(0xffffffffu, ref_nxt, t & 31);
    const uint32_t ref = (j0 + t < win + 32) ? rc : rn;
    if (lane < cnt && j0 + t < win + 64) {
      const bool is_miss = (ref & 0x80000000u) != 0;
      if (!is_miss) prefetch_l2(a.x + (size_t)ref * a.x_ld, a.copy_bytes);
      else if (a.miss_bulk) prefetch_l2(a.miss + (size_t)(ref & 0x7FFFFFFFu) * a.miss_ld, a.copy_bytes);
    }
  };
  const uint32_t PF = a.ring_prefetch;

  // prologue: fill the ring
  for (uint32_t gi = 0; gi < R && (gi << Gs) < n_edges; gi++) issue_group(gi, gi);
  for (uint32_t gi = R; gi < R + PF; gi++) prefetch_group(gi);

  uint32_t row = r_begin;
  uint32_t row_end = __shfl_sync(0xffffffffu, rend, 0);
  // two packed pairs per float4 column: one packed fused multiply-add covers two elements
  float2 acc[TILES][2];
#pragma unroll
  for (int t = 0; t < TILES; t++) acc[t][0] = acc[t][1] = make_float2(0.0f, 0.0f);

  auto finish_row = [&]() {      // write the accumulated row, move to the next one
    float *out = a.y + (size_t)row * a.y_ld;
    const float *act = MASK ? a.act + (size_t)row * a.F : nullptr;
#pragma unroll
    for (int t = 0; t < TILES; t++) {
      const uint32_t col = (lane + 32 * t) * 4;
      if (col < a.F) {
        float r[4] = {acc[t][0].x, acc[t][0].y, acc[t][1].x, acc[t][1].y};
#pragma unroll
        for (int c = 0; c < 4; c++) {
          if (col + c < a.F) {
            if constexpr (MASK) r[c] = __ldg(act + col + c) > 0.0f ? __fmul_rn(r[c], a.act_scale) : 0.0f;
          }
        }
        // streaming stores: the output is consumed by a later kernel that streams it once; keeping it out of the
        // way leaves L2 to the source rows, which are re-read by other destinations
        if (a.out_vec == 4) {
          if (a.y_stream) __stcs(reinterpret_cast<float4 *>(out + col), make_float4(r[0], r[1], r[2], r[3]));
          else *reinterpret_cast<float4 *>(out + col) = make_float4(r[0], r[1], r[2], r[3]);
        } else if (a.out_vec == 2) {
          if (col + 1 < a.F) __stcs(reinterpret_cast<float2 *>(out + col), make_float2(r[0], r[1]));
          if (col + 3 < a.F) __stcs(reinterpret_cast<float2 *>(out + col + 2), make_float2(r[2], r[3]));
        } else {
#pragma unroll
          for (int c = 0; c < 4; c++)
            if (col + c < a.F) __stcs(out + col + c, r[c]);
        }
      }
      acc[t][0] = acc[t][1] = make_float2(0.0f, 0.0f);
    }
    row++;
    if (row < r_end) {
      if (row - rw_base >= 32) {
        rw_base = row;
        rend = (rw_base + lane < r_end) ? __ldg(a.offs + rw_base + lane + 1) : j1;
      }
      row_end = __shfl_sync(0xffffffffu, rend, row - rw_base);
    }
  };

  uint32_t cur_gs = 0, cur_parity = 0;                        // ring position and phase of the group being consumed
  for (uint32_t j = j0; j < j1; j++) {
    while (j == row_end && row < r_end) finish_row();        // rows without (more) edges
    if (j - win >= 32) {                                      // consume window moves on; fetch the one after
      win += 32;
      ref_cur = ref_nxt; w_cur = finish_weight(f_nxt, nr_nxt); f_cur = f_nxt;
      load_edge(win + 32, ref_nxt, f_nxt, nr_nxt);
    }
    const uint32_t t = j - j0, in_group = t & (G - 1);
    if (in_group == 0) {                                      // first edge of a group: wait for the group's copies
      if (t != 0 && ++cur_gs == R) { cur_gs = 0; cur_parity ^= 1u; }
      const uint32_t bar = bar0 + 8 * cur_gs;
      uint32_t spins = 0;
      while (!(a.wait_ns ? mbar_try_wait_hint(bar, cur_parity, a.wait_ns) : mbar_try_wait(bar, cur_parity))) {
        if (++spins > kWaitLimit) {
          if (lane == 0) atomicOr(&g_tma_spmm_error, 1u);
          for (uint32_t k = 0; k < kWaitLimit && !mbar_try_wait(bar, cur_parity); k++) {}
          return;
        }
      }
    }
    __syncwarp();
    const float wu = __shfl_sync(0xffffffffu, w_cur, t & 31);   // the edge's weight, formed when its window was loaded
    const float4 *rowp =
        reinterpret_cast<const float4 *>(my_smem + (size_t)((cur_gs << Gs) + in_group) * a.slot_bytes);
    const float2 wu2 = make_float2(wu, wu);
#pragma unroll
    for (int tl = 0; tl < TILES; tl++) {
      const uint32_t q = lane + 32 * tl;
      if (q * 4 < a.F) {
        const float4 v = rowp[q];
        acc[tl][0] = fma2_rn(make_float2(v.x, v.y), wu2, acc[tl][0]);
        acc[tl][1] = fma2_rn(make_float2(v.z, v.w), wu2, acc[tl][1]);
      }
    }
    // last edge of the group: its slots are free, refill them with the group R groups ahead
    if ((in_group == G - 1 || j + 1 == j1) && (((t >> Gs) + R) << Gs) < n_edges) {
      __syncwarp();            // every lane has read the slots
      fence_proxy_async();     // order those reads before the async-proxy refill
      issue_group((t >> Gs) + R, cur_gs);
      if (PF) prefetch_group((t >> Gs) + R + PF);
    }
  }
  while (row < r_end) finish_row();
}

// ref[j] / w[j] for the gather-fused form: the row reference of edge j is the cache slot of its source
// (or the global id with bit 31 set when the source is not cached), the weight is the GCN weight.
__global__ void gather_refs_kernel(const uint32_t *__restrict__ offs, const uint32_t *__restrict__ idx, uint32_t v,
                                   uint32_t e, const uint32_t *__restrict__ source,
                                   const uint32_t *__restrict__ hashmap, bool feat_is_hit,
                                   const float *__restrict__ norm_idx, const float *__restrict__ norm_row,
                                   uint32_t *__restrict__ ref, float *__restrict__ w) {
  for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < e; j += (uint64_t)gridDim.x * blockDim.x) {
    const uint32_t li = idx[j];
    const uint32_t g = source[li];
    const uint32_t slot = hashmap ? hashmap[g] : 0xFFFFFFFFu;
    ref[j] = slot != 0xFFFFFFFFu ? slot : (feat_is_hit ? g : (g | 0x80000000u));
    uint32_t lo = 0, hi = v;
    while (hi - lo > 1) {
      const uint32_t mid = (lo + hi) >> 1;
      if (offs[mid] <= (uint32_t)j) lo = mid; else hi = mid;
    }
    w[j] = __fdiv_rn(1.0f, __fmul_rn(norm_idx[li], norm_row[lo]));
  }
}

template <int TILES, bool MASK>
static int launch_tiles(const TmaSpmmArgs &a, size_t smem, cudaStream_t stream) {
  static PerDeviceOnce configured;   // the attribute is kept per device
  if (configured.need()) {
    NB_CUDA(cudaFuncSetAttribute(spmm_tma_kernel<TILES, MASK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 200 * 1024));
    configured.done();
  }
  const unsigned need = (unsigned)(((uint64_t)a.n * a.panels + kTmaWarps - 1) / kTmaWarps);
  const unsigned grid = need < (unsigned)num_sms() ? need : (unsigned)num_sms();
  spmm_tma_kernel<TILES, MASK><<<grid, kTmaWarps * 32, smem, stream>>>(a);
  NB_LAUNCH_CHECK();
  return 0;
}

template <int TILES, bool MASK, int WARPS>
static int launch_ring_tiles(const TmaSpmmArgs &a, size_t smem, cudaStream_t stream) {
  static PerDeviceOnce configured;   // the attribute is kept per device
  if (configured.need()) {
    NB_CUDA(cudaFuncSetAttribute(spmm_ring_kernel<TILES, MASK, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 227 * 1024));
    configured.done();
  }
  // enough CTAs that every warp gets at least a few rows, at most one CTA per SM
  const unsigned want = (a.n + WARPS * 4 - 1) / (WARPS * 4);
  // one CTA per SM; SMs held by a kernel that runs beside this one (a gradient all-reduce on another stream) would
  // make their CTAs wait for a second wave, so the caller can keep a few SMs out of the grid
  const int reserve = tuning().reserve_sms > 0 ? tuning().reserve_sms : 0;
  const unsigned sms = (unsigned)(num_sms() > reserve + 1 ? num_sms() - reserve : 1);
  const unsigned grid = want < sms ? (want ? want : 1) : sms;
  NB_CUDA(launch_chained(spmm_ring_kernel<TILES, MASK, WARPS>, dim3(grid), dim3(WARPS * 32), smem, stream, a));
  NB_LAUNCH_CHECK();
  return 0;
}

template <bool MASK, int WARPS>
static int launch_ring_w(const TmaSpmmArgs &a, size_t smem, cudaStream_t stream) {
  switch ((a.F + 127) / 128) {
    case 1: return launch_ring_tiles<1, MASK, WARPS>(a, smem, stream);
    case 2: return launch_ring_tiles<2, MASK, WARPS>(a, smem, stream);
    case 3: return launch_ring_tiles<3, MASK, WARPS>(a, smem, stream);
    case 4: return launch_ring_tiles<4, MASK, WARPS>(a, smem, stream);
    case 5: return launch_ring_tiles<5, MASK, WARPS>(a, smem, stream);
    case 6: return launch_ring_tiles<6, MASK, WARPS>(a, smem, stream);
    case 7: return launch_ring_tiles<7, MASK, WARPS>(a, smem, stream);
    case 8: return launch_ring_tiles<8, MASK, WARPS>(a, smem, stream);
    default: return fail(NB_ERR_INVALID, "spmm (ring): feature width above 1024");
  }
}

template <bool MASK>
static int launch_ring(const TmaSpmmArgs &a, int warps, size_t smem, cudaStream_t stream) {
  switch (warps) {
    case 24: return launch_ring_w<MASK, 24>(a, smem, stream);
    case 22: return launch_ring_w<MASK, 22>(a, smem, stream);
    default: return launch_ring_w<MASK, kRingWarps>(a, smem, stream);
  }
}

template <bool MASK>
static int launch_mask(const TmaSpmmArgs &a, size_t smem, cudaStream_t stream) {
  switch ((a.panel_floats + 127) / 128) {
    case 1: return launch_tiles<1, MASK>(a, smem, stream);
    case 2: return launch_tiles<2, MASK>(a, smem, stream);
    case 3: return launch_tiles<3, MASK>(a, smem, stream);
    case 4: return launch_tiles<4, MASK>(a, smem, stream);
    case 5: return launch_tiles<5, MASK>(a, smem, stream);
    case 6: return launch_tiles<6, MASK>(a, smem, stream);
    case 7: return launch_tiles<7, MASK>(a, smem, stream);
    case 8: return launch_tiles<8, MASK>(a, smem, stream);
    default: return fail(NB_ERR_INVALID, "spmm (staged): feature width above 1024");
  }
}

// Staging pays off for wide rows (one bulk copy moves a kilobyte or more); narrow rows are faster with
// direct vector loads at high occupancy (measured on B200: F = 100..128 direct, F = 602 staged).
bool tma_spmm_applicable(const float *x, size_t x_ld, uint32_t F) {
  if (x == nullptr || F < (uint32_t)tuning().staged_min_width || F > 1024) return false;
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || (x_ld & 3) != 0) return false;
  return (size_t)((F + 3) / 4) * 4 <= x_ld;   // the 16-byte-granular copy stays inside the row pitch
}

int launch_spmm_tma(TmaSpmmArgs a, cudaStream_t stream) {
  if (a.n == 0) return 0;
  a.fpad = ((a.F + 3) / 4) * 4;
  if (a.y_ld == 0) a.y_ld = a.F;
  a.l2_prefetch = tuning().l2_prefetch;
  a.l2_hint = tuning().l2_hint;
  a.ring_prefetch = 0;
  a.wait_ns = (uint32_t)(tuning().ring_wait_ns > 0 ? tuning().ring_wait_ns : 0);
  a.keep_uses = a.l2_hint == 2 ? 1.5f : (a.l2_hint == 3 ? (float)tuning().l2_keep_min_uses - 0.5f : 3.0e38f);
  a.y_stream = tuning().y_stream_stores;
  a.balance = tuning().ring_balance;
  // Column panels: when the distinct source rows of the block exceed what L2 keeps, the row is cut
  // into panels whose working set fits, and panels are processed one after the other.
  uint32_t panels = 1;
  if (a.src_rows_hint > 0 && tuning().l2_panel_bytes > 0) {
    const uint64_t working_set = (uint64_t)a.src_rows_hint * a.fpad * 4;
    panels = (uint32_t)((working_set + tuning().l2_panel_bytes - 1) / tuning().l2_panel_bytes);
    const uint32_t max_panels = (a.fpad + 63) / 64;            // keep copies at 256 bytes or more
    if (panels > max_panels) panels = max_panels;
    if (panels < 1) panels = 1;
  }
  if (panels == 1 && tuning().spmm_ring) {
    // ring variant: whole rows, per-warp ring of R slots out of about 13.5 KB
    a.panels = 1; a.panel_floats = a.fpad; a.copy_bytes = a.fpad * 4; a.slot_bytes = a.copy_bytes;
    // the CTA's warps share its shared memory as row slots; more warps (22, 24) are taken only where each still gets
    // the four slots that two pairs in flight need
    auto slots_for = [&](int w) -> uint32_t {
      if (w == kRingWarps) return (216u * 1024u / (uint32_t)w) / a.slot_bytes;          // the measured default
      for (uint32_t sl = 16; sl >= 1; sl--) {
        const uint32_t groups = sl >= 4 ? sl >> tuning().ring_group_shift : sl;
        if ((uint64_t)w * ((uint64_t)sl * a.slot_bytes + groups * 8ull) <= kRingSmemMax) return sl;
      }
      return 0;
    };
    int warps = tuning().ring_warps == 22 || tuning().ring_warps == 24 ? tuning().ring_warps : kRingWarps;
    if (slots_for(warps) < 4) warps = kRingWarps;
    uint32_t slots = slots_for(warps);
    if (slots > 16) slots = 16;
    // two rows per barrier (one wait and one refill per pair of edges) where at least two pairs fit; measured on the
    // layer-0 block of the Reddit-shaped model: 78 us against 81 us with a barrier per row (65 against 75 from L2)
    const uint32_t shift = slots >= 4 ? tuning().ring_group_shift : 0;
    const uint32_t R = slots >> shift;                         // groups of 1 << shift slots
    if (R >= 2) {
      a.seg = R;
      a.grp_shift = shift;
      // groups prefetched into L2 beyond the ring, while their references are still inside the operand windows
      const uint32_t max_pf = (32u >> shift) > R + 1 ? (32u >> shift) - R - 1 : 0;
      a.ring_prefetch = (uint32_t)tuning().ring_prefetch < max_pf ? (uint32_t)tuning().ring_prefetch : max_pf;
      const size_t smem = (size_t)warps * (R << shift) * a.slot_bytes + (size_t)warps * R * sizeof(uint64_t);
      return a.act ? launch_ring<true>(a, warps, smem, stream) : launch_ring<false>(a, warps, smem, stream);
    }
  }
  if (a.ref == nullptr) return fail(NB_ERR_INVALID, "spmm (staged): the segment kernel needs per-edge references");
  a.panel_floats = ((a.fpad / 4 + panels - 1) / panels) * 4;   // multiple of 4 floats = 16 bytes
  a.panels = (a.fpad + a.panel_floats - 1) / a.panel_floats;
  a.copy_bytes = a.panel_floats * 4;
  a.slot_bytes = a.copy_bytes;
  const uint32_t per_warp_budget = 24 * 1024;   // two stages
  uint32_t seg = per_warp_budget / (kTmaStages * a.slot_bytes);
  if (seg < 1) seg = 1;
  if (seg > 32) seg = 32;
  a.seg = seg;
  const size_t smem = (size_t)kTmaWarps * kTmaStages * seg * a.slot_bytes + kTmaWarps * kTmaStages * sizeof(uint64_t);
  if (smem > 200 * 1024) return fail(NB_ERR_INVALID, "spmm (staged): row too wide for the shared-memory ring");
  if ((uint64_t)a.n * a.panels > 0xFFFFFFFFull) return fail(NB_ERR_INVALID, "spmm (staged): too many work items");
  return a.act ? launch_mask<true>(a, smem, stream) : launch_mask<false>(a, smem, stream);
}

int launch_gather_refs(const uint32_t *offs, const uint32_t *idx, uint32_t v, uint32_t e, const uint32_t *source,
                       const uint32_t *hashmap, bool feat_is_hit, const float *norm_idx, const float *norm_row,
                       uint32_t *ref, float *w, cudaStream_t stream) {
  if (e == 0) return 0;
  gather_refs_kernel<<<grid_for(e, 256), 256, 0, stream>>>(offs, idx, v, e, source, hashmap, feat_is_hit, norm_idx,
                                                          norm_row, ref, w);
  NB_LAUNCH_CHECK();
  return 0;
}

int read_tma_error_flag(unsigned int *value) {
  NB_CUDA(cudaMemcpyFromSymbol(value, g_tma_spmm_error, sizeof(unsigned int)));
  return 0;
}
int reset_tma_error_flag() {
  const unsigned int zero = 0;
  NB_CUDA(cudaMemcpyToSymbol(g_tma_spmm_error, &zero, sizeof(unsigned int)));
  return 0;
}

}  // namespace nb
