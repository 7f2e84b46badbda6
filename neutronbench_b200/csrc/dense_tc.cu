// fp32 GEMM on the 5th-generation tensor cores (tcgen05.mma, kind::tf32) with fp32-level accuracy.
//
//   C[M x N] = op(A) op(B)            NN (Y W), TN (Y^T dZ, split over the long reduction), NT (dZ W^T)
//
// Accuracy: every fp32 operand is split as x = hi + lo with hi = x truncated to TF32 (the tensor core
// drops the low 13 mantissa bits itself) and lo = x - hi (exact).  Three MMAs per K step accumulate
// hi*hi + hi*lo + lo*hi into the same fp32 TMEM accumulator; the dropped lo*lo term is below 2^-22 of
// the product.  mode 2 issues only hi*hi (plain TF32).
//
// This file: the kernel for operands that cannot have a TMA tensor map (pitch not a multiple of 16 bytes).  Raw
// fp32 tiles are copied global -> shared with cp.async in 4/8/16-byte pieces straight into the layouts the tensor
// core reads (see "Tile layouts" below), three to six stages deep; every staging thread then writes lo for exactly
// the pieces it copied (the raw words stay in place and serve as hi), fences them towards the tensor core's proxy
// and arrives on the stage's mbarrier; a separate warp issues tcgen05.mma from shared-memory descriptors; the
// accumulator lives in tensor memory and is read back with tcgen05.ld (a warp reaches its own 32 TMEM lanes).  A
// tcgen05.commit mbarrier per stage tells when the MMAs that read it have finished.  dense_tma.cu holds the TMA-fed
// kernels, which issue the same MMAs in the same order.
#include "common.cuh"
#include "tc_common.cuh"

namespace nb {

__device__ unsigned int g_tc_gemm_error = 0;

// Tile layouts in shared memory (floats).  A tile holds ROWS rows (M or N index) by kBK reduction elements.
//
//   K-major   (the operand is contiguous along K in global memory): no swizzle; core matrices of 8 rows x
//             4 k (16 bytes per row).  K-cores of a row group are 144 bytes apart (LBO), 8-row groups
//             kKCores*144 bytes (SBO).  The 16 bytes of padding per core put the pieces that consecutive
//             threads write on different banks.
//   MN-major  (the operand is contiguous along its row index: a transposed operand).  For kind::tf32 the
//             tensor core reads MN-major operands only in the "128-byte swizzle with 32-byte atoms" mode
//             (descriptor layout type 1): a line is 32 rows (128 bytes) of one k; four lines (k & 3) form
//             a 512-byte atom inside which the 32-byte quarter (row >> 3) & 3 of a line is stored at
//             quarter ^ (k & 3).  Atoms of consecutive k groups are SBO = 512 bytes apart, 32-row blocks
//             LBO = kBK/4 * 512 bytes.  Measured on the device with a selector matrix, not taken from a
//             manual.  A quarter-warp writes one whole 128-byte line, so there are no bank conflicts.
//
// Strides and the swizzle mode are descriptor fields, so the transposed operands need no transposition
// pass: rows are copied with 16-byte pieces along their contiguous direction either way.
constexpr uint32_t kCoreFloats = 36;                   // K-major: 128-byte core matrix + 16 bytes of padding
constexpr uint32_t kKCores = kBK / 4;                  // K-major core matrices along K per chunk
constexpr uint32_t kGroupFloats = kKCores * kCoreFloats;
constexpr uint32_t kMnAtomFloats = 128;                // MN-major: 4 k x 32 rows
constexpr uint32_t kMnBlockFloats = (kBK / 4) * kMnAtomFloats;   // one 32-row block of a chunk

template <bool MN>
__device__ __forceinline__ uint32_t tile_off(uint32_t r, uint32_t k) {
  if (MN)
    return (r >> 5) * kMnBlockFloats + (k >> 2) * kMnAtomFloats + (k & 3) * 32 + ((((r >> 3) & 3) ^ (k & 3)) << 3) + (r & 7);
  return (r >> 3) * kGroupFloats + (k >> 2) * kCoreFloats + (r & 7) * 4 + (k & 3);
}
// float offset of 16-byte piece q of a tile, q in [0, ROWS * kBK / 4): any order that covers the data
template <bool MN>
__device__ __forceinline__ uint32_t quad_off(uint32_t q) {
  if (MN) return q * 4;   // the MN-major tile is dense
  constexpr uint32_t PER_GROUP = 8 * kKCores;
  return (q / PER_GROUP) * kGroupFloats + ((q % PER_GROUP) >> 3) * kCoreFloats + (q & 7) * 4;
}
template <int ROWS>
struct TileFloats {   // the K-major tile is the larger of the two; rounded up to 1 KB so that every tile of a
                      // stage ring keeps the alignment the swizzle pattern is defined on
  static constexpr uint32_t value = (((ROWS / 8) * kGroupFloats) + 255) / 256 * 256;
};
template <bool MN> struct DescStride {};
template <> struct DescStride<false> {
  static constexpr uint32_t lbo = kCoreFloats * 4, sbo = kGroupFloats * 4, kstep = 2 * kCoreFloats * 4, layout = 0;
};
template <> struct DescStride<true> {
  static constexpr uint32_t lbo = kMnBlockFloats * 4, sbo = kMnAtomFloats * 4, kstep = 2 * kMnAtomFloats * 4, layout = 1;
};


template <int BYTES>
__device__ __forceinline__ void cp_async(uint32_t dst, const void *src, int valid) {
  // `valid` bytes are read, the rest of the BYTES-wide destination is zero-filled
  if (BYTES == 16)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(valid) : "memory");
  else if (BYTES == 8)
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(valid) : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(valid) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Per-thread copy plan of one operand.  A tile is moved in pieces of `vec` floats along the operand's
// contiguous direction; piece `item` = tid + i * T (T threads per CTA) of every chunk is the same (row, k) place, so
// the source pointer, the destination offsets and the bounds predicate are computed once and the main
// loop only advances the pointer.
//   K-major:  piece = item % (kBK/vec) along k, row = item / (kBK/vec)
//   MN-major: piece = item % (ROWS/vec) along the rows, k = item / (ROWS/vec)
// The pitch of a dense row-major operand equals its extent along the contiguous direction and is a
// multiple of `vec`, so a piece never straddles the matrix edge.
template <int ROWS, bool MN, int T>
struct CopyPlan {
  static constexpr int kMaxPieces = (ROWS * kBK) / T > 0 ? (ROWS * kBK) / T : 1;   // at vec = 1
  const float *src;        // this thread's first piece in chunk 0 (clamped into the matrix when out of range)
  int64_t step;            // elements between a thread's consecutive pieces
  int64_t chunk_step;      // elements between chunks
  uint32_t dst[kMaxPieces];   // byte offsets in the tile
  int vec, pieces, valid;  // valid: bit i set when piece i lies inside the matrix rows
  // for the bounds-checked tail chunk
  int64_t s_row, s_k, row0, rows_total;
  const float *base;

  __device__ void init(const float *base_, int64_t s_row_, int64_t s_k_, int64_t row0_, int64_t rows_total_,
                       int64_t k0, int vec_) {
    base = base_; s_row = s_row_; s_k = s_k_; row0 = row0_; rows_total = rows_total_; vec = vec_;
    const int tid = threadIdx.x;
    valid = 0;
    const int per_line = (MN ? ROWS : kBK) / vec;           // pieces along the contiguous direction
    const int total = (ROWS * kBK) / vec;
    pieces = total / T;
    if (pieces < 1) pieces = tid < total ? 1 : 0;
    const int piece = tid % per_line, line0 = tid / per_line;
    const int lstep = T / per_line > 0 ? T / per_line : 1;
    if (MN) {
      const int r = piece * vec;                            // row within the tile, k = line
      const bool row_ok = row0 + r < rows_total;
      src = base + (k0 + line0) * s_k + (row_ok ? row0 + r : 0);
      step = (int64_t)lstep * s_k;
#pragma unroll
      for (int i = 0; i < kMaxPieces; i++) {
        dst[i] = tile_off<true>(r, line0 + i * lstep) * 4;
        if (i < pieces && row_ok) valid |= 1 << i;
      }
    } else {
      const int k = piece * vec;                            // k within the chunk, row = line
      src = base + (row0 + line0) * s_row + k0 + k;
      step = (int64_t)lstep * s_row;
#pragma unroll
      for (int i = 0; i < kMaxPieces; i++) {
        const int r = line0 + i * lstep;
        dst[i] = tile_off<false>(r < ROWS ? r : 0, k) * 4;
        if (i < pieces && row0 + r < rows_total) valid |= 1 << i;
      }
    }
    chunk_step = (int64_t)kBK * s_k;
  }

  template <int VEC>
  __device__ __forceinline__ void issue_vec(uint32_t tile_s, const float *p) const {
    constexpr int N = kMaxPieces / VEC > 0 ? kMaxPieces / VEC : 1;   // pieces per thread at this width
#pragma unroll
    for (int i = 0; i < N; i++) {
      if (N > 1 || i < pieces) {
        const bool ok = (valid >> i) & 1;
        cp_async<VEC * 4>(tile_s + dst[i], ok ? p + (int64_t)i * step : base, ok ? VEC * 4 : 0);
      }
    }
  }
  // Copies of one full chunk (all kBK reduction elements inside the matrix); rows outside are zero-filled.
  __device__ __forceinline__ void issue(uint32_t tile_s, int chunk) const {
    const float *p = src + (int64_t)chunk * chunk_step;
    if (vec == 4) issue_vec<4>(tile_s, p);
    else if (vec == 2) issue_vec<2>(tile_s, p);
    else issue_vec<1>(tile_s, p);
  }
  // lo = raw - hi of exactly the pieces this thread copied (after its own cp.async.wait_group) into the same
  // offsets of `lo`; the raw words stay in place as hi.  No other thread's data is touched, so the staging
  // threads need no barrier among themselves.  Zero-filled pieces are processed too (lo must be zero there).
  template <int VEC>
  __device__ __forceinline__ void split_vec(unsigned char *raw, unsigned char *lo, bool split) const {
    constexpr int N = kMaxPieces / VEC > 0 ? kMaxPieces / VEC : 1;
#pragma unroll
    for (int i = 0; i < N; i++) {
      if (N > 1 || i < pieces) {
        float x[VEC], h[VEC], l[VEC];
        if (VEC == 4) *reinterpret_cast<float4 *>(x) = *reinterpret_cast<const float4 *>(raw + dst[i]);
        else if (VEC == 2) *reinterpret_cast<float2 *>(x) = *reinterpret_cast<const float2 *>(raw + dst[i]);
        else x[0] = *reinterpret_cast<const float *>(raw + dst[i]);
#pragma unroll
        for (int e = 0; e < VEC; e++) tc_split(x[e], h[e], l[e]);
        if (!split) continue;   // the raw words serve as hi: the tensor core ignores their low 13 mantissa bits
        if (VEC == 4) *reinterpret_cast<float4 *>(lo + dst[i]) = *reinterpret_cast<float4 *>(l);
        else if (VEC == 2) *reinterpret_cast<float2 *>(lo + dst[i]) = *reinterpret_cast<float2 *>(l);
        else *reinterpret_cast<float *>(lo + dst[i]) = l[0];
      }
    }
  }
  __device__ __forceinline__ void split_own(float *raw, float *lo, bool split) const {
    unsigned char *r = reinterpret_cast<unsigned char *>(raw), *l = reinterpret_cast<unsigned char *>(lo);
    if (vec == 4) split_vec<4>(r, l, split);
    else if (vec == 2) split_vec<2>(r, l, split);
    else split_vec<1>(r, l, split);
  }
  // The same for the tail chunk, whose elements were copied one by one by issue_tail.
  __device__ void split_tail(float *raw, float *lo, bool split) const {
    for (int item = threadIdx.x; item < ROWS * kBK; item += T) {
      const int r = MN ? item % ROWS : item / kBK, k = MN ? item / ROWS : item % kBK;
      const uint32_t off = tile_off<MN>(r, k);
      float h, l;
      tc_split(raw[off], h, l);
      if (split) lo[off] = l;
    }
  }
  // The one chunk with a K tail: element by element with bounds checks.
  __device__ void issue_tail(uint32_t tile_s, int64_t k0, int64_t k_end) const {
    for (int item = threadIdx.x; item < ROWS * kBK; item += T) {
      const int r = MN ? item % ROWS : item / kBK, k = MN ? item / ROWS : item % kBK;
      const int64_t gr = row0 + r, gk = k0 + k;
      const bool ok = gr < rows_total && gk < k_end;
      cp_async<4>(tile_s + tile_off<MN>(r, k) * 4, ok ? base + gr * s_row + gk * s_k : base, ok ? 4 : 0);
    }
  }
};

// In place: raw -> hi (low 13 mantissa bits cleared); lo = raw - hi goes to `lo`.  Works piece by piece on
// the same offsets in both buffers, so it does not care which layout the tile has.
template <int ROWS, bool MN, int T>
struct SplitPlan {
  static constexpr int QUADS = ROWS * kBK / 4;
  static constexpr int N = (QUADS + T - 1) / T;
  uint32_t off[N];
  __device__ void init() {
#pragma unroll
    for (int i = 0; i < N; i++) {
      const int q = threadIdx.x + i * T;
      off[i] = q < QUADS ? quad_off<MN>(q) : 0xFFFFFFFFu;
    }
  }
  __device__ __forceinline__ void run(float *raw, float *lo, bool split) const {
#pragma unroll
    for (int i = 0; i < N; i++) {
      if (off[i] == 0xFFFFFFFFu) continue;
      const float4 x = *reinterpret_cast<const float4 *>(raw + off[i]);
      float h[4], l[4];
      tc_split(x.x, h[0], l[0]); tc_split(x.y, h[1], l[1]); tc_split(x.z, h[2], l[2]); tc_split(x.w, h[3], l[3]);
      *reinterpret_cast<float4 *>(raw + off[i]) = make_float4(h[0], h[1], h[2], h[3]);
      if (split) *reinterpret_cast<float4 *>(lo + off[i]) = make_float4(l[0], l[1], l[2], l[3]);
    }
  }
};

// Warp-specialised main loop.  NS staging threads (256, or 512 when the CTA has an SM to itself) copy and split operand tiles; one more warp only
// issues MMAs.  The two sides meet through mbarriers alone:
//   full[s]  (count = staging threads) a staging thread arrives once its own pieces of the chunk in stage s are
//            copied, split and fenced towards the tensor core's proxy;
//   empty[s] (count = 1) tcgen05.commit arrives when the MMAs that read stage s have finished.
// A staging thread splits exactly the pieces it copied itself, so it waits only for its own cp.async group
// and never for another staging thread: there is no block-wide barrier in the loop, and the latency of
// issuing MMAs is off the staging path.
template <int BN, bool A_MN, bool B_MN, int S, int NS>
__global__ void __launch_bounds__(NS + 32, S <= 3 ? kCtasPerSM : 1) gemm_tc_kernel(const TcGemmArgs g) {
  extern __shared__ __align__(1024) unsigned char tc_smem[];
  constexpr int T = NS;   // staging threads; one more warp issues the MMAs
  constexpr uint32_t A_TILE = TileFloats<kBM>::value;
  constexpr uint32_t B_TILE = TileFloats<BN>::value;
  float *a_raw = reinterpret_cast<float *>(tc_smem);                 // [S][A_TILE]  (becomes hi)
  float *b_raw = a_raw + S * A_TILE;                                 // [S][B_TILE]
  float *a_lo = b_raw + S * B_TILE;                                  // [S][A_TILE]
  float *b_lo = a_lo + S * A_TILE;                                   // [S][B_TILE]
  uint64_t *full = reinterpret_cast<uint64_t *>(b_lo + S * B_TILE);  // [S]
  uint64_t *empty = full + S;                                        // [S]
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(empty + S);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool is_stager = tid < T;
  const bool split = g.mode == 1;
  const int64_t row0 = (int64_t)blockIdx.x * kBM, col0 = (int64_t)blockIdx.y * BN;
  const int64_t k_begin = (int64_t)blockIdx.z * g.k_per_split;
  const int64_t k_end = min(g.K, k_begin + g.k_per_split);
  const int nchunks = (int)((k_end - k_begin + kBK - 1) / kBK);

  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(tmem_slot)),
                 "r"((uint32_t)BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < S; s++) {
      tc_mbar_init(tc_smem_u32(&full[s]), T);
      tc_mbar_init(tc_smem_u32(&empty[s]), 1);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // instruction descriptor: D = F32, A = B = TF32, bit 15 / 16 = A / B is MN-major, N = BN, M = 128
  const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                         ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
  bool ok = true;
  const int full_chunks = (int)((k_end - k_begin) / kBK);   // chunks without a K tail

  if (is_stager) {
    CopyPlan<kBM, A_MN, T> plan_a;
    CopyPlan<BN, B_MN, T> plan_b;
    plan_a.init(g.a, g.a_row, g.a_k, row0, g.M, k_begin, g.a_vec);
    plan_b.init(g.b, g.b_row, g.b_k, col0, g.N, k_begin, g.b_vec);

    // A K-major operand is read 64 bytes per row and chunk; every kPrefetchChunks chunks one thread per row
    // asks L2 for the row's next kPrefetchChunks * 64 bytes in whole lines, so that DRAM sees long bursts.
    constexpr int kPrefetchChunks = 8;
    auto prefetch_rows = [&](int chunk_lo) {
      if (A_MN || tid >= kBM || row0 + tid >= g.M) return;
      const int64_t k_lo = k_begin + (int64_t)chunk_lo * kBK;
      const int64_t k_hi = min(k_end, k_lo + (int64_t)kPrefetchChunks * kBK);
      if (k_lo >= k_hi) return;
      const char *row = reinterpret_cast<const char *>(g.a + (row0 + tid) * g.a_row);
      const char *lo = reinterpret_cast<const char *>(reinterpret_cast<uintptr_t>(row + k_lo * 4) & ~(uintptr_t)127);
      const char *hi = row + k_hi * 4;
      for (const char *q = lo; q < hi; q += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(q));
    };
    // copies of chunk `chunk` into its stage; one cp.async group per call, empty past the end, so that the
    // wait count below is a constant
    auto start_copy = [&](int chunk) {
      if (chunk < nchunks) {
        const int st = chunk % S;
        if (chunk >= S) {   // the stage is being reused: the MMAs of chunk - S must have finished reading it
          if (!tc_mbar_wait(tc_smem_u32(&empty[st]), ((chunk / S) - 1) & 1)) ok = false;
        }
        if (ok) {
          if (chunk < full_chunks) {
            plan_a.issue(tc_smem_u32(a_raw + st * A_TILE), chunk);
            plan_b.issue(tc_smem_u32(b_raw + st * B_TILE), chunk);
          } else {
            const int64_t k0 = k_begin + (int64_t)chunk * kBK;
            plan_a.issue_tail(tc_smem_u32(a_raw + st * A_TILE), k0, k_end);
            plan_b.issue_tail(tc_smem_u32(b_raw + st * B_TILE), k0, k_end);
          }
        }
      }
      cp_async_commit();
    };
    // Chunks in flight ahead of the one being split.  Refilling the stage of chunk c-1 would wait for MMAs
    // that have only just been issued, so with four or more stages the copy goes S-2 chunks ahead (into the
    // stage chunk c-2 used); three stages (two CTAs per SM, which cover for each other) leave one.
    constexpr int kAhead = S >= 4 ? S - 2 : 1;
    prefetch_rows(0);
    prefetch_rows(kPrefetchChunks);
#pragma unroll
    for (int c = 0; c < kAhead; c++) start_copy(c);
    for (int c = 0; c < nchunks && ok; c++) {
      const int st = c % S;
      start_copy(c + kAhead);                 // into a stage whose MMAs are done (waits for them if not)
      if (c % kPrefetchChunks == 0) prefetch_rows(c + 2 * kPrefetchChunks);
      cp_async_wait<kAhead>();                // this thread's copies of chunk c have landed
      if (c < full_chunks) {
        plan_a.split_own(a_raw + st * A_TILE, a_lo + st * A_TILE, split);
        plan_b.split_own(b_raw + st * B_TILE, b_lo + st * B_TILE, split);
      } else {
        plan_a.split_tail(a_raw + st * A_TILE, a_lo + st * A_TILE, split);
        plan_b.split_tail(b_raw + st * B_TILE, b_lo + st * B_TILE, split);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> tensor-core reads
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc_smem_u32(&full[st])) : "memory");
    }
    cp_async_wait<0>();   // nothing of ours may still be landing in shared memory when the CTA winds down
  } else {
    // MMA warp: waits for a full stage, issues its MMAs from one lane, commits to the stage's empty barrier
    for (int c = 0; c < nchunks; c++) {
      const int st = c % S;
      if (!tc_mbar_wait(tc_smem_u32(&full[st]), (c / S) & 1)) { ok = false; break; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t a_h = tc_smem_u32(a_raw + st * A_TILE), a_l = tc_smem_u32(a_lo + st * A_TILE);
        const uint32_t b_h = tc_smem_u32(b_raw + st * B_TILE), b_l = tc_smem_u32(b_lo + st * B_TILE);
#pragma unroll
        for (int kk = 0; kk < kBK / 8; kk++) {
          // one K step = 8 tf32: two K-major core matrices, or one MN-major core matrix, further along K
          using SA = DescStride<A_MN>;
          using SB = DescStride<B_MN>;
          const uint32_t ka = kk * SA::kstep, kb = kk * SB::kstep;
          const uint64_t da_h = tc_make_desc(a_h + ka, SA::lbo, SA::sbo, SA::layout);
          const uint64_t db_h = tc_make_desc(b_h + kb, SB::lbo, SB::sbo, SB::layout);
          tc_mma_tf32(tmem, da_h, db_h, idesc, (c > 0 || kk > 0) ? 1u : 0u);
          if (split) {
            const uint64_t da_l = tc_make_desc(a_l + ka, SA::lbo, SA::sbo, SA::layout);
            const uint64_t db_l = tc_make_desc(b_l + kb, SB::lbo, SB::sbo, SB::layout);
            tc_mma_tf32(tmem, da_h, db_l, idesc, 1u);
            tc_mma_tf32(tmem, da_l, db_h, idesc, 1u);
          }
        }
        tc_commit(tc_smem_u32(&empty[st]));
      }
      __syncwarp();
    }
  }

  // all MMAs done: the last commit covers every earlier one
  if (ok && nchunks > 0) {
    const int last = nchunks - 1;
    ok = tc_mbar_wait(tc_smem_u32(&empty[last % S]), (last / S) & 1);
  }
  ok = __syncthreads_and(ok);
  if (!ok && tid == 0) atomicExch(&g_tc_gemm_error, 1u);
  tc_fence_after();

  if (ok && is_stager) {
    // Warp w reads TMEM lanes 32*(w%4)..+31 (the only ones it can reach); warps 0-3 take the left half
    // of the columns, warps 4-7 the right half.
    float *out = g.c + (int64_t)blockIdx.z * g.M * g.N;
    const int quarter = warp & 3, part = warp >> 2;
    constexpr int CB = BN / 32;                      // 32-column blocks in the tile
    constexpr int PARTS = T / 128;                   // groups of four warps sharing the column blocks
#pragma unroll
    for (int cbi = 0; cbi < (CB + PARTS - 1) / PARTS; cbi++) {
      const int cb = cbi * PARTS + part;
      if (cb >= CB) continue;
      uint32_t r[32];
      const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16) + cb * 32;
      if (nchunks > 0) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
              "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
              "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(taddr) : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      } else {
#pragma unroll
        for (int q = 0; q < 32; q++) r[q] = 0u;
      }
      // Transpose through shared memory (the operand stages are free by now) so that a warp writes
      // one C row segment of 128 contiguous bytes per instruction instead of 32 scattered words.
      float *stage = reinterpret_cast<float *>(tc_smem) + warp * (32 * 33);
      __syncwarp();
#pragma unroll
      for (int q = 0; q < 32; q++) stage[lane * 33 + q] = __uint_as_float(r[q]);
      __syncwarp();
      {
        const int64_t gj = col0 + cb * 32 + lane;
        for (int rr = 0; rr < 32; rr++) {
          const int64_t grow = row0 + quarter * 32 + rr;
          if (grow < g.M && gj < g.N) out[grow * g.N + gj] = stage[rr * 33 + lane];
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)BN) : "memory");
  }
}

template <int BN, bool A_MN, bool B_MN, int S, int NS>
static int launch_tc_s(const TcGemmArgs &g, dim3 grid, cudaStream_t stream) {
  constexpr size_t smem = (size_t)(2 * S * (TileFloats<kBM>::value + TileFloats<BN>::value)) * sizeof(float) + 128;
  static PerDeviceOnce configured;   // the attribute is kept per device
  if (configured.need()) {
    NB_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BN, A_MN, B_MN, S, NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured.done();
  }
  gemm_tc_kernel<BN, A_MN, B_MN, S, NS><<<grid, NS + 32, smem, stream>>>(g);
  NB_LAUNCH_CHECK();
  return 0;
}

__global__ void tc_splitk_reduce_kernel(const float *__restrict__ partial, float *__restrict__ c, int64_t mn,
                                        int splits) {
  pdl_enter();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < mn; i += (int64_t)gridDim.x * blockDim.x) {
    float s = partial[i];
    for (int z = 1; z < splits; z++) s += partial[(int64_t)z * mn + i];
    c[i] = s;
  }
}

// Six stages (the whole shared memory of an SM) when every CTA has an SM to itself, three when the grid can put
// two CTAs on an SM.
template <int BN, bool A_MN, bool B_MN>
static int launch_tc(const TcGemmArgs &g, dim3 grid, cudaStream_t stream) {
  const int64_t ctas = (int64_t)grid.x * grid.y * grid.z;
  int stages = ctas <= num_sms() ? 6 : 3;
  int stagers = stages >= 4 ? 512 : 256;
  if (stages >= 6) {
    if (stagers == 512) return launch_tc_s<BN, A_MN, B_MN, 6, 512>(g, grid, stream);
    return launch_tc_s<BN, A_MN, B_MN, 6, 256>(g, grid, stream);
  }
  return launch_tc_s<BN, A_MN, B_MN, 3, 256>(g, grid, stream);
}

// The three operand layouts of the GCN step: Y W (B transposed in memory relative to K-major), Y^T dZ
// (both), dZ W^T (neither).
template <int BN>
static int launch_layout(const TcGemmArgs &g, int trans_a, int trans_b, dim3 grid, cudaStream_t stream) {
  if (!trans_a && !trans_b) return launch_tc<BN, false, true>(g, grid, stream);
  if (trans_a && !trans_b) return launch_tc<BN, true, true>(g, grid, stream);
  if (!trans_a && trans_b) return launch_tc<BN, false, false>(g, grid, stream);
  return launch_tc<BN, true, false>(g, grid, stream);
}

static int vec_of(const float *p, int64_t ld) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  if ((a & 15) == 0 && (ld & 3) == 0) return 4;
  if ((a & 7) == 0 && (ld & 1) == 0) return 2;
  return 1;
}

// Tensor-core GEMM front end; same contract as the CUDA-core path in dense.cu.  Two environment switches exist for
// tests and comparisons: NB_TC_NO_TMA (set: always the cp.async kernel) and NB_TC_NO_ROWS_FORM (set: Y W in plain
// 128-row tiles); results are bit-identical either way.
int gemm_tensor_core(nb_ws *ws, const float *d_a, int64_t lda, const float *d_b, int64_t ldb, float *d_c, int64_t M,
                     int64_t N, int64_t K, int trans_a, int trans_b, int mode, cudaStream_t stream, const ReluEpi *epi,
                     bool *applied) {
  if (applied) *applied = false;
  TcGemmArgs g{};
  g.a = d_a; g.b = d_b; g.M = M; g.N = N; g.K = K; g.mode = mode;
  // op(A)(i,k): NN/NT -> A[i*lda + k];  TN -> A[k*lda + i]
  g.a_row = trans_a ? 1 : lda;  g.a_k = trans_a ? lda : 1;
  // op(B)^T(j,k) = op(B)(k,j): NN/TN -> B[k*ldb + j];  NT -> B[j*ldb + k]
  g.b_row = trans_b ? ldb : 1;  g.b_k = trans_b ? 1 : ldb;
  // widest piece that is aligned and divides the extent along the contiguous direction (a padded pitch must
  // not let a piece reach into the padding)
  auto piece = [](const float *p, int64_t ld, int64_t extent) {
    int v = vec_of(p, ld);
    while (v > 1 && extent % v != 0) v >>= 1;
    return v;
  };
  g.a_vec = piece(d_a, lda, trans_a ? M : K);
  g.b_vec = piece(d_b, ldb, trans_b ? K : N);
  const int bn = N > 64 ? 128 : (N > 32 ? 64 : 32);
  const int64_t tiles = ((M + kBM - 1) / kBM) * ((N + bn - 1) / bn);
  // Split-K towards one CTA per SM; ranges are multiples of 32 so that both kernels cut K at the same places.
  int splits = 1;
  if (tiles < num_sms() && K >= 512) {
    splits = (int)(num_sms() / tiles);
    const int64_t max_splits = K / 256;
    if (splits > max_splits) splits = (int)max_splits;
    if (splits < 1) splits = 1;
  }
  g.k_per_split = ((K + splits - 1) / splits + 31) / 32 * 32;
  splits = (int)((K + g.k_per_split - 1) / g.k_per_split);
  // TMA tensor loads need 16-byte aligned bases and pitches, and boxes that fit inside the tensor
  const bool a_mn = trans_a != 0, b_mn = trans_b == 0;
  const bool use_tma = !getenv("NB_TC_NO_TMA") && tma_gemm_applicable(d_a, lda, d_b, ldb) && K >= 32 &&
                       (a_mn ? M >= 32 : M >= kBM) && (b_mn ? N >= 32 : N >= bn);
  WsScope scope(ws);
  float *partial = nullptr;
  if (splits > 1) {
    NB_REQUIRE(ws != nullptr, "nb_gemm: split-K needs a workspace");
    partial = ws->alloc_n<float>((size_t)splits * M * N);
    if (!partial) return fail(NB_ERR_NOMEM, "nb_gemm: workspace arena exhausted");
  }
  g.c = splits > 1 ? partial : d_c;
  dim3 grid((unsigned)((M + kBM - 1) / kBM), (unsigned)((N + bn - 1) / bn), (unsigned)splits);
  if (grid.y > 65535) return fail(NB_ERR_INVALID, "nb_gemm: N too large for one launch");
  int st;
  // Y W with a short W: rows dealt evenly to the SMs (one wave whatever the row count, up to 160 rows per SM)
  const bool rows_form = use_tma && !trans_a && !trans_b && splits == 1 && !getenv("NB_TC_NO_ROWS_FORM") &&
                         tma_rows_form_applicable(M, N, K);
  // ReLU + dropout in the epilogue: whole quads of four elements per row, final values (no split-K partials)
  const bool epi_ok = epi != nullptr && epi->on && applied != nullptr && splits == 1 && (N % 4) == 0 && use_tma;
  if (rows_form) {
    st = gemm_tma_rows_launch(d_a, lda, d_b, ldb, d_c, M, N, K, mode, stream, epi_ok ? epi : nullptr);
    if (st == 0 && epi_ok) *applied = true;
  } else if (use_tma) {
    st = gemm_tma_launch(d_a, lda, d_b, ldb, g.c, M, N, K, trans_a, trans_b, bn, splits, g.k_per_split, mode, stream,
                         epi_ok ? epi : nullptr);
    if (st == 0 && epi_ok) *applied = true;
  } else {
    switch (bn) {
      case 128: st = launch_layout<128>(g, trans_a, trans_b, grid, stream); break;
      case 64: st = launch_layout<64>(g, trans_a, trans_b, grid, stream); break;
      default: st = launch_layout<32>(g, trans_a, trans_b, grid, stream); break;
    }
  }
  if (st != 0) return st;
  if (splits > 1) {
    NB_CUDA(launch_chained(tc_splitk_reduce_kernel, dim3(grid_for(M * N, 256)), dim3(256), 0, stream, partial, d_c, M * N,
                           splits));
    NB_LAUNCH_CHECK();
  }
  return 0;
}

int read_tc_error_flag(unsigned int *value) {
  unsigned int a = 0, b = 0;
  NB_CUDA(cudaMemcpyFromSymbol(&a, g_tc_gemm_error, sizeof(unsigned int)));
  NB_TRY(read_tma_gemm_error_flag(&b));
  *value = a | b;
  return 0;
}
int reset_tc_error_flag() {
  const unsigned int zero = 0;
  NB_CUDA(cudaMemcpyToSymbol(g_tc_gemm_error, &zero, sizeof(unsigned int)));
  return reset_tma_gemm_error_flag();
}

}  // namespace nb
