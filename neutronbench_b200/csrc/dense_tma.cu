// fp32 GEMM on tcgen05 (kind::tf32, three-term hi/lo split) with the operands brought into shared memory by
// TMA tensor loads: one thread issues one cp.async.bulk.tensor per tile (four per transposed tile) and the tile
// arrives already in the swizzled layout the tensor core reads, so no thread computes a source address or
// issues a copy for an element, and the hi/lo split runs as a straight pass over whole tiles.
//
// Used when both operands qualify for a tensor map: base 16-byte aligned and pitch a multiple of 4 floats.  The
// cp.async kernel of dense_tc.cu serves everything else.  Both issue the same MMAs in the same order (K steps of 8
// ascending; hi*hi, hi*lo, lo*hi per step; split-K ranges in multiples of 32), so they give identical bits.
//
// Layouts (measured, see the notes on MN-major operands in dense_tc.cu):
//   K-major operand   box {32 floats of K, ROWS rows}, CU_TENSOR_MAP_SWIZZLE_128B; descriptor layout type 2,
//                     SBO = 1024 bytes (8 rows of 128 bytes), K step of 8 = +32 bytes inside the swizzle line.
//   MN-major operand  boxes {32 rows, 32 k}, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, one per block of 32 rows (4 KB
//                     each); descriptor layout type 1, LBO = 4096 (row blocks), SBO = 512 (groups of 4 k),
//                     K step of 8 = +1024 bytes.
// Rows beyond the matrix and the K tail are zero-filled by the TMA unit (out-of-bounds box elements).
//
// Warp roles: warps 0-7 compute the lo tiles (lo = x - hi; the raw tile itself serves as hi) and run the epilogue, warp 8 issues the tensor loads, warp 9 the
// MMAs.  Three barriers per stage: loaded (TMA transaction bytes), split (256 arrivals), free (tcgen05.commit).
// Every wait is bounded; a wait that runs out sets the error word read by nb_device_error_flags.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <cstdlib>

#include "common.cuh"
#include "philox.cuh"
#include "tc_common.cuh"

namespace nb {

__device__ unsigned int g_tma_gemm_error = 0;

constexpr int kTmaBK = 32;            // K per chunk: one 128-byte swizzle line
constexpr int kTmaStages = 3;
constexpr int kSplitThreads = 256;    // warps 0-7
constexpr int kTmaThreads = kSplitThreads + 64;

struct TmaGemmArgs {
  float *c;                 // output, or split-K partials [splits][M][N]
  int64_t M, N, K;
  int64_t k_per_split;      // multiple of kTmaBK
  int mode;                 // 1: 3xTF32, 2: 1xTF32
  ReluEpi epi;              // ReLU + dropout on the way out (needs N % 4 == 0 and no split-K)
};

// What nb_relu_dropout does to one element, given the element's Philox word.
__device__ __forceinline__ uint32_t relu_drop_bits(uint32_t zbits, uint32_t rnd, const ReluEpi &e) {
  const float z = __uint_as_float(zbits);
  float val = z > 0.0f ? z : 0.0f;
  if (e.p > 0.0f) {
    const float u = (float)(rnd >> 8) * (1.0f / 16777216.0f);
    val = (u >= e.p) ? __fmul_rn(val, e.scale) : 0.0f;
  }
  return __float_as_uint(val);
}

template <bool MN> struct TmaDesc {};
template <> struct TmaDesc<false> { static constexpr uint32_t lbo = 16, sbo = 1024, kstep = 32, layout = 2; };
template <> struct TmaDesc<true> { static constexpr uint32_t lbo = 4096, sbo = 512, kstep = 1024, layout = 1; };

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

// One operand tile of a chunk: ROWS rows starting at row0, K range [k0, k0 + 32).
template <int ROWS, bool MN>
__device__ __forceinline__ void tma_load_tile(uint32_t dst, const CUtensorMap *map, int row0, int k0, uint32_t bar) {
  if (MN) {
#pragma unroll
    for (int rb = 0; rb < ROWS / 32; rb++) tma_load_2d(dst + rb * 4096, map, row0 + rb * 32, k0, bar);
  } else {
    tma_load_2d(dst, map, k0, row0, bar);
  }
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kTmaThreads, 1) gemm_tma_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                  const __grid_constant__ CUtensorMap map_b,
                                                                  const TmaGemmArgs g) {
  extern __shared__ __align__(1024) unsigned char tc_smem[];
  pdl_enter();
  constexpr int S = kTmaStages;
  constexpr uint32_t A_BYTES = kBM * kTmaBK * 4, B_BYTES = BN * kTmaBK * 4;   // 16 KB, and 4 / 8 / 16 KB
  constexpr uint32_t STAGE = 2 * (A_BYTES + B_BYTES);                        // raw A | raw B | lo A | lo B
  uint64_t *bars = reinterpret_cast<uint64_t *>(tc_smem + (size_t)S * STAGE);
  uint64_t *loaded = bars, *split_done = bars + S, *freed = bars + 2 * S;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * S);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool split = g.mode == 1;
  const int row0 = (int)blockIdx.x * kBM, col0 = (int)blockIdx.y * BN;
  const int64_t k_begin = (int64_t)blockIdx.z * g.k_per_split;
  const int64_t k_end = min(g.K, k_begin + g.k_per_split);
  const int nchunks = (int)((k_end - k_begin + kTmaBK - 1) / kTmaBK);

  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(tmem_slot)),
                 "r"((uint32_t)BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < S; s++) {
      tc_mbar_init(tc_smem_u32(&loaded[s]), 1);
      tc_mbar_init(tc_smem_u32(&split_done[s]), kSplitThreads);
      tc_mbar_init(tc_smem_u32(&freed[s]), 1);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                         ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
  bool ok = true;

  if (warp == 8) {
    // ---- producer: tensor loads, one stage ahead of nothing but the free barrier
    if (lane == 0) {
      for (int c = 0; c < nchunks; c++) {
        const int st = c % S;
        if (c >= S && !tc_mbar_wait(tc_smem_u32(&freed[st]), ((c / S) - 1) & 1)) { ok = false; break; }
        const uint32_t bar = tc_smem_u32(&loaded[st]);
        const uint32_t a_dst = tc_smem_u32(tc_smem + (size_t)st * STAGE), b_dst = a_dst + A_BYTES;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(A_BYTES + B_BYTES) : "memory");
        const int k0 = (int)(k_begin + (int64_t)c * kTmaBK);
        tma_load_tile<kBM, A_MN>(a_dst, &map_a, row0, k0, bar);
        tma_load_tile<BN, B_MN>(b_dst, &map_b, col0, k0, bar);
      }
    }
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
  } else if (warp == 9) {
    // ---- MMA issuer
    for (int c = 0; c < nchunks; c++) {
      const int st = c % S;
      if (!tc_mbar_wait(tc_smem_u32(&split_done[st]), (c / S) & 1)) { ok = false; break; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t a_h = tc_smem_u32(tc_smem + (size_t)st * STAGE), b_h = a_h + A_BYTES;
        const uint32_t a_l = a_h + A_BYTES + B_BYTES, b_l = a_l + A_BYTES;
        using DA = TmaDesc<A_MN>;
        using DB = TmaDesc<B_MN>;
#pragma unroll
        for (int kk = 0; kk < kTmaBK / 8; kk++) {
          const uint64_t da_h = tc_make_desc(a_h + kk * DA::kstep, DA::lbo, DA::sbo, DA::layout);
          const uint64_t db_h = tc_make_desc(b_h + kk * DB::kstep, DB::lbo, DB::sbo, DB::layout);
          tc_mma_tf32(tmem, da_h, db_h, idesc, (c > 0 || kk > 0) ? 1u : 0u);
          if (split) {
            const uint64_t da_l = tc_make_desc(a_l + kk * DA::kstep, DA::lbo, DA::sbo, DA::layout);
            const uint64_t db_l = tc_make_desc(b_l + kk * DB::kstep, DB::lbo, DB::sbo, DB::layout);
            tc_mma_tf32(tmem, da_h, db_l, idesc, 1u);
            tc_mma_tf32(tmem, da_l, db_h, idesc, 1u);
          }
        }
        tc_commit(tc_smem_u32(&freed[st]));
      }
      __syncwarp();
    }
  } else {
    // ---- splitters: lo = x - hi (hi = x with the low 13 mantissa bits cleared) into the second half of the stage.
    // The raw fp32 words stay where TMA put them and serve as hi: kind::tf32 ignores the low 13 mantissa bits of
    // its operands (measured: rewriting them as zeros gives the same bits), which saves a third of the pass's
    // shared-memory traffic.  Element by element and position-preserving, so the swizzle pattern does not matter.
    constexpr int QUADS = (A_BYTES + B_BYTES) / 16;
    for (int c = 0; c < nchunks && ok; c++) {
      const int st = c % S;
      if (!tc_mbar_wait(tc_smem_u32(&loaded[st]), (c / S) & 1)) { ok = false; break; }
      float4 *raw = reinterpret_cast<float4 *>(tc_smem + (size_t)st * STAGE);
      float4 *lo = raw + QUADS;
#pragma unroll 4
      for (int q = tid; q < QUADS; q += kSplitThreads) {
        const float4 x = raw[q];
        float h[4], l[4];
        tc_split(x.x, h[0], l[0]); tc_split(x.y, h[1], l[1]); tc_split(x.z, h[2], l[2]); tc_split(x.w, h[3], l[3]);
        if (split) lo[q] = make_float4(l[0], l[1], l[2], l[3]);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> tensor-core reads
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc_smem_u32(&split_done[st])) : "memory");
    }
  }

  // all MMAs done: the last commit covers every earlier one
  if (ok && nchunks > 0) {
    const int last = nchunks - 1;
    ok = tc_mbar_wait(tc_smem_u32(&freed[last % S]), (last / S) & 1);
  }
  ok = __syncthreads_and(ok);
  if (!ok && tid == 0) atomicExch(&g_tma_gemm_error, 1u);
  tc_fence_after();

  if (ok && warp < 8) {
    // Warp w reads TMEM lanes 32*(w%4)..+31; warps 0-3 and 4-7 alternate over the 32-column blocks.  The values go
    // through shared memory (the stages are free by now) so that a warp writes whole 128-byte row segments of C.
    float *out = g.c + (int64_t)blockIdx.z * g.M * g.N;
    const int quarter = warp & 3, part = warp >> 2;
    constexpr int CB = BN / 32;
#pragma unroll
    for (int cbi = 0; cbi < (CB + 1) / 2; cbi++) {
      const int cb = cbi * 2 + part;
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
      if (g.epi.on) {
        // this thread holds columns col0 + cb*32 .. +31 of row row0 + quarter*32 + lane: eight whole Philox quads
        const int64_t e0 = (row0 + quarter * 32 + lane) * g.N + col0 + cb * 32;
#pragma unroll
        for (int q8 = 0; q8 < 8; q8++) {
          uint32_t rnd[4] = {0u, 0u, 0u, 0u};
          if (g.epi.p > 0.0f)
            philox4x32_10((uint32_t)((e0 + 4 * q8) >> 2), g.epi.layer, g.epi.step, 1u, g.epi.seed_lo, g.epi.seed_hi, rnd);
#pragma unroll
          for (int k = 0; k < 4; k++) r[4 * q8 + k] = relu_drop_bits(r[4 * q8 + k], rnd[k], g.epi);
        }
      }
      float *stage = reinterpret_cast<float *>(tc_smem) + warp * (32 * 33);
      __syncwarp();
#pragma unroll
      for (int q = 0; q < 32; q++) stage[lane * 33 + q] = __uint_as_float(r[q]);
      __syncwarp();
      const int64_t gj = col0 + cb * 32 + lane;
      for (int rr = 0; rr < 32; rr++) {
        const int64_t grow = row0 + quarter * 32 + rr;
        if (grow < g.M && gj < g.N) out[grow * g.N + gj] = stage[rr * 33 + lane];
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)BN) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------
// Row-balanced form of C = Y W for a wide, short W (N <= 128): the product is computed as C^T = W^T Y^T, so the
// rows of Y become the N dimension of the MMA, which can be any multiple of 16 up to 256 instead of exactly 128.
// Every CTA takes ceil(M / #SMs) rows (rounded up to 16, at most kRowsMax), which keeps a product of, say, 150
// row tiles of 128 in ONE wave over 148 SMs instead of two.  W^T is the MN-major A operand (128 outputs, zero rows
// beyond N), the rows of Y the K-major B operand.  The three MMAs per K step are issued in the order
// hi*hi, lo(W)*hi(Y), hi(W)*lo(Y), i.e. the same three products in the same order as the plain form, so both
// forms give identical bits.  The accumulator holds C^T (lane = output column, TMEM column = row), which the
// epilogue writes straight out: a warp stores 32 consecutive output columns of one row per instruction.
constexpr int kRowsMax = 160;

struct TmaRowsArgs {
  float *c;
  int64_t M, N, K;
  int rows_per_cta;         // multiple of 16, <= kRowsMax
  int mode;
  ReluEpi epi;              // ReLU + dropout on the way out (needs N % 4 == 0)
};

__global__ void __launch_bounds__(kTmaThreads, 1) gemm_tma_rows_kernel(const __grid_constant__ CUtensorMap map_y,
                                                                       const __grid_constant__ CUtensorMap map_w,
                                                                       const TmaRowsArgs g) {
  extern __shared__ __align__(1024) unsigned char tc_smem[];
  pdl_enter();
  constexpr int S = kTmaStages;
  constexpr uint32_t W_BYTES = kBM * kTmaBK * 4;                 // W^T tile: 128 outputs x 32 k
  constexpr uint32_t Y_MAX = kRowsMax * kTmaBK * 4;              // Y tile: up to 160 rows x 32 k
  constexpr uint32_t STAGE = 2 * (W_BYTES + Y_MAX);              // raw W | raw Y | lo W | lo Y
  uint64_t *bars = reinterpret_cast<uint64_t *>(tc_smem + (size_t)S * STAGE);
  uint64_t *loaded = bars, *split_done = bars + S, *freed = bars + 2 * S;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * S);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool split = g.mode == 1;
  const int rows = g.rows_per_cta;
  const int row0 = (int)blockIdx.x * rows;
  const uint32_t y_bytes = (uint32_t)rows * kTmaBK * 4;
  const int nchunks = (int)((g.K + kTmaBK - 1) / kTmaBK);

  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(tmem_slot)),
                 "r"(256u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
#pragma unroll
    for (int s = 0; s < S; s++) {
      tc_mbar_init(tc_smem_u32(&loaded[s]), 1);
      tc_mbar_init(tc_smem_u32(&split_done[s]), kSplitThreads);
      tc_mbar_init(tc_smem_u32(&freed[s]), 1);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // A = W^T is MN-major (bit 15), B = Y rows K-major; N = rows of this CTA, M = 128
  const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | ((uint32_t)(rows >> 3) << 17) |
                         ((uint32_t)(kBM >> 4) << 24);
  bool ok = true;

  if (warp == 8) {
    if (lane == 0) {
      for (int c = 0; c < nchunks; c++) {
        const int st = c % S;
        if (c >= S && !tc_mbar_wait(tc_smem_u32(&freed[st]), ((c / S) - 1) & 1)) { ok = false; break; }
        const uint32_t bar = tc_smem_u32(&loaded[st]);
        const uint32_t w_dst = tc_smem_u32(tc_smem + (size_t)st * STAGE), y_dst = w_dst + W_BYTES;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(W_BYTES + y_bytes) : "memory");
        const int k0 = c * kTmaBK;
        tma_load_tile<kBM, true>(w_dst, &map_w, 0, k0, bar);
        tma_load_2d(y_dst, &map_y, k0, row0, bar);     // box {32 k, rows}
      }
    }
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
  } else if (warp == 9) {
    for (int c = 0; c < nchunks; c++) {
      const int st = c % S;
      if (!tc_mbar_wait(tc_smem_u32(&split_done[st]), (c / S) & 1)) { ok = false; break; }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t w_h = tc_smem_u32(tc_smem + (size_t)st * STAGE), y_h = w_h + W_BYTES;
        const uint32_t w_l = w_h + W_BYTES + Y_MAX, y_l = w_l + W_BYTES;
        using DW = TmaDesc<true>;
        using DY = TmaDesc<false>;
#pragma unroll
        for (int kk = 0; kk < kTmaBK / 8; kk++) {
          const uint64_t dw_h = tc_make_desc(w_h + kk * DW::kstep, DW::lbo, DW::sbo, DW::layout);
          const uint64_t dy_h = tc_make_desc(y_h + kk * DY::kstep, DY::lbo, DY::sbo, DY::layout);
          tc_mma_tf32(tmem, dw_h, dy_h, idesc, (c > 0 || kk > 0) ? 1u : 0u);
          if (split) {
            const uint64_t dw_l = tc_make_desc(w_l + kk * DW::kstep, DW::lbo, DW::sbo, DW::layout);
            const uint64_t dy_l = tc_make_desc(y_l + kk * DY::kstep, DY::lbo, DY::sbo, DY::layout);
            tc_mma_tf32(tmem, dw_l, dy_h, idesc, 1u);   // hi(Y) * lo(W): second term of the plain form
            tc_mma_tf32(tmem, dw_h, dy_l, idesc, 1u);   // lo(Y) * hi(W): third term
          }
        }
        tc_commit(tc_smem_u32(&freed[st]));
      }
      __syncwarp();
    }
  } else {
    const int w_quads = W_BYTES / 16, y_quads = (int)(y_bytes / 16);
    for (int c = 0; c < nchunks && ok; c++) {
      const int st = c % S;
      if (!tc_mbar_wait(tc_smem_u32(&loaded[st]), (c / S) & 1)) { ok = false; break; }
      float4 *raw = reinterpret_cast<float4 *>(tc_smem + (size_t)st * STAGE);
      float4 *lo = raw + (W_BYTES + Y_MAX) / 16;
      // the W tile and the used part of the Y tile; the two sit W_BYTES / 16 quads apart in both halves
      for (int q = tid; q < w_quads + y_quads; q += kSplitThreads) {
        const float4 x = raw[q];
        float h[4], l[4];
        tc_split(x.x, h[0], l[0]); tc_split(x.y, h[1], l[1]); tc_split(x.z, h[2], l[2]); tc_split(x.w, h[3], l[3]);
        if (split) lo[q] = make_float4(l[0], l[1], l[2], l[3]);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc_smem_u32(&split_done[st])) : "memory");
    }
  }

  if (ok && nchunks > 0) {
    const int last = nchunks - 1;
    ok = tc_mbar_wait(tc_smem_u32(&freed[last % S]), (last / S) & 1);
  }
  ok = __syncthreads_and(ok);
  if (!ok && tid == 0) atomicExch(&g_tma_gemm_error, 1u);
  tc_fence_after();

  if (ok && warp < 8) {
    // lane = output column 32*(w%4) + lane, TMEM column = row of this CTA; warps 0-3 / 4-7 alternate over the
    // blocks of 32 rows
    const int quarter = warp & 3, part = warp >> 2;
    const int64_t col = quarter * 32 + lane;
    for (int cb = part; cb * 32 < rows; cb += 2) {
      uint32_t r[32];
      const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16) + cb * 32;
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
      if (g.epi.on) {
        // This thread holds ONE column of 32 rows, while a Philox call yields the words of four neighbouring columns
        // of one row.  The four lanes that share a quad of columns each draw for one of four rows and pass the words
        // round: in round u lane d reads from the lane of its group that drew for row (d + u) & 3 the word of d's
        // own column.
        const uint32_t k = lane & 3;
#pragma unroll
        for (int jb = 0; jb < 8; jb++) {
          uint32_t got[4] = {0u, 0u, 0u, 0u};
          if (g.epi.p > 0.0f) {
            const int64_t e0 = ((int64_t)row0 + cb * 32 + jb * 4 + k) * g.N + (col & ~(int64_t)3);
            uint32_t pr[4];
            philox4x32_10((uint32_t)(e0 >> 2), g.epi.layer, g.epi.step, 1u, g.epi.seed_lo, g.epi.seed_hi, pr);
#pragma unroll
            for (int u = 0; u < 4; u++) {
              const uint32_t sel = (k - u) & 3;
              const uint32_t give = sel == 0 ? pr[0] : (sel == 1 ? pr[1] : (sel == 2 ? pr[2] : pr[3]));
              got[u] = __shfl_sync(0xffffffffu, give, (lane & ~3u) + ((lane + u) & 3));
            }
          }
#pragma unroll
          for (int t = 0; t < 4; t++) {
            const uint32_t u = ((uint32_t)t - k) & 3;     // the round in which row jb*4 + t came round
            const uint32_t rnd = u == 0 ? got[0] : (u == 1 ? got[1] : (u == 2 ? got[2] : got[3]));
            r[jb * 4 + t] = relu_drop_bits(r[jb * 4 + t], rnd, g.epi);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 32; j++) {
        const int64_t grow = (int64_t)row0 + cb * 32 + j;
        if (cb * 32 + j < rows && grow < g.M && col < g.N) g.c[grow * g.N + col] = __uint_as_float(r[j]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u) : "memory");
  }
}

// ------------------------------------------------------------------------------------------------ host side
static PFN_cuTensorMapEncodeTiled tensor_map_encoder() {
  static PFN_cuTensorMapEncodeTiled fn = nullptr;
  static bool tried = false;
  if (!tried) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(p);
    tried = true;
  }
  return fn;
}

// Tensor map of one operand.  K-major: the matrix is [rows x K] with pitch ld; boxes of 32 k by box_rows rows.
// MN-major: the matrix is [K x rows] with pitch ld; boxes of 32 rows by 32 k.
static bool make_operand_map(CUtensorMap *map, const float *base, bool mn, int64_t rows, int64_t K, int64_t ld,
                             int box_rows) {
  PFN_cuTensorMapEncodeTiled encode = tensor_map_encoder();
  if (!encode) return false;
  cuuint64_t dims[2], strides[1] = {(cuuint64_t)ld * 4};
  cuuint32_t box[2], estr[2] = {1, 1};
  CUtensorMapSwizzle swz;
  if (mn) {
    dims[0] = (cuuint64_t)rows; dims[1] = (cuuint64_t)K;
    box[0] = 32; box[1] = kTmaBK;
    swz = CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
  } else {
    dims[0] = (cuuint64_t)K; dims[1] = (cuuint64_t)rows;
    box[0] = kTmaBK; box[1] = (cuuint32_t)box_rows;
    swz = CU_TENSOR_MAP_SWIZZLE_128B;
  }
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, bool A_MN, bool B_MN>
static int launch_tma(const CUtensorMap &ma, const CUtensorMap &mb, const TmaGemmArgs &g, dim3 grid, cudaStream_t stream) {
  constexpr size_t smem = (size_t)kTmaStages * 2 * (kBM + BN) * kTmaBK * 4 + 256;
  static PerDeviceOnce configured;   // the attribute is kept per device
  if (configured.need()) {
    NB_CUDA(cudaFuncSetAttribute(gemm_tma_kernel<BN, A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured.done();
  }
  NB_CUDA(launch_chained(gemm_tma_kernel<BN, A_MN, B_MN>, grid, dim3(kTmaThreads), smem, stream, ma, mb, g));
  NB_LAUNCH_CHECK();
  return 0;
}

template <int BN>
static int launch_tma_layout(const CUtensorMap &ma, const CUtensorMap &mb, const TmaGemmArgs &g, bool a_mn, bool b_mn,
                             dim3 grid, cudaStream_t stream) {
  if (!a_mn && b_mn) return launch_tma<BN, false, true>(ma, mb, g, grid, stream);
  if (a_mn && b_mn) return launch_tma<BN, true, true>(ma, mb, g, grid, stream);
  if (!a_mn && !b_mn) return launch_tma<BN, false, false>(ma, mb, g, grid, stream);
  return launch_tma<BN, true, false>(ma, mb, g, grid, stream);
}

bool tma_gemm_applicable(const float *d_a, int64_t lda, const float *d_b, int64_t ldb) {
  auto ok = [](const float *p, int64_t ld) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0 && (ld & 3) == 0 && ld > 0; };
  return ok(d_a, lda) && ok(d_b, ldb) && tensor_map_encoder() != nullptr;
}

// C (or the split-K partials) = op(A) op(B) for one launch; `c` is dense [splits][M][N].
int gemm_tma_launch(const float *d_a, int64_t lda, const float *d_b, int64_t ldb, float *c, int64_t M, int64_t N,
                    int64_t K, int trans_a, int trans_b, int bn, int splits, int64_t k_per_split, int mode,
                    cudaStream_t stream, const ReluEpi *epi) {
  const bool a_mn = trans_a != 0, b_mn = trans_b == 0;
  CUtensorMap ma, mb;
  if (!make_operand_map(&ma, d_a, a_mn, M, K, lda, kBM) || !make_operand_map(&mb, d_b, b_mn, N, K, ldb, bn))
    return fail(NB_ERR_CUDA, "nb_gemm: cuTensorMapEncodeTiled failed");
  TmaGemmArgs g{};
  g.c = c; g.M = M; g.N = N; g.K = K; g.k_per_split = k_per_split; g.mode = mode;
  if (epi && splits == 1 && (N % 4) == 0) g.epi = *epi;
  dim3 grid((unsigned)((M + kBM - 1) / kBM), (unsigned)((N + bn - 1) / bn), (unsigned)splits);
  switch (bn) {
    case 128: return launch_tma_layout<128>(ma, mb, g, a_mn, b_mn, grid, stream);
    case 64: return launch_tma_layout<64>(ma, mb, g, a_mn, b_mn, grid, stream);
    default: return launch_tma_layout<32>(ma, mb, g, a_mn, b_mn, grid, stream);
  }
}

// C = Y W in the row-balanced form; applicable to NN products with N <= 128 and no split-K.
bool tma_rows_form_applicable(int64_t M, int64_t N, int64_t K) {
  if (N > kBM || N < 32 || K < kTmaBK || M < 8192) return false;   // small products: plain tiles and split-K
  const int64_t rows = ((M + num_sms() - 1) / num_sms() + 15) / 16 * 16;
  return rows <= kRowsMax && M >= rows;
}

int gemm_tma_rows_launch(const float *d_y, int64_t ldy, const float *d_w, int64_t ldw, float *c, int64_t M, int64_t N,
                         int64_t K, int mode, cudaStream_t stream, const ReluEpi *epi) {
  const int rows = (int)(((M + num_sms() - 1) / num_sms() + 15) / 16 * 16);
  CUtensorMap my, mw;
  if (!make_operand_map(&my, d_y, false, M, K, ldy, rows) || !make_operand_map(&mw, d_w, true, N, K, ldw, 0))
    return fail(NB_ERR_CUDA, "nb_gemm: cuTensorMapEncodeTiled failed");
  TmaRowsArgs g{};
  g.c = c; g.M = M; g.N = N; g.K = K; g.rows_per_cta = rows; g.mode = mode;
  if (epi && (N % 4) == 0) g.epi = *epi;
  constexpr size_t smem = (size_t)kTmaStages * 2 * (kBM + kRowsMax) * kTmaBK * 4 + 256;
  static PerDeviceOnce configured;   // the attribute is kept per device
  if (configured.need()) {
    NB_CUDA(cudaFuncSetAttribute(gemm_tma_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured.done();
  }
  const unsigned grid = (unsigned)((M + rows - 1) / rows);
  NB_CUDA(launch_chained(gemm_tma_rows_kernel, dim3(grid), dim3(kTmaThreads), smem, stream, my, mw, g));
  NB_LAUNCH_CHECK();
  return 0;
}

int read_tma_gemm_error_flag(unsigned int *value) {
  NB_CUDA(cudaMemcpyFromSymbol(value, g_tma_gemm_error, sizeof(unsigned int)));
  return 0;
}
int reset_tma_gemm_error_flag() {
  const unsigned int zero = 0;
  NB_CUDA(cudaMemcpyToSymbol(g_tma_gemm_error, &zero, sizeof(unsigned int)));
  return 0;
}

}  // namespace nb
