// Dense layer pieces: fp32 GEMM (CUDA-core path with split-K), ReLU+dropout, softmax/NLL loss with
// gradient, Adam.  The reference runs these through libtorch (core/NtsScheduler.hpp:712-715, 794-811;
// toolkits/GCN_GPU_NEIGHBOR.hpp:715-728; utils/torch_func.hpp:67-82).
#include "common.cuh"
#include "philox.cuh"

namespace nb {


// ------------------------------------------------------------------------------------ GEMM (SIMT)
// C[M x N] = op(A) op(B), element access through strides so that NN / TN / NT share one kernel.
// 64 x 64 x 16 tiles, 256 threads, 4 x 4 outputs per thread.  blockIdx.z walks split-K slices whose
// partial products are summed afterwards in slice order (deterministic).
constexpr int kTM = 64, kTN = 64, kTK = 16;

struct GemmArgs {
  const float *a, *b;
  float *c;          // final output, or partial buffer [splits][M][N] when splits > 1
  int64_t M, N, K;
  int64_t sa_i, sa_k, sb_k, sb_j;
  int64_t k_per_split;
  int splits;
};

__global__ void __launch_bounds__(256) gemm_simt_kernel(const GemmArgs g) {
  __shared__ float As[kTK][kTM + 4];
  __shared__ float Bs[kTK][kTN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, each 4 x 4
  const int64_t row0 = (int64_t)blockIdx.x * kTM, col0 = (int64_t)blockIdx.y * kTN;
  const int64_t k_begin = (int64_t)blockIdx.z * g.k_per_split;
  const int64_t k_end = min(g.K, k_begin + g.k_per_split);
  float acc[4][4] = {};
  for (int64_t k0 = k_begin; k0 < k_end; k0 += kTK) {
    // A tile: 64 x 16 elements, 4 per thread.  The faster-varying thread index follows the unit stride.
#pragma unroll
    for (int t = 0; t < 4; t++) {
      const int idx = tid + t * 256;
      int i, k;
      if (g.sa_k == 1) { k = idx & 15; i = idx >> 4; } else { i = idx & 63; k = idx >> 6; }
      const int64_t gi = row0 + i, gk = k0 + k;
      As[k][i] = (gi < g.M && gk < k_end) ? __ldg(g.a + gi * g.sa_i + gk * g.sa_k) : 0.0f;
    }
#pragma unroll
    for (int t = 0; t < 4; t++) {
      const int idx = tid + t * 256;
      int j, k;
      if (g.sb_j == 1) { j = idx & 63; k = idx >> 6; } else { k = idx & 15; j = idx >> 4; }
      const int64_t gj = col0 + j, gk = k0 + k;
      Bs[k][j] = (gj < g.N && gk < k_end) ? __ldg(g.b + gk * g.sb_k + gj * g.sb_j) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kTK; k++) {
      const float4 av = *reinterpret_cast<const float4 *>(&As[k][ty * 4]);
      const float4 bv = *reinterpret_cast<const float4 *>(&Bs[k][tx * 4]);
      const float a4[4] = {av.x, av.y, av.z, av.w};
      const float b4[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a4[i], b4[j], acc[i][j]);
    }
    __syncthreads();
  }
  float *out = g.c + (int64_t)blockIdx.z * g.M * g.N;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int64_t gi = row0 + ty * 4 + i;
    if (gi >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int64_t gj = col0 + tx * 4 + j;
      if (gj < g.N) out[gi * g.N + gj] = acc[i][j];
    }
  }
}

__global__ void splitk_reduce_kernel(const float *__restrict__ partial, float *__restrict__ c, int64_t mn, int splits) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < mn; i += (int64_t)gridDim.x * blockDim.x) {
    float s = partial[i];
    for (int z = 1; z < splits; z++) s += partial[(int64_t)z * mn + i];
    c[i] = s;
  }
}

// ------------------------------------------------------------------------------------ ReLU + dropout
__global__ void relu_dropout_kernel(float *z, int64_t n, float p, float scale, uint32_t seed_lo, uint32_t seed_hi,
                                    uint32_t layer, uint32_t step) {
  pdl_enter();
  const int64_t quads = (n + 3) >> 2;
  for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < quads; q += (int64_t)gridDim.x * blockDim.x) {
    uint32_t r[4] = {0, 0, 0, 0};
    if (p > 0.0f) philox4x32_10((uint32_t)q, layer, step, 1u, seed_lo, seed_hi, r);
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const int64_t i = q * 4 + k;
      if (i >= n) break;
      float val = z[i] > 0.0f ? z[i] : 0.0f;
      if (p > 0.0f) {
        const float u = (float)(r[k] >> 8) * (1.0f / 16777216.0f);
        val = (u >= p) ? __fmul_rn(val, scale) : 0.0f;
      }
      z[i] = val;
    }
  }
}

// ------------------------------------------------------------------------------------ loss
// Set (never cleared by the kernels) when a label was outside [0, C): that row then counts with loss 0, no hit and a
// zero gradient instead of indexing the logits with it.
__device__ unsigned int g_loss_error = 0;

// One warp per row: max, log-sum-exp, NLL at the label, gradient (softmax - onehot)/B, argmax hit.
__global__ void softmax_nll_rows_kernel(const float *__restrict__ logits, const int64_t *__restrict__ label, int64_t B,
                                        int64_t C, float *dlogits, float *row_loss, float *row_hit) {
  const unsigned lane = threadIdx.x & 31;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < B; i += warps) {
    const float *z = logits + i * C;
    float m = -INFINITY;
    int64_t arg = 0;
    for (int64_t c = lane; c < C; c += 32)
      if (z[c] > m) { m = z[c]; arg = c; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const int64_t oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (om > m || (om == m && oa < arg)) { m = om; arg = oa; }  // first maximum wins, like argmax
    }
    float sum = 0.0f;
    for (int64_t c = lane; c < C; c += 32) sum += expf(z[c] - m);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float lse = logf(sum);
    const int64_t y = label[i];
    const bool labelled = y >= 0 && y < C;
    if (lane == 0) {
      if (!labelled) atomicOr(&g_loss_error, 1u);
      row_loss[i] = labelled ? -((z[y] - m) - lse) : 0.0f;
      row_hit[i] = (labelled && arg == y) ? 1.0f : 0.0f;
    }
    if (dlogits) {
      const float inv_b = 1.0f / (float)B;
      for (int64_t c = lane; c < C; c += 32) {
        const float pr = expf(z[c] - m - lse);
        dlogits[i * C + c] = labelled ? (pr - (c == y ? 1.0f : 0.0f)) * inv_b : 0.0f;
      }
    }
  }
}

// Fixed-shape reduction (one block of 1024 threads, strided partial sums, shared-memory tree): the
// result does not depend on scheduling.
__global__ void __launch_bounds__(1024) loss_reduce_kernel(const float *__restrict__ row_loss,
                                                           const float *__restrict__ row_hit, int64_t B,
                                                           float *stats) {
  __shared__ float sl[1024], sh[1024];
  float l = 0.0f, h = 0.0f;
  for (int64_t i = threadIdx.x; i < B; i += 1024) { l += row_loss[i]; h += row_hit[i]; }
  sl[threadIdx.x] = l; sh[threadIdx.x] = h;
  __syncthreads();
  for (int o = 512; o > 0; o >>= 1) {
    if (threadIdx.x < o) { sl[threadIdx.x] += sl[threadIdx.x + o]; sh[threadIdx.x] += sh[threadIdx.x + o]; }
    __syncthreads();
  }
  if (threadIdx.x == 0) { stats[0] = sl[0] / (float)B; stats[1] = sh[0]; }
}

// Multi-label loss (CLASSES > 1): one warp per row; per row the BCE sum and the three F1 counters.
__global__ void sigmoid_bce_rows_kernel(const float *__restrict__ logits, const int64_t *__restrict__ label, int64_t B,
                                        int64_t C, float *dlogits, float4 *row_part) {
  const unsigned lane = threadIdx.x & 31;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const float inv_n = 1.0f / ((float)B * (float)C);
  for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < B; i += warps) {
    float loss = 0.0f, tp = 0.0f, pre = 0.0f, tru = 0.0f;
    for (int64_t c = lane; c < C; c += 32) {
      const float z = logits[i * C + c];
      const float p = 1.0f / (1.0f + expf(-z));
      const bool y = label[i * C + c] != 0;
      const float lp = fmaxf(logf(p), -100.0f), lq = fmaxf(logf(1.0f - p), -100.0f);
      loss -= y ? lp : lq;
      const bool pred = p > 0.5f;
      tp += (pred && y) ? 1.0f : 0.0f;
      pre += pred ? 1.0f : 0.0f;
      tru += y ? 1.0f : 0.0f;
      if (dlogits) {
        const float den = fmaxf((1.0f - p) * p, 1e-12f);
        dlogits[i * C + c] = (p - (y ? 1.0f : 0.0f)) / den * (p * (1.0f - p)) * inv_n;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      loss += __shfl_xor_sync(0xffffffffu, loss, o);
      tp += __shfl_xor_sync(0xffffffffu, tp, o);
      pre += __shfl_xor_sync(0xffffffffu, pre, o);
      tru += __shfl_xor_sync(0xffffffffu, tru, o);
    }
    if (lane == 0) row_part[i] = make_float4(loss, tp, pre, tru);
  }
}

// Fixed-shape reduction of the row partials: stats = {mean loss, predicted-and-true, predicted, true}.
__global__ void __launch_bounds__(1024) bce_reduce_kernel(const float4 *__restrict__ row_part, int64_t B, int64_t C,
                                                          float *stats) {
  __shared__ float4 sm[1024];
  float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (int64_t i = threadIdx.x; i < B; i += 1024) {
    const float4 r = row_part[i];
    a.x += r.x; a.y += r.y; a.z += r.z; a.w += r.w;
  }
  sm[threadIdx.x] = a;
  __syncthreads();
  for (int o = 512; o > 0; o >>= 1) {
    if (threadIdx.x < o) {
      float4 x = sm[threadIdx.x];
      const float4 y = sm[threadIdx.x + o];
      x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w;
      sm[threadIdx.x] = x;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    stats[0] = sm[0].x / ((float)B * (float)C);
    stats[1] = sm[0].y; stats[2] = sm[0].z; stats[3] = sm[0].w;
  }
}

// ------------------------------------------------------------------------------------ fused output layer
// Last GCN layer with one label per vertex: logits = Y W, softmax / NLL, dZ, dY = dZ W^T and the per-CTA part of
// dW = Y^T dZ in one launch; a second launch adds the parts up in CTA order and reduces loss and hits.  The layer is
// small (1,024 x 128 x 41 on the Reddit-shaped model) and was six launch-latency-bound kernels before.
// One warp per row.  Lane c (and c + 32) owns class c for the logits; lane h (+32q) owns hidden unit h for dY.
constexpr int kOutRows = 8;          // rows per CTA = warps per CTA
constexpr int kOutMaxC = 64;

// Where the aggregate of the last block comes from when the kernel forms it itself (x != nullptr) instead of reading it
// from y: row r of the aggregate = sum over the edges j of column r, in edge order, of fma(x[idx[j]], w_j, .) with
// w_j = 1 / (norm_idx[idx[j]] * norm_row[r]) - what nb_spmm_csc_fwd_fused computes, element for element.
struct OutAgg {
  const float *x;             // rows of the layer's input (H floats each, 16-byte aligned, pitch x_ld), or null
  size_t x_ld;
  const uint32_t *offs, *idx;
  const float *norm_idx, *norm_row;
};

__global__ void __launch_bounds__(kOutRows * 32) output_layer_rows_kernel(
    const float *__restrict__ y, const float *__restrict__ w, const int64_t *__restrict__ label_table,
    const uint32_t *__restrict__ dst, uint32_t B, uint32_t H, uint32_t C, uint32_t CP, int train, float *dy,
    float *dw_part, float *row_loss, float *row_hit, const OutAgg ag) {
  pdl_enter();
  extern __shared__ float out_smem[];
  float *ws = out_smem;                       // [H][CP]
  float *ys = ws + (size_t)H * CP;            // [kOutRows][H]
  float *dzs = ys + (size_t)kOutRows * H;     // [kOutRows][kOutMaxC]
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t row = blockIdx.x * kOutRows + warp;
  for (uint32_t i = threadIdx.x; i < H * C; i += blockDim.x) ws[(i / C) * CP + (i % C)] = w[i];
  if (row < B && ag.x != nullptr) {
    // the warp aggregates its row: lane holds float4 columns 4*lane + 128*t (H <= 256, a multiple of 4)
    const uint32_t start = __ldg(ag.offs + row), end = __ldg(ag.offs + row + 1);
    const float nr = __ldg(ag.norm_row + row);
    float2 acc[2][2];
#pragma unroll
    for (int t = 0; t < 2; t++) acc[t][0] = acc[t][1] = make_float2(0.0f, 0.0f);
    for (uint32_t base = start; base < end; base += 32) {
      const uint32_t j = base + lane;
      const float *my_ptr = nullptr;
      float my_w = 0.0f;
      if (j < end) {
        const uint32_t li = __ldg(ag.idx + j);
        my_w = __fdiv_rn(1.0f, __fmul_rn(__ldg(ag.norm_idx + li), nr));
        my_ptr = ag.x + (size_t)li * ag.x_ld;
      }
      const uint32_t cnt = min(32u, end - base);
      for (uint32_t jj = 0; jj < cnt; jj += 8) {
        float4 v[8][2];
        float wu[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
          const uintptr_t p = __shfl_sync(0xffffffffu, (unsigned long long)(uintptr_t)my_ptr, (jj + u) & 31);
          wu[u] = __shfl_sync(0xffffffffu, my_w, (jj + u) & 31);
          const bool valid = jj + u < cnt;
#pragma unroll
          for (int t = 0; t < 2; t++) {
            const uint32_t col = 4 * lane + 128 * t;
            v[u][t] = (valid && col < H) ? __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p) + col))
                                         : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          }
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
          if (jj + u < cnt) {
            const float2 w2 = make_float2(wu[u], wu[u]);
#pragma unroll
            for (int t = 0; t < 2; t++) {
              acc[t][0] = fma2_rn(make_float2(v[u][t].x, v[u][t].y), w2, acc[t][0]);
              acc[t][1] = fma2_rn(make_float2(v[u][t].z, v[u][t].w), w2, acc[t][1]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int t = 0; t < 2; t++) {
      const uint32_t col = 4 * lane + 128 * t;
      if (col < H) {
        ys[warp * H + col] = acc[t][0].x; ys[warp * H + col + 1] = acc[t][0].y;
        ys[warp * H + col + 2] = acc[t][1].x; ys[warp * H + col + 3] = acc[t][1].y;
      }
    }
  } else if (row < B) {
    for (uint32_t h = lane; h < H; h += 32) ys[warp * H + h] = y[(size_t)row * H + h];
  } else {
    for (uint32_t h = lane; h < H; h += 32) ys[warp * H + h] = 0.0f;
  }
  dzs[warp * kOutMaxC + lane] = 0.0f;
  dzs[warp * kOutMaxC + lane + 32] = 0.0f;
  __syncthreads();

  if (row < B) {
    const uint32_t c0 = lane, c1 = lane + 32;
    float z0 = 0.0f, z1 = 0.0f;
    for (uint32_t h = 0; h < H; h++) {
      const float yh = ys[warp * H + h];
      if (c0 < C) z0 = fmaf(yh, ws[h * CP + c0], z0);
      if (c1 < C) z1 = fmaf(yh, ws[h * CP + c1], z1);
    }
    // max / argmax (first maximum wins), log-sum-exp
    float m = c0 < C ? z0 : -INFINITY;
    uint32_t arg = c0;
    if (c1 < C && z1 > m) { m = z1; arg = c1; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const uint32_t oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (om > m || (om == m && oa < arg)) { m = om; arg = oa; }
    }
    float sum = (c0 < C ? expf(z0 - m) : 0.0f) + (c1 < C ? expf(z1 - m) : 0.0f);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float lse = logf(sum);
    const int64_t lab = label_table[dst[row]];
    const bool labelled = lab >= 0 && lab < (int64_t)C;
    const float z_lab = __shfl_sync(0xffffffffu, (lab >= 32) ? z1 : z0, (unsigned)(lab & 31));
    if (lane == 0) {
      if (!labelled) atomicOr(&g_loss_error, 1u);
      row_loss[row] = labelled ? -((z_lab - m) - lse) : 0.0f;
      row_hit[row] = (labelled && (int64_t)arg == lab) ? 1.0f : 0.0f;
    }
    if (train) {
      const float inv_b = labelled ? 1.0f / (float)B : 0.0f;   // a row without a valid label has no gradient
      if (c0 < C) dzs[warp * kOutMaxC + c0] = (expf(z0 - m - lse) - ((int64_t)c0 == lab ? 1.0f : 0.0f)) * inv_b;
      if (c1 < C) dzs[warp * kOutMaxC + c1] = (expf(z1 - m - lse) - ((int64_t)c1 == lab ? 1.0f : 0.0f)) * inv_b;
      __syncwarp();
      if (dy) {
        for (uint32_t h = lane; h < H; h += 32) {
          float acc = 0.0f;
          for (uint32_t c = 0; c < C; c++) acc = fmaf(dzs[warp * kOutMaxC + c], ws[h * CP + c], acc);
          dy[(size_t)row * H + h] = acc;
        }
      }
    }
  }
  if (!train) return;
  __syncthreads();
  // this CTA's part of dW = Y^T dZ: rows in order, one (h, c) pair per thread and step
  float *part = dw_part + (size_t)blockIdx.x * H * C;
  for (uint32_t i = threadIdx.x; i < H * C; i += blockDim.x) {
    const uint32_t h = i / C, c = i % C;
    float acc = 0.0f;
#pragma unroll
    for (int r = 0; r < kOutRows; r++) acc = fmaf(ys[r * H + h], dzs[r * kOutMaxC + c], acc);
    part[i] = acc;
  }
}

// Blocks 0 .. n-2: dW[i] = sum of the CTA parts in CTA order.  Last block: loss and hits, fixed-shape tree.
__global__ void __launch_bounds__(256) output_layer_reduce_kernel(const float *__restrict__ dw_part, uint32_t parts,
                                                                  uint32_t hc, float *dw, const float *__restrict__ row_loss,
                                                                  const float *__restrict__ row_hit, uint32_t B, float *stats) {
  pdl_enter();
  if (blockIdx.x + 1 < gridDim.x) {
    if (dw == nullptr) return;
    const uint32_t i = blockIdx.x * 256 + threadIdx.x;
    if (i >= hc) return;
    float acc = 0.0f;
    for (uint32_t p = 0; p < parts; p++) acc += dw_part[(size_t)p * hc + i];
    dw[i] = acc;
    return;
  }
  __shared__ float sl[256], sh[256];
  float l = 0.0f, h = 0.0f;
  for (uint32_t i = threadIdx.x; i < B; i += 256) { l += row_loss[i]; h += row_hit[i]; }
  sl[threadIdx.x] = l; sh[threadIdx.x] = h;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) { sl[threadIdx.x] += sl[threadIdx.x + o]; sh[threadIdx.x] += sh[threadIdx.x + o]; }
    __syncthreads();
  }
  if (threadIdx.x == 0) { stats[0] = sl[0] / (float)B; stats[1] = sh[0]; }
}

// ------------------------------------------------------------------------------------ Adam
__global__ void adam_kernel(float *W, const float *__restrict__ grad, float *M, float *V, int64_t n, float alpha,
                            float b1, float b2, float eps, float wd, float c1, float c2) {
  pdl_enter();
  const float one_m_b1 = 1.0f - b1, one_m_b2 = 1.0f - b2;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float w = W[i];
    const float g = __fadd_rn(grad[i], __fmul_rn(wd, w));
    const float m = __fadd_rn(__fmul_rn(b1, M[i]), __fmul_rn(one_m_b1, g));
    const float v = __fadd_rn(__fmul_rn(b2, V[i]), __fmul_rn(one_m_b2, __fmul_rn(g, g)));
    M[i] = m;
    V[i] = v;
    const float mt = __fdiv_rn(m, c1), vt = __fdiv_rn(v, c2);
    W[i] = __fsub_rn(w, __fdiv_rn(__fmul_rn(alpha, mt), __fadd_rn(__fsqrt_rn(vt), eps)));
  }
}

}  // namespace nb

using namespace nb;

NB_API int nb_gemm(nb_ws *ws, const float *d_a, const float *d_b, float *d_c, int64_t M, int64_t N, int64_t K,
                   int trans_a, int trans_b, void *stream_) {
  return nb::gemm_ld(ws, d_a, trans_a ? M : K, d_b, trans_b ? K : N, d_c, M, N, K, trans_a, trans_b, as_stream(stream_));
}

namespace nb {

bool gemm_uses_tensor_cores(int64_t M, int64_t N, int64_t K) {
  const bool tiny = 2.0 * (double)M * (double)N * (double)K < 4.0e7 && tuning().gemm_force_tc == 0;
  return tuning().gemm_mode != 0 && !tiny;
}

// nb_gemm with operand pitches (floats): A is stored with pitch lda >= its row length, B with ldb; C is dense.
int gemm_ld(nb_ws *ws, const float *d_a, int64_t lda, const float *d_b, int64_t ldb, float *d_c, int64_t M, int64_t N,
            int64_t K, int trans_a, int trans_b, cudaStream_t stream, const ReluEpi *epi, bool *applied) {
  if (applied) *applied = false;
  if (M == 0 || N == 0) return 0;
  NB_REQUIRE(d_a && d_b && d_c, "nb_gemm: null pointer");
  NB_REQUIRE(M > 0 && N > 0 && K >= 0, "nb_gemm: negative dimension");
  NB_REQUIRE(!(trans_a && trans_b), "nb_gemm: TT is not supported");
  NB_REQUIRE(lda >= (trans_a ? M : K) && ldb >= (trans_b ? K : N), "nb_gemm: pitch shorter than a row");
  if (K == 0) {
    NB_CUDA(cudaMemsetAsync(d_c, 0, (size_t)(M * N) * sizeof(float), stream));
    return 0;
  }
  // Small products (the output layer and its gradients) finish sooner on the CUDA cores than the
  // tensor-core kernel takes to set up its pipeline (TMEM allocation, 200 KB of staging buffers).
  if (gemm_uses_tensor_cores(M, N, K))
    return gemm_tensor_core(ws, d_a, lda, d_b, ldb, d_c, M, N, K, trans_a, trans_b, tuning().gemm_mode, stream, epi,
                            applied);
  GemmArgs g{};
  g.a = d_a; g.b = d_b; g.M = M; g.N = N; g.K = K;
  g.sa_i = trans_a ? 1 : lda;  g.sa_k = trans_a ? lda : 1;
  g.sb_k = trans_b ? 1 : ldb;  g.sb_j = trans_b ? ldb : 1;
  const int64_t tiles = ((M + kTM - 1) / kTM) * ((N + kTN - 1) / kTN);
  int splits = 1;
  if (tiles < 2 * num_sms() && K >= 4 * kTK * 8) {
    splits = (int)((2 * num_sms() + tiles - 1) / tiles);
    const int64_t max_splits = K / (kTK * 8);
    if (splits > max_splits) splits = (int)max_splits;
    if (splits < 1) splits = 1;
  }
  g.splits = splits;
  g.k_per_split = ((K + splits - 1) / splits + kTK - 1) / kTK * kTK;
  splits = (int)((K + g.k_per_split - 1) / g.k_per_split);
  g.splits = splits;
  WsScope scope(ws);
  float *partial = nullptr;
  if (splits > 1) {
    NB_REQUIRE(ws != nullptr, "nb_gemm: split-K needs a workspace");
    partial = ws->alloc_n<float>((size_t)splits * M * N);
    if (!partial) return fail(NB_ERR_NOMEM, "nb_gemm: workspace arena exhausted");
  }
  g.c = splits > 1 ? partial : d_c;
  dim3 grid((unsigned)((M + kTM - 1) / kTM), (unsigned)((N + kTN - 1) / kTN), (unsigned)splits);
  if (grid.y > 65535) return fail(NB_ERR_INVALID, "nb_gemm: N too large for one launch");
  gemm_simt_kernel<<<grid, 256, 0, stream>>>(g);
  NB_LAUNCH_CHECK();
  if (splits > 1) {
    splitk_reduce_kernel<<<grid_for(M * N, 256), 256, 0, stream>>>(partial, d_c, M * N, splits);
    NB_LAUNCH_CHECK();
  }
  return 0;
}

}  // namespace nb

namespace nb {
int read_loss_error_flag(unsigned int *value) {
  NB_CUDA(cudaMemcpyFromSymbol(value, g_loss_error, sizeof(unsigned int)));
  return 0;
}
int reset_loss_error_flag() {
  const unsigned int zero = 0;
  NB_CUDA(cudaMemcpyToSymbol(g_loss_error, &zero, sizeof(unsigned int)));
  return 0;
}
}  // namespace nb

NB_API int nb_set_gemm_mode(int mode) {
  nb::Tuning &t = nb::default_tuning();
  const int old = t.gemm_mode;
  if (mode >= 0 && mode <= 2) { t.gemm_mode = mode; t.gemm_force_tc = 0; }
  if (mode >= 16 && mode <= 18) { t.gemm_mode = mode - 16; t.gemm_force_tc = 1; }   // 17 / 18: tensor cores for every size
  return old;
}

NB_API int nb_relu_dropout(float *d_z, int64_t n, float p, uint64_t seed, uint32_t layer, uint32_t step,
                           void *stream) {
  if (n == 0) return 0;
  NB_REQUIRE(d_z != nullptr && n > 0, "nb_relu_dropout: null pointer");
  NB_REQUIRE(p >= 0.0f && p < 1.0f, "nb_relu_dropout: drop rate must be in [0,1)");
  const float scale = p > 0.0f ? 1.0f / (1.0f - p) : 1.0f;
  NB_CUDA(launch_chained(relu_dropout_kernel, dim3(grid_for((n + 3) / 4, 256)), dim3(256), 0, as_stream(stream), d_z, n, p, scale, (uint32_t)seed,
                         (uint32_t)(seed >> 32), layer, step));
  NB_LAUNCH_CHECK();
  return 0;
}

NB_API int nb_softmax_nll(nb_ws *ws, const float *d_logits, const int64_t *d_label, int64_t B, int64_t C,
                          float *d_dlogits, float *d_stats, void *stream_) {
  NB_REQUIRE(ws && d_logits && d_label && d_stats, "nb_softmax_nll: null pointer");
  NB_REQUIRE(B > 0 && C > 0, "nb_softmax_nll: empty batch or no classes");
  cudaStream_t stream = as_stream(stream_);
  WsScope scope(ws);
  float *row_loss = ws->alloc_n<float>((size_t)B);
  float *row_hit = ws->alloc_n<float>((size_t)B);
  if (!row_loss || !row_hit) return fail(NB_ERR_NOMEM, "nb_softmax_nll: workspace arena exhausted");
  softmax_nll_rows_kernel<<<grid_for((uint64_t)B * 32, 256), 256, 0, stream>>>(d_logits, d_label, B, C, d_dlogits,
                                                                               row_loss, row_hit);
  NB_LAUNCH_CHECK();
  loss_reduce_kernel<<<1, 1024, 0, stream>>>(row_loss, row_hit, B, d_stats);
  NB_LAUNCH_CHECK();
  return 0;
}

NB_API int nb_sigmoid_bce(nb_ws *ws, const float *d_logits, const int64_t *d_label, int64_t B, int64_t C,
                          float *d_dlogits, float *d_stats, void *stream_) {
  NB_REQUIRE(ws && d_logits && d_label && d_stats, "nb_sigmoid_bce: null pointer");
  NB_REQUIRE(B > 0 && C > 0, "nb_sigmoid_bce: empty batch or no classes");
  NB_REQUIRE((double)B * (double)C < 16777216.0, "nb_sigmoid_bce: more than 2^24 label slots in one batch");
  cudaStream_t stream = as_stream(stream_);
  WsScope scope(ws);
  float4 *row_part = ws->alloc_n<float4>((size_t)B);
  if (!row_part) return fail(NB_ERR_NOMEM, "nb_sigmoid_bce: workspace arena exhausted");
  sigmoid_bce_rows_kernel<<<grid_for((uint64_t)B * 32, 256), 256, 0, stream>>>(d_logits, d_label, B, C, d_dlogits,
                                                                               row_part);
  NB_LAUNCH_CHECK();
  bce_reduce_kernel<<<1, 1024, 0, stream>>>(row_part, B, C, d_stats);
  NB_LAUNCH_CHECK();
  return 0;
}

static size_t output_layer_smem(uint32_t H, uint32_t C) {
  const uint32_t CP = C | 1u;
  return ((size_t)H * CP + (size_t)kOutRows * H + (size_t)kOutRows * kOutMaxC) * sizeof(float);
}

NB_API int nb_output_layer_supported(uint32_t H, uint32_t C) {
  return (H > 0 && C > 0 && C <= (uint32_t)kOutMaxC && output_layer_smem(H, C) <= 96 * 1024) ? 1 : 0;
}

namespace nb {
static int output_layer_impl(nb_ws *ws, const float *d_y, const OutAgg &ag, const float *d_w, const int64_t *d_label,
                             const uint32_t *d_dst, uint32_t B, uint32_t H, uint32_t C, int train, float *d_dw, float *d_dy,
                             float *d_stats, void *stream_);

// nb_output_layer with the aggregation of the last block done by the same kernel: the aggregate never goes to memory.
bool output_layer_can_aggregate(const float *d_x, size_t x_ld, uint32_t H, uint32_t C) {
  return nb_output_layer_supported(H, C) && H <= 256 && (H & 3) == 0 && (x_ld & 3) == 0 &&
         (reinterpret_cast<uintptr_t>(d_x) & 15) == 0;
}
int output_layer_aggregating(nb_ws *ws, const float *d_x, size_t x_ld, const uint32_t *d_row_indices,
                             const uint32_t *d_column_offset, const float *d_src_norm, const float *d_dst_norm,
                             const float *d_w, const int64_t *d_label, const uint32_t *d_dst, uint32_t B, uint32_t H,
                             uint32_t C, int train, float *d_dw, float *d_dy, float *d_stats, void *stream) {
  NB_REQUIRE(d_x && d_row_indices && d_column_offset && d_src_norm && d_dst_norm, "nb_output_layer: null pointer");
  NB_REQUIRE(output_layer_can_aggregate(d_x, x_ld, H, C), "nb_output_layer: rows not usable by the aggregating form");
  OutAgg ag{d_x, x_ld, d_column_offset, d_row_indices, d_src_norm, d_dst_norm};
  return output_layer_impl(ws, nullptr, ag, d_w, d_label, d_dst, B, H, C, train, d_dw, d_dy, d_stats, stream);
}
}  // namespace nb

NB_API int nb_output_layer(nb_ws *ws, const float *d_y, const float *d_w, const int64_t *d_label, const uint32_t *d_dst,
                           uint32_t B, uint32_t H, uint32_t C, int train, float *d_dw, float *d_dy, float *d_stats,
                           void *stream_) {
  NB_REQUIRE(d_y != nullptr, "nb_output_layer: null pointer");
  return nb::output_layer_impl(ws, d_y, nb::OutAgg{}, d_w, d_label, d_dst, B, H, C, train, d_dw, d_dy, d_stats, stream_);
}

namespace nb {
static int output_layer_impl(nb_ws *ws, const float *d_y, const OutAgg &ag, const float *d_w, const int64_t *d_label,
                             const uint32_t *d_dst, uint32_t B, uint32_t H, uint32_t C, int train, float *d_dw, float *d_dy,
                             float *d_stats, void *stream_) {
  NB_REQUIRE(ws && d_w && d_label && d_dst && d_stats, "nb_output_layer: null pointer");
  NB_REQUIRE(B > 0, "nb_output_layer: empty batch");
  NB_REQUIRE(nb_output_layer_supported(H, C), "nb_output_layer: layer too wide for the fused form (C <= 64, H*C*4 <= ~90 KB)");
  NB_REQUIRE(!train || d_dw, "nb_output_layer: training needs the weight-gradient buffer");
  cudaStream_t stream = as_stream(stream_);
  WsScope scope(ws);
  const uint32_t ctas = (B + kOutRows - 1) / kOutRows, hc = H * C;
  float *row_loss = ws->alloc_n<float>(B), *row_hit = ws->alloc_n<float>(B);
  float *part = train ? ws->alloc_n<float>((size_t)ctas * hc) : nullptr;
  if (!row_loss || !row_hit || (train && !part)) return fail(NB_ERR_NOMEM, "nb_output_layer: workspace arena exhausted");
  const size_t smem = output_layer_smem(H, C);
  static PerDeviceOnce configured;   // the attribute is kept per device
  if (configured.need()) {
    NB_CUDA(cudaFuncSetAttribute(output_layer_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    configured.done();
  }
  NB_CUDA(launch_chained(output_layer_rows_kernel, dim3(ctas), dim3(kOutRows * 32), smem, stream, d_y, d_w, d_label, d_dst, B,
                         H, C, C | 1u, train ? 1 : 0, train ? d_dy : (float *)nullptr, part, row_loss, row_hit, ag));
  NB_LAUNCH_CHECK();
  const unsigned blocks = (train ? (hc + 255) / 256 : 0) + 1;
  NB_CUDA(launch_chained(output_layer_reduce_kernel, dim3(blocks), dim3(256), 0, stream, (const float *)part, ctas, hc,
                         train ? d_dw : (float *)nullptr, (const float *)row_loss, (const float *)row_hit, B, d_stats));
  NB_LAUNCH_CHECK();
  return 0;
}
}  // namespace nb

NB_API int nb_set_pdl(int enabled) {
  const int old = nb::default_tuning().use_pdl;
  nb::default_tuning().use_pdl = enabled != 0;
  return old;
}

NB_API int nb_adam(float *d_W, const float *d_grad, float *d_M, float *d_V, int64_t n, float alpha, float b1,
                   float b2, float eps, float wd, float b1_t, float b2_t, void *stream) {
  if (n == 0) return 0;
  NB_REQUIRE(d_W && d_grad && d_M && d_V && n > 0, "nb_adam: null pointer");
  NB_CUDA(launch_chained(adam_kernel, dim3(grid_for(n, 256)), dim3(256), 0, as_stream(stream), d_W, d_grad, d_M, d_V, n, alpha,
                         b1, b2, eps, wd, 1.0f - b1_t, 1.0f - b2_t));
  NB_LAUNCH_CHECK();
  return 0;
}

// ------------------------------------------------------------------------------------ loss without a workspace
// Some hosts of this library cannot hand it scratch memory at call time: a serving or training process
// that gave the whole device to its own pool at start-up (a later cudaMalloc fails or fragments the
// pool), or a plugin slot whose contract forbids allocation once initialisation is over.  For them the
// loss is also available with its per-row scratch in a fixed device array that is part of the library
// image: every GPU that loads the library carries these 512 KiB until the process exits.
constexpr int64_t kNoAllocMaxRows = 65536;
static __device__ __align__(256) float g_loss_scratch[2 * kNoAllocMaxRows];   // [row_loss | row_hit]

namespace {
float *g_loss_scratch_addr[nb::kMaxDevices] = {};   // device address of g_loss_scratch, per device
}  // namespace

// In host code `g_loss_scratch` names a host-side shadow of the symbol, not device memory, so the
// device address has to be asked for once per device, with that device current.
static int loss_scratch_address(float **out) {
  int dev = -1;
  NB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= nb::kMaxDevices) return nb::fail(NB_ERR_INVALID, "nb_softmax_nll_static: device index out of range");
  float *p = __atomic_load_n(&g_loss_scratch_addr[dev], __ATOMIC_ACQUIRE);
  if (p == nullptr) {
    void *addr = nullptr;
    NB_CUDA(cudaGetSymbolAddress(&addr, g_loss_scratch));
    p = static_cast<float *>(addr);
    __atomic_store_n(&g_loss_scratch_addr[dev], p, __ATOMIC_RELEASE);   // same value from any racing thread
  }
  *out = p;
  return 0;
}

NB_API int nb_softmax_nll_static(const float *d_logits, const int64_t *d_label, int64_t B, int64_t C,
                                 float *d_dlogits, float *d_stats, void *stream_) {
  NB_REQUIRE(d_logits && d_label && d_stats, "nb_softmax_nll_static: null pointer");
  NB_REQUIRE(B > 0 && C > 0, "nb_softmax_nll_static: empty batch or no classes");
  if (B > kNoAllocMaxRows) {
    nb::set_error("nb_softmax_nll_static: batch of %lld rows exceeds the built-in scratch of %lld rows; "
                  "use nb_softmax_nll with a workspace", (long long)B, (long long)kNoAllocMaxRows);
    return NB_ERR_INVALID;
  }
  float *scratch = nullptr;
  NB_TRY(loss_scratch_address(&scratch));
  float *row_loss = scratch, *row_hit = scratch + kNoAllocMaxRows;
  cudaStream_t stream = nb::as_stream(stream_);
  // Rows 0..B-1 of both halves are fully rewritten below before they are read, so nothing left over
  // from an earlier call (of any batch size) can leak into this one; no clearing is needed.
  nb::softmax_nll_rows_kernel<<<nb::grid_for((uint64_t)B * 32, 256), 256, 0, stream>>>(d_logits, d_label, B, C,
                                                                                    d_dlogits, row_loss, row_hit);
  NB_LAUNCH_CHECK();
  nb::loss_reduce_kernel<<<1, 1024, 0, stream>>>(row_loss, row_hit, B, d_stats);
  NB_LAUNCH_CHECK();
  return 0;
}
