/*
 * CPU oracle for the sampled mini-batch GCN path of NeutronBench (toolkit GCN_GPU_NEIGHBOR /
 * GCN_CPU_NEIGHBOR).  TEST INFRASTRUCTURE ONLY: it is the checker the CUDA path is compared with and
 * the timed host-CPU baseline; nothing shipped may call it.
 *
 * It is a plain-C restatement (not a copy) of the reference algorithms.  Every function cites the
 * reference file:line it follows (paths are relative to the reference project root).  Integer outputs
 * are meant to be bit-identical to the reference's; floating-point kernels use the reference's
 * operation order (multiply, then add, edge by edge) and are compiled with -ffp-contract=off so that
 * no fused multiply-add changes the rounding.
 *
 * Pinning: the reference has no golden vectors of its own (its test/ directory only prints tensors).
 * This file is pinned against outputs of the reference's own headers compiled with single-rank shims
 * (oracle/ref_harness.cpp -> oracle/_ref/), stored as fixtures under tests/golden/.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

typedef uint32_t vid_t; /* dep/gemini/type.hpp:28  VertexId = uint32_t */

/* --------------------------------------------------------------------------------------------
 * a1  Whole-graph CSC from the binary edge list.
 * core/FullyRepGraph.hpp:485-560 (ReadRepGraphFromRawFile): pass 1 counts in-edges per destination,
 * prefix sum, pass 2 places each source at the cursor of its destination, in file order (stable).
 * `edges` holds E pairs (src,dst) of little-endian u32 exactly as the .edge file does
 * (core/graph.hpp:1059-1060).  Offsets are 64-bit here so that graphs with more than 2^32 edges fit
 * (the reference keeps 32-bit offsets, core/FullyRepGraph.hpp:424).
 * ------------------------------------------------------------------------------------------ */
ORC_API void orc_build_csc(const vid_t *edges, uint64_t E, vid_t V, uint64_t *column_offset /*V+1*/,
                           vid_t *row_indices /*E*/) {
  uint64_t *cursor = (uint64_t *)calloc((size_t)V + 1, sizeof(uint64_t));
  for (uint64_t e = 0; e < E; e++) cursor[edges[2 * e + 1] + 1]++;
  for (vid_t i = 0; i < V; i++) cursor[i + 1] += cursor[i];
  memcpy(column_offset, cursor, ((size_t)V + 1) * sizeof(uint64_t));
  for (uint64_t e = 0; e < E; e++) row_indices[cursor[edges[2 * e + 1]]++] = edges[2 * e];
  free(cursor);
}

/* In/out degree arrays as Graph::load_directed fills them (core/graph.hpp:1050-1440), with the
 * clamp to >= 1 that generate_backward_structure applies (core/graph.hpp:3983-3986).  The degree
 * cache policy sorts by out_degree_for_backward (toolkits/GCN_GPU_NEIGHBOR.hpp:940-943). */
ORC_API void orc_degrees(const vid_t *edges, uint64_t E, vid_t V, vid_t *out_degree, vid_t *in_degree,
                         int clamp_to_one) {
  memset(out_degree, 0, (size_t)V * sizeof(vid_t));
  memset(in_degree, 0, (size_t)V * sizeof(vid_t));
  for (uint64_t e = 0; e < E; e++) {
    out_degree[edges[2 * e]]++;
    in_degree[edges[2 * e + 1]]++;
  }
  if (clamp_to_one)
    for (vid_t i = 0; i < V; i++) {
      if (out_degree[i] == 0) out_degree[i] = 1;
      if (in_degree[i] == 0) in_degree[i] = 1;
    }
}

/* --------------------------------------------------------------------------------------------
 * a2  Per-hop column offsets.
 * core/FullyRepGraph.hpp:199-209 (init_co) with the neighbour-count rule of
 * core/ntsSampler.hpp:914-923: min(deg, fanout), or deg when fanout < 0.  Returns e (edge count).
 * ------------------------------------------------------------------------------------------ */
ORC_API vid_t orc_init_co(const uint64_t *g_column_offset, const vid_t *dst, vid_t v, int fanout,
                          vid_t *column_offset /*v+1*/) {
  vid_t off = 0;
  for (vid_t i = 0; i < v; i++) {
    column_offset[i] = off;
    int64_t nbrs = (int64_t)(g_column_offset[dst[i] + 1] - g_column_offset[dst[i]]);
    off += (vid_t)((fanout < 0) ? nbrs : (nbrs < fanout ? nbrs : fanout));
  }
  column_offset[v] = off;
  return off;
}

/* SAMPLE_RATE mode of the training sampler (core/ntsSampler.hpp:901-912): per destination
 * max(int(nbrs * sample_rate), min(lower_fanout, nbrs)); the product is a float multiply truncated to int. */
ORC_API vid_t orc_init_co_rate(const uint64_t *g_column_offset, const vid_t *dst, vid_t v, float sample_rate,
                               int lower_fanout, vid_t *column_offset /*v+1*/) {
  vid_t off = 0;
  for (vid_t i = 0; i < v; i++) {
    column_offset[i] = off;
    int nbrs = (int)(g_column_offset[dst[i] + 1] - g_column_offset[dst[i]]);
    int lower = lower_fanout < nbrs ? lower_fanout : nbrs;
    int by_rate = (int)((float)nbrs * sample_rate);
    int k = by_rate > lower ? by_rate : lower;
    if (k > nbrs) k = nbrs;
    if (k < 0) k = 0;
    off += (vid_t)k;
  }
  column_offset[v] = off;
  return off;
}

/* --------------------------------------------------------------------------------------------
 * Counter-based random numbers: Philox4x32-10 (Salmon et al., SC'11), the published algorithm.
 * The reference draws from a thread-local std::mt19937(2000) under OpenMP (utils/rand.hpp:6-13), so
 * which edges it samples depends on thread scheduling; parity on sampling is therefore defined on
 * identical sampled edge lists, and this generator only has to match the CUDA sampler's.
 * ------------------------------------------------------------------------------------------ */
static inline void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                 uint32_t k1, uint32_t out[4]) {
  for (int r = 0; r < 10; r++) {
    uint64_t p0 = (uint64_t)0xD2511F53u * c0;
    uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
    uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
    uint32_t n1 = (uint32_t)p1;
    uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
    uint32_t n3 = (uint32_t)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

ORC_API void orc_philox(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1,
                        uint32_t *out4) {
  philox4x32_10(c0, c1, c2, c3, k0, k1, out4);
}

/* Uniform integer in [0, n) from one 32-bit word: multiply-shift (Lemire, without the rejection
 * step; bias < n / 2^32). */
static inline uint32_t bounded(uint32_t r, uint32_t n) { return (uint32_t)(((uint64_t)r * n) >> 32); }

/* --------------------------------------------------------------------------------------------
 * a2  Fan-out sampling of one hop.
 * core/ntsSampler.hpp:936-1042: a destination whose degree exceeds the fanout gets `fanout` DISTINCT
 * neighbour positions drawn uniformly (the reference rejects duplicates with an unordered_set,
 * :998-1005); otherwise all neighbours are copied in CSC order (:1033-1040).  Global source ids are
 * written to row_indices and their bits set in the hop's bitmap.
 * The distinct positions are drawn with Floyd's subset algorithm from the stream
 * Philox(counter = (draw/4, local dst index, hop, 0), key = (seed_lo, seed_hi)); position t of the
 * subset uses draw t.  Within a column the order is Floyd's insertion order.
 * ------------------------------------------------------------------------------------------ */
#define ORC_FLOYD_MAX 128u
ORC_API void orc_sample_hop(const uint64_t *g_column_offset, const vid_t *g_row_indices,
                            const vid_t *dst, vid_t v, int fanout, const vid_t *column_offset,
                            uint64_t seed, uint32_t hop, vid_t *row_indices /*e, global ids*/) {
  for (vid_t i = 0; i < v; i++) {
    uint64_t base = g_column_offset[dst[i]];
    uint32_t deg = (uint32_t)(g_column_offset[dst[i] + 1] - base);
    vid_t pos = column_offset[i];
    uint32_t k = column_offset[i + 1] - pos;
    (void)fanout;   /* the counts in column_offset already carry the fan-out rule */
    if (k >= deg) {
      for (uint32_t j = 0; j < deg; j++) row_indices[pos + j] = g_row_indices[base + j];
      continue;
    }
    if (k > ORC_FLOYD_MAX) {
      /* Large subsets (SAMPLE_RATE on hub vertices): selection sampling, one draw per neighbour in
       * column order, stream tag 2 in the fourth counter word; picks exactly k, ascending positions. */
      uint32_t r[4], m = 0;
      for (uint32_t j = 0; j < deg && m < k; j++) {
        if ((j & 3) == 0) philox4x32_10(j >> 2, i, hop, 2, (uint32_t)seed, (uint32_t)(seed >> 32), r);
        if (bounded(r[j & 3], deg - j) < k - m) row_indices[pos + m++] = g_row_indices[base + j];
      }
      continue;
    }
    uint32_t *chosen = (uint32_t *)malloc(sizeof(uint32_t) * k);
    uint32_t r[4];
    for (uint32_t t = 0; t < k; t++) {
      if ((t & 3) == 0) philox4x32_10(t >> 2, i, hop, 0, (uint32_t)seed, (uint32_t)(seed >> 32), r);
      uint32_t j = deg - k + t;          /* Floyd: candidate range grows by one each draw */
      uint32_t c = bounded(r[t & 3], j + 1);
      for (uint32_t q = 0; q < t; q++)
        if (chosen[q] == c) { c = j; break; }
      chosen[t] = c;
      row_indices[pos + t] = g_row_indices[base + c];
    }
    free(chosen);
  }
}

/* --------------------------------------------------------------------------------------------
 * a3  Dedup + reindex of one hop.
 * core/ntsSampler.hpp:1004,1039 (bitmap marks) and core/coocsc.hpp:338-425 (postprocessing):
 * source[] = set bits of the |V|-bit bitmap in ascending id order (the reference scans 64-bit words
 * low bit first, :373-391), node_idx[g] = rank, row_indices[j] = node_idx[row_indices[j]].
 * Returns src_size.
 * ------------------------------------------------------------------------------------------ */
ORC_API vid_t orc_dedup_reindex(vid_t V, vid_t *row_indices /*e: global in, local out*/, vid_t e,
                                vid_t *source /*<= min(V,e)*/) {
  size_t words = ((size_t)V >> 6) + 1; /* dep/gemini/bitmap.hpp:27 */
  uint64_t *bits = (uint64_t *)calloc(words, sizeof(uint64_t));
  vid_t *node_idx = (vid_t *)malloc((size_t)V * sizeof(vid_t));
  for (vid_t j = 0; j < e; j++) bits[row_indices[j] >> 6] |= 1ull << (row_indices[j] & 63);
  vid_t s = 0;
  for (size_t w = 0; w < words; w++) {
    uint64_t word = bits[w];
    vid_t id = (vid_t)(w << 6);
    while (word) {
      if (word & 1) {
        source[s] = id;
        node_idx[id] = s++;
      }
      id++;
      word >>= 1;
    }
  }
  for (vid_t j = 0; j < e; j++) row_indices[j] = node_idx[row_indices[j]];
  free(bits);
  free(node_idx);
  return s;
}

/* --------------------------------------------------------------------------------------------
 * a4  CSR of the block from its CSC (transpose by stable counting sort).
 * core/coocsc.hpp:243-309 (generate_csr_from_csc): count per local source, prefix sum, then walk
 * destinations in order so every source row lists its local destinations in ascending order.
 * ------------------------------------------------------------------------------------------ */
ORC_API void orc_csr_from_csc(const vid_t *column_offset, const vid_t *row_indices, vid_t v, vid_t s,
                              vid_t *row_offset /*s+1*/, vid_t *column_indices /*e*/) {
  vid_t e = column_offset[v];
  memset(row_offset, 0, ((size_t)s + 1) * sizeof(vid_t));
  for (vid_t j = 0; j < e; j++) row_offset[row_indices[j] + 1]++;
  for (vid_t i = 1; i <= s; i++) row_offset[i] += row_offset[i - 1];
  for (vid_t i = 0; i < v; i++)
    for (vid_t j = column_offset[i]; j < column_offset[i + 1]; j++)
      column_indices[row_offset[row_indices[j]]++] = i;
  for (vid_t i = s; i > 0; i--) row_offset[i] = row_offset[i - 1];
  row_offset[0] = 0;
}

/* --------------------------------------------------------------------------------------------
 * a5  GCN edge weights of the block.
 * core/coocsc.hpp:166-216 (update_degree): in-degree of a destination = its column length, out-degree
 * of a source = its CSR row length (degrees of the SAMPLED block).  core/ntsBaseOp.hpp:183-186
 * (nts_norm_degree): 1 / ((float)sqrt(out[src]) * (float)sqrt(in[dst])), square roots taken in double
 * (std::sqrt on an integer) and rounded to float before the float multiply.
 * core/coocsc.hpp:136-163: forward weights in CSC order, backward weights in CSR order.
 * src_norm/dst_norm receive the per-vertex (float)sqrt(degree) factors.
 * ------------------------------------------------------------------------------------------ */
ORC_API void orc_block_weights(const vid_t *column_offset, const vid_t *row_indices,
                               const vid_t *row_offset, const vid_t *column_indices, vid_t v, vid_t s,
                               float *src_norm /*s*/, float *dst_norm /*v*/, float *w_fwd /*e*/,
                               float *w_bwd /*e*/) {
  for (vid_t i = 0; i < s; i++) src_norm[i] = (float)sqrt((double)(row_offset[i + 1] - row_offset[i]));
  for (vid_t i = 0; i < v; i++)
    dst_norm[i] = (float)sqrt((double)(column_offset[i + 1] - column_offset[i]));
  if (w_fwd)
    for (vid_t i = 0; i < v; i++)
      for (vid_t j = column_offset[i]; j < column_offset[i + 1]; j++)
        w_fwd[j] = 1.0f / (src_norm[row_indices[j]] * dst_norm[i]);
  if (w_bwd)
    for (vid_t i = 0; i < s; i++)
      for (vid_t j = row_offset[i]; j < row_offset[i + 1]; j++)
        w_bwd[j] = 1.0f / (src_norm[i] * dst_norm[column_indices[j]]);
}

/* --------------------------------------------------------------------------------------------
 * a9  Forward aggregation  Y[d,:] = sum_j w_fwd[j] * X[row_indices[j],:]  over column d.
 * core/ntsMiniBatchGraphOp.hpp:154-184 (MiniBatchFuseOp::forward) with nts_comp
 * (core/ntsBaseOp.hpp:76-97): output += input * weight, edge after edge in CSC order, into a zeroed
 * output.  The reference builds with -O3 -march=native, where its _mm256_add_ps(_mm256_mul_ps(..)) and the
 * scalar tail are contracted into fused multiply-adds, so the operator's arithmetic is
 * out = fma(in, w, out) per element (single rounding): restated here with fmaf, which reproduces the
 * compiled reference bit for bit (tests/test_golden_cpu.py).  The reference's GPU kernel
 * (cuda/ntsCUDAFuseKernel.cuh:272-290) rounds the product before its atomicAdd and so differs from the
 * reference's own CPU operator in the last bit of some sums.
 * ------------------------------------------------------------------------------------------ */
ORC_API void orc_spmm_fwd(const float *x, float *y, const float *w, const vid_t *row_indices,
                          const vid_t *column_offset, vid_t v, vid_t F) {
#pragma omp parallel for schedule(dynamic, 64)
  for (vid_t d = 0; d < v; d++) {
    float *out = y + (size_t)d * F;
    for (vid_t k = 0; k < F; k++) out[k] = 0.0f;
    for (vid_t j = column_offset[d]; j < column_offset[d + 1]; j++) {
      const float *in = x + (size_t)row_indices[j] * F;
      float wj = w[j];
      for (vid_t k = 0; k < F; k++) out[k] = fmaf(in[k], wj, out[k]);
    }
  }
}

/* --------------------------------------------------------------------------------------------
 * a10 Backward aggregation  gX[s,:] = sum_j w_bwd[j] * gY[column_indices[j],:]  over CSR row s.
 * core/ntsMiniBatchGraphOp.hpp:214-240 (pull mode) ; GPU kernel cuda/ntsCUDAFuseKernel.cuh:450-468.
 * `act` (nullable, s x F) fuses the gradient of dropout(relu(.)) that follows in the chain rule:
 * the sum is multiplied by `scale` where act > 0 and zeroed elsewhere
 * (toolkits/GCN_GPU_NEIGHBOR.hpp:715-728 is the forward this differentiates).
 * ------------------------------------------------------------------------------------------ */
ORC_API void orc_spmm_bwd(const float *gy, float *gx, const float *w, const vid_t *row_offset,
                          const vid_t *column_indices, vid_t s, vid_t F, const float *act,
                          float scale) {
#pragma omp parallel for schedule(dynamic, 64)
  for (vid_t r = 0; r < s; r++) {
    float *out = gx + (size_t)r * F;
    for (vid_t k = 0; k < F; k++) out[k] = 0.0f;
    for (vid_t j = row_offset[r]; j < row_offset[r + 1]; j++) {
      const float *in = gy + (size_t)column_indices[j] * F;
      float wj = w[j];
      for (vid_t k = 0; k < F; k++) out[k] = fmaf(in[k], wj, out[k]);
    }
    if (act) {
      const float *a = act + (size_t)r * F;
      for (vid_t k = 0; k < F; k++) out[k] = a[k] > 0.0f ? out[k] * scale : 0.0f;
    }
  }
}

/* --------------------------------------------------------------------------------------------
 * a7  Feature gather  X0[i,:] = feat[source[i],:].
 * core/ntsSampler.hpp:364-376 + cuda/ntsCUDATransferKernel.cuh:96-108 (no cache) and
 * core/ntsSampler.hpp:424-469 + cuda/ntsCUDATransferKernel.cuh:153-182 (cache: a row whose
 * cache_node_hashmap entry is not 0xFFFFFFFF is read from cache slot hashmap[id]).  CPU twin:
 * core/ntsMiniBatchGraphOp.hpp:77-91.
 * ------------------------------------------------------------------------------------------ */
ORC_API void orc_feature_gather(float *x0, const float *feat, const vid_t *source, vid_t n, vid_t F,
                                const float *cache, const vid_t *hashmap) {
#pragma omp parallel for
  for (vid_t i = 0; i < n; i++) {
    vid_t g = source[i];
    const float *row = (cache && hashmap && hashmap[g] != 0xFFFFFFFFu) ? cache + (size_t)hashmap[g] * F
                                                                      : feat + (size_t)g * F;
    memcpy(x0 + (size_t)i * F, row, (size_t)F * sizeof(float));
  }
}

/* a8  Label gather lab[i] = label[dst[i]]  (core/ntsSampler.hpp:501-529,
 * cuda/ntsCUDATransferKernel.cuh:184-203; label_size > 1 copies rows of a multi-label matrix). */
ORC_API void orc_label_gather(int64_t *lab, const int64_t *label, const vid_t *dst, vid_t n,
                              vid_t label_size) {
  for (vid_t i = 0; i < n; i++)
    for (vid_t k = 0; k < label_size; k++)
      lab[(size_t)i * label_size + k] = label[(size_t)dst[i] * label_size + k];
}

/* Degree-ordered cache map: toolkits/GCN_GPU_NEIGHBOR.hpp:919-943,1214-1243.  Nodes sorted by
 * descending out degree; the first cache_num get slots 0..cache_num-1, everyone else 0xFFFFFFFF.
 * std::sort leaves the order of equal degrees unspecified; ties are broken here by ascending id. */
typedef struct { vid_t deg, id; } deg_id_t;
static int cmp_deg_desc(const void *a, const void *b) {
  const deg_id_t *x = (const deg_id_t *)a, *y = (const deg_id_t *)b;
  if (x->deg != y->deg) return x->deg > y->deg ? -1 : 1;
  return x->id < y->id ? -1 : (x->id > y->id);
}
ORC_API void orc_cache_by_degree(const vid_t *out_degree, vid_t V, vid_t cache_num, vid_t *hashmap /*V*/,
                                 vid_t *cache_ids /*cache_num*/) {
  deg_id_t *a = (deg_id_t *)malloc((size_t)V * sizeof(deg_id_t));
  for (vid_t i = 0; i < V; i++) { a[i].deg = out_degree[i]; a[i].id = i; }
  qsort(a, V, sizeof(deg_id_t), cmp_deg_desc);
  for (vid_t i = 0; i < V; i++) hashmap[i] = 0xFFFFFFFFu;
  for (vid_t i = 0; i < cache_num && i < V; i++) { hashmap[a[i].id] = i; cache_ids[i] = a[i].id; }
  free(a);
}

/* --------------------------------------------------------------------------------------------
 * a11 Dense layer, loss and their gradients.
 * Parameter::forward  x.mm(W)                                   core/NtsScheduler.hpp:712-715
 * vertexForward       dropout(relu(Y*W)), last layer Y*W        toolkits/GCN_GPU_NEIGHBOR.hpp:715-728
 * Loss                nll_loss(log_softmax(out,1), target) mean utils/torch_func.hpp:67-82
 * get_correct         argmax(1) == target                       utils/torch_func.hpp:11-29
 * Dropout keeps element i of layer l at step t when the Philox word
 * Philox(counter = (i/4, l, t, 1), key = seed)[i%4] scaled to [0,1) is >= p, and multiplies the kept
 * value by 1/(1-p) (torch::dropout semantics; the reference's mask comes from libtorch's own
 * generator, so mask-level parity with the reference needs DROP_RATE:0).
 * ------------------------------------------------------------------------------------------ */
ORC_API void orc_gemm_nn(const float *a, const float *b, float *c, int64_t M, int64_t K, int64_t N) {
#pragma omp parallel for
  for (int64_t i = 0; i < M; i++) {
    float *ci = c + i * N;
    for (int64_t n = 0; n < N; n++) ci[n] = 0.0f;
    for (int64_t k = 0; k < K; k++) {
      float aik = a[i * K + k];
      const float *bk = b + k * N;
      for (int64_t n = 0; n < N; n++) ci[n] += aik * bk[n];
    }
  }
}

/* C[K x N] = A^T[K x M] * B[M x N]  (weight gradient Y^T dZ), accumulated in double. */
ORC_API void orc_gemm_tn(const float *a, const float *b, float *c, int64_t M, int64_t K, int64_t N) {
  double *acc = (double *)calloc((size_t)(K * N), sizeof(double));
  for (int64_t i = 0; i < M; i++)
    for (int64_t k = 0; k < K; k++) {
      double aik = a[i * K + k];
      if (aik == 0.0) continue;
      const float *bi = b + i * N;
      double *ck = acc + k * N;
      for (int64_t n = 0; n < N; n++) ck[n] += aik * bi[n];
    }
  for (int64_t i = 0; i < K * N; i++) c[i] = (float)acc[i];
  free(acc);
}

/* C[M x K] = A[M x N] * B^T  with B[K x N]  (input gradient dZ W^T). */
ORC_API void orc_gemm_nt(const float *a, const float *b, float *c, int64_t M, int64_t N, int64_t K) {
#pragma omp parallel for
  for (int64_t i = 0; i < M; i++)
    for (int64_t k = 0; k < K; k++) {
      float acc = 0.0f;
      for (int64_t n = 0; n < N; n++) acc += a[i * N + n] * b[k * N + n];
      c[i * K + k] = acc;
    }
}

ORC_API void orc_relu_dropout(float *z, int64_t n, float p, uint64_t seed, uint32_t layer,
                              uint32_t step) {
  float scale = p > 0.0f ? 1.0f / (1.0f - p) : 1.0f;
  uint32_t r[4];
  for (int64_t i = 0; i < n; i++) {
    float val = z[i] > 0.0f ? z[i] : 0.0f;
    if (p > 0.0f) {
      if ((i & 3) == 0)
        philox4x32_10((uint32_t)(i >> 2), layer, step, 1, (uint32_t)seed, (uint32_t)(seed >> 32), r);
      float u = (float)(r[i & 3] >> 8) * (1.0f / 16777216.0f);
      val = (u >= p) ? val * scale : 0.0f;
    }
    z[i] = val;
  }
}

/* Returns the mean NLL loss; writes dlogits = (softmax - onehot)/B and the number of correct
 * argmax predictions. */
ORC_API float orc_softmax_nll(const float *logits, const int64_t *label, int64_t B, int64_t C,
                              float *dlogits, int64_t *correct) {
  double loss = 0.0;
  int64_t ok = 0;
  for (int64_t i = 0; i < B; i++) {
    const float *z = logits + i * C;
    float m = z[0];
    int64_t arg = 0;
    for (int64_t c = 1; c < C; c++)
      if (z[c] > m) { m = z[c]; arg = c; }
    double sum = 0.0;
    for (int64_t c = 0; c < C; c++) sum += exp((double)(z[c] - m));
    double lse = log(sum);
    loss += -((double)(z[label[i]] - m) - lse);
    if (arg == label[i]) ok++;
    if (dlogits)
      for (int64_t c = 0; c < C; c++) {
        double pr = exp((double)(z[c] - m) - lse);
        dlogits[i * C + c] = (float)((pr - (c == label[i] ? 1.0 : 0.0)) / (double)B);
      }
  }
  if (correct) *correct = ok;
  return (float)(loss / (double)B);
}

/* Multi-label loss and F1 counters (CLASSES > 1): Loss = binary_cross_entropy(sigmoid(z), y), mean over all
 * B*C elements with each log clamped at -100 (utils/torch_func.hpp:67-75; the clamp is libtorch's);
 * dlogits follows libtorch's backward pair: (p - y) / max((1 - p) p, 1e-12) * p (1 - p) / (B*C).
 * counters (utils/torch_func.hpp:31-60, f1_score): [0] predicted-and-true, [1] predicted (sigmoid > 0.5),
 * [2] true labels.  label: B x C, zero / non-zero.  Returns the mean loss. */
ORC_API float orc_sigmoid_bce(const float *logits, const int64_t *label, int64_t B, int64_t C, float *dlogits,
                              int64_t counters[3]) {
  double loss = 0.0;
  int64_t tp = 0, pre = 0, tru = 0;
  const double n = (double)B * (double)C;
  for (int64_t i = 0; i < B * C; i++) {
    /* the sigmoid is an fp32 tensor in the reference: it saturates to exactly 0 or 1 beyond |z| of about 17,
     * which is what brings the clamp into play */
    const float pf = 1.0f / (1.0f + expf(-logits[i]));
    const double p = (double)pf;
    const double y = label[i] != 0 ? 1.0 : 0.0;
    double lp = log(p), lq = log((double)(1.0f - pf));
    if (lp < -100.0) lp = -100.0;
    if (lq < -100.0) lq = -100.0;
    loss += -(y * lp + (1.0 - y) * lq);
    const int pred = pf > 0.5f;
    tp += (pred && label[i] != 0);
    pre += pred;
    tru += (label[i] != 0);
    if (dlogits) {
      double den = (double)(1.0f - pf) * p;
      if (den < 1e-12) den = 1e-12;
      dlogits[i] = (float)((p - y) / den * (p * (double)(1.0f - pf)) / n);
    }
  }
  if (counters) { counters[0] = tp; counters[1] = pre; counters[2] = tru; }
  return (float)(loss / n);
}

/* --------------------------------------------------------------------------------------------
 * a13 Adam with weight decay, as Parameter::learnC2G_with_decay_Adam
 * (core/NtsScheduler.hpp:794-811) followed by next() (:700-711):
 *   g = grad + wd*W ; M = b1*M + (1-b1)*g ; V = b2*V + (1-b2)*g*g ;
 *   W -= alpha * (M/(1-b1^t)) / (sqrt(V/(1-b2^t)) + eps)
 * b1^t / b2^t are carried as float products exactly like beta1_t / beta2_t (first step uses b1, b2).
 * toolkits/GCN_GPU_NEIGHBOR.hpp:214-217: b1 = .9, b2 = .999, eps = 1e-9.
 * ------------------------------------------------------------------------------------------ */
ORC_API void orc_adam(float *W, const float *grad, float *M, float *V, int64_t n, float alpha, float b1,
                      float b2, float eps, float wd, float b1_t, float b2_t) {
  float one_m_b1 = 1.0f - b1, one_m_b2 = 1.0f - b2;
  float c1 = 1.0f - b1_t, c2 = 1.0f - b2_t;
  for (int64_t i = 0; i < n; i++) {
    float g = grad[i] + wd * W[i];
    float m = b1 * M[i] + one_m_b1 * g;
    float v = b2 * V[i] + one_m_b2 * (g * g);
    M[i] = m;
    V[i] = v;
    float mt = m / c1, vt = v / c2;
    W[i] = W[i] - (alpha * mt) / (sqrtf(vt) + eps);
  }
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
ORC_API void orc_set_threads(int n) {
#ifdef _OPENMP
  omp_set_num_threads(n);
#else
  (void)n;
#endif
}
