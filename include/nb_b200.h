/*
 * nb_b200.h — C ABI of libnb_b200.so: hand-written sm_100a CUDA for the sampled mini-batch GCN
 * path of NeutronBench (ALGORITHM:GCNNEIGHBORGPU).
 *
 * Conventions
 *   - Every pointer named d_* is DEVICE memory of the current CUDA device unless the comment says
 *     "host" or "pinned".  Vertex ids and block-local indices are uint32_t (the reference's
 *     VertexId, dep/gemini/type.hpp:28); whole-graph CSC offsets are uint64_t so that graphs with
 *     more than 2^32 edges fit; features, weights and gradients are fp32 row-major.
 *   - `stream` is a cudaStream_t passed as void*.  Kernels are enqueued on it and the call returns
 *     without synchronising unless stated (the reference synchronises after every kernel,
 *     cuda/ntsCUDAGraphOP.cu:366-373; results are identical because all work is stream-ordered).
 *   - Return value: 0 (NB_OK) on success, a negative nb_status otherwise; nb_last_error() returns a
 *     message for the calling thread.  Nothing here calls exit() (the reference prints and exits,
 *     cuda/ntsCUDAGraphOP.cu:13-20).
 *   - The library never frees or reallocates caller memory.  Scratch memory lives in an nb_ws
 *     workspace that the caller creates and destroys.
 *   - There is no CPU fallback: without a CUDA device every compute entry point fails with
 *     NB_ERR_CUDA.
 */
#ifndef NB_B200_H
#define NB_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum nb_status {
  NB_OK = 0,
  NB_ERR_INVALID = -1,   /* bad argument (null pointer, zero width, size over a stated limit) */
  NB_ERR_CUDA = -2,      /* a CUDA runtime call or kernel launch failed                        */
  NB_ERR_NOMEM = -3,     /* workspace arena exhausted                                          */
  NB_ERR_OVERFLOW = -4   /* a device-side bounded wait or capacity check gave up               */
} nb_status;

const char *nb_last_error(void);
int nb_version(void);
/* Number of CUDA kernels this library has launched in the calling process so far. */
uint64_t nb_launch_count(void);

/* ------------------------------------------------------------------------------------------------
 * Workspace: a bump arena of device scratch memory plus a small pinned host mailbox used to read
 * sizes back.  If `d_arena` is NULL the workspace allocates `bytes` with cudaMalloc and frees it in
 * nb_ws_destroy; otherwise it sub-allocates from the caller's buffer and never frees it.
 * Replaces sampCSC::alloc_dev_array's cudaMalloc/cudaFree churn with 1.2x growth
 * (core/coocsc.hpp:621-671).  One workspace serves one stream at a time.
 * ---------------------------------------------------------------------------------------------- */
typedef struct nb_ws nb_ws;
int nb_ws_create(nb_ws **out, void *d_arena, size_t bytes);
int nb_ws_destroy(nb_ws *ws);
int nb_ws_reset(nb_ws *ws);                 /* forget all sub-allocations               */
size_t nb_ws_used(const nb_ws *ws);         /* bytes currently handed out               */
size_t nb_ws_high_water(const nb_ws *ws);   /* largest value nb_ws_used ever had        */

/* ------------------------------------------------------------------------------------------------
 * Aggregation (SpMM).
 *
 * nb_spmm_csc_fwd replaces Cuda_Stream::Gather_By_Dst_From_Src with with_weight=true
 * (cuda/ntsCUDA.hpp:124-128, cuda/ntsCUDAGraphOP.cu:186-210, kernel
 * cuda/ntsCUDAFuseKernel.cuh:272-290; caller core/ntsMiniBatchGraphOp.hpp:311-315):
 *     y[d,:] = sum_{j in [column_offset[d], column_offset[d+1])} w[j] * x[row_indices[j],:]
 * Every row of y is written (empty columns become zero), so y need not be zeroed first.  The sum is
 * taken edge after edge in CSC order with one fused multiply-add per element, y = fma(x, w, y): the
 * arithmetic of the reference's CPU operator (nts_comp, core/ntsBaseOp.hpp:76-97, as its -O3 -march=native
 * build compiles it), whose results it reproduces bit for bit; results do not depend on the launch shape.
 * (The reference's CUDA kernel rounds the product before its atomicAdd and differs in the last bit.)
 *
 * nb_spmm_csr_bwd replaces Cuda_Stream::Gather_By_Src_From_Dst (cuda/ntsCUDA.hpp:139-143,
 * cuda/ntsCUDAGraphOP.cu:269-292, kernel cuda/ntsCUDAFuseKernel.cuh:450-468; caller
 * core/ntsMiniBatchGraphOp.hpp:365-368):
 *     gx[s,:] = sum_{j in [row_offset[s], row_offset[s+1])} w[j] * gy[column_indices[j],:]
 * Atomics-free; the order within a row is the CSR order, so it is deterministic.
 *
 * The *_fused variants take no per-edge weight array: the GCN weight
 * 1/(sqrt(out_deg[src]) * sqrt(in_deg[dst])) (core/ntsBaseOp.hpp:183-186) is formed per edge from the
 * per-vertex factors src_norm[s] = (float)sqrt(out_deg), dst_norm[v] = (float)sqrt(in_deg) that
 * nb_block_build emits; the value is bit-identical to the reference's edge_weight_forward /
 * edge_weight_backward (core/coocsc.hpp:136-163).  nb_spmm_csr_bwd_fused additionally applies the
 * gradient of the dropout(relu(.)) that produced the block's input: where d_act (s x F, nullable) is
 * > 0 the sum is multiplied by act_scale, elsewhere it becomes 0.
 * ---------------------------------------------------------------------------------------------- */
int nb_spmm_csc_fwd(const float *d_x, float *d_y, const float *d_w, const uint32_t *d_row_indices,
                    const uint32_t *d_column_offset, uint32_t v, uint32_t F, void *stream);
int nb_spmm_csr_bwd(const float *d_gy, float *d_gx, const float *d_w, const uint32_t *d_row_offset,
                    const uint32_t *d_column_indices, uint32_t s, uint32_t F, void *stream);
int nb_spmm_csc_fwd_fused(const float *d_x, float *d_y, const uint32_t *d_row_indices,
                          const uint32_t *d_column_offset, const float *d_src_norm,
                          const float *d_dst_norm, uint32_t v, uint32_t F, void *stream);
int nb_spmm_csr_bwd_fused(const float *d_gy, float *d_gx, const uint32_t *d_row_offset,
                          const uint32_t *d_column_indices, const float *d_src_norm,
                          const float *d_dst_norm, const float *d_act, float act_scale, uint32_t s,
                          uint32_t F, void *stream);

/* Layer-0 aggregation straight from the feature store, without materialising the gathered input:
 *     y[d,:] = sum_j w_j * row(source[row_indices[j]])
 * where row(g) is the cached row d_cache[hashmap[g]] when d_hashmap != NULL and hashmap[g] !=
 * 0xFFFFFFFF, else feat[g] (device, mapped pinned host, or a peer GPU's memory).  Equals
 * nb_feature_gather followed by nb_spmm_csc_fwd_fused (core/ntsSampler.hpp:364-376 then
 * core/ntsMiniBatchGraphOp.hpp:288-318) bit for bit.  cache_ld / feat_ld are the row pitches in
 * floats (>= F); s and e are the block's source and edge counts; ws (nullable) provides 8*e bytes
 * of scratch for the staged path. */
int nb_spmm_csc_fwd_gather_fused(nb_ws *ws, const float *feat, size_t feat_ld, const float *d_cache,
                                 size_t cache_ld, const uint32_t *d_hashmap,
                                 const uint32_t *d_source, float *d_y,
                                 const uint32_t *d_row_indices, const uint32_t *d_column_offset,
                                 const float *d_src_norm, const float *d_dst_norm, uint32_t v,
                                 uint32_t s, uint32_t e, uint32_t F, void *stream);

/* Where the rows are 16-byte aligned (base aligned, width a multiple of 4 floats or a padded pitch)
 * and F <= 1024, the aggregation entry points above stage source rows through shared memory with
 * non-multicast TMA bulk copies; otherwise they use direct vector loads.  Both give identical bits.
 * By default only rows of 256 floats or more are staged (narrow rows are faster with direct loads).
 * nb_set_staged_spmm(0) forces the direct-load path, 1 is the default (per-warp ring of row slots,
 * one copy barrier per pair of rows), 2 stages every width the alignment rules allow, 3 / 4 are 1 / 2
 * with the two-stage segment kernel instead of the ring, 5 is 1 with a barrier per row; returns the
 * previous on/off setting.
 * nb_device_error_flags reads (and so synchronises with) the device-side error word: bit 0 is set
 * when a bounded wait on a copy barrier gave up, bit 1 when a wait on a tensor-core completion
 * barrier gave up, bit 2 when a gather or gather-fused aggregation met a vertex id that no table holds (beyond
 * the last shard, or not cached and no table given; the row is skipped or counts as zeros), bit 3 when a loss
 * kernel met a label outside [0, C) (the row counts with loss 0, no hit, zero gradient).  The word belongs to the
 * process and the device, not to a workspace or handle. */
int nb_set_staged_spmm(int enabled);
/* The staged gather-fused aggregation cuts wide rows into column panels whose distinct source data
 * (s rows x panel width) stays below this many bytes, so that reuse of a source row hits L2
 * (0 = never cut, the default).  Returns the previous value. */
uint64_t nb_set_l2_panel_bytes(uint64_t bytes);
int nb_device_error_flags(uint32_t *flags);
/* Clears the error word (it is sticky otherwise); synchronises like nb_device_error_flags. */
int nb_device_error_reset(void);

/* ------------------------------------------------------------------------------------------------
 * Block construction.
 *
 * nb_block_build turns one hop's raw sampled edge list into the reference's sampCSC block
 * (core/coocsc.hpp:792-813), on the device and without sorting the vertex set:
 *   dedup + reindex   sampCSC::postprocessing, core/coocsc.hpp:338-425
 *                     source[] = distinct global ids ascending; row_indices become local ranks
 *   CSR transpose     sampCSC::generate_csr_from_csc, core/coocsc.hpp:243-309
 *                     ascending local destinations within each source row
 *   degrees, weights  sampCSC::update_degree + compute_weight_forward/backward,
 *                     core/coocsc.hpp:136-216
 * and replaces the eight host->device copies per layer of copy_data_to_device_async
 * (core/coocsc.hpp:737-773).  Results are bit-identical to the reference's arrays.
 *
 * In:  d_row_indices[e] global source ids in CSC order (overwritten with local ranks),
 *      d_column_offset[v+1], num_vertices = |V| of the whole graph.
 * Out: d_source[>= min(|V|, e)], *src_size (host; the call synchronises the stream once to read it),
 *      d_row_offset[>= min(|V|,e)+1], d_column_indices[e], d_src_norm[>= min(|V|,e)], d_dst_norm[v],
 *      d_w_fwd[e] / d_w_bwd[e] (either may be NULL when only the fused SpMM variants are used).
 * Scratch: ws; about |V|/4 + 8*min(|V|,e) bytes.
 * ---------------------------------------------------------------------------------------------- */
int nb_block_build(nb_ws *ws, uint32_t num_vertices, uint32_t *d_row_indices,
                   const uint32_t *d_column_offset, uint32_t v, uint32_t e, uint32_t *d_source,
                   uint32_t *src_size, uint32_t *d_row_offset, uint32_t *d_column_indices,
                   float *d_src_norm, float *d_dst_norm, float *d_w_fwd, float *d_w_bwd,
                   void *stream);

/* ------------------------------------------------------------------------------------------------
 * Fan-out sampling of one hop (Sampler::sample_one, core/ntsSampler.hpp:843-1083, one iteration of
 * its layer loop up to and excluding postprocessing; init_co core/FullyRepGraph.hpp:199-209).
 *
 * nb_sample_hop_offsets: column_offset[i] = prefix sum of min(deg(dst[i]), fanout) (deg when
 * fanout < 0); *e_size (host) receives the edge count; synchronises the stream once.
 * nb_sample_hop: for every destination, `fanout` distinct neighbour positions drawn uniformly
 * (Floyd's subset algorithm on a per-destination Philox4x32-10 stream keyed by `seed`, counter
 * (draw/4, local destination index, hop, 0)) when deg > fanout, else all neighbours in CSC order;
 * writes GLOBAL source ids to d_row_indices in the layout nb_block_build consumes.
 * The reference draws with a thread-local mt19937 under OpenMP (utils/rand.hpp:6-13), so its sampled
 * sets are not reproducible across runs; parity with it is defined on identical edge lists.
 * ---------------------------------------------------------------------------------------------- */
int nb_sample_hop_offsets(nb_ws *ws, const uint64_t *d_graph_column_offset, const uint32_t *d_dst,
                          uint32_t v, int fanout, uint32_t *d_column_offset, uint32_t *e_size,
                          void *stream);
/* SAMPLE_RATE mode of the training sampler (core/ntsSampler.hpp:901-912): the count of destination i is
 * max(int(deg * sample_rate), min(lower_fanout, deg)) instead of min(deg, fanout).  nb_sample_hop takes its
 * counts from the offsets, so it follows with fanout = -1; subsets of more than 128 positions are drawn
 * by selection sampling (one Philox draw per neighbour, counter word 3 = 2) instead of Floyd's algorithm. */
int nb_sample_hop_offsets_rate(nb_ws *ws, const uint64_t *d_graph_column_offset, const uint32_t *d_dst,
                               uint32_t v, float sample_rate, int lower_fanout, uint32_t *d_column_offset,
                               uint32_t *e_size, void *stream);
int nb_sample_hop(const uint64_t *d_graph_column_offset, const uint32_t *d_graph_row_indices,
                  const uint32_t *d_dst, uint32_t v, int fanout, const uint32_t *d_column_offset,
                  uint64_t seed, uint32_t hop, uint32_t *d_row_indices, void *stream);

/* Whole-graph CSC from a device-resident edge list (u32 src, u32 dst pairs as in the .edge file),
 * stable in file order like FullyRepGraph::ReadRepGraphFromRawFile (core/FullyRepGraph.hpp:485-560).
 * d_out_degree / d_in_degree (nullable, |V| each) receive the raw degrees. */
int nb_graph_build_csc(nb_ws *ws, const uint32_t *d_edges, uint64_t num_edges, uint32_t num_vertices,
                       uint64_t *d_column_offset, uint32_t *d_row_indices, uint32_t *d_out_degree,
                       uint32_t *d_in_degree, void *stream);

/* ------------------------------------------------------------------------------------------------
 * Feature and label movement.
 *
 * nb_feature_gather: x0[i,:] = row(source[i]) for i < n, with row(g) as in
 * nb_spmm_csc_fwd_gather_fused.  One call replaces Cuda_Stream::zero_copy_feature_move_gpu
 * (cuda/ntsCUDAGraphOP.cu:379-396) when d_hashmap is NULL, and the pair
 * zero_copy_feature_move_gpu_cache + gather_feature_from_gpu_cache (cuda/ntsCUDAGraphOP.cu:398-423)
 * including the serial host-side hit/miss split of Sampler::load_feature_gpu_cache
 * (core/ntsSampler.hpp:444-456) otherwise.  `feat` may be device memory, the device alias of mapped
 * pinned host memory, or (feat_shards != NULL) a table sharded by contiguous node-id range over
 * `num_shards` pointers (own memory or peer GPUs reached with plain loads): owner = g / shard_rows.
 *
 * nb_label_gather: lab[i,:] = label[dst[i],:] with label_size int64 per row
 * (global_copy_label_move_gpu / global_copy_mulilabel_move_gpu, cuda/ntsCUDATransferKernel.cuh:184-203).
 *
 * nb_cache_fill: cache[hashmap[g],:] = feat[g,:] for every g < num_vertices with a slot
 * (gater_cpu_cache_feature_and_trans_to_gpu, toolkits/GCN_GPU_NEIGHBOR.hpp:899-918).
 * The slot map itself (descending degree, cache_high_degree + mark_cache_node,
 * toolkits/GCN_GPU_NEIGHBOR.hpp:919-943) is one-time host work and stays on the host side.
 * ---------------------------------------------------------------------------------------------- */
int nb_feature_gather(float *d_x0, const float *feat, size_t feat_ld, const float *const *feat_shards,
                      uint32_t num_shards, uint32_t shard_rows, const float *d_cache, size_t cache_ld,
                      const uint32_t *d_hashmap, const uint32_t *d_source, uint32_t n, uint32_t F,
                      void *stream);
/* The index-list form of the reference's cache path, for callers that keep its host-side hit/miss split
 * (Sampler::load_feature_gpu_cache, core/ntsSampler.hpp:424-469): for i < n, with lid = local_idx[i],
 *     x0[lid,:] = table[source[lid],:]              when d_slot_map == NULL
 *                 (Cuda_Stream::zero_copy_feature_move_gpu_cache, cuda/ntsCUDAGraphOP.cu:398-409), or
 *     x0[lid,:] = table[slot_map[source[lid]],:]    otherwise
 *                 (Cuda_Stream::gather_feature_from_gpu_cache, cuda/ntsCUDAGraphOP.cu:411-423).
 * Rows whose slot is 0xFFFFFFFF are skipped and reported through nb_device_error_flags (bit 2). */
int nb_feature_gather_indexed(float *d_x0, size_t x0_ld, const float *table, size_t table_ld,
                              const uint32_t *d_source, const uint32_t *d_local_idx, const uint32_t *d_slot_map,
                              uint32_t n, uint32_t F, void *stream);
/* Shards of a feature table that other processes of the job read (one process per GPU): a shard is an allocation of
 * its own (cudaMalloc), so that its inter-process handle names exactly that buffer.
 *   nb_shard_alloc / nb_shard_free   device memory of the current device
 *   nb_shard_upload                  copies `bytes` from `src` (host or device memory) into a shard; synchronous
 *   nb_shard_export                  64-byte handle of a shard of THIS process (cudaIpcGetMemHandle)
 *   nb_shard_open / nb_shard_close   maps a shard of ANOTHER process on the same machine into this process; the
 *                                    returned pointer is valid on the current device, which reads the owner's memory
 *                                    with plain loads over NVLink; nothing is copied.  Open each handle once.
 * The pointers, own and opened, go into the d_feat_shards table of nb_gcn_config / nb_feature_gather.  The owner
 * must keep a shard allocated until every peer has closed it. */
int nb_shard_alloc(void **d_ptr, size_t bytes);
int nb_shard_free(void *d_ptr);
int nb_shard_upload(void *d_dst, const void *src, size_t bytes);
int nb_shard_export(void *d_ptr, unsigned char handle[64]);
int nb_shard_open(const unsigned char handle[64], void **d_ptr);
int nb_shard_close(void *d_ptr);
int nb_label_gather(int64_t *d_lab, const int64_t *d_label, const uint32_t *d_dst, uint32_t n,
                    uint32_t label_size, void *stream);
int nb_cache_fill(float *d_cache, size_t cache_ld, const float *feat, size_t feat_ld,
                  const uint32_t *d_hashmap, uint32_t num_vertices, uint32_t F, void *stream);
/* d_counts[id] += 1 for every id of the list: the per-node sampling frequency that CACHE_POLICY:sample ranks
 * nodes by (cache_sample, toolkits/GCN_GPU_NEIGHBOR.hpp:974-999, counts every block's source list over one
 * dry-run epoch).  d_counts: num_vertices words, zeroed by the caller before the first call. */
int nb_count_ids(const uint32_t *d_ids, uint64_t n, uint32_t num_vertices, uint32_t *d_counts, void *stream);

/* ------------------------------------------------------------------------------------------------
 * Dense layer, loss, optimizer (the libtorch calls of vertexForward / Loss / Parameter,
 * toolkits/GCN_GPU_NEIGHBOR.hpp:715-728, utils/torch_func.hpp:67-82, core/NtsScheduler.hpp:712-715,
 * 794-811).  fp32 in, fp32 out, fp32 accumulation.
 *
 * nb_gemm: C[M x N] = op(A) * op(B).  trans_a = 0: A is M x K row-major; 1: A is K x M (A^T used).
 *          trans_b likewise for B (K x N, or N x K when 1).  Supported: NN, TN, NT.
 *          nb_set_gemm_mode selects the arithmetic: 0 = CUDA cores (fp32 FMA), 1 = tcgen05 tensor cores
 *          with a three-term TF32 split (fp32-level accuracy), 2 = tcgen05 plain TF32.  Products below
 *          about 40 MFLOP run on the CUDA cores in every mode (faster there); 17 / 18 are modes 1 / 2
 *          with that shortcut off.  Returns the previous mode.
 * nb_relu_dropout: z = dropout(relu(z)) in place; keeps element i when the Philox word
 *          (counter (i/4, layer, step, 1), key seed) mapped to [0,1) is >= p, scaling by 1/(1-p).
 * nb_softmax_nll: mean negative log-likelihood of log_softmax(logits) at `label`, its gradient
 *          (softmax - onehot)/B into d_dlogits (nullable), argmax hits into d_stats[1];
 *          d_stats[0] = loss (two floats, device).
 * nb_adam: g = grad + wd*W; M = b1 M + (1-b1) g; V = b2 V + (1-b2) g^2;
 *          W -= alpha * (M/(1-b1_t)) / (sqrt(V/(1-b2_t)) + eps).
 * ---------------------------------------------------------------------------------------------- */
int nb_set_gemm_mode(int mode);
int nb_gemm(nb_ws *ws, const float *d_a, const float *d_b, float *d_c, int64_t M, int64_t N, int64_t K,
            int trans_a, int trans_b, void *stream);
int nb_relu_dropout(float *d_z, int64_t n, float p, uint64_t seed, uint32_t layer, uint32_t step,
                    void *stream);
int nb_softmax_nll(nb_ws *ws, const float *d_logits, const int64_t *d_label, int64_t B, int64_t C,
                   float *d_dlogits, float *d_stats, void *stream);
/* No counterpart in the reference.  Same result as nb_softmax_nll, for callers that cannot provide
 * scratch memory when they call: processes that committed all device memory to their own pool at
 * start-up, or hosts whose rules forbid any allocation after initialisation.  The per-row scratch
 * (two floats per row) lives in a fixed 512 KiB device array inside the library image, which every GPU
 * that loads the library keeps until the process ends.  Limits and rules:
 *   - B <= 65536 rows; larger batches are refused with NB_ERR_INVALID (use nb_softmax_nll).
 *   - The call performs no cudaMalloc / cudaFree and uses no workspace.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress with that
 *     device current); make that first call outside any stream capture.
 *   - All calls on a device share the one array: two calls whose kernels can overlap on the GPU
 *     (different streams without an ordering between them) corrupt each other's loss.  The array keeps
 *     the previous call's rows; the kernels rewrite every row they read, so no clearing is required. */
int nb_softmax_nll_static(const float *d_logits, const int64_t *d_label, int64_t B, int64_t C,
                          float *d_dlogits, float *d_stats, void *stream);
/* The last GCN layer with one label per vertex in two launches instead of six: logits = Y W (B x H times H x C),
 * Loss and get_correct (utils/torch_func.hpp:16-29, 67-82) on the labels label[dst[i]], and for train != 0 the
 * gradients d_dw = Y^T dZ (H x C) and d_dy = dZ W^T (B x H, nullable).  d_stats as nb_softmax_nll.  Same values as
 * nb_gemm + nb_label_gather + nb_softmax_nll + two nb_gemm up to summation order.  nb_output_layer_supported tells
 * whether a layer fits the fused form (C <= 64 and W in about 90 KB of shared memory). */
int nb_output_layer_supported(uint32_t H, uint32_t C);
/* Programmatic dependent launch for the kernels of the training half of a step (aggregation, dense layers, output
 * layer, Adam): a kernel may be scheduled while its predecessor on the stream drains and waits for it at its first
 * instruction.  On by default; same results either way.  Returns the previous setting. */
int nb_set_pdl(int enabled);
/* nb_gcn_step / nb_gcn_compute use nb_output_layer for the last layer where it applies; 0 switches that off
 * (the layer then runs as separate calls).  Returns the previous setting. */
int nb_set_fused_output_layer(int enabled);
int nb_output_layer(nb_ws *ws, const float *d_y, const float *d_w, const int64_t *d_label, const uint32_t *d_dst,
                    uint32_t B, uint32_t H, uint32_t C, int train, float *d_dw, float *d_dy, float *d_stats,
                    void *stream);
/* Multi-label loss and F1 counters (CLASSES > 1; Loss with onelabel = false and f1_score,
 * utils/torch_func.hpp:31-75): loss = mean over B*C of binary_cross_entropy(sigmoid(z), y) with libtorch's
 * clamp of each log at -100; d_dlogits (nullable) = its gradient; d_label: B x C, zero / non-zero.
 * d_stats (device, 4 floats) = {mean loss, predicted-and-true, predicted (sigmoid > 0.5), true}; the batch's
 * F1 is 2PR/(P+R) with P = stats[1]/stats[2], R = stats[1]/stats[3], and 0 when stats[1] or stats[2] is 0. */
int nb_sigmoid_bce(nb_ws *ws, const float *d_logits, const int64_t *d_label, int64_t B, int64_t C,
                   float *d_dlogits, float *d_stats, void *stream);
int nb_adam(float *d_W, const float *d_grad, float *d_M, float *d_V, int64_t n, float alpha, float b1,
            float b2, float eps, float wd, float b1_t, float b2_t, void *stream);

/* ------------------------------------------------------------------------------------------------
 * Whole training step in one call: the body of the batch loop of
 * GCN_GPU_NEIGHBOR_impl::zerocopy_version (toolkits/GCN_GPU_NEIGHBOR.hpp:604-713) — sample_one,
 * feature / label gather, per layer runGraphOp<SingleGPUSampleGraphOp> + vertexForward, Loss,
 * self_backward (core/ntsContext.hpp:285-366; the input-side block is not back-propagated) — issued
 * from native code on the caller's stream, with every per-step buffer taken from the workspace arena
 * (which the call resets first).  The caller owns the graph, the feature store, the labels and the
 * flat parameter buffers; nb_gcn_update applies Adam (Parameter::learnC2G_with_decay_Adam + next,
 * core/NtsScheduler.hpp:794-811, 700-711) to the gradient that nb_gcn_step left in d_grad, so that a
 * data-parallel caller can sum d_grad over ranks in between.
 * ---------------------------------------------------------------------------------------------- */
#define NB_MAX_LAYERS 8
typedef struct nb_gcn_config {
  uint32_t num_layers;                      /* L: number of GCN layers = number of hops            */
  uint32_t layer_size[NB_MAX_LAYERS + 1];   /* LAYERS a-b-c                                         */
  int32_t fanout[NB_MAX_LAYERS];            /* hop order, seeds first; negative = all neighbours    */
  uint32_t num_vertices;
  float learn_rate, weight_decay, drop_rate, beta1, beta2, epsilon;
  uint64_t seed;
  int fuse_gather;                          /* layer 0 aggregates straight from the feature store   */
  const uint64_t *d_graph_column_offset;    /* whole-graph CSC                                      */
  const uint32_t *d_graph_row_indices;
  const float *feat;   size_t feat_ld;      /* feature table (device or mapped pinned host), may be NULL when all rows are cached */
  const float *d_cache; size_t cache_ld;    /* GPU feature cache and its slot map, or NULL          */
  const uint32_t *d_hashmap;
  const int64_t *d_label;                   /* one label per vertex                                 */
  float *d_W, *d_grad, *d_M, *d_V;          /* flat parameter bucket, sum of layer_size[l]*layer_size[l+1] floats each */
  float sample_rate;                        /* SAMPLE_RATE > 0: training batches use nb_sample_hop_offsets_rate */
  int32_t lower_fanout;                     /* LOWER_FANOUT of that mode                             */
  uint32_t classes;                         /* CLASSES: 0 or 1 = one label per vertex (NLL loss); > 1 = that many
                                               zero/non-zero labels per vertex in d_label (BCE loss, 4 stats)  */
  /* Feature table sharded by contiguous node-id range (replaces `feat`; the reference keeps remote rows behind an
   * MPI RPC, core/ntsPeerRPC.hpp:44-46): d_feat_shards is a DEVICE array of num_shards row pointers, shard k holds
   * the rows of vertices [k*shard_rows, (k+1)*shard_rows) with pitch feat_ld; a pointer may name this GPU's memory
   * or a peer GPU's (mapped by the caller; read with plain loads only).  Needs stage_misses.                     */
  const float *const *d_feat_shards;
  uint32_t num_shards, shard_rows;
  /* stage_misses != 0: the rows of the input block's distinct sources that have no cache slot are copied, once each,
   * into a staging table in the batch's workspace by the sampling half (nb_gcn_sample*), and the layer-0 aggregation
   * reads cache and staging table only.  For tables in mapped host memory or on peer GPUs: a row used by k edges
   * crosses the link once instead of k times, and does so while the previous batch trains.  Same results.        */
  int stage_misses;
} nb_gcn_config;

typedef struct nb_gcn_step_info {
  uint32_t v[NB_MAX_LAYERS], s[NB_MAX_LAYERS], e[NB_MAX_LAYERS];   /* block sizes, index 0 = input side */
  uint64_t agg_bytes;                        /* algorithmic bytes of the step's aggregation launches */
} nb_gcn_step_info;

typedef struct nb_gcn nb_gcn;
int nb_gcn_create(nb_gcn **out, const nb_gcn_config *cfg, nb_ws *ws);
int nb_gcn_destroy(nb_gcn *g);
/* One batch.  d_seeds: n_seeds vertex ids on the device.  train != 0: dropout on, gradient of the
 * weights left in d_grad; train == 0: forward and loss only.  d_stats[0] = mean loss, d_stats[1] =
 * number of correct argmax predictions (device; with classes > 1 the four values of nb_sigmoid_bce).  info (nullable, host) receives the block sizes. */
int nb_gcn_step(nb_gcn *g, const uint32_t *d_seeds, uint32_t n_seeds, int train, float *d_stats,
                nb_gcn_step_info *info, void *stream);
int nb_gcn_update(nb_gcn *g, void *stream);
/* The update may run on a stream of its own, so that the gradient sum over ranks and Adam overlap the layer-0
 * aggregation of the next batch (which does not read the weights): nb_gcn_wait_gradients makes `stream` wait for
 * the gradients of the last step / compute call (enqueue the all-reduce on it afterwards), nb_gcn_update on that
 * stream then orders itself after them, and the next step waits for the update before its first weight read. */
int nb_gcn_wait_gradients(nb_gcn *g, void *stream);
/* The same step in two halves, so that sampling batch i+1 overlaps the training of batch i — the
 * reference's pipelined batch loop (pipeline_version, toolkits/GCN_GPU_NEIGHBOR.hpp:399-505, where each
 * pipeline thread owns its SampledSubgraph and three streams).  A nb_gcn_batch is one SampledSubgraph
 * whose arrays live in a workspace of its own (not the model's).
 *   nb_gcn_sample  draws the batch on `stream` (d_seeds: device or pinned host memory, copied into the
 *                  batch; train != 0 selects the training sampler's SAMPLE_RATE mode when configured); it synchronises that stream for the block sizes, and first waits for the
 *                  compute call that last used this batch.
 *   nb_gcn_compute makes `stream` wait for the batch's sampling, then runs forward, loss and backward
 *                  exactly as nb_gcn_step; it never blocks the host.
 * Batches must be sampled in the order they are trained on (the sampler stream position advances per
 * nb_gcn_sample); results are bit-identical to nb_gcn_step on the same sequence of batches. */
typedef struct nb_gcn_batch nb_gcn_batch;
int nb_gcn_batch_create(nb_gcn_batch **out, nb_ws *ws);
int nb_gcn_batch_destroy(nb_gcn_batch *batch);
int nb_gcn_sample(nb_gcn *g, nb_gcn_batch *batch, const uint32_t *d_seeds, uint32_t n_seeds, int train,
                  void *stream);
int nb_gcn_compute(nb_gcn *g, nb_gcn_batch *batch, int train, float *d_stats, nb_gcn_step_info *info,
                   void *stream);
/* nb_gcn_sample with the drawing replaced by the caller's sampled edge lists: for a host that keeps the
 * reference's CPU sampler (Sampler::sample_one, core/ntsSampler.hpp:843-1106, whose draws come from a thread-local
 * mt19937 and cannot be reproduced on the device), and for parity runs, which are defined on identical sampled
 * edge lists.  d_hop_edges: host array with one device (or pinned host) pointer per hop, seeds first; entry h
 * holds the global source ids of hop h in CSC order, min(degree, fanout[h]) (the whole neighbourhood when the
 * fan-out is negative) per destination, where hop 0's destinations are the seeds and hop h's the distinct sources
 * of hop h-1 in ascending id order; hop_edge_counts (host) their lengths, checked against the column offsets.
 * The sampler's own stream of draws does not advance.  Blocks, and so nb_gcn_compute's results, are what the
 * reference builds from the same lists (sampCSC::postprocessing .. compute_weight, core/coocsc.hpp:136-425). */
int nb_gcn_sample_from_edges(nb_gcn *g, nb_gcn_batch *batch, const uint32_t *d_seeds, uint32_t n_seeds,
                             const uint32_t *const *d_hop_edges, const uint32_t *hop_edge_counts, void *stream);
/* nb_gcn_sample on a thread of the library (started at the first call, joined by nb_gcn_destroy), so that the
 * caller's thread is free to enqueue the training of the previous batch meanwhile; requests run in the order
 * they were made.  d_seeds must stay valid until the batch has been sampled.  nb_gcn_compute on the batch blocks
 * until then and returns the sampling's error, if any.  nb_gcn_batch_destroy: only after that. */
int nb_gcn_sample_async(nb_gcn *g, nb_gcn_batch *batch, const uint32_t *d_seeds, uint32_t n_seeds, int train,
                        void *stream);
/* Number of library threads that serve nb_gcn_sample_async (default 1, at most 8).  With more than one,
 * several batches are drawn at the same time, each on the stream its request named (use one stream per
 * batch); every request takes its place in the sampler's sequence of draws when it is made, so results do
 * not depend on the number of threads. */
int nb_gcn_set_sampler_threads(nb_gcn *g, int threads);
/* Tuning switches of one handle.  A handle starts with the process defaults (the nb_set_* calls above change those
 * and act on the stand-alone entry points and on handles created afterwards) and keeps its own copy, which is in
 * force on the calling thread while one of its nb_gcn_* entry points runs; handles and threads do not share
 * settings.  Names: "gemm_mode" (as nb_set_gemm_mode), "pdl", "fused_output_layer", "staged_spmm", "spmm_ring",
 * "staged_min_width", "ring_group_shift", "l2_panel_bytes", "l2_prefetch", "l2_hint" (0 off; 1 rows that a single
 * edge of the launch uses are copied with the L2 evict-first policy; 2 the others evict-last as well),
 * "y_stream_stores" (streaming stores for the wide layer-0 aggregate), "ring_warps" (20, 22 or 24 warps per CTA of the wide-row aggregation kernel, four row
 * slots each; 24 fill the shared memory of an SM), "ring_balance" (1: the warps of the wide-row
 * aggregation kernel take shares of equal edge count cut at row boundaries; 0: of equal row count), "reserve_sms" (SMs that the
 * one-CTA-per-SM aggregation kernel leaves free for a collective running beside it).  Results never depend on them. */
int nb_gcn_set_option(nb_gcn *g, const char *name, int64_t value);
/* The same switch on the process defaults: in force for the stand-alone entry points (nb_spmm_*, nb_gemm_*, ...) and
 * copied by handles created afterwards.  "hub_min_edges" (rows of at least this many edges of an aggregation over a
 * plain table, i.e. popular sources in the backward pass, are walked by a team of warps with one column per lane
 * instead of by one warp; 0 switches that off; same bits either way) and "fuse_relu" (ReLU + dropout of a hidden layer
 * leave with the product from the tensor-core GEMM's epilogue instead of a kernel of their own; same bits) and
 * "fuse_last_aggregation" (the fused output layer forms the last block's aggregate itself; same bits),
 * "blocking_sync" (host waits of the sampling half sleep on blocking events instead of spinning: for nodes with fewer
 * cores than sampler threads) are accepted by both calls. */
int nb_set_option(const char *name, int64_t value);
/* nb_count_ids over the source list of every block of a sampled batch (one step of the dry-run epoch of
 * CACHE_POLICY:sample); waits for the batch's sampling like nb_gcn_compute. */
int nb_gcn_count_sources(nb_gcn *g, nb_gcn_batch *batch, uint32_t *d_counts, void *stream);
/* Measurement aid: with timing on, every aggregation launch of nb_gcn_step is bracketed by CUDA events on the
 * step's stream; nb_gcn_read_timing waits for them and returns the summed device time, the summed
 * algorithmic bytes and the launch count since timing was switched on (or last read).  enabled == 2 brackets only the
 * layer-0 forward aggregation (two event records per step instead of eight; an event record between two kernels
 * keeps the second from starting under the first one's tail, so full timing costs several microseconds per step). */
int nb_gcn_set_timing(nb_gcn *g, int enabled);
int nb_gcn_read_timing(nb_gcn *g, double *agg_ms, uint64_t *agg_bytes, uint64_t *agg_launches);
/* The same, split in two classes: [0] the layer-0 forward aggregation (the launch that reads the feature rows,
 * the dominant kernel of a step), [1] all other aggregation launches. */
int nb_gcn_read_timing_by_class(nb_gcn *g, double ms[2], uint64_t bytes[2], uint64_t launches[2]);
/* The four per-phase times of the reference's epoch log line (toolkits/GCN_GPU_NEIGHBOR.hpp:60-72, 750-761,
 * 1499-1505) since timing was switched on or last read, in milliseconds: [0] sample = wall time the sampling halves
 * took on their threads (they overlap the training half when batches are drawn ahead), [1] trans = device time
 * of staging rows that are not cached, [2] graph = device time of the aggregation launches, [3] nn = device time
 * of the training half minus graph.  Consumes the same event pairs as the two calls above. */
int nb_gcn_read_phase_times(nb_gcn *g, double ms[4]);

/* ------------------------------------------------------------------------------------------------
 * Gradient sum over the ranks of a data-parallel job (libnb_b200_comm.so, a thin layer over NCCL; optional: a host
 * that already has a collective library, such as torch.distributed, sums the gradient bucket itself between
 * nb_gcn_compute and nb_gcn_update).  Replaces Parameter::all_reduce_to_gradient -> Network_simple::all_reduce_sum
 * (core/NtsScheduler.hpp:692-695, comm/network.h:189-193: device -> host copy, MPI_Allreduce(MPI_SUM), host -> device)
 * and Parameter::init_parameter -> Network_simple::broadcast (core/NtsScheduler.hpp:691) with one in-place call on
 * the device buffer, enqueued on the caller's stream.
 *   nb_comm_unique_id   rank 0 creates the 128-byte id and hands it to the other ranks (MPI_Bcast, a file, a store)
 *   nb_comm_create      collective over all ranks, with the GPU of the rank current
 * ---------------------------------------------------------------------------------------------- */
typedef struct nb_comm nb_comm;
int nb_comm_unique_id(unsigned char id[128]);
int nb_comm_create(nb_comm **out, const unsigned char id[128], int world, int rank);
int nb_comm_destroy(nb_comm *comm);
int nb_allreduce_sum_f32(nb_comm *comm, float *d_buf, size_t n, void *stream);
int nb_broadcast_f32(nb_comm *comm, float *d_buf, size_t n, int root, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* NB_B200_H */
