// Whole training step issued from native code: the batch-loop body of the reference toolkit
// (toolkits/GCN_GPU_NEIGHBOR.hpp:604-713) as a sequence of this library's kernels on one stream.
// No kernels of its own: it exists so that a step costs one host call and no per-step allocations.
#include <chrono>
#include <condition_variable>
#include <deque>
#include <mutex>
#include <new>
#include <string>
#include <thread>
#include <vector>

#include "common.cuh"

struct BlockArrays {
  uint32_t v, s, e;
  uint32_t *destination, *source, *column_offset, *row_indices, *row_offset, *column_indices;
  float *src_norm, *dst_norm;
};

// One sampled subgraph (SampledSubgraph, core/ntsSampler.hpp:843-1106): its arrays live in the arena of `ws`.
struct nb_gcn_batch {
  nb_ws *ws = nullptr;
  uint32_t layers = 0;
  BlockArrays blk[NB_MAX_LAYERS];   // index 0 = input side (core/ntsSampler.hpp:1088)
  float *stage = nullptr;           // rows of the input block's sources that have no cache slot (row li), or null
  size_t stage_ld = 0;
  cudaEvent_t sampled = nullptr;    // recorded when the last sampling kernel is enqueued
  cudaEvent_t consumed = nullptr;   // recorded after the last kernel that reads the arrays
  bool in_use = false;              // a compute call has been enqueued since the last sample call
  // nb_gcn_sample_async: set under the model's mutex
  bool pending = false;             // queued or being sampled by the sampler thread
  int status = 0;                   // result of that sampling
  std::string error;
};

struct SampleJob {
  int train;
  uint32_t draw;        // position of this batch in the sampler's stream of draws
  nb_gcn_batch *batch;
  const uint32_t *seeds;
  uint32_t n;
  void *stream;
};

struct nb_gcn {
  nb_gcn_config cfg;
  nb::Tuning tuning;   // this handle's switches: the process defaults at creation, then nb_gcn_set_option
  nb_ws *ws;
  nb_gcn_batch own;    // the batch nb_gcn_step samples into: shares `ws` with the activations
  uint32_t draws;      // sample_one calls so far: part of the Philox counter of the sampler
  uint32_t steps;      // optimizer steps so far: part of the Philox counter of the dropout mask
  float beta1_t, beta2_t;
  size_t w_off[NB_MAX_LAYERS + 1];
  // optional timing of the aggregation launches with CUDA events on the step's stream
  int timing = 0;                    // 0 off, 1 every class, 2 only the layer-0 forward aggregation (class 0)
  std::vector<cudaEvent_t> ev_pool;   // pairs: start, stop
  size_t ev_used = 0;
  uint64_t timed_bytes = 0;
  std::vector<int> ev_class;         // per pair: 0 = layer-0 forward aggregation, 1 = any other aggregation,
                                     // 2 = a whole compute call (forward, loss, backward), 3 = staging of uncached rows
  double sample_host_ms = 0.0;       // wall time the sampling halves took on their threads while timing was on
  // event pairs already read out, per class: one set for each of the two readers, cleared by its reader
  double cls_ms[4] = {}, phase_ms[4] = {};
  uint64_t cls_bytes[4] = {}, cls_launches[4] = {};
  std::vector<uint64_t> ev_bytes;
  // cross-stream ordering of gradients and weights when the caller runs the update on a stream of its own
  cudaEvent_t ev_grad = nullptr;      // recorded after the last kernel of a compute call
  cudaEvent_t ev_updated = nullptr;   // recorded after Adam
  bool updated_recorded = false;
  // sampler thread (one of the reference's pipeline threads, toolkits/GCN_GPU_NEIGHBOR.hpp:399-505, reduced to
  // the part that blocks on the device): started by the first nb_gcn_sample_async
  int device = 0;
  std::vector<std::thread> samplers;
  int sampler_threads = 1;
  std::mutex mu;
  std::condition_variable cv_job, cv_done;
  std::deque<SampleJob> jobs;
  bool stop = false;
};


namespace {

using Block = BlockArrays;

template <typename T>
int arena(nb_ws *ws, size_t n, T **out) {
  *out = ws->alloc_n<T>(n ? n : 1);
  if (!*out) return nb::fail(NB_ERR_NOMEM, "nb_gcn_step: workspace arena exhausted");
  return 0;
}

uint64_t bytes_fwd(const Block &b, uint32_t F, bool gather, bool cached) {
  uint64_t x = 4ull * F * (b.s + b.v) + 4ull * b.e + 4ull * (b.v + 1) + 4ull * (b.s + b.v);
  if (gather) x += 4ull * b.s + (cached ? 4ull * b.s : 0);
  return x;
}
uint64_t bytes_bwd(const Block &b, uint32_t F) {
  return 4ull * F * (b.v + b.s) + 4ull * b.e + 4ull * (b.s + 1) + 4ull * (b.s + b.v) + 4ull * F * b.s;
}

// Brackets one aggregation launch with events when timing is on.
struct AggTimer {
  nb_gcn *g;
  cudaStream_t st;
  bool on;
  cudaEvent_t stop = nullptr;
  // The pool is shared by the thread that enqueues the training half and the sampler threads (class 3): a pair is
  // reserved under the handle's mutex and its two events are recorded outside it.
  AggTimer(nb_gcn *g_, void *stream, uint64_t bytes, int cls = 1) : g(g_), st(nb::as_stream(stream)), on(g_->timing == 1 || (g_->timing == 2 && cls == 0)) {
    if (!on) return;
    cudaEvent_t start;
    {
      std::lock_guard<std::mutex> lk(g->mu);
      if (g->ev_used + 2 > g->ev_pool.size()) {
        cudaEvent_t a, b;
        if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) { on = false; return; }
        g->ev_pool.push_back(a);
        g->ev_pool.push_back(b);
      }
      start = g->ev_pool[g->ev_used];
      stop = g->ev_pool[g->ev_used + 1];
      g->ev_used += 2;
      g->timed_bytes += bytes;
      g->ev_class.push_back(cls);
      g->ev_bytes.push_back(bytes);
    }
    cudaEventRecord(start, st);
  }
  ~AggTimer() {
    if (on) cudaEventRecord(stop, st);
  }
};

}  // namespace

NB_API int nb_gcn_create(nb_gcn **out, const nb_gcn_config *cfg, nb_ws *ws) {
  NB_REQUIRE(out && cfg && ws, "nb_gcn_create: null pointer");
  NB_REQUIRE(cfg->num_layers >= 1 && cfg->num_layers <= NB_MAX_LAYERS, "nb_gcn_create: 1..8 layers");
  NB_REQUIRE(cfg->d_graph_column_offset && cfg->d_graph_row_indices && cfg->d_label, "nb_gcn_create: null graph or labels");
  NB_REQUIRE(cfg->d_W && cfg->d_grad && cfg->d_M && cfg->d_V, "nb_gcn_create: null parameter buffers");
  NB_REQUIRE(cfg->feat || cfg->d_feat_shards || (cfg->d_cache && cfg->d_hashmap), "nb_gcn_create: no feature store");
  NB_REQUIRE(cfg->d_feat_shards == nullptr || (cfg->num_shards > 0 && cfg->shard_rows > 0 &&
                                               (uint64_t)cfg->num_shards * cfg->shard_rows >= cfg->num_vertices),
             "nb_gcn_create: the shards of the feature table do not cover every vertex");
  NB_REQUIRE(cfg->d_feat_shards == nullptr || cfg->stage_misses,
             "nb_gcn_create: a sharded feature table is read through the staging table (set stage_misses)");
  NB_REQUIRE(cfg->drop_rate >= 0.0f && cfg->drop_rate < 1.0f, "nb_gcn_create: drop rate must be in [0,1)");
  NB_REQUIRE(cfg->classes <= 1 || cfg->classes == cfg->layer_size[cfg->num_layers],
             "nb_gcn_create: with classes > 1 the last layer must have one output per class");
  NB_REQUIRE(cfg->sample_rate >= 0.0f && cfg->sample_rate <= 1.0f && cfg->lower_fanout >= 0,
             "nb_gcn_create: sample rate must be in [0,1] and the lower fan-out non-negative");
  for (uint32_t l = 0; l <= cfg->num_layers; l++) NB_REQUIRE(cfg->layer_size[l] > 0, "nb_gcn_create: zero layer width");
  for (uint32_t l = 0; l < cfg->num_layers; l++) NB_REQUIRE(cfg->fanout[l] != 0, "nb_gcn_create: zero fanout");
  nb_gcn *g = new (std::nothrow) nb_gcn();
  if (!g) return nb::fail(NB_ERR_NOMEM, "nb_gcn_create: out of host memory");
  g->cfg = *cfg;
  g->tuning = nb::default_tuning();
  g->ws = ws;
  g->own.ws = ws;
  NB_CUDA(cudaGetDevice(&g->device));
  NB_CUDA(cudaEventCreateWithFlags(&g->ev_grad, cudaEventDisableTiming));
  NB_CUDA(cudaEventCreateWithFlags(&g->ev_updated, cudaEventDisableTiming));
  g->draws = 0;
  g->steps = 0;
  g->beta1_t = cfg->beta1;
  g->beta2_t = cfg->beta2;
  g->w_off[0] = 0;
  for (uint32_t l = 0; l < cfg->num_layers; l++)
    g->w_off[l + 1] = g->w_off[l] + (size_t)cfg->layer_size[l] * cfg->layer_size[l + 1];
  *out = g;
  return 0;
}

NB_API int nb_gcn_destroy(nb_gcn *g) {
  if (g) {
    if (!g->samplers.empty()) {
      {
        std::lock_guard<std::mutex> lk(g->mu);
        g->stop = true;
      }
      g->cv_job.notify_all();
      for (std::thread &t : g->samplers) t.join();
    }
    for (cudaEvent_t e : g->ev_pool) cudaEventDestroy(e);
    if (g->ev_grad) cudaEventDestroy(g->ev_grad);
    if (g->ev_updated) cudaEventDestroy(g->ev_updated);
    if (g->own.sampled) cudaEventDestroy(g->own.sampled);
    if (g->own.consumed) cudaEventDestroy(g->own.consumed);
  }
  delete g;
  return 0;
}

NB_API int nb_gcn_set_timing(nb_gcn *g, int enabled) {
  NB_REQUIRE(g != nullptr, "nb_gcn_set_timing: null pointer");
  std::lock_guard<std::mutex> lk(g->mu);
  g->timing = enabled == 2 ? 2 : (enabled != 0 ? 1 : 0);
  g->sample_host_ms = 0.0;
  for (int k = 0; k < 4; k++) { g->cls_ms[k] = g->phase_ms[k] = 0.0; g->cls_bytes[k] = g->cls_launches[k] = 0; }
  g->ev_used = 0;
  g->timed_bytes = 0;
  g->ev_class.clear();
  g->ev_bytes.clear();
  return 0;
}

namespace {
// Adds the recorded event pairs to the per-class totals of both readers and forgets the pairs.  Caller holds g->mu.
int drain_events(nb_gcn *g) {
  for (size_t i = 0; i + 1 < g->ev_used; i += 2) {
    NB_CUDA(cudaEventSynchronize(g->ev_pool[i + 1]));
    float t = 0.0f;
    NB_CUDA(cudaEventElapsedTime(&t, g->ev_pool[i], g->ev_pool[i + 1]));
    const int k = g->ev_class[i / 2] & 3;
    g->cls_ms[k] += t;
    g->phase_ms[k] += t;
    g->cls_bytes[k] += g->ev_bytes[i / 2];
    g->cls_launches[k]++;
  }
  g->ev_used = 0;
  g->timed_bytes = 0;
  g->ev_class.clear();
  g->ev_bytes.clear();
  return 0;
}
}  // namespace

NB_API int nb_gcn_read_timing_by_class(nb_gcn *g, double ms[2], uint64_t bytes[2], uint64_t launches[2]) {
  NB_REQUIRE(g && ms && bytes && launches, "nb_gcn_read_timing_by_class: null pointer");
  std::lock_guard<std::mutex> lk(g->mu);
  NB_TRY(drain_events(g));
  for (int k = 0; k < 4; k++) {
    if (k < 2) { ms[k] = g->cls_ms[k]; bytes[k] = g->cls_bytes[k]; launches[k] = g->cls_launches[k]; }
    g->cls_ms[k] = 0.0;
    g->cls_bytes[k] = g->cls_launches[k] = 0;
  }
  return 0;
}

NB_API int nb_gcn_read_phase_times(nb_gcn *g, double ms[4]) {
  NB_REQUIRE(g && ms, "nb_gcn_read_phase_times: null pointer");
  std::lock_guard<std::mutex> lk(g->mu);
  NB_TRY(drain_events(g));
  const double *m = g->phase_ms;
  ms[0] = g->sample_host_ms;
  ms[1] = m[3];
  ms[2] = m[0] + m[1];
  ms[3] = m[2] > ms[2] ? m[2] - ms[2] : 0.0;
  g->sample_host_ms = 0.0;
  for (int k = 0; k < 4; k++) g->phase_ms[k] = 0.0;
  return 0;
}

NB_API int nb_gcn_read_timing(nb_gcn *g, double *agg_ms, uint64_t *agg_bytes, uint64_t *agg_launches) {
  NB_REQUIRE(g && agg_ms && agg_bytes && agg_launches, "nb_gcn_read_timing: null pointer");
  double ms[2];
  uint64_t bytes[2], launches[2];
  NB_TRY(nb_gcn_read_timing_by_class(g, ms, bytes, launches));
  *agg_ms = ms[0] + ms[1];
  *agg_bytes = bytes[0] + bytes[1];
  *agg_launches = launches[0] + launches[1];
  return 0;
}

namespace {

int ensure_events(nb_gcn_batch *bt) {
  if (!bt->sampled) NB_CUDA(cudaEventCreateWithFlags(&bt->sampled, cudaEventDisableTiming));
  // a sampler thread may wait long for a slot to be consumed: with blocking_sync it sleeps instead of spinning
  if (!bt->consumed)
    NB_CUDA(cudaEventCreateWithFlags(&bt->consumed, cudaEventDisableTiming |
                                                        (nb::tuning().blocking_sync ? cudaEventBlockingSync : 0)));
  return 0;
}

// sample_one: hop 0 starts at the seeds, hop h at the sources of hop h-1 (core/ntsSampler.hpp:843-1106).
// With `ext_edges` (host array of one device pointer per hop, seeds first) the hop's global source ids are copied
// from the caller instead of being drawn: the hop's column offsets still follow the fan-out rule and the supplied
// list must have exactly that many entries.
int sample_into(nb_gcn *g, nb_gcn_batch *bt, uint32_t draw, const uint32_t *d_seeds, uint32_t n_seeds, int train,
                void *stream, const uint32_t *const *ext_edges = nullptr, const uint32_t *ext_counts = nullptr) {
  const nb_gcn_config &c = g->cfg;
  const uint32_t L = c.num_layers;
  nb_ws *ws = bt->ws;
  struct HostTimer {   // wall time of this call, added to the handle's sampling total while timing is on
    nb_gcn *g;
    std::chrono::steady_clock::time_point t0 = std::chrono::steady_clock::now();
    ~HostTimer() {
      if (!g->timing) return;
      const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
      std::lock_guard<std::mutex> lk(g->mu);
      g->sample_host_ms += ms;
    }
  } host_timer{g};
  NB_TRY(ensure_events(bt));
  if (bt->in_use) {   // the arrays of the batch sampled here before may still be read by a compute call
    NB_CUDA(cudaEventSynchronize(bt->consumed));
    bt->in_use = false;
  }
  ws->used = 0;
  // The batch keeps its own copy of the seeds: the caller may reuse its buffer for the next batch at once.
  uint32_t *seeds;
  NB_TRY(arena(ws, n_seeds, &seeds));
  NB_CUDA(cudaMemcpyAsync(seeds, d_seeds, 4ull * n_seeds, cudaMemcpyDefault, nb::as_stream(stream)));
  Block hops[NB_MAX_LAYERS];
  const uint32_t *dst = seeds;
  uint32_t v = n_seeds;
  for (uint32_t h = 0; h < L; h++) {
    Block &b = hops[h];
    b.v = v;
    b.destination = const_cast<uint32_t *>(dst);
    NB_TRY(arena(ws, (size_t)v + 1, &b.column_offset));
    const bool by_rate = train && c.sample_rate > 0.0f;   // core/ntsSampler.hpp:901-912
    if (by_rate)
      NB_TRY(nb_sample_hop_offsets_rate(ws, c.d_graph_column_offset, dst, v, c.sample_rate, c.lower_fanout,
                                        b.column_offset, &b.e, stream));
    else
      NB_TRY(nb_sample_hop_offsets(ws, c.d_graph_column_offset, dst, v, c.fanout[h], b.column_offset, &b.e, stream));
    NB_TRY(arena(ws, b.e, &b.row_indices));
    uint32_t *marked = nullptr;
    if (ext_edges) {
      NB_REQUIRE(ext_counts[h] == b.e, "nb_gcn_sample_from_edges: a hop's edge list does not have the length its "
                                       "column offsets (min(degree, fan-out) per destination) give");
      if (b.e) NB_CUDA(cudaMemcpyAsync(b.row_indices, ext_edges[h], 4ull * b.e, cudaMemcpyDefault, nb::as_stream(stream)));
    } else {
      // the sampler marks the dedup bitmap of the hop while it writes the ids (cleared here, |V| bits + 4 flag words)
      const size_t words = ((size_t)c.num_vertices + 31) / 32;
      NB_TRY(arena(ws, words + 4, &marked));
      NB_CUDA(cudaMemsetAsync(marked, 0, (words + 4) * sizeof(uint32_t), nb::as_stream(stream)));
      NB_TRY(nb::sample_hop_impl(c.d_graph_column_offset, c.d_graph_row_indices, dst, v, by_rate ? -1 : c.fanout[h],
                                 b.column_offset, c.seed, (draw << 8) | h, b.row_indices, marked, stream));
    }
    const size_t cap = b.e < c.num_vertices ? (b.e ? b.e : 1) : c.num_vertices;
    NB_TRY(arena(ws, cap, &b.source));
    NB_TRY(arena(ws, cap + 1, &b.row_offset));
    NB_TRY(arena(ws, b.e, &b.column_indices));
    NB_TRY(arena(ws, cap, &b.src_norm));
    NB_TRY(arena(ws, v, &b.dst_norm));
    NB_TRY(nb::block_build_impl(ws, c.num_vertices, b.row_indices, b.column_offset, v, b.e, b.source, &b.s, b.row_offset,
                                b.column_indices, b.src_norm, b.dst_norm, nullptr, nullptr, b.e > 0 ? marked : nullptr,
                                stream));
    dst = b.source;
    v = b.s;
  }
  bt->layers = L;
  for (uint32_t l = 0; l < L; l++) bt->blk[l] = hops[L - 1 - l];
  // Rows of the input block's sources that are not cached, fetched here, in the sampling half, once per distinct
  // source: from mapped host memory or from the GPU that owns the row's shard (plain loads).  The aggregation then
  // reads device memory only.
  bt->stage = nullptr;
  bt->stage_ld = 0;
  if (c.stage_misses && c.fuse_gather && (c.feat || c.d_feat_shards) && bt->blk[0].s > 0) {
    const Block &b0 = bt->blk[0];
    const uint32_t F0 = c.layer_size[0];
    bt->stage_ld = (F0 + 3) / 4 * 4;
    NB_TRY(arena(ws, (size_t)b0.s * bt->stage_ld, &bt->stage));
    AggTimer t(g, stream, 0, 3);
    // A copy over the host link is bound by that link: a few CTAs keep it busy and leave the SMs to the training half
    // that runs beside this stream.  Peer reads over NVLink need more in flight.
    const uint32_t ctas = nb::tuning().stage_ctas > 0 ? (uint32_t)nb::tuning().stage_ctas
                                                      : (c.d_feat_shards ? 2u * (uint32_t)nb::num_sms() : 32u);
    NB_TRY(nb::feature_gather_impl(bt->stage, bt->stage_ld, c.d_hashmap != nullptr, c.feat, c.feat_ld, c.d_feat_shards,
                                   c.num_shards, c.shard_rows, c.d_cache, c.cache_ld, c.d_hashmap, b0.source, b0.s, F0,
                                   stream, ctas));
  }
  NB_CUDA(cudaEventRecord(bt->sampled, nb::as_stream(stream)));
  return 0;
}

int compute_from(nb_gcn *g, nb_gcn_batch *bt, int train, float *d_stats, nb_gcn_step_info *info, void *stream) {
  const nb_gcn_config &c = g->cfg;
  const uint32_t L = c.num_layers;
  NB_REQUIRE(bt->layers == L && bt->sampled, "nb_gcn_compute: the batch holds no sampled subgraph of this model");
  nb_ws *ws = g->ws;
  if (bt->ws != ws) {
    ws->used = 0;   // activations of the previous step are dead; later kernels are stream-ordered after its users
    NB_CUDA(cudaStreamWaitEvent(nb::as_stream(stream), bt->sampled, 0));
  }
  const Block *blk = bt->blk;
  uint64_t agg_bytes = 0;
  AggTimer whole(g, stream, 0, 2);   // the whole training half of the step, for the per-phase epoch times

  // ---- forward
  const float p = train ? c.drop_rate : 0.0f;
  const float scale = p > 0.0f ? 1.0f / (1.0f - p) : 1.0f;
  float *Y[NB_MAX_LAYERS], *X[NB_MAX_LAYERS + 1];
  size_t y_ld[NB_MAX_LAYERS];
  X[0] = nullptr;
  bool fused_out = false, fused_agg = false;
  for (uint32_t l = 0; l < L; l++) {
    const Block &b = blk[l];
    const uint32_t Fi = c.layer_size[l], Fo = c.layer_size[l + 1];
    // Rows of the layer-0 aggregate are padded to 16 bytes when the dense layer runs on the tensor cores, so that
    // its TMA tensor loads apply to any feature width (602 -> 604); the padding is never read.
    y_ld[l] = Fi;
    if (l == 0 && c.fuse_gather && nb::gemm_uses_tensor_cores(b.v, Fo, Fi)) y_ld[l] = (Fi + 3) / 4 * 4;
    NB_TRY(arena(ws, (size_t)b.v * y_ld[l], &Y[l]));
    if (l == 0) {
      if (c.fuse_gather) {
        AggTimer t(g, stream, bytes_fwd(b, Fi, true, c.d_hashmap != nullptr), 0);
        NB_TRY(nb::spmm_csc_fwd_gather_fused_ld(ws, c.feat, c.feat_ld, c.d_cache, c.cache_ld, c.d_hashmap, b.source,
                                                Y[0], y_ld[0], b.row_indices, b.column_offset, b.src_norm, b.dst_norm,
                                                b.v, b.s, b.e, Fi, stream, bt->stage, bt->stage_ld));
        agg_bytes += bytes_fwd(b, Fi, true, c.d_hashmap != nullptr);
      } else {
        NB_TRY(arena(ws, (size_t)b.s * Fi, &X[0]));
        NB_TRY(nb_feature_gather(X[0], c.feat, c.feat_ld, c.d_feat_shards, c.num_shards, c.shard_rows, c.d_cache,
                                 c.cache_ld, c.d_hashmap, b.source, b.s, Fi, stream));
        AggTimer t(g, stream, bytes_fwd(b, Fi, false, false), 0);
        NB_TRY(nb_spmm_csc_fwd_fused(X[0], Y[0], b.row_indices, b.column_offset, b.src_norm, b.dst_norm, b.v, Fi,
                                     stream));
        agg_bytes += bytes_fwd(b, Fi, false, false);
      }
    } else {
      // The last block of a model with one label per vertex: the fused output layer forms the aggregate itself, row by
      // row, and it never goes to memory (same arithmetic and edge order as nb_spmm_csc_fwd_fused).
      fused_agg = l + 1 == L && c.classes <= 1 && nb::tuning().fuse_output_layer && nb::tuning().fuse_last_aggregation &&
                  nb_output_layer_supported(Fi, Fo) && nb::output_layer_can_aggregate(X[l], Fi, Fi, Fo);
      if (!fused_agg) {
        AggTimer t(g, stream, bytes_fwd(b, Fi, false, false));
        NB_TRY(nb_spmm_csc_fwd_fused(X[l], Y[l], b.row_indices, b.column_offset, b.src_norm, b.dst_norm, b.v, Fi, stream));
      }
      agg_bytes += bytes_fwd(b, Fi, false, false);
    }
    // First reader of the weights in this step: if the previous update ran on another stream, wait for it here,
    // after the layer-0 aggregation (which does not touch the weights) has been enqueued.
    if (l == 0 && g->updated_recorded) NB_CUDA(cudaStreamWaitEvent(nb::as_stream(stream), g->ev_updated, 0));
    // The last layer with one label per vertex runs fused with the loss and its own gradients (nb_output_layer).
    fused_out = l + 1 == L && c.classes <= 1 && y_ld[l] == Fi && nb::tuning().fuse_output_layer && nb_output_layer_supported(Fi, Fo);
    if (fused_out) break;
    NB_TRY(arena(ws, (size_t)b.v * Fo, &X[l + 1]));
    // hidden layers: ReLU + dropout leave with the product where the GEMM kernel that runs can apply them
    nb::ReluEpi epi{};
    if (l + 1 < L && nb::tuning().fuse_relu) {
      epi.on = 1; epi.p = p; epi.scale = scale;
      epi.seed_lo = (uint32_t)c.seed; epi.seed_hi = (uint32_t)(c.seed >> 32); epi.layer = l; epi.step = g->steps;
    }
    bool relu_done = false;
    NB_TRY(nb::gemm_ld(ws, Y[l], y_ld[l], c.d_W + g->w_off[l], Fo, X[l + 1], b.v, Fo, Fi, 0, 0, nb::as_stream(stream),
                       epi.on ? &epi : nullptr, &relu_done));
    if (l + 1 < L && !relu_done) NB_TRY(nb_relu_dropout(X[l + 1], (int64_t)b.v * Fo, p, c.seed, l, g->steps, stream));
  }

  // ---- loss (utils/torch_func.hpp:67-82)
  const Block &last = blk[L - 1];
  const int64_t B = last.v, C = c.layer_size[L];
  const bool multi = c.classes > 1;   // CLASSES > 1: C labels per vertex, BCE loss (utils/torch_func.hpp:67-75)
  float *dZ = nullptr, *dY_out = nullptr;
  if (fused_out) {
    const uint32_t H = c.layer_size[L - 1];
    if (train && L > 1) NB_TRY(arena(ws, (size_t)B * H, &dY_out));
    if (fused_agg)
      NB_TRY(nb::output_layer_aggregating(ws, X[L - 1], H, last.row_indices, last.column_offset, last.src_norm,
                                          last.dst_norm, c.d_W + g->w_off[L - 1], c.d_label, last.destination, (uint32_t)B,
                                          H, (uint32_t)C, train, c.d_grad + g->w_off[L - 1], dY_out, d_stats, stream));
    else
      NB_TRY(nb_output_layer(ws, Y[L - 1], c.d_W + g->w_off[L - 1], c.d_label, last.destination, (uint32_t)B, H,
                             (uint32_t)C, train, c.d_grad + g->w_off[L - 1], dY_out, d_stats, stream));
  } else {
    int64_t *lab;
    NB_TRY(arena(ws, (size_t)(multi ? B * C : B), &lab));
    NB_TRY(nb_label_gather(lab, c.d_label, last.destination, last.v, multi ? (uint32_t)C : 1u, stream));
    if (train) NB_TRY(arena(ws, (size_t)(B * C), &dZ));
    if (multi)
      NB_TRY(nb_sigmoid_bce(ws, X[L], lab, B, C, dZ, d_stats, stream));
    else
      NB_TRY(nb_softmax_nll(ws, X[L], lab, B, C, dZ, d_stats, stream));
  }

  // ---- backward: dW_l = Y_l^T dZ_l; dY_l = dZ_l W_l^T; dZ_{l-1} = (A_l^T dY_l) masked by X_l > 0
  if (train) {
    for (int l = (int)L - 1; l >= 0; l--) {
      const Block &b = blk[l];
      const uint32_t Fi = c.layer_size[l], Fo = c.layer_size[l + 1];
      const bool from_fused = fused_out && l + 1 == (int)L;   // dW and dY of the last layer are already there
      if (!from_fused)
        NB_TRY(nb::gemm_ld(ws, Y[l], y_ld[l], dZ, Fo, c.d_grad + g->w_off[l], Fi, Fo, b.v, 1, 0, nb::as_stream(stream)));
      if (l == 0) break;   // the input-side block is never back-propagated (core/ntsContext.hpp:292)
      float *dY = dY_out, *dX;
      if (!from_fused) {
        NB_TRY(arena(ws, (size_t)b.v * Fi, &dY));
        NB_TRY(nb_gemm(ws, dZ, c.d_W + g->w_off[l], dY, b.v, Fi, Fo, 0, 1, stream));
      }
      NB_TRY(arena(ws, (size_t)b.s * Fi, &dX));
      AggTimer t(g, stream, bytes_bwd(b, Fi));
      NB_TRY(nb_spmm_csr_bwd_fused(dY, dX, b.row_offset, b.column_indices, b.src_norm, b.dst_norm, X[l], scale, b.s, Fi,
                                   stream));
      agg_bytes += bytes_bwd(b, Fi);
      dZ = dX;
    }
  }
  if (info) {
    for (uint32_t l = 0; l < L; l++) { info->v[l] = blk[l].v; info->s[l] = blk[l].s; info->e[l] = blk[l].e; }
    info->agg_bytes = agg_bytes;
  }
  NB_CUDA(cudaEventRecord(bt->consumed, nb::as_stream(stream)));
  NB_CUDA(cudaEventRecord(g->ev_grad, nb::as_stream(stream)));
  bt->in_use = true;
  return 0;
}

// Blocks until the sampler thread has finished with `bt`; returns the sampling's status.
int wait_sampled(nb_gcn *g, nb_gcn_batch *bt) {
  std::unique_lock<std::mutex> lk(g->mu);
  g->cv_done.wait(lk, [&] { return !bt->pending; });
  if (bt->status != 0) return nb::fail((nb_status)bt->status, bt->error.c_str());
  return 0;
}

void sampler_main(nb_gcn *g) {
  cudaSetDevice(g->device);
  for (;;) {
    SampleJob job;
    {
      std::unique_lock<std::mutex> lk(g->mu);
      g->cv_job.wait(lk, [&] { return g->stop || !g->jobs.empty(); });
      if (g->jobs.empty()) return;   // stop requested and nothing left to do
      job = g->jobs.front();
      g->jobs.pop_front();
    }
    nb::TuningScope scope(&g->tuning);
    const int st = sample_into(g, job.batch, job.draw, job.seeds, job.n, job.train, job.stream);
    {
      std::lock_guard<std::mutex> lk(g->mu);
      job.batch->status = st;
      job.batch->error = st ? nb_last_error() : "";
      job.batch->pending = false;
    }
    g->cv_done.notify_all();
  }
}

}  // namespace

NB_API int nb_gcn_batch_create(nb_gcn_batch **out, nb_ws *ws) {
  NB_REQUIRE(out && ws, "nb_gcn_batch_create: null pointer");
  nb_gcn_batch *bt = new (std::nothrow) nb_gcn_batch();
  if (!bt) return nb::fail(NB_ERR_NOMEM, "nb_gcn_batch_create: out of host memory");
  bt->ws = ws;
  *out = bt;
  return 0;
}

NB_API int nb_gcn_batch_destroy(nb_gcn_batch *bt) {
  if (bt) {
    if (bt->sampled) cudaEventDestroy(bt->sampled);
    if (bt->consumed) cudaEventDestroy(bt->consumed);
  }
  delete bt;
  return 0;
}

NB_API int nb_gcn_sample(nb_gcn *g, nb_gcn_batch *batch, const uint32_t *d_seeds, uint32_t n_seeds, int train,
                         void *stream) {
  NB_REQUIRE(g && batch && d_seeds, "nb_gcn_sample: null pointer");
  NB_REQUIRE(n_seeds > 0, "nb_gcn_sample: empty batch");
  NB_REQUIRE(batch->ws != g->ws, "nb_gcn_sample: a batch needs a workspace of its own, not the model's");
  uint32_t draw;
  {
    std::unique_lock<std::mutex> lk(g->mu);
    g->cv_done.wait(lk, [&] { return !batch->pending; });
    draw = g->draws++;
  }
  nb::TuningScope scope(&g->tuning);
  return sample_into(g, batch, draw, d_seeds, n_seeds, train, stream);
}

NB_API int nb_gcn_sample_from_edges(nb_gcn *g, nb_gcn_batch *batch, const uint32_t *d_seeds, uint32_t n_seeds,
                                    const uint32_t *const *d_hop_edges, const uint32_t *hop_edge_counts, void *stream) {
  NB_REQUIRE(g && batch && d_seeds && d_hop_edges && hop_edge_counts, "nb_gcn_sample_from_edges: null pointer");
  NB_REQUIRE(n_seeds > 0, "nb_gcn_sample_from_edges: empty batch");
  NB_REQUIRE(batch->ws != g->ws, "nb_gcn_sample_from_edges: a batch needs a workspace of its own, not the model's");
  for (uint32_t h = 0; h < g->cfg.num_layers; h++)
    NB_REQUIRE(d_hop_edges[h] || hop_edge_counts[h] == 0, "nb_gcn_sample_from_edges: null edge list");
  {
    std::unique_lock<std::mutex> lk(g->mu);
    g->cv_done.wait(lk, [&] { return !batch->pending; });
  }
  nb::TuningScope scope(&g->tuning);
  return sample_into(g, batch, 0, d_seeds, n_seeds, 0, stream, d_hop_edges, hop_edge_counts);
}

NB_API int nb_gcn_sample_async(nb_gcn *g, nb_gcn_batch *batch, const uint32_t *d_seeds, uint32_t n_seeds, int train,
                               void *stream) {
  NB_REQUIRE(g && batch && d_seeds, "nb_gcn_sample_async: null pointer");
  NB_REQUIRE(n_seeds > 0, "nb_gcn_sample_async: empty batch");
  NB_REQUIRE(batch->ws != g->ws, "nb_gcn_sample_async: a batch needs a workspace of its own, not the model's");
  std::lock_guard<std::mutex> lk(g->mu);
  NB_REQUIRE(!batch->pending, "nb_gcn_sample_async: this batch is still being sampled");
  while ((int)g->samplers.size() < g->sampler_threads) {
    try {
      g->samplers.emplace_back(sampler_main, g);
    } catch (...) {
      if (g->samplers.empty()) return nb::fail(NB_ERR_NOMEM, "nb_gcn_sample_async: cannot start a sampler thread");
      break;
    }
  }
  batch->pending = true;
  batch->status = 0;
  g->jobs.push_back(SampleJob{train, g->draws++, batch, d_seeds, n_seeds, stream});
  g->cv_job.notify_one();
  return 0;
}

NB_API int nb_gcn_count_sources(nb_gcn *g, nb_gcn_batch *batch, uint32_t *d_counts, void *stream) {
  NB_REQUIRE(g && batch && d_counts, "nb_gcn_count_sources: null pointer");
  NB_TRY(wait_sampled(g, batch));
  NB_REQUIRE(batch->layers == g->cfg.num_layers && batch->sampled, "nb_gcn_count_sources: the batch holds no sampled subgraph");
  if (batch->ws != g->ws) NB_CUDA(cudaStreamWaitEvent(nb::as_stream(stream), batch->sampled, 0));
  for (uint32_t l = 0; l < batch->layers; l++)
    NB_TRY(nb_count_ids(batch->blk[l].source, batch->blk[l].s, g->cfg.num_vertices, d_counts, stream));
  NB_CUDA(cudaEventRecord(batch->consumed, nb::as_stream(stream)));
  batch->in_use = true;
  return 0;
}

NB_API int nb_set_fused_output_layer(int enabled) {
  const int old = nb::default_tuning().fuse_output_layer;
  nb::default_tuning().fuse_output_layer = enabled != 0;
  return old;
}

static int apply_option(nb::Tuning &t, const char *name, int64_t value) {
  const std::string n(name);
  if (n == "gemm_mode") {
    NB_REQUIRE((value >= 0 && value <= 2) || (value >= 16 && value <= 18), "nb_gcn_set_option: gemm_mode is 0..2 or 16..18");
    t.gemm_mode = (int)(value & 15);
    t.gemm_force_tc = value >= 16;
  } else if (n == "pdl") t.use_pdl = value != 0;
  else if (n == "fused_output_layer") t.fuse_output_layer = value != 0;
  else if (n == "staged_spmm") t.staged_spmm = value != 0;
  else if (n == "spmm_ring") t.spmm_ring = value != 0;
  else if (n == "staged_min_width") t.staged_min_width = (int)(value > 0 ? value : 1);
  else if (n == "ring_group_shift") t.ring_group_shift = value != 0 ? 1u : 0u;
  else if (n == "l2_panel_bytes") t.l2_panel_bytes = (uint64_t)(value > 0 ? value : 0);
  else if (n == "l2_prefetch") t.l2_prefetch = value != 0;
  else if (n == "l2_hint") {
    NB_REQUIRE(value >= 0 && value <= 3, "nb_gcn_set_option: l2_hint is 0..3");
    t.l2_hint = (int)value;
  } else if (n == "l2_keep_min_uses") {
    NB_REQUIRE(value >= 2 && value <= 1000000, "nb_gcn_set_option: l2_keep_min_uses is at least 2");
    t.l2_keep_min_uses = (int)value;
  } else if (n == "y_stream_stores") t.y_stream_stores = value != 0;
  else if (n == "ring_balance") t.ring_balance = value != 0;
  else if (n == "fuse_relu") t.fuse_relu = value != 0;
  else if (n == "fuse_last_aggregation") t.fuse_last_aggregation = value != 0;
  else if (n == "ring_warps") {
    NB_REQUIRE(value == 20 || value == 22 || value == 24, "nb_gcn_set_option: ring_warps is 20, 22 or 24");
    t.ring_warps = (int)value;
  }
  else if (n == "blocking_sync") t.blocking_sync = value != 0;
  else if (n == "hub_min_edges") t.hub_min_edges = (int)(value > 0 ? (value < 32 ? 32 : value) : 0);
  else if (n == "ring_prefetch") t.ring_prefetch = (int)(value > 0 ? (value < 14 ? value : 14) : 0);
  else if (n == "ring_wait_ns") t.ring_wait_ns = (int)(value > 0 ? (value < 100000 ? value : 100000) : 0);
  else if (n == "stage_ctas") t.stage_ctas = (int)(value > 0 ? value : 0);
  else if (n == "wide_direct") t.wide_direct = value != 0;
  else if (n == "wide_col_split") {
    NB_REQUIRE(value >= 1 && value <= 4, "nb_gcn_set_option: wide_col_split is 1..4");
    t.wide_col_split = (int)value;
  } else if (n == "wide_rows_in_flight") {
    NB_REQUIRE(value == 1 || value == 2 || value == 4, "nb_gcn_set_option: wide_rows_in_flight is 1, 2 or 4");
    t.wide_rows_in_flight = (int)value;
  }
  else if (n == "reserve_sms") {
    NB_REQUIRE(value >= 0 && value < 64, "nb_gcn_set_option: reserve_sms is 0..63");
    t.reserve_sms = (int)value;
  } else return nb::fail(NB_ERR_INVALID, "nb_gcn_set_option: unknown option");
  return 0;
}

NB_API int nb_gcn_set_option(nb_gcn *g, const char *name, int64_t value) {
  NB_REQUIRE(g && name, "nb_gcn_set_option: null pointer");
  return apply_option(g->tuning, name, value);
}

NB_API int nb_set_option(const char *name, int64_t value) {
  NB_REQUIRE(name != nullptr, "nb_set_option: null pointer");
  return apply_option(nb::default_tuning(), name, value);
}

NB_API int nb_gcn_set_sampler_threads(nb_gcn *g, int threads) {
  NB_REQUIRE(g != nullptr, "nb_gcn_set_sampler_threads: null pointer");
  NB_REQUIRE(threads >= 1 && threads <= 8, "nb_gcn_set_sampler_threads: 1..8 threads");
  std::lock_guard<std::mutex> lk(g->mu);
  NB_REQUIRE((int)g->samplers.size() <= threads, "nb_gcn_set_sampler_threads: threads cannot be taken away");
  g->sampler_threads = threads;
  return 0;
}

NB_API int nb_gcn_compute(nb_gcn *g, nb_gcn_batch *batch, int train, float *d_stats, nb_gcn_step_info *info,
                          void *stream) {
  NB_REQUIRE(g && batch && d_stats, "nb_gcn_compute: null pointer");
  NB_TRY(wait_sampled(g, batch));
  nb::TuningScope scope(&g->tuning);
  return compute_from(g, batch, train, d_stats, info, stream);
}

NB_API int nb_gcn_step(nb_gcn *g, const uint32_t *d_seeds, uint32_t n_seeds, int train, float *d_stats,
                       nb_gcn_step_info *info, void *stream) {
  NB_REQUIRE(g && d_seeds && d_stats, "nb_gcn_step: null pointer");
  NB_REQUIRE(n_seeds > 0, "nb_gcn_step: empty batch");
  g->own.in_use = false;   // same stream and same arena: stream order alone protects the arrays
  uint32_t draw;
  {
    std::lock_guard<std::mutex> lk(g->mu);
    draw = g->draws++;
  }
  nb::TuningScope scope(&g->tuning);
  NB_TRY(sample_into(g, &g->own, draw, d_seeds, n_seeds, train, stream));
  return compute_from(g, &g->own, train, d_stats, info, stream);
}

NB_API int nb_gcn_wait_gradients(nb_gcn *g, void *stream) {
  NB_REQUIRE(g != nullptr, "nb_gcn_wait_gradients: null pointer");
  NB_CUDA(cudaStreamWaitEvent(nb::as_stream(stream), g->ev_grad, 0));
  return 0;
}

NB_API int nb_gcn_update(nb_gcn *g, void *stream) {
  NB_REQUIRE(g != nullptr, "nb_gcn_update: null pointer");
  nb::TuningScope scope(&g->tuning);
  const nb_gcn_config &c = g->cfg;
  NB_CUDA(cudaStreamWaitEvent(nb::as_stream(stream), g->ev_grad, 0));   // no-op on the stream that computed them
  NB_TRY(nb_adam(c.d_W, c.d_grad, c.d_M, c.d_V, (int64_t)g->w_off[c.num_layers], c.learn_rate, c.beta1, c.beta2,
                 c.epsilon, c.weight_decay, g->beta1_t, g->beta2_t, stream));
  NB_CUDA(cudaEventRecord(g->ev_updated, nb::as_stream(stream)));
  g->updated_recorded = true;
  g->beta1_t *= c.beta1;   // Parameter::next (core/NtsScheduler.hpp:700-711)
  g->beta2_t *= c.beta2;
  g->steps++;
  return 0;
}
