// Reference-backed oracle: runs the REFERENCE's own code for the sampled mini-batch GCN path and dumps
// its outputs, so that the plain-C restatement (nts_oracle.c) and the CUDA path can be pinned to them.
// TEST INFRASTRUCTURE ONLY.  Nothing of the reference is copied: its headers are included in place
// from the reference tree (-I<reference root>), with single-rank stand-ins for <mpi.h>, <numa.h>,
// <metis.h> (oracle/shims/) and host-memory stand-ins for the reference's CUDA allocation/copy helpers
// (oracle/shims/cuda_stubs.cpp), because the reference's CPU path allocates "device" arrays
// unconditionally (core/ntsSampler.hpp:1098).
//
// What runs (all reference code):
//   FullyRepGraph::ReadRepGraphFromRawFile            core/FullyRepGraph.hpp:485-560
//   Sampler::sample_one -> init_co, sample_processing, sampCSC::postprocessing,
//     generate_csr_from_csc, update_degree, compute_weight_forward/backward
//                                                     core/ntsSampler.hpp:843-1106, core/coocsc.hpp
//   nts::op::MiniBatchFuseOp::forward / backward      core/ntsMiniBatchGraphOp.hpp:154-244
//
// usage: ref_harness <edge_file> <vertices> <seeds.u32> <fanout hop order, comma list> <F> <out_dir> [in_dir]
//   (with in_dir the aggregation operands are read from in_dir/block<l>_x.f32, block<l>_gy.f32 instead of torch::randn)
// Output: raw little-endian arrays <out_dir>/<name>.bin plus <out_dir>/index.txt (name dtype count).
#define CUDA_ENABLE 1
#include "core/neutronstar.hpp"
#include "utils/torch_func.hpp"

#include <cstdio>
#include <fstream>
#include <sstream>
#include <string>
#include <vector>

static std::string g_out;
static std::ofstream g_index;

template <typename T>
static void dump(const std::string &name, const char *dtype, const T *data, size_t n) {
  std::ofstream f(g_out + "/" + name + ".bin", std::ios::binary);
  f.write(reinterpret_cast<const char *>(data), (std::streamsize)(n * sizeof(T)));
  g_index << name << " " << dtype << " " << n << "\n";
}

// ---------------------------------------------------------------------------------------------
// bench mode: times the reference's CPU training path on this machine's host cores, batch by batch,
// with the call sequence of GCN_CPU_NEIGHBOR_impl::Forward (toolkits/GCN_CPU_NEIGHBOR.hpp:300-366):
// sample_one -> get_feature / get_label -> runGraphOp<MiniBatchFuseOp> + vertexForward per layer ->
// Loss -> appendNNOp -> self_backward -> all_reduce_to_gradient + learnC2C_with_decay_Adam + next.
// usage: ref_harness bench <edge_file> <vertices> <feat.f32> <label.i64> <seeds.u32> <fanouts>
//                          <layers a-b-c> <batch> <warmup batches> <timed batches> <drop> <lr> <wd> [threads]
// threads: the cfg key THREADS (0 or absent = the reference's default, ncpus/2 - 1, core/ntsSampler.hpp:221-228).
// prints one line: REFBENCH ms_per_batch=<..> agg_edges_per_batch=<..> omp_threads=<..> batches=<..>
// ---------------------------------------------------------------------------------------------
static int bench_main(int argc, char **argv) {
  if (argc < 15) {
    fprintf(stderr, "bench: not enough arguments\n");
    return 2;
  }
  const std::string edge_file = argv[2];
  const VertexId V = (VertexId)std::stoul(argv[3]);
  const std::string feat_file = argv[4], label_file = argv[5], seeds_file = argv[6];
  std::vector<int> fanout, sizes;
  {
    std::stringstream ss(argv[7]);
    std::string t;
    while (std::getline(ss, t, ',')) fanout.push_back(std::stoi(t));
    std::stringstream s2(argv[8]);
    while (std::getline(s2, t, '-')) sizes.push_back(std::stoi(t));
  }
  const VertexId batch = (VertexId)std::stoul(argv[9]);
  const int warm = std::stoi(argv[10]), timed = std::stoi(argv[11]);
  const float drop = std::stof(argv[12]), lr = std::stof(argv[13]), wd = std::stof(argv[14]);
  const int cfg_threads = argc > 15 ? std::stoi(argv[15]) : 0;
  const int L = (int)fanout.size();

  std::vector<VertexId> seeds;
  {
    std::ifstream f(seeds_file, std::ios::binary);
    VertexId x;
    while (f.read(reinterpret_cast<char *>(&x), sizeof(x))) seeds.push_back(x);
  }
  const EdgeId E = (EdgeId)(file_size(edge_file.c_str()) / (2 * sizeof(VertexId)));
  Graph<Empty> *graph = new Graph<Empty>();
  graph->filename = edge_file;
  graph->vertices = V;
  graph->edges = E;
  graph->partition_offset = new VertexId[2]{0, V};
  graph->owned_vertices = V;
  graph->in_degree_for_backward = new VertexId[V]();
  graph->out_degree_for_backward = new VertexId[V]();
  graph->gnnctx = new GNNContext();
  graph->gnnctx->layer_size = sizes;
  graph->gnnctx->fanout = fanout;
  graph->gnnctx->val_fanout = fanout;
  graph->config->batch_size = batch;
  graph->config->batch_type = SEQUENCE;
  graph->config->sample_rate = -1;
  graph->config->mini_pull = 1;
  graph->config->classes = 1;
  if (cfg_threads > 0) graph->config->threads = cfg_threads;

  FullyRepGraph *frg = new FullyRepGraph(graph);
  frg->ReadRepGraphFromRawFile();
  Sampler *sampler = new Sampler(frg, seeds);
  SampledSubgraph *ssg = sampler->subgraph;

  const long F0 = sizes[0];
  NtsVar F = torch::empty({(long)V, F0}, torch::kFloat);
  {
    std::ifstream f(feat_file, std::ios::binary);
    f.read(reinterpret_cast<char *>(F.data_ptr<float>()), (std::streamsize)((size_t)V * F0 * sizeof(float)));
  }
  NtsVar labels = torch::empty({(long)V}, torch::kLong);
  {
    std::ifstream f(label_file, std::ios::binary);
    f.read(reinterpret_cast<char *>(labels.data_ptr<long>()), (std::streamsize)((size_t)V * sizeof(long)));
  }
  torch::manual_seed(2000);
  std::vector<Parameter *> P;
  for (int i = 0; i < L; i++) P.push_back(new Parameter(sizes[i], sizes[i + 1], lr, 0.9, 0.999, 1e-9, wd));
  nts::ctx::NtsContext *ctx = new nts::ctx::NtsContext();
  ctx->train();
  std::vector<NtsVar> X(L + 1);
  int cur_layer = 0;
  auto vertexForward = [&](NtsVar &n_i) -> NtsVar {
    if (cur_layer == L - 1) return P[cur_layer]->forward(n_i);
    return torch::dropout(torch::relu(P[cur_layer]->forward(n_i)), drop, true);
  };

  double total = 0;
  uint64_t edges = 0;
  int done = 0;
  for (int b = 0; b < warm + timed && sampler->sample_not_finished(); b++) {
    const double t0 = get_time();
    for (auto p : P) p->zero_grad();
    sampler->sample_one(ssg, 0, false);
    X[0] = nts::op::get_feature(ssg->sampled_sgs[0]->src().data(), ssg->sampled_sgs[0]->src_size, F, graph);
    NtsVar target = nts::op::get_label(ssg->sampled_sgs.back()->dst().data(), ssg->sampled_sgs.back()->v_size, labels,
                                       graph);
    for (int l = 0; l < L; l++) {
      cur_layer = l;
      NtsVar Y = ctx->runGraphOp<nts::op::MiniBatchFuseOp>(ssg, graph, l, X[l]);
      X[l + 1] = ctx->runVertexForward([&](NtsVar n_i) { return vertexForward(n_i); }, Y);
    }
    auto loss = Loss(X[L], target, true);
    volatile float lv = loss.item<float>();
    (void)lv;
    ctx->appendNNOp(X[L], loss);
    ctx->self_backward(false);
    for (auto p : P) {
      p->all_reduce_to_gradient(p->W.grad());
      p->learnC2C_with_decay_Adam();
      p->next();
    }
    const double dt = get_time() - t0;
    if (b >= warm) {
      total += dt;
      done++;
      for (int l = 0; l < L; l++) edges += ssg->sampled_sgs[l]->e_size;
      for (int l = 1; l < L; l++) edges += ssg->sampled_sgs[l]->e_size;
    }
  }
  printf("REFBENCH ms_per_batch=%.4f agg_edges_per_batch=%.1f omp_threads=%d batches=%d\n",
         done ? 1e3 * total / done : 0.0, done ? (double)edges / done : 0.0,
         (cfg_threads > 0 && cfg_threads <= numa_num_configured_cpus()) ? cfg_threads
                                                                        : std::max(1, numa_num_configured_cpus() / 2 - 1),
         done);
  fflush(stdout);
  _exit(0);   // the reference's destructors free members they never initialised
}

// ---------------------------------------------------------------------------------------------
// train mode: the reference's CPU trainer (call sequence of GCN_CPU_NEIGHBOR_impl::Forward,
// toolkits/GCN_CPU_NEIGHBOR.hpp:300-366, with DROP_RATE 0 so that no libtorch random stream is
// involved) for a number of epochs over a fixed seed list, dumping everything another implementation
// needs to replay the run batch by batch and everything it must reproduce:
//   W0_<l>                 initial weights of layer l (xavier_uniform_ under torch::manual_seed(2000))
//   b<k>_h<h>_edges        global source ids of hop h (seeds first) of batch k in CSC order, i.e.
//                          source[row_indices] of the hop's block: the sampled edge list
//   b<k>_h<h>_offsets      the hop's column offsets
//   loss                   mean NLL of every batch, in the order trained   (Loss, utils/torch_func.hpp:67-82)
//   correct                get_correct of every batch                      (utils/torch_func.hpp:11-29)
//   W_<l>                  weights after the last batch (learnC2C_with_decay_Adam + next,
//                          core/NtsScheduler.hpp:716-734, 700-711)
// usage: ref_harness train <edge_file> <vertices> <feat.f32> <label.i64> <seeds.u32> <fanouts>
//                          <layers a-b-c> <batch> <epochs> <lr> <wd> <out_dir>
// ---------------------------------------------------------------------------------------------
static int train_main(int argc, char **argv) {
  if (argc < 14) {
    fprintf(stderr, "train: not enough arguments\n");
    return 2;
  }
  const std::string edge_file = argv[2];
  const VertexId V = (VertexId)std::stoul(argv[3]);
  const std::string feat_file = argv[4], label_file = argv[5], seeds_file = argv[6];
  std::vector<int> fanout, sizes;
  {
    std::stringstream ss(argv[7]);
    std::string t;
    while (std::getline(ss, t, ',')) fanout.push_back(std::stoi(t));
    std::stringstream s2(argv[8]);
    while (std::getline(s2, t, '-')) sizes.push_back(std::stoi(t));
  }
  const VertexId batch = (VertexId)std::stoul(argv[9]);
  const int epochs = std::stoi(argv[10]);
  const float lr = std::stof(argv[11]), wd = std::stof(argv[12]);
  g_out = argv[13];
  g_index.open(g_out + "/index.txt");
  const int L = (int)fanout.size();

  std::vector<VertexId> seeds;
  {
    std::ifstream f(seeds_file, std::ios::binary);
    VertexId x;
    while (f.read(reinterpret_cast<char *>(&x), sizeof(x))) seeds.push_back(x);
  }
  const EdgeId E = (EdgeId)(file_size(edge_file.c_str()) / (2 * sizeof(VertexId)));
  Graph<Empty> *graph = new Graph<Empty>();
  graph->filename = edge_file;
  graph->vertices = V;
  graph->edges = E;
  graph->partition_offset = new VertexId[2]{0, V};
  graph->owned_vertices = V;
  graph->in_degree_for_backward = new VertexId[V]();
  graph->out_degree_for_backward = new VertexId[V]();
  graph->gnnctx = new GNNContext();
  graph->gnnctx->layer_size = sizes;
  graph->gnnctx->fanout = fanout;
  graph->gnnctx->val_fanout = fanout;
  graph->config->batch_size = batch;
  graph->config->batch_type = SEQUENCE;
  graph->config->sample_rate = -1;
  graph->config->mini_pull = 1;
  graph->config->classes = 1;
  graph->config->threads = 1;

  FullyRepGraph *frg = new FullyRepGraph(graph);
  frg->ReadRepGraphFromRawFile();
  Sampler *sampler = new Sampler(frg, seeds);
  SampledSubgraph *ssg = sampler->subgraph;

  const long F0 = sizes[0];
  NtsVar F = torch::empty({(long)V, F0}, torch::kFloat);
  {
    std::ifstream f(feat_file, std::ios::binary);
    f.read(reinterpret_cast<char *>(F.data_ptr<float>()), (std::streamsize)((size_t)V * F0 * sizeof(float)));
  }
  NtsVar labels = torch::empty({(long)V}, torch::kLong);
  {
    std::ifstream f(label_file, std::ios::binary);
    f.read(reinterpret_cast<char *>(labels.data_ptr<long>()), (std::streamsize)((size_t)V * sizeof(long)));
  }
  torch::manual_seed(2000);
  std::vector<Parameter *> P;
  for (int i = 0; i < L; i++) P.push_back(new Parameter(sizes[i], sizes[i + 1], lr, 0.9, 0.999, 1e-9, wd));
  for (int i = 0; i < L; i++)
    dump("W0_" + std::to_string(i), "f32", P[i]->W.data_ptr<float>(), (size_t)P[i]->W.numel());
  nts::ctx::NtsContext *ctx = new nts::ctx::NtsContext();
  ctx->train();
  std::vector<NtsVar> X(L + 1);
  int cur_layer = 0;
  auto vertexForward = [&](NtsVar &n_i) -> NtsVar {   // DROP_RATE 0: dropout is the identity
    if (cur_layer == L - 1) return P[cur_layer]->forward(n_i);
    return torch::relu(P[cur_layer]->forward(n_i));
  };

  std::vector<float> losses;
  std::vector<VertexId> corrects;
  int k = 0;
  for (int ep = 0; ep < epochs; ep++) {
    while (sampler->sample_not_finished()) {
      for (auto p : P) p->zero_grad();
      sampler->sample_one(ssg, 0, false);
      for (int h = 0; h < L; h++) {   // hop h is block L-1-h after the reverse of core/ntsSampler.hpp:1088
        sampCSC *b = ssg->sampled_sgs[L - 1 - h];
        std::vector<VertexId> raw(b->e_size);
        for (VertexId j = 0; j < b->e_size; j++) raw[j] = b->source[b->row_indices[j]];
        const std::string p = "b" + std::to_string(k) + "_h" + std::to_string(h) + "_";
        dump(p + "edges", "u32", raw.data(), raw.size());
        dump(p + "offsets", "u32", b->column_offset.data(), (size_t)b->v_size + 1);
      }
      X[0] = nts::op::get_feature(ssg->sampled_sgs[0]->src().data(), ssg->sampled_sgs[0]->src_size, F, graph);
      NtsVar target = nts::op::get_label(ssg->sampled_sgs.back()->dst().data(), ssg->sampled_sgs.back()->v_size,
                                         labels, graph);
      for (int l = 0; l < L; l++) {
        cur_layer = l;
        NtsVar Y = ctx->runGraphOp<nts::op::MiniBatchFuseOp>(ssg, graph, l, X[l]);
        X[l + 1] = ctx->runVertexForward([&](NtsVar n_i) { return vertexForward(n_i); }, Y);
      }
      auto loss = Loss(X[L], target, true);
      losses.push_back(loss.item<float>());
      corrects.push_back((VertexId)get_correct(X[L], target, true));
      ctx->appendNNOp(X[L], loss);
      ctx->self_backward(false);
      for (auto p : P) {
        p->all_reduce_to_gradient(p->W.grad());
        p->learnC2C_with_decay_Adam();
        p->next();
      }
      k++;
    }
    sampler->restart();
  }
  dump("loss", "f32", losses.data(), losses.size());
  dump("correct", "u32", corrects.data(), corrects.size());
  for (int i = 0; i < L; i++)
    dump("W_" + std::to_string(i), "f32", P[i]->W.data_ptr<float>(), (size_t)P[i]->W.numel());
  g_index.close();
  printf("ref_harness train: %d batches, wrote %s\n", k, g_out.c_str());
  fflush(stdout);
  _exit(0);   // the reference's destructors free members they never initialised
}

int main(int argc, char **argv) {
  if (argc > 1 && std::string(argv[1]) == "bench") return bench_main(argc, argv);
  if (argc > 1 && std::string(argv[1]) == "train") return train_main(argc, argv);
  if (argc < 7) {
    fprintf(stderr, "usage: %s edge_file vertices seeds.u32 fanouts F out_dir\n", argv[0]);
    return 2;
  }
  const std::string edge_file = argv[1];
  const VertexId V = (VertexId)std::stoul(argv[2]);
  const std::string seeds_file = argv[3];
  std::vector<int> fanout;
  {
    std::stringstream ss(argv[4]);
    std::string t;
    while (std::getline(ss, t, ',')) fanout.push_back(std::stoi(t));
  }
  const int F = std::stoi(argv[5]);
  g_out = argv[6];
  g_index.open(g_out + "/index.txt");

  std::vector<VertexId> seeds;
  {
    std::ifstream f(seeds_file, std::ios::binary);
    VertexId x;
    while (f.read(reinterpret_cast<char *>(&x), sizeof(x))) seeds.push_back(x);
  }
  const long file_bytes = file_size(edge_file.c_str());
  const EdgeId E = (EdgeId)(file_bytes / (2 * sizeof(VertexId)));

  // A single-rank Graph object with just the fields the sampled path reads.
  Graph<Empty> *graph = new Graph<Empty>();
  graph->filename = edge_file;
  graph->vertices = V;
  graph->edges = E;
  graph->partition_offset = new VertexId[2]{0, V};
  graph->owned_vertices = V;
  graph->in_degree_for_backward = new VertexId[V]();
  graph->out_degree_for_backward = new VertexId[V]();
  graph->gnnctx = new GNNContext();
  graph->gnnctx->layer_size.assign(fanout.size() + 1, F);
  graph->gnnctx->fanout = fanout;       // hop order, as the toolkit holds it after its reverse()
  graph->gnnctx->val_fanout = fanout;
  graph->config->batch_size = (VertexId)seeds.size();
  graph->config->batch_type = SEQUENCE;
  graph->config->sample_rate = -1;
  graph->config->mini_pull = 1;
  graph->config->classes = 1;
  graph->config->threads = 1;   // one sampling thread: the thread-local mt19937(2000) stream is reproducible

  FullyRepGraph *frg = new FullyRepGraph(graph);
  frg->ReadRepGraphFromRawFile();
  dump("graph_column_offset", "u32", frg->column_offset, (size_t)V + 1);
  dump("graph_row_indices", "u32", frg->row_indices, (size_t)E);

  Sampler *sampler = new Sampler(frg, seeds);
  SampledSubgraph *ssg = sampler->subgraph;
  sampler->sample_one(ssg, 0, false);   // phase=false: plain fan-out rule, no batch-type special cases

  const int L = (int)fanout.size();
  for (int l = 0; l < L; l++) {
    sampCSC *b = ssg->sampled_sgs[l];
    const std::string p = "block" + std::to_string(l) + "_";
    VertexId sizes[3] = {b->v_size, b->e_size, b->src_size};
    dump(p + "sizes", "u32", sizes, 3);
    dump(p + "destination", "u32", b->destination.data(), b->v_size);
    dump(p + "source", "u32", b->source.data(), b->src_size);
    dump(p + "column_offset", "u32", b->column_offset.data(), (size_t)b->v_size + 1);
    dump(p + "row_indices", "u32", b->row_indices.data(), b->e_size);
    dump(p + "row_offset", "u32", b->row_offset.data(), (size_t)b->src_size + 1);
    dump(p + "column_indices", "u32", b->column_indices.data(), b->e_size);
    dump(p + "edge_weight_forward", "f32", b->edge_weight_forward.data(), b->e_size);
    dump(p + "edge_weight_backward", "f32", b->edge_weight_backward.data(), b->e_size);
  }

  // Aggregation through the reference operator on seeded inputs.
  torch::manual_seed(2000);
  for (int l = 0; l < L; l++) {
    sampCSC *b = ssg->sampled_sgs[l];
    const std::string p = "block" + std::to_string(l) + "_";
    NtsVar x = torch::randn({(long)b->src_size, (long)F}, torch::kFloat);
    NtsVar gy = torch::randn({(long)b->v_size, (long)F}, torch::kFloat);
    if (argc > 7) {   // operands supplied by the caller: <in_dir>/block<l>_x.f32 and block<l>_gy.f32
      std::ifstream fx(std::string(argv[7]) + "/" + p + "x.f32", std::ios::binary);
      std::ifstream fg(std::string(argv[7]) + "/" + p + "gy.f32", std::ios::binary);
      if (!fx.read(reinterpret_cast<char *>(x.data_ptr<float>()), (std::streamsize)(x.numel() * sizeof(float))) ||
          !fg.read(reinterpret_cast<char *>(gy.data_ptr<float>()), (std::streamsize)(gy.numel() * sizeof(float)))) {
        fprintf(stderr, "ref_harness: operand files of block %d are missing or short\n", l);
        return 3;
      }
    }
    nts::op::MiniBatchFuseOp op(ssg, graph, l);
    NtsVar y = op.forward(x);
    NtsVar gx = op.backward(gy);
    dump(p + "x", "f32", x.data_ptr<float>(), (size_t)x.numel());
    dump(p + "gy", "f32", gy.data_ptr<float>(), (size_t)gy.numel());
    dump(p + "y", "f32", y.data_ptr<float>(), (size_t)y.numel());
    dump(p + "gx", "f32", gx.data_ptr<float>(), (size_t)gx.numel());
  }
  g_index.close();
  printf("ref_harness: wrote %s\n", g_out.c_str());
  return 0;
}
