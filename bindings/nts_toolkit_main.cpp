// `nts_b200 <file.cfg>`: the reference's own GPU mini-batch trainer class, unmodified, on this library.
//
// The reference's executable is toolkits/main.cpp + core/GraphSegment.cpp + comm/network.cpp linked against its CUDA
// static library (CMakeLists.txt:136-150).  This file takes the place of main.cpp for ALGORITHM:GCNNEIGHBORGPU
// (toolkits/main.cpp:116-137): it includes toolkits/GCN_GPU_NEIGHBOR.hpp where it lies, reads the .cfg with the
// reference's InputInfo::readFromCfgFile (core/GraphSegment.cpp:196), constructs GCN_GPU_NEIGHBOR_impl and calls
// init_graph / init_nn / run exactly as main.cpp does.  Every Cuda_Stream member, allocation and copy helper the class
// calls resolves to libnts_cuda_b200.so, i.e. to the sm_100a kernels of libnb_b200.so; the dense half stays libtorch,
// as in the reference.
//
// One difference from main.cpp, for one rank: Graph::load_directed + generate_backward_structure
// (core/graph.hpp) exchange the edge list between ranks over MPI, and this build has the single-rank stand-in for
// <mpi.h> only.  The GPU mini-batch trainer reads just a handful of fields those two calls leave behind (the vertex and
// edge counts, the partition offsets, the degree arrays, the per-socket edge totals that init_gnnctx sums); they are
// filled here from one pass over the edge file.  The sampled path itself takes its topology from
// FullyRepGraph::ReadRepGraphFromRawFile, which reads the edge file again on its own.
#include <sys/stat.h>

#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <string>
#include <vector>

// main.cpp pulls utils/cuda_memory.hpp (get_gpu_mem) in through an earlier toolkit header; the GPU trainer relies on it.
#include "core/neutronstar.hpp"
#include "utils/cuda_memory.hpp"
#include "toolkits/GCN_GPU_NEIGHBOR.hpp"

static void prepare_single_rank_graph(Graph<Empty> *graph) {
  const std::string &path = graph->config->edge_file;
  struct stat st;
  if (stat(path.c_str(), &st) != 0) {
    fprintf(stderr, "nts_b200: cannot stat edge file %s\n", path.c_str());
    exit(2);
  }
  const VertexId V = graph->config->vertices;
  const EdgeId E = (EdgeId)(st.st_size / (2 * sizeof(VertexId)));
  graph->filename = path;
  graph->vertices = V;
  graph->edges = E;
  graph->partition_offset = new VertexId[graph->partitions + 1];
  graph->partition_offset[0] = 0;
  for (int p = 1; p <= graph->partitions; p++) graph->partition_offset[p] = V;
  graph->owned_vertices = V;
  graph->local_partition_offset = new VertexId[graph->sockets + 1];
  graph->local_partition_offset[0] = 0;
  for (int s = 1; s <= graph->sockets; s++) graph->local_partition_offset[s] = V;
  graph->in_degree_for_backward = new VertexId[V]();
  graph->out_degree_for_backward = new VertexId[V]();
  graph->in_degree = graph->in_degree_for_backward;
  graph->out_degree = graph->out_degree_for_backward;
  {
    std::ifstream f(path, std::ios::binary);
    std::vector<VertexId> buf(1 << 20);
    EdgeId left = E * 2;
    while (left > 0) {
      const EdgeId n = std::min<EdgeId>(left, buf.size());
      f.read(reinterpret_cast<char *>(buf.data()), (std::streamsize)(n * sizeof(VertexId)));
      for (EdgeId i = 0; i + 1 < n; i += 2) {
        const VertexId src = buf[i], dst = buf[i + 1];
        if (src >= V || dst >= V) {
          fprintf(stderr, "nts_b200: edge (%u,%u) outside VERTICES:%u\n", src, dst, V);
          exit(2);
        }
        graph->out_degree_for_backward[src]++;
        graph->in_degree_for_backward[dst]++;
      }
      left -= n;
    }
  }
  // init_gnnctx adds incoming_adj_index_backward[socket][vertices] over the sockets to get the local edge count.
  graph->incoming_adj_index_backward = new EdgeId *[graph->sockets];
  for (int s = 0; s < graph->sockets; s++) {
    graph->incoming_adj_index_backward[s] = new EdgeId[(size_t)V + 1]();
    graph->incoming_adj_index_backward[s][V] = s == 0 ? E : 0;
  }
}

int main(int argc, char **argv) {
  MPI_Instance mpi(&argc, &argv);
  if (argc < 2) {
    printf("configuration file missed \n");
    exit(-1);
  }
  double exec_time = -get_time();
  Graph<Empty> *graph = new Graph<Empty>();
  graph->config->readFromCfgFile(argv[1]);
  if (graph->partition_id == 0) graph->config->print();
  int iterations = graph->config->epochs;
  graph->replication_threshold = graph->config->repthreshold;
  if (graph->config->algorithm != std::string("GCNNEIGHBORGPU")) {
    fprintf(stderr, "nts_b200: ALGORITHM:%s is not the GPU mini-batch path (GCNNEIGHBORGPU)\n",
            graph->config->algorithm.c_str());
    return 2;
  }
  if (graph->partitions != 1) {
    fprintf(stderr, "nts_b200: built with the single-rank <mpi.h> stand-in; run one process\n");
    return 2;
  }
  prepare_single_rank_graph(graph);

  GCN_GPU_NEIGHBOR_impl *ntsGCN = new GCN_GPU_NEIGHBOR_impl(graph, iterations);
  ntsGCN->init_graph();
  ntsGCN->init_nn();
  std::vector<float> best_val_accs;
  for (int i = 0; i < graph->config->runs; ++i) {
    if (i > 0) ntsGCN->init_active();
    best_val_accs.push_back(ntsGCN->run());
  }
  std::cout << "\nmain(): Best-val-acc: ";
  for (auto &it : best_val_accs) std::cout << it << " ";
  std::cout << std::endl;
  float mean, var;
  std::tie(mean, var) = get_mean_var(best_val_accs);
  printf("Val-mean-var %d runs: %.4f(%.4f)\n", graph->config->runs, mean, var);
  std::cout << "edge_file: " << graph->config->edge_file << std::endl;
  exec_time += get_time();
  if (graph->partition_id == 0) printf("exec_time=%lf(s)\n", exec_time);
  return 0;
}
