// The reference's host<->CUDA layer (cuda/ntsCUDA.hpp: class Cuda_Stream and the free allocation / copy helpers)
// implemented on libnb_b200.so.  This file is compiled against the reference's UNCHANGED header and takes the place
// of its static library `cuda_propagate` (cuda/ntsCUDAGraphOP.cu): link a reference build against this object and
// libnb_b200.so and NtsContext::runGraphOp<SingleGPUSampleGraphOp>, Sampler::load_feature_gpu[_cache],
// Sampler::load_label_gpu and sampCSC's device mirrors run on the sm_100a kernels without a source change.
//
// Every method on the sampled mini-batch GCN path forwards to the C ABI (include/nb_b200.h).  Methods of the class
// that belong to other toolkits (GAT edge softmax, the distributed engine's message kernels) keep the reference's
// error convention for a missing implementation: a message and exit (cuda/ntsCUDAGraphOP.cu:13-20).
//
// Build: make -C bindings   (needs the reference tree for its header; output bindings/_build/)
#define CUDA_ENABLE 1
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>

#include "cuda_type.h"
#include "ntsCUDA.hpp"
#include "nb_b200.h"

namespace {

void check_cuda(cudaError_t st, int line) {
  if (st != cudaSuccess) {   // the reference's CHECK_CUDA_RESULT: print and exit
    printf("CUDA call on line %d returned error %d (%s)\n", line, (int)st, cudaGetErrorString(st));
    exit(1);
  }
}
void check_nb(int st, const char *what) {
  if (st != 0) {
    printf("%s failed with status %d: %s\n", what, st, nb_last_error());
    exit(1);
  }
}
[[noreturn]] void not_on_this_path(const char *name) {
  printf("Cuda_Stream::%s is not part of the sampled mini-batch GCN path that libnb_b200 implements\n", name);
  exit(1);
}
#define CUDA_OK(call) check_cuda((call), __LINE__)

}  // namespace

// ---------------------------------------------------------------- allocation and copies (cuda/ntsCUDAGraphOP.cu:22-60, 560-700)
void *getDevicePointer(void *host_data_to_device) {
  void *dev = nullptr;
  CUDA_OK(cudaHostGetDevicePointer(&dev, host_data_to_device, 0));
  return dev;
}
void *cudaMallocPinned(long size_of_bytes) {
  void *data = nullptr;
  CUDA_OK(cudaHostAlloc(&data, size_of_bytes > 0 ? (size_t)size_of_bytes : 1, cudaHostAllocMapped));
  return data;
}
void ntsFreeHost(void *buffer) { CUDA_OK(cudaFreeHost(buffer)); }
void *cudaMallocGPU(long size_of_bytes) {
  void *data = nullptr;
  CUDA_OK(cudaMalloc(&data, size_of_bytes > 0 ? (size_t)size_of_bytes : 1));
  return data;
}
void move_bytes_in(void *d_pointer, void *h_pointer, long bytes, bool sync) {
  CUDA_OK(cudaMemcpy(d_pointer, h_pointer, (size_t)bytes, cudaMemcpyHostToDevice));
  if (sync) CUDA_OK(cudaDeviceSynchronize());
}
void move_bytes_in_async(void *d_pointer, void *h_pointer, long bytes, cudaStream_t cs) {
  CUDA_OK(cudaMemcpyAsync(d_pointer, h_pointer, (size_t)bytes, cudaMemcpyHostToDevice, cs));
}
void move_data_in(float *d_pointer, float *h_pointer, int start, int end, int feature_size, bool sync) {
  move_bytes_in(d_pointer, h_pointer, (long)(end - start) * feature_size * (long)sizeof(float), sync);
}
void move_edge_in(VertexId_CUDA *d_pointer, VertexId_CUDA *h_pointer, VertexId_CUDA start, VertexId_CUDA end,
                  int feature_size, bool sync) {
  move_bytes_in(d_pointer, h_pointer, (long)(end - start) * feature_size * (long)sizeof(VertexId_CUDA), sync);
}
void move_result_out(float *output, float *input, int src, int dst, int feature_size, bool sync) {
  CUDA_OK(cudaMemcpy(output, input, (size_t)(dst - src) * feature_size * sizeof(float), cudaMemcpyDeviceToHost));
  if (sync) CUDA_OK(cudaDeviceSynchronize());
}
void allocate_gpu_buffer(float **input, int size) { *input = (float *)cudaMallocGPU((long)size * (long)sizeof(float)); }
void allocate_gpu_edge(VertexId_CUDA **input, int size) {
  *input = (VertexId_CUDA *)cudaMallocGPU((long)size * (long)sizeof(VertexId_CUDA));
}
void allocate_gpu_buffer_async(float **input, int size, cudaStream_t cs) {
  CUDA_OK(cudaMallocAsync((void **)input, (size_t)(size > 0 ? size : 1) * sizeof(float), cs));
}
void allocate_gpu_edge_async(VertexId_CUDA **input, int size, cudaStream_t cs) {
  CUDA_OK(cudaMallocAsync((void **)input, (size_t)(size > 0 ? size : 1) * sizeof(VertexId_CUDA), cs));
}
void FreeBuffer(float *buffer) { CUDA_OK(cudaFree(buffer)); }
void FreeEdge(VertexId_CUDA *buffer) { CUDA_OK(cudaFree(buffer)); }
void FreeBufferAsync(float *buffer, cudaStream_t cs) { CUDA_OK(cudaFreeAsync(buffer, cs)); }
void FreeEdgeAsync(VertexId_CUDA *buffer, cudaStream_t cs) { CUDA_OK(cudaFreeAsync(buffer, cs)); }
void zero_buffer(float *buffer, int size) { CUDA_OK(cudaMemset(buffer, 0, (size_t)size * sizeof(float))); }
void CUDA_DEVICE_SYNCHRONIZE() { CUDA_OK(cudaDeviceSynchronize()); }
void ResetDevice() { CUDA_OK(cudaDeviceReset()); }
void aggregate_comm_result(float *, float *, int, int, int, bool) { not_on_this_path("aggregate_comm_result (free function)"); }

// ---------------------------------------------------------------- the stream object (cuda/ntsCUDAGraphOP.cu:62-80, 340-373)
Cuda_Stream::Cuda_Stream() { CUDA_OK(cudaStreamCreate(&stream)); }
Cuda_Stream::~Cuda_Stream() {}
void Cuda_Stream::destory_Stream() { CUDA_OK(cudaStreamDestroy(stream)); }
cudaStream_t Cuda_Stream::getStream() { return stream; }
void Cuda_Stream::setNewStream(cudaStream_t cudaStream) {   // adopts the caller's stream; destroys the one it created
  destory_Stream();
  this->stream = cudaStream;
}
void Cuda_Stream::CUDA_DEVICE_SYNCHRONIZE() { CUDA_OK(cudaStreamSynchronize(stream)); }

void Cuda_Stream::move_result_out(float *output, float *input, VertexId_CUDA src, VertexId_CUDA dst, int feature_size,
                                  bool sync) {
  CUDA_OK(cudaMemcpyAsync(output, input, (size_t)(dst - src) * feature_size * sizeof(float), cudaMemcpyDeviceToHost, stream));
  if (sync) CUDA_OK(cudaStreamSynchronize(stream));
}
void Cuda_Stream::move_data_in(float *d_pointer, float *h_pointer, VertexId_CUDA start, VertexId_CUDA end,
                               int feature_size, bool sync) {
  CUDA_OK(cudaMemcpyAsync(d_pointer, h_pointer, (size_t)(end - start) * feature_size * sizeof(float), cudaMemcpyHostToDevice,
                          stream));
  if (sync) CUDA_OK(cudaStreamSynchronize(stream));
}
void Cuda_Stream::move_edge_in(VertexId_CUDA *d_pointer, VertexId_CUDA *h_pointer, VertexId_CUDA start,
                               VertexId_CUDA end, int feature_size, bool sync) {
  CUDA_OK(cudaMemcpyAsync(d_pointer, h_pointer, (size_t)(end - start) * feature_size * sizeof(VertexId_CUDA),
                          cudaMemcpyHostToDevice, stream));
  if (sync) CUDA_OK(cudaStreamSynchronize(stream));
}

// ---------------------------------------------------------------- aggregation (cuda/ntsCUDAGraphOP.cu:186-292)
// y[d,:] = sum_j w[j] * x[row_indices[j] - src_start,:].  The reference adds into an output it zeroed beforehand;
// nb_spmm_csc_fwd writes every row, which gives the same values.  The caller synchronises afterwards itself
// (core/ntsMiniBatchGraphOp.hpp:316).
void Cuda_Stream::Gather_By_Dst_From_Src(float *input, float *output, float *weight_forward, VertexId_CUDA *row_indices,
                                         VertexId_CUDA *column_offset, VertexId_CUDA src_start, VertexId_CUDA,
                                         VertexId_CUDA, VertexId_CUDA, VertexId_CUDA, VertexId_CUDA batch_size,
                                         VertexId_CUDA feature_size, bool with_weight, bool tensor_weight) {
  if (!with_weight || tensor_weight) not_on_this_path("Gather_By_Dst_From_Src without scalar edge weights");
  check_nb(nb_spmm_csc_fwd(input - (size_t)src_start * feature_size, output, weight_forward, row_indices, column_offset,
                           batch_size, feature_size, stream),
           "nb_spmm_csc_fwd");
}
void Cuda_Stream::Gather_By_Dst_From_Src_Optim(float *input, float *output, float *weight_forward,
                                               VertexId_CUDA *row_indices, VertexId_CUDA *column_offset,
                                               VertexId_CUDA src_start, VertexId_CUDA src_end, VertexId_CUDA dst_start,
                                               VertexId_CUDA dst_end, VertexId_CUDA edges, VertexId_CUDA batch_size,
                                               VertexId_CUDA feature_size, bool with_weight, bool tensor_weight) {
  Gather_By_Dst_From_Src(input, output, weight_forward, row_indices, column_offset, src_start, src_end, dst_start, dst_end,
                         edges, batch_size, feature_size, with_weight, tensor_weight);
}
// gx[s,:] = sum_j w[j] * gy[column_indices[j] - dst_start,:]
void Cuda_Stream::Gather_By_Src_From_Dst(float *input, float *output, float *weight_backward, VertexId_CUDA *row_offset,
                                         VertexId_CUDA *column_indices, VertexId_CUDA, VertexId_CUDA,
                                         VertexId_CUDA dst_start, VertexId_CUDA, VertexId_CUDA, VertexId_CUDA batch_size,
                                         VertexId_CUDA feature_size, bool with_weight, bool tensor_weight) {
  if (!with_weight || tensor_weight) not_on_this_path("Gather_By_Src_From_Dst without scalar edge weights");
  check_nb(nb_spmm_csr_bwd(input - (size_t)dst_start * feature_size, output, weight_backward, row_offset, column_indices,
                           batch_size, feature_size, stream),
           "nb_spmm_csr_bwd");
}
void Cuda_Stream::Gather_By_Src_From_Dst_Optim(float *input, float *output, float *weight_backward,
                                               VertexId_CUDA *row_offset, VertexId_CUDA *column_indices,
                                               VertexId_CUDA src_start, VertexId_CUDA src_end, VertexId_CUDA dst_start,
                                               VertexId_CUDA dst_end, VertexId_CUDA edges, VertexId_CUDA batch_size,
                                               VertexId_CUDA feature_size, bool with_weight, bool tensor_weight) {
  Gather_By_Src_From_Dst(input, output, weight_backward, row_offset, column_indices, src_start, src_end, dst_start, dst_end,
                         edges, batch_size, feature_size, with_weight, tensor_weight);
}

// ---------------------------------------------------------------- feature and label movement (cuda/ntsCUDAGraphOP.cu:379-450)
// Each of these synchronises the stream before it returns, as the reference's do.
void Cuda_Stream::zero_copy_feature_move_gpu(float *dev_feature, float *pinned_host_feature, VertexId_CUDA *src_vertex,
                                             VertexId_CUDA feature_size, VertexId_CUDA vertex_size) {
  check_nb(nb_feature_gather(dev_feature, pinned_host_feature, feature_size, nullptr, 0, 0, nullptr, 0, nullptr, src_vertex,
                             vertex_size, feature_size, stream),
           "nb_feature_gather");
  CUDA_DEVICE_SYNCHRONIZE();
}
void Cuda_Stream::zero_copy_feature_move_gpu_cache(float *dev_feature, float *host_pinned_feature,
                                                   VertexId_CUDA *src_vertex, VertexId_CUDA feature_size,
                                                   VertexId_CUDA vertex_size, VertexId_CUDA *local_idx) {
  check_nb(nb_feature_gather_indexed(dev_feature, feature_size, host_pinned_feature, feature_size, src_vertex, local_idx,
                                     nullptr, vertex_size, feature_size, stream),
           "nb_feature_gather_indexed");
  CUDA_DEVICE_SYNCHRONIZE();
}
void Cuda_Stream::gather_feature_from_gpu_cache(float *dev_feature, float *dev_cache_feature, VertexId_CUDA *src_vertex,
                                                VertexId_CUDA feature_size, VertexId_CUDA vertex_size,
                                                VertexId_CUDA *local_idx, VertexId_CUDA *cache_node_hashmap) {
  check_nb(nb_feature_gather_indexed(dev_feature, feature_size, dev_cache_feature, feature_size, src_vertex, local_idx,
                                     cache_node_hashmap, vertex_size, feature_size, stream),
           "nb_feature_gather_indexed");
  CUDA_DEVICE_SYNCHRONIZE();
}
void Cuda_Stream::global_copy_label_move_gpu(long *dev_label, long *global_dev_label, VertexId_CUDA *dst_vertex,
                                             VertexId_CUDA vertex_size) {
  check_nb(nb_label_gather((int64_t *)dev_label, (const int64_t *)global_dev_label, dst_vertex, vertex_size, 1, stream),
           "nb_label_gather");
  CUDA_DEVICE_SYNCHRONIZE();
}
void Cuda_Stream::global_copy_mulilabel_move_gpu(long *dev_label, long *global_dev_label, VertexId_CUDA *dst_vertex,
                                                 VertexId_CUDA vertex_size, VertexId_CUDA label_size) {
  check_nb(nb_label_gather((int64_t *)dev_label, (const int64_t *)global_dev_label, dst_vertex, vertex_size, label_size,
                           stream),
           "nb_label_gather");
  CUDA_DEVICE_SYNCHRONIZE();
}
void Cuda_Stream::zero_copy_embedding_move_gpu(float *dev_feature, float *pinned_host_feature,
                                               VertexId_CUDA feature_size, VertexId_CUDA vertex_size) {
  CUDA_OK(cudaMemcpyAsync(dev_feature, pinned_host_feature, (size_t)vertex_size * feature_size * sizeof(float),
                          cudaMemcpyDefault, stream));
  CUDA_DEVICE_SYNCHRONIZE();
}

// ---------------------------------------------------------------- other toolkits' kernels: not built
void Cuda_Stream::aggregate_comm_result(float *, float *, VertexId_CUDA, int, int, bool) { not_on_this_path("aggregate_comm_result"); }
void Cuda_Stream::deSerializeToGPU(float *, float *, VertexId_CUDA, VertexId_CUDA, VertexId_CUDA, VertexId_CUDA, bool) {
  not_on_this_path("deSerializeToGPU");
}
void Cuda_Stream::aggregate_comm_result_debug(float *, float *, VertexId_CUDA, VertexId_CUDA, VertexId_CUDA, VertexId_CUDA,
                                              bool) {
  not_on_this_path("aggregate_comm_result_debug");
}
void Cuda_Stream::Scatter_Src_Mirror_to_Msg(float *, float *, VertexId_CUDA *, VertexId_CUDA *, VertexId_CUDA *,
                                            VertexId_CUDA, VertexId_CUDA) {
  not_on_this_path("Scatter_Src_Mirror_to_Msg");
}
void Cuda_Stream::Gather_Msg_To_Src_Mirror(float *, float *, VertexId_CUDA *, VertexId_CUDA *, VertexId_CUDA *,
                                           VertexId_CUDA, VertexId_CUDA) {
  not_on_this_path("Gather_Msg_To_Src_Mirror");
}
void Cuda_Stream::Scatter_Dst_to_Msg(float *, float *, VertexId_CUDA *, VertexId_CUDA *, VertexId_CUDA, VertexId_CUDA) {
  not_on_this_path("Scatter_Dst_to_Msg");
}
void Cuda_Stream::Gather_Msg_to_Dst(float *, float *, VertexId_CUDA *, VertexId_CUDA *, VertexId_CUDA, VertexId_CUDA) {
  not_on_this_path("Gather_Msg_to_Dst");
}
void Cuda_Stream::Edge_Softmax_Forward_Block(float *, float *, float *, VertexId_CUDA *, VertexId_CUDA *, VertexId_CUDA,
                                             VertexId_CUDA) {
  not_on_this_path("Edge_Softmax_Forward_Block");
}
void Cuda_Stream::Edge_Softmax_Backward_Block(float *, float *, float *, VertexId_CUDA *, VertexId_CUDA *, VertexId_CUDA,
                                              VertexId_CUDA) {
  not_on_this_path("Edge_Softmax_Backward_Block");
}
void Cuda_Stream::Gather_By_Dst_From_Message(float *, float *, VertexId_CUDA *, VertexId_CUDA *, VertexId_CUDA, VertexId_CUDA,
                                             VertexId_CUDA, VertexId_CUDA, VertexId_CUDA, VertexId_CUDA, VertexId_CUDA, bool,
                                             bool) {
  not_on_this_path("Gather_By_Dst_From_Message");
}
void Cuda_Stream::Scatter_Grad_Back_To_Message(float *, float *, VertexId_CUDA *, VertexId_CUDA *, VertexId_CUDA,
                                               VertexId_CUDA, VertexId_CUDA, VertexId_CUDA, VertexId_CUDA, VertexId_CUDA,
                                               VertexId_CUDA, bool) {
  not_on_this_path("Scatter_Grad_Back_To_Message");
}
