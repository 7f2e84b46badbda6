// Host-memory stand-ins for the reference's CUDA helpers (declared in cuda/ntsCUDA.hpp, defined in
// cuda/ntsCUDAGraphOP.cu, which needs a GPU).  The reference's CPU sampling path calls them
// unconditionally to mirror every block on the device (core/coocsc.hpp:621-671); here the "device"
// arrays are plain host allocations that nothing reads.  Test infrastructure only.
#include <cstdlib>
#include <cstring>
#include <cuda_runtime.h>
#include "cuda_type.h"
#include "ntsCUDA.hpp"

Cuda_Stream::Cuda_Stream() { stream = nullptr; }
// sampCSC's destructor frees members it never initialised (core/coocsc.hpp:100-116); leak instead.
void FreeBuffer(float *) {}
void FreeEdge(VertexId_CUDA *) {}
void allocate_gpu_buffer(float **input, int size) { *input = (float *)calloc(size > 0 ? size : 1, sizeof(float)); }
void allocate_gpu_edge(VertexId_CUDA **input, int size) {
  *input = (VertexId_CUDA *)calloc(size > 0 ? size : 1, sizeof(VertexId_CUDA));
}
// comm/network.cpp allocates its message buffers "pinned"; ordinary host memory serves a single rank.
void *cudaMallocPinned(long size_of_bytes) { return calloc(size_of_bytes > 0 ? (size_t)size_of_bytes : 1, 1); }
