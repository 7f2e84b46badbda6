// Gradient sum over the ranks of a data-parallel job for hosts that do not bring their own collective library: a thin
// layer over NCCL (one communicator per process and GPU).  Built as a library of its own, libnb_b200_comm.so, so that
// libnb_b200.so itself depends on nothing but the CUDA runtime.  Replaces Network_simple::all_reduce_sum / broadcast
// (comm/network.h:189-193, 195-200; MPI over host buffers in the reference) on device buffers.
#include <nccl.h>

#include <new>

#include "common.cuh"

struct nb_comm {
  ncclComm_t comm = nullptr;
  int world = 0, rank = 0;
};

static_assert(sizeof(ncclUniqueId) == 128, "the C ABI passes the NCCL unique id as 128 bytes");

#define NB_NCCL(call)                                                                          \
  do {                                                                                         \
    ncclResult_t r__ = (call);                                                                 \
    if (r__ != ncclSuccess) {                                                                  \
      nb::set_error("%s:%d %s -> %s", __FILE__, __LINE__, #call, ncclGetErrorString(r__));     \
      return (int)NB_ERR_CUDA;                                                                 \
    }                                                                                          \
  } while (0)

NB_API int nb_comm_unique_id(unsigned char id[128]) {
  NB_REQUIRE(id != nullptr, "nb_comm_unique_id: null pointer");
  ncclUniqueId u;
  NB_NCCL(ncclGetUniqueId(&u));
  memcpy(id, &u, sizeof(u));
  return 0;
}

NB_API int nb_comm_create(nb_comm **out, const unsigned char id[128], int world, int rank) {
  NB_REQUIRE(out && id, "nb_comm_create: null pointer");
  NB_REQUIRE(world >= 1 && rank >= 0 && rank < world, "nb_comm_create: rank outside [0, world)");
  nb_comm *c = new (std::nothrow) nb_comm();
  if (!c) return nb::fail(NB_ERR_NOMEM, "nb_comm_create: out of host memory");
  ncclUniqueId u;
  memcpy(&u, id, sizeof(u));
  const ncclResult_t r = ncclCommInitRank(&c->comm, world, u, rank);
  if (r != ncclSuccess) {
    delete c;
    nb::set_error("nb_comm_create: ncclCommInitRank -> %s", ncclGetErrorString(r));
    return (int)NB_ERR_CUDA;
  }
  c->world = world;
  c->rank = rank;
  *out = c;
  return 0;
}

NB_API int nb_comm_destroy(nb_comm *c) {
  if (c) {
    if (c->comm) ncclCommDestroy(c->comm);
    delete c;
  }
  return 0;
}

NB_API int nb_allreduce_sum_f32(nb_comm *c, float *d_buf, size_t n, void *stream) {
  NB_REQUIRE(c && c->comm && (d_buf || n == 0), "nb_allreduce_sum_f32: null pointer");
  if (n == 0) return 0;
  NB_NCCL(ncclAllReduce(d_buf, d_buf, n, ncclFloat32, ncclSum, c->comm, nb::as_stream(stream)));
  return 0;
}

NB_API int nb_broadcast_f32(nb_comm *c, float *d_buf, size_t n, int root, void *stream) {
  NB_REQUIRE(c && c->comm && (d_buf || n == 0), "nb_broadcast_f32: null pointer");
  NB_REQUIRE(root >= 0 && root < c->world, "nb_broadcast_f32: root outside [0, world)");
  if (n == 0) return 0;
  NB_NCCL(ncclBroadcast(d_buf, d_buf, n, ncclFloat32, root, c->comm, nb::as_stream(stream)));
  return 0;
}
