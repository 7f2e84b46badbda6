/* Single-rank stand-in for <mpi.h>, just enough for the reference's headers to compile and run as
 * one process (rank 0 of 1).  Test infrastructure for the reference-backed oracle only. */
#ifndef NB_ORACLE_SHIM_MPI_H
#define NB_ORACLE_SHIM_MPI_H
#include <string.h>
#include <sys/time.h>
typedef int MPI_Comm;
typedef int MPI_Datatype;
typedef int MPI_Op;
typedef int MPI_Request;
typedef int MPI_Message;
typedef struct { int MPI_SOURCE, MPI_TAG, MPI_ERROR, count_; } MPI_Status;
#define MPI_COMM_WORLD 0
#define MPI_SUCCESS 0
#define MPI_CHAR 1
#define MPI_UNSIGNED_CHAR 1
#define MPI_UINT8_T 1
#define MPI_INT 4
#define MPI_UNSIGNED 4
#define MPI_UINT 4
#define MPI_FLOAT 4
#define MPI_LONG 8
#define MPI_UNSIGNED_LONG 8
#define MPI_DOUBLE 8
#define MPI_SUM 0
#define MPI_MIN 1
#define MPI_MAX 2
#define MPI_IN_PLACE ((void *)1)
#define MPI_STATUS_IGNORE ((MPI_Status *)0)
#define MPI_ANY_SOURCE (-1)
#define MPI_ANY_TAG (-1)
#define MPI_THREAD_SINGLE 0
#define MPI_THREAD_FUNNELED 1
#define MPI_THREAD_SERIALIZED 2
#define MPI_THREAD_MULTIPLE 3
static inline int MPI_Init_thread(int *, char ***, int required, int *provided) { if (provided) *provided = required; return 0; }
static inline int MPI_Initialized(int *flag) { *flag = 1; return 0; }
static inline int MPI_Finalize(void) { return 0; }
static inline int MPI_Abort(MPI_Comm, int) { return 0; }
static inline int MPI_Comm_rank(MPI_Comm, int *r) { *r = 0; return 0; }
static inline int MPI_Comm_size(MPI_Comm, int *s) { *s = 1; return 0; }
static inline int MPI_Barrier(MPI_Comm) { return 0; }
static inline double MPI_Wtime(void) { struct timeval tv; gettimeofday(&tv, 0); return tv.tv_sec + tv.tv_usec * 1e-6; }
/* one rank: a sum / min / max over ranks is the identity */
static inline int MPI_Allreduce(const void *s, void *r, int n, MPI_Datatype t, MPI_Op, MPI_Comm) {
  if (s != MPI_IN_PLACE && s != r) memcpy(r, s, (size_t)n * (size_t)t);
  return 0;
}
static inline int MPI_Bcast(void *, int, MPI_Datatype, int, MPI_Comm) { return 0; }
static inline int MPI_Send(const void *, int, MPI_Datatype, int, int, MPI_Comm) { return 0; }
static inline int MPI_Issend(const void *, int, MPI_Datatype, int, int, MPI_Comm, MPI_Request *) { return 0; }
static inline int MPI_Recv(void *, int, MPI_Datatype, int, int, MPI_Comm, MPI_Status *) { return 0; }
static inline int MPI_Probe(int, int, MPI_Comm, MPI_Status *) { return 0; }
static inline int MPI_Iprobe(int, int, MPI_Comm, int *flag, MPI_Status *) { *flag = 0; return 0; }
static inline int MPI_Improbe(int, int, MPI_Comm, int *flag, MPI_Message *, MPI_Status *) { *flag = 0; return 0; }
static inline int MPI_Test(MPI_Request *, int *flag, MPI_Status *) { *flag = 1; return 0; }
static inline int MPI_Get_count(const MPI_Status *, MPI_Datatype, int *c) { *c = 0; return 0; }
#endif
