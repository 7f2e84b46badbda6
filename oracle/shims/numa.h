/* Single-node stand-in for <numa.h> (libnuma is not installed): one node, plain malloc. */
#ifndef NB_ORACLE_SHIM_NUMA_H
#define NB_ORACLE_SHIM_NUMA_H
#include <stdlib.h>
#include <string.h>
#include <unistd.h>
struct bitmask { unsigned long size; unsigned long *maskp; };
static inline int numa_available(void) { return 0; }
static inline int numa_num_configured_cpus(void) { long n = sysconf(_SC_NPROCESSORS_ONLN); return n > 0 ? (int)n : 1; }
static inline int numa_num_configured_nodes(void) { return 1; }
static inline void *numa_alloc_onnode(size_t n, int) { return calloc(1, n ? n : 1); }
static inline void *numa_alloc_interleaved(size_t n) { return calloc(1, n ? n : 1); }
static inline void *numa_realloc(void *p, size_t, size_t n) { return realloc(p, n); }
static inline void numa_free(void *p, size_t) { free(p); }
static inline int numa_run_on_node(int) { return 0; }
static inline void numa_tonode_memory(void *, size_t, int) {}
static inline struct bitmask *numa_parse_nodestring(const char *) { static struct bitmask b; return &b; }
static inline void numa_set_interleave_mask(struct bitmask *) {}
#endif
