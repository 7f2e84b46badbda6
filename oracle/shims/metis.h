/* Stand-in for <metis.h> (the METIS submodule is not vendored in the reference tree).  BATCH_TYPE:metis
 * is outside the sampled-GCN hot path; the entry points only have to exist for the headers to compile. */
#ifndef NB_ORACLE_SHIM_METIS_H
#define NB_ORACLE_SHIM_METIS_H
#include <stdint.h>
typedef int64_t idx_t;
typedef float real_t;
#define METIS_NOPTIONS 40
enum { METIS_OK = 1, METIS_ERROR_INPUT = -2, METIS_ERROR_MEMORY = -3, METIS_ERROR = -4 };
enum { METIS_OPTION_PTYPE, METIS_OPTION_OBJTYPE, METIS_OPTION_CTYPE, METIS_OPTION_IPTYPE, METIS_OPTION_RTYPE,
       METIS_OPTION_DBGLVL, METIS_OPTION_NIPARTS, METIS_OPTION_NITER, METIS_OPTION_NCUTS, METIS_OPTION_SEED,
       METIS_OPTION_ONDISK, METIS_OPTION_MINCONN, METIS_OPTION_CONTIG, METIS_OPTION_COMPRESS, METIS_OPTION_CCORDER,
       METIS_OPTION_PFACTOR, METIS_OPTION_NSEPS, METIS_OPTION_UFACTOR, METIS_OPTION_NUMBERING, METIS_OPTION_DROPEDGES };
enum { METIS_OBJTYPE_CUT, METIS_OBJTYPE_VOL, METIS_OBJTYPE_NODE };
static inline int METIS_SetDefaultOptions(idx_t *) { return METIS_OK; }
static inline int METIS_PartGraphKway(idx_t *, idx_t *, idx_t *, idx_t *, idx_t *, idx_t *, idx_t *, idx_t *, real_t *,
                                      real_t *, idx_t *, idx_t *, idx_t *) { return METIS_ERROR; }
static inline int METIS_PartGraphRecursive(idx_t *, idx_t *, idx_t *, idx_t *, idx_t *, idx_t *, idx_t *, idx_t *,
                                           real_t *, real_t *, idx_t *, idx_t *, idx_t *) { return METIS_ERROR; }
#endif
