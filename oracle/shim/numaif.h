/*
 * Stand-in for libnuma's <numaif.h> (TEST INFRASTRUCTURE ONLY), on the include path of the recipe that compiles
 * the reference project's ESA retrieval backend (ucm/sparse/esa/retrieval/cpy/retrieval_backend.cpp) on machines
 * without libnuma.  That file includes <numaif.h> unconditionally but only calls set_mempolicy when it is built with
 * NUMA_ENABLED, which the recipe does not define.  The two memory-policy calls are declared here as thin wrappers over
 * the raw system calls, so a build that did enable them would still link.
 */
#ifndef UCMR_ORACLE_NUMAIF_SHIM_H_
#define UCMR_ORACLE_NUMAIF_SHIM_H_

#include <sys/syscall.h>
#include <unistd.h>

#define MPOL_DEFAULT 0
#define MPOL_PREFERRED 1
#define MPOL_BIND 2
#define MPOL_INTERLEAVE 3

static inline long set_mempolicy(int mode, const unsigned long* nodemask, unsigned long maxnode)
{
    return syscall(SYS_set_mempolicy, mode, nodemask, maxnode);
}

static inline long mbind(void* addr, unsigned long len, int mode, const unsigned long* nodemask,
                         unsigned long maxnode, unsigned flags)
{
    return syscall(SYS_mbind, addr, len, mode, nodemask, maxnode, flags);
}

#endif
