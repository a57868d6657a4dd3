/* No-op stand-in for libnuma (mlp_omp.cc:10,33-38,429-433): the reference binds
 * each OpenMP thread to its socket's memory node; without libnuma the binding is
 * skipped and every "socket" shares the machine's memory.  Checker infrastructure. */
#ifndef B2_SHIM_NUMA_H
#define B2_SHIM_NUMA_H
struct bitmask { int unused; };
static inline struct bitmask* numa_allocate_nodemask(void) { static struct bitmask m; return &m; }
static inline void numa_bitmask_clearall(struct bitmask*) {}
static inline void numa_bitmask_setbit(struct bitmask*, unsigned) {}
static inline void numa_bind(struct bitmask*) {}
static inline void numa_bitmask_free(struct bitmask*) {}
#endif
