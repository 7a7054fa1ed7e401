// SPDX-License-Identifier: Apache-2.0
/* Empty stand-in for hwloc: the reference project's CPU-affinity helpers in
 * src/threading/dynamic_scheduler.cpp are compiled but never called. Enough types and inline
 * no-ops for that file to compile; nothing here does any work. */
#ifndef CS_BASELINE_HWLOC_SHIM_H
#define CS_BASELINE_HWLOC_SHIM_H
typedef struct hwloc_topology *hwloc_topology_t;
typedef struct hwloc_bitmap_s *hwloc_bitmap_t;
typedef hwloc_bitmap_t hwloc_cpuset_t;
typedef const struct hwloc_bitmap_s *hwloc_const_cpuset_t;
struct hwloc_obj { unsigned os_index; };
typedef struct hwloc_obj *hwloc_obj_t;
typedef enum { HWLOC_OBJ_PU = 3 } hwloc_obj_type_t;
#define HWLOC_CPUBIND_THREAD 2
static inline int hwloc_topology_init(hwloc_topology_t *t) { *t = 0; return 0; }
static inline int hwloc_topology_load(hwloc_topology_t t) { (void)t; return 0; }
static inline void hwloc_topology_destroy(hwloc_topology_t t) { (void)t; }
static inline hwloc_bitmap_t hwloc_bitmap_alloc(void) { return 0; }
static inline void hwloc_bitmap_free(hwloc_bitmap_t b) { (void)b; }
static inline int hwloc_bitmap_set(hwloc_bitmap_t b, unsigned i) { (void)b; (void)i; return 0; }
static inline int hwloc_bitmap_and(hwloc_bitmap_t r, hwloc_bitmap_t a, hwloc_bitmap_t b) { (void)r; (void)a; (void)b; return 0; }
static inline int hwloc_bitmap_iszero(hwloc_bitmap_t b) { (void)b; return 1; }
static inline int hwloc_bitmap_first(hwloc_bitmap_t b) { (void)b; return -1; }
static inline int hwloc_bitmap_next(hwloc_bitmap_t b, int p) { (void)b; (void)p; return -1; }
static inline int hwloc_bitmap_weight(hwloc_bitmap_t b) { (void)b; return 0; }
static inline hwloc_bitmap_t hwloc_bitmap_dup(hwloc_bitmap_t b) { return b; }
static inline int hwloc_bitmap_only(hwloc_bitmap_t b, unsigned i) { (void)b; (void)i; return 0; }
static inline int hwloc_bitmap_singlify(hwloc_bitmap_t b) { (void)b; return 0; }
static inline int hwloc_get_nbobjs_by_type(hwloc_topology_t t, hwloc_obj_type_t ty) { (void)t; (void)ty; return 0; }
static inline hwloc_obj_t hwloc_get_obj_by_type(hwloc_topology_t t, hwloc_obj_type_t ty, unsigned i) { (void)t; (void)ty; (void)i; return 0; }
static inline int hwloc_set_cpubind(hwloc_topology_t t, hwloc_const_cpuset_t s, int f) { (void)t; (void)s; (void)f; return 0; }
static inline int hwloc_get_cpubind(hwloc_topology_t t, hwloc_cpuset_t s, int f) { (void)t; (void)s; (void)f; return 0; }
#endif
