// SPDX-License-Identifier: Apache-2.0
/* Stand-in for hwloc's NVML helper (see ../hwloc.h): never called. */
#ifndef CS_BASELINE_HWLOC_NVML_SHIM_H
#define CS_BASELINE_HWLOC_NVML_SHIM_H
#include <nvml.h>

#include "../hwloc.h"
static inline int hwloc_nvml_get_device_cpuset(hwloc_topology_t t, nvmlDevice_t d, hwloc_cpuset_t s) { (void)t; (void)d; (void)s; return 0; }
#endif
