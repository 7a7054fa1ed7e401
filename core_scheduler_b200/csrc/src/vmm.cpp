// SPDX-License-Identifier: Apache-2.0
// See vmm.h.
#include "vmm.h"

#include <cuda_runtime.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <cstdlib>
#include <cstring>

namespace cs::communication::vmm {
namespace {
#ifndef SYS_pidfd_open
#define SYS_pidfd_open 434
#endif
#ifndef SYS_pidfd_getfd
#define SYS_pidfd_getfd 438
#endif

// Driver entry points are resolved at run time: the library links only the CUDA runtime.
struct Driver {
  CUresult (*MemCreate)(CUmemGenericAllocationHandle *, size_t, const CUmemAllocationProp *, unsigned long long);
  CUresult (*MemRelease)(CUmemGenericAllocationHandle);
  CUresult (*MemAddressReserve)(CUdeviceptr *, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*MemAddressFree)(CUdeviceptr, size_t);
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*MemUnmap)(CUdeviceptr, size_t);
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc *, size_t);
  CUresult (*MemExportToShareableHandle)(void *, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle *, void *, CUmemAllocationHandleType);
  CUresult (*MemGetAllocationGranularity)(size_t *, const CUmemAllocationProp *, CUmemAllocationGranularity_flags);
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle *, const CUmulticastObjectProp *);
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
  CUresult (*MulticastGetGranularity)(size_t *, const CUmulticastObjectProp *, CUmulticastGranularity_flags);
  CUresult (*DeviceGet)(CUdevice *, int);
  CUresult (*DeviceGetAttribute)(int *, CUdevice_attribute, CUdevice);
  bool ok{false};
};

template <typename Fn>
bool resolve(Fn *&fn, const char *name) {
  void *ptr = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &ptr, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !ptr) {
    (void)cudaGetLastError();
    return false;
  }
  fn = reinterpret_cast<Fn *>(ptr);
  return true;
}

const Driver &driver() {
  static const Driver d = [] {
    Driver x{};
    x.ok = resolve(x.MemCreate, "cuMemCreate") && resolve(x.MemRelease, "cuMemRelease") &&
           resolve(x.MemAddressReserve, "cuMemAddressReserve") && resolve(x.MemAddressFree, "cuMemAddressFree") &&
           resolve(x.MemMap, "cuMemMap") && resolve(x.MemUnmap, "cuMemUnmap") && resolve(x.MemSetAccess, "cuMemSetAccess") &&
           resolve(x.MemExportToShareableHandle, "cuMemExportToShareableHandle") &&
           resolve(x.MemImportFromShareableHandle, "cuMemImportFromShareableHandle") &&
           resolve(x.MemGetAllocationGranularity, "cuMemGetAllocationGranularity") && resolve(x.DeviceGet, "cuDeviceGet") &&
           resolve(x.DeviceGetAttribute, "cuDeviceGetAttribute");
    // multicast entry points are optional (older drivers): their absence only disables multicast
    if (!(resolve(x.MulticastCreate, "cuMulticastCreate") && resolve(x.MulticastAddDevice, "cuMulticastAddDevice") &&
          resolve(x.MulticastBindMem, "cuMulticastBindMem") && resolve(x.MulticastUnbind, "cuMulticastUnbind") &&
          resolve(x.MulticastGetGranularity, "cuMulticastGetGranularity")))
      x.MulticastCreate = nullptr;
    return x;
  }();
  return d;
}

std::string key(const char *what, int rank) { return std::string(what) + "/" + std::to_string(rank); }

// Every rank publishes whether its step worked and reads everybody's answer: all ranks take the same branch.
bool all_ok(Exchange &ex, const char *what, int rank, int size, bool mine) {
  ex.put(key(what, rank), mine ? "1" : "0");
  bool ok = true;
  for (int p = 0; p < size; ++p) ok = (ex.get(key(what, p)) == "1") && ok;
  return ok;
}

bool map_range(const Driver &d, CUmemGenericAllocationHandle handle, int64_t bytes, size_t granularity, int device, char **out) {
  CUdeviceptr va = 0;
  if (d.MemAddressReserve(&va, static_cast<size_t>(bytes), granularity, 0, 0) != CUDA_SUCCESS) return false;
  if (d.MemMap(va, static_cast<size_t>(bytes), 0, handle, 0) != CUDA_SUCCESS) {
    d.MemAddressFree(va, static_cast<size_t>(bytes));
    return false;
  }
  CUmemAccessDesc access{};
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = device;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  if (d.MemSetAccess(va, static_cast<size_t>(bytes), &access, 1) != CUDA_SUCCESS) {
    d.MemUnmap(va, static_cast<size_t>(bytes));
    d.MemAddressFree(va, static_cast<size_t>(bytes));
    return false;
  }
  *out = reinterpret_cast<char *>(va);
  return true;
}

void unmap_range(const Driver &d, char *va, int64_t bytes) {
  if (!va) return;
  d.MemUnmap(reinterpret_cast<CUdeviceptr>(va), static_cast<size_t>(bytes));
  d.MemAddressFree(reinterpret_cast<CUdeviceptr>(va), static_cast<size_t>(bytes));
}

// "pid:fd" <-> handle
std::string describe(int fd) { return std::to_string(static_cast<long long>(getpid())) + ":" + std::to_string(fd); }
bool import_described(const Driver &d, const std::string &text, CUmemGenericAllocationHandle *out) {
  const auto colon = text.find(':');
  if (colon == std::string::npos) return false;
  const int pid = std::atoi(text.substr(0, colon).c_str()), fd = std::atoi(text.substr(colon + 1).c_str());
  const int local = duplicate_descriptor(pid, fd);
  if (local < 0) return false;
  const CUresult r = d.MemImportFromShareableHandle(out, reinterpret_cast<void *>(static_cast<uintptr_t>(local)),
                                                    CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  close(local);
  return r == CUDA_SUCCESS;
}
}  // namespace

int duplicate_descriptor(int pid, int fd) {
  if (pid == static_cast<int>(getpid())) return dup(fd);
  const long pidfd = syscall(SYS_pidfd_open, pid, 0);
  if (pidfd < 0) return -1;
  const long local = syscall(SYS_pidfd_getfd, static_cast<int>(pidfd), fd, 0);
  close(static_cast<int>(pidfd));
  return local < 0 ? -1 : static_cast<int>(local);
}

bool create(Arena *out, int rank, int size, int device, int64_t bytes, bool want_multicast, Exchange &ex, std::string *why) {
  const Driver &d = driver();
  Arena a{};
  a.device = device;
  a.rank = rank;
  a.peer_va.assign(static_cast<size_t>(size), nullptr);
  a.handles.assign(static_cast<size_t>(size), 0);
  auto fail = [&](const char *what) {
    if (why) *why = what;
    destroy(&a);
    return false;
  };

  // ---- 1. own allocation, exported as a file descriptor --------------------------------------
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t granularity = 2 << 20;
  int own_fd = -1;
  bool ok = d.ok;
  CUdevice cu_device = 0;
  int multicast_supported = 0;
  CUmulticastObjectProp mc_prop{};
  if (ok) {
    ok = d.DeviceGet(&cu_device, device) == CUDA_SUCCESS &&
         d.MemGetAllocationGranularity(&granularity, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS;
  }
  if (ok && want_multicast && d.MulticastCreate) {
    if (d.DeviceGetAttribute(&multicast_supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cu_device) != CUDA_SUCCESS)
      multicast_supported = 0;
    if (multicast_supported) {
      mc_prop.numDevices = static_cast<unsigned>(size);
      mc_prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
      mc_prop.size = static_cast<size_t>(bytes);
      size_t mc_gran = 0;
      if (d.MulticastGetGranularity(&mc_gran, &mc_prop, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mc_gran > granularity)
        granularity = mc_gran;
    }
  }
  if (ok) {
    a.bytes = (bytes + static_cast<int64_t>(granularity) - 1) / static_cast<int64_t>(granularity) * static_cast<int64_t>(granularity);
    ok = d.MemCreate(&a.handles[rank], static_cast<size_t>(a.bytes), &prop, 0) == CUDA_SUCCESS;
    if (!ok) a.handles[rank] = 0;
  }
  if (ok)
    ok = d.MemExportToShareableHandle(&own_fd, a.handles[rank], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) == CUDA_SUCCESS;
  ex.put(key("vmm/handle", rank), ok ? describe(own_fd) : std::string("none"));
  if (!all_ok(ex, "vmm/created", rank, size, ok)) {
    if (own_fd >= 0) close(own_fd);
    return fail("cuMemCreate / export of the arena failed on a rank");
  }

  // ---- 2. import and map every peer ------------------------------------------------------------
  ok = map_range(d, a.handles[rank], a.bytes, granularity, device, &a.peer_va[rank]);
  for (int p = 0; ok && p < size; ++p) {
    if (p == rank) continue;
    ok = import_described(d, ex.get(key("vmm/handle", p)), &a.handles[p]);
    if (!ok) {
      a.handles[p] = 0;
      break;
    }
    ok = map_range(d, a.handles[p], a.bytes, granularity, device, &a.peer_va[p]);
  }
  const bool mapped = all_ok(ex, "vmm/mapped", rank, size, ok);  // also: nobody needs our descriptor any more
  close(own_fd);
  if (!mapped) return fail("importing or mapping a peer's arena failed on a rank (pidfd_getfd / cuMemImportFromShareableHandle / cuMemMap)");

  // ---- 3. multicast object over the same pages (optional) ---------------------------------------
  bool mc = all_ok(ex, "vmm/mc_supported", rank, size, multicast_supported != 0 && want_multicast);
  if (mc) {
    int mc_fd = -1;
    mc_prop.size = static_cast<size_t>(a.bytes);
    bool step = true;
    if (rank == 0) {
      step = d.MulticastCreate(&a.multicast_handle, &mc_prop) == CUDA_SUCCESS;
      if (!step) a.multicast_handle = 0;
      if (step) step = d.MemExportToShareableHandle(&mc_fd, a.multicast_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) == CUDA_SUCCESS;
      ex.put("vmm/mc_handle", step ? describe(mc_fd) : std::string("none"));
    } else {
      step = import_described(d, ex.get("vmm/mc_handle"), &a.multicast_handle);
      if (!step) a.multicast_handle = 0;
    }
    mc = all_ok(ex, "vmm/mc_imported", rank, size, step);
    if (mc_fd >= 0) close(mc_fd);
    if (mc) mc = all_ok(ex, "vmm/mc_added", rank, size, d.MulticastAddDevice(a.multicast_handle, cu_device) == CUDA_SUCCESS);
    if (mc) {
      // every device has been added (agreed above) before anyone binds memory
      step = d.MulticastBindMem(a.multicast_handle, 0, a.handles[rank], 0, static_cast<size_t>(a.bytes), 0) == CUDA_SUCCESS;
      a.multicast_bound = step;
      mc = all_ok(ex, "vmm/mc_bound", rank, size, step);
    }
    if (mc) mc = all_ok(ex, "vmm/mc_mapped", rank, size, map_range(d, a.multicast_handle, a.bytes, granularity, device, &a.multicast_va));
    if (!mc) {
      // peer mappings stay usable; drop whatever part of the multicast object exists
      if (a.multicast_va) unmap_range(d, a.multicast_va, a.bytes);
      a.multicast_va = nullptr;
      if (a.multicast_bound) d.MulticastUnbind(a.multicast_handle, cu_device, 0, static_cast<size_t>(a.bytes));
      a.multicast_bound = false;
      if (a.multicast_handle) d.MemRelease(a.multicast_handle);
      a.multicast_handle = 0;
      ex.barrier("vmm/mc_dropped");
    }
  }
  *out = a;
  return true;
}

void destroy(Arena *arena) {
  const Driver &d = driver();
  if (!d.ok || !arena) return;
  if (arena->multicast_va) unmap_range(d, arena->multicast_va, arena->bytes);
  arena->multicast_va = nullptr;
  if (arena->multicast_handle) {
    CUdevice dev = 0;
    if (arena->multicast_bound && d.DeviceGet(&dev, arena->device) == CUDA_SUCCESS)
      d.MulticastUnbind(arena->multicast_handle, dev, 0, static_cast<size_t>(arena->bytes));
    d.MemRelease(arena->multicast_handle);
  }
  arena->multicast_handle = 0;
  arena->multicast_bound = false;
  for (size_t p = 0; p < arena->peer_va.size(); ++p) {
    unmap_range(d, arena->peer_va[p], arena->bytes);
    arena->peer_va[p] = nullptr;
  }
  for (auto &h : arena->handles) {
    if (h) d.MemRelease(h);
    h = 0;
  }
}
}  // namespace cs::communication::vmm
