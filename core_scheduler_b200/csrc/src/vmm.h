// SPDX-License-Identifier: Apache-2.0
// Virtual-memory-management allocation of the symmetric arena, shared between the processes of one
// NVSwitch domain, with an NVLink multicast object bound over the same pages.
//
// What this gives the kernels: besides one mapping per peer (plain loads and stores to one GPU's
// copy) a single "multicast" address range whose loads can be reduced inside the switch
// (multimem.ld_reduce) and whose stores are replicated to every GPU (multimem.st). The reference
// project reaches those switch features only through NCCL (src/communication/all_reduce.cpp:107-113);
// its own peer-to-peer backend is declared and never written (include/communication/communication.h:51).
//
// Handles cross process boundaries as POSIX file descriptors: the exporting rank publishes
// (pid, fd) through the communicator's store and every importer duplicates the descriptor with
// pidfd_getfd(2). No daemon and no socket are involved. Every step reports failure instead of
// throwing, so that the caller can fall back to cudaMalloc + CUDA IPC (no multicast).
#pragma once
#include <cuda.h>

#include <cstdint>
#include <string>
#include <vector>

namespace cs::communication::vmm {
struct Arena {
  std::vector<char *> peer_va;   // peer_va[p]: rank p's allocation mapped here (peer_va[rank] = our own)
  char *multicast_va{nullptr};   // null when the device or the driver has no multicast support
  int64_t bytes{0};              // mapped size (rounded up to the allocation granularity)
  // teardown state
  std::vector<CUmemGenericAllocationHandle> handles;
  CUmemGenericAllocationHandle multicast_handle{0};
  bool multicast_bound{false};
  int device{0};
  int rank{0};
};

// Exchange callbacks, implemented by the caller on top of its key/value store.
struct Exchange {
  // Publishes `value` under `key` / waits for and reads the value another rank published.
  virtual void put(const std::string &key, const std::string &value) = 0;
  virtual std::string get(const std::string &key) = 0;
  // Returns once every rank has called it with the same name.
  virtual void barrier(const std::string &name) = 0;
  virtual ~Exchange() = default;
};

// Collective over `size` ranks. Returns false (with `why` filled in, nothing left allocated) when the
// driver lacks an entry point, a handle cannot be exported or imported, or a mapping fails; in that
// case every rank returns false (failures are agreed on through the exchange before anything is used).
bool create(Arena *out, int rank, int size, int device, int64_t bytes, bool want_multicast, Exchange &exchange, std::string *why);
// Unbinds, unmaps and releases everything `create` set up. Call it on every rank, after the device is idle.
void destroy(Arena *arena);

// Duplicates descriptor `fd` of process `pid` into this process (pidfd_open + pidfd_getfd); -1 on failure.
int duplicate_descriptor(int pid, int fd);
}  // namespace cs::communication::vmm
