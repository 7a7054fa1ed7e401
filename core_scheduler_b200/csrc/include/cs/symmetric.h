// SPDX-License-Identifier: Apache-2.0
// Peer-mapped ("symmetric") device memory for the ranks of one NVSwitch domain, a caching
// sub-allocator on top of it, and the collectives / fused paths that run as this library's
// own kernels over peer pointers.
//
// The reference declares an NVLink peer-to-peer backend (BackendType::kNVP2P,
// include/communication/communication.h:51 of the reference project) without implementing it;
// this is that backend. Every rank creates one arena with the driver's virtual-memory API
// (cuMemCreate), shares it with the other processes as a file descriptor through the
// communicator's store and maps every peer's arena, so a kernel on rank r can load/store rank
// p's buffer at the same offset. On NVSwitch systems an NVLink multicast object is bound over the
// same pages: `multicast_base + offset` addresses every rank's copy at once, which lets kernels
// reduce inside the switch (multimem.ld_reduce) and broadcast with one store (multimem.st).
// When the virtual-memory path is unavailable (or CS_SYMMETRIC_IPC=1 asks for it) the arena is a
// cudaMalloc block shared through CUDA IPC, without multicast. NCCL_NVLS_ENABLE=0 also switches
// the multicast object off (multi-rank tests in which a rank may leave early run that way).
// Waits on peer flags are bounded: a kernel that gives up records a status word that the host
// turns into cs::Error.
#pragma once
#include "cs/communication.h"

namespace cs::communication {
struct SymmetricBlock {
  int64_t offset{0};  // bytes from the arena base, identical on every rank
  int64_t bytes{0};
};

struct CS_API SymmetricContext {
  int rank{0};
  int size{1};
  int device{0};
  int64_t arena_bytes{0};
  std::vector<char *> bases;       // bases[p]: rank p's arena as mapped into this process
  std::vector<uint32_t *> flags;   // flags[p]: rank p's signal pad (kFlagWords words)
  char *multicast_base{nullptr};   // the arena of every rank at once (NVLink multicast mapping); null = none
  bool virtual_memory{false};      // arena created with cuMemCreate (else cudaMalloc + CUDA IPC)
  void *status{nullptr};           // kernels::DeviceStatus in device memory
  uint32_t epoch{0};               // monotonically increasing generation of the stand-alone barrier
  // Per-channel state of the barriers that the collective kernels carry inside them: launches so far and
  // blocks launched so far (kernels/collectives.h describes the channels).
  uint32_t channel_epoch[16] = {};
  uint32_t channel_blocks[16] = {};
  static constexpr int kFlagWords = 4096;

  // Caching sub-allocator. Blocks are handed out in the same order on every rank, so equal
  // call sequences yield equal offsets (the symmetric-address property kernels rely on).
  SymmetricBlock allocate(int64_t bytes);
  void release(const SymmetricBlock &block);
  [[nodiscard]] int64_t bytes_in_use() const { return in_use_; }
  [[nodiscard]] int64_t cached_blocks() const { return static_cast<int64_t>(free_.size()); }
  // A tensor view over a block of this rank's arena (storage is not owned by the tensor).
  [[nodiscard]] at::Tensor tensor(const SymmetricBlock &block, at::IntArrayRef sizes, at::ScalarType dtype) const;
  // True when [ptr, ptr+bytes) lies inside this rank's arena; *offset receives the position.
  bool locate(const void *ptr, int64_t bytes, int64_t *offset) const;
  // Device-side barrier of all ranks on the current stream (bounded wait).
  void barrier();
  // Loopback emulation only (see create_loopback_contexts): marks every peer flag of this rank's pad as set.
  void prime_loopback();
  // Reusable staging block of at least `bytes` (same offset on every rank when every rank asks
  // for the same sizes in the same order).
  SymmetricBlock staging(int64_t bytes);
  ~SymmetricContext();

 private:
  friend std::shared_ptr<SymmetricContext> create_symmetric_context(const Comm &, int64_t);
  int64_t bump_{0};
  int64_t in_use_{0};
  std::vector<SymmetricBlock> free_;
  SymmetricBlock staging_{};
  bool owns_{false};
  std::vector<void *> opened_;  // IPC mappings to close
  std::shared_ptr<void> vmm_;   // virtual-memory arena state (vmm::Arena), released with the context
  std::shared_ptr<void> loopback_;  // shared owner of the emulated ranks' arenas and pads
  friend std::vector<std::shared_ptr<SymmetricContext>> create_loopback_contexts(int, int64_t);
};

// Collective: every rank of `comm` must call it with the same size. Attaches the context to
// the communicator (comm.impl()->symmetric).
CS_API std::shared_ptr<SymmetricContext> create_symmetric_context(const Comm &comm, int64_t arena_bytes);

// Single-GPU emulation of `ranks` ranks for kernel tests and profiling: one context per emulated rank, all in this
// process and on the current device, over arenas and signal pads that are plain device allocations ("every peer's
// memory" is local memory, so there is no multicast mapping). Only one emulated rank's kernel runs at a time, so the
// peers' flags cannot arrive; prime_loopback() therefore marks every flag a kernel of this context may wait for as
// already set. Call it before each launch, then run the same collective for rank 0, 1, ... in turn: after the last
// one the arenas hold what a real run would have produced.
CS_API std::vector<std::shared_ptr<SymmetricContext>> create_loopback_contexts(int ranks, int64_t arena_bytes);

// The collectives below run on the current stream; they return false when the tensors are
// not eligible (the caller then uses the library path).
// `ranges` are contiguous 1-D views (adjacent arena slots already merged by the caller).
CS_API bool symmetric_all_reduce(SymmetricContext &ctx, const std::vector<at::Tensor> &ranges, Operation op);
CS_API bool symmetric_all_gather(SymmetricContext &ctx, const std::vector<std::vector<at::Tensor>> &recv,
                                 const std::vector<at::Tensor> &send);
CS_API bool symmetric_reduce_scatter(SymmetricContext &ctx, const std::vector<at::Tensor> &recv,
                                     const std::vector<std::vector<at::Tensor>> &send, Operation op);
CS_API bool symmetric_all_to_all(SymmetricContext &ctx, const std::vector<at::Tensor> &recv,
                                 const std::vector<at::Tensor> &send);
// Reads (and clears) the device status word; raises cs::Error when a kernel reported a
// timed-out wait.
CS_API void check_device_status(SymmetricContext &ctx, const char *where);
}  // namespace cs::communication
