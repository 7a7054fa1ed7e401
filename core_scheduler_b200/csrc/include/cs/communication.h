// SPDX-License-Identifier: Apache-2.0
// Communicators and collectives as scheduler tasks on the comm stream.
//
// Capability parity (reference project paths): include/communication/communication.h:25-59,
// src/communication/communication.cpp:33-151 (rendezvous + process-group creation),
// all_reduce.h:23-36 / all_reduce.cpp:43-179 (run_inplace, byte-threshold bucket),
// all_gather.h, reduce_scatter.h, all_to_all.h and their sources.
//
// Differences: ranks rendezvous through the torchrun-style environment (RANK, WORLD_SIZE,
// LOCAL_RANK, MASTER_ADDR, MASTER_PORT) and a TCP store instead of MPI; a communicator can
// also wrap a torch.distributed backend (NCCL on GPUs, Gloo on CPUs); multi-tensor
// all-reduce reduces adjacent arena views as one contiguous range and every tensor of a
// bucket receives the reduced value; kNVP2P is implemented: collectives run as this
// library's own kernels over peer-mapped symmetric memory (see cs/symmetric.h).
#pragma once
#ifdef CS_WITH_MPI
#include <mpi.h>
#endif
#include <functional>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>

#include "cs/core.h"

namespace cs::communication {
enum BackendType { kMPI = 0, kNCCL, kNVP2P, kGLOO, kTHREADS };
enum Operation { kSUM = 0, kAVG };

struct SymmetricContext;  // cs/symmetric.h

struct CS_API Comm {
  struct Impl;
  Comm() = default;
  explicit Comm(std::shared_ptr<Impl> impl) : impl_{std::move(impl)} {}
  [[nodiscard]] int64_t get_rank() const;
  [[nodiscard]] int64_t get_size() const;
  [[nodiscard]] const std::shared_ptr<Impl> &impl() const { return impl_; }
  [[nodiscard]] bool defined() const { return impl_ != nullptr; }

 private:
  std::shared_ptr<Impl> impl_;
};

struct Comm::Impl {
  c10::intrusive_ptr<c10d::Store> store;      // may be null for wrapped backends
  c10::intrusive_ptr<c10d::Backend> backend;  // null for a single-rank communicator
  BackendType type{kNCCL};
  int64_t rank{0};
  int64_t size{1};
  std::shared_ptr<SymmetricContext> symmetric;  // peer-mapped memory (kNVP2P and fused paths)
  // Injected failure for host-side fault tests: the next `fail_after` collectives succeed,
  // the one after raises cs::Error (negative = never).
  int64_t fail_after{-1};
};

struct CS_API Bucket {
  virtual ~Bucket() = default;
  virtual void apply(const Scheduler &scheduler, const Comm &comm) const;
};

#ifdef CS_WITH_MPI
// Communicator over the ranks of an MPI group (the reference's entry point, include/communication/communication.h:55).
// Available when the library is built with -DCS_WITH_MPI against an MPI installation: rank and size come from the
// group, the store address is broadcast from the group's rank 0, and the collectives run on `backend_type`.
CS_API Comm get_comm(MPI_Comm group, BackendType backend_type);
#endif
// World communicator from the launcher environment. With WORLD_SIZE unset or 1 the result is
// a single-rank communicator whose collectives are local no-ops/copies.
CS_API Comm get_comm_world(BackendType backend_type = kNCCL);
// All ranks of this node (identical to the world on a single node).
CS_API Comm get_comm_node(BackendType backend_type = kNCCL);
// Wraps an existing c10d backend (e.g. the one torch.distributed created).
CS_API Comm wrap_backend(c10::intrusive_ptr<c10d::Backend> backend, int64_t rank, int64_t size, BackendType type,
                         c10::intrusive_ptr<c10d::Store> store = {});
// Single-process communicator of size 1.
CS_API Comm get_comm_self();
// In-process group for host-side tests (kTHREADS): `size` communicators, one per rank, to be used from `size`
// threads of this process (each with a scheduler of its own). A collective that not every rank joins within
// `timeout_ms` raises cs::Error on the ranks that did, and the group stays broken afterwards.
CS_API std::vector<Comm> create_thread_comms(int64_t size, int64_t timeout_ms = 30000);
// Fault injection for such a group: this rank sleeps `delay_ms` before it joins each collective.
CS_API void set_thread_comm_delay(const Comm &comm, int64_t delay_ms);
// Collectives the group has started so far.
CS_API int64_t thread_comm_collectives(const Comm &comm);
// Shuts down and forgets the communicators created from the environment (get_comm_world / get_comm_node). Call
// it before main() returns: their NCCL process groups must go while the CUDA driver is still up.
CS_API void finalize();

struct CS_API AllReduce {
  static void run_inplace(const Scheduler &scheduler, const Comm &comm, const std::vector<Tensor> &tensors,
                          Operation operation);
};

struct CS_API AllReduceBucket : Bucket {
  AllReduceBucket(int64_t byteThreshold, Operation operation);
  // Queues a tensor; launches one all-reduce over everything queued once the byte threshold
  // is reached.
  void push_back(const Scheduler &scheduler, const Comm &comm, Tensor tensor) const;
  // Flushes whatever is queued (call once after the last push_back of a step).
  void sync(const Scheduler &scheduler, const Comm &comm) const;
  void apply(const Scheduler &scheduler, const Comm &comm) const override { sync(scheduler, comm); }
  [[nodiscard]] int64_t launches() const;
  // Hook that runs after every flush: it receives the tensors of the bucket that was just reduced and the
  // stream class that orders work after the reduction (the communication stream; a single rank reduces nothing
  // but still hands its buckets over there). An optimizer attached here updates a bucket's parameters while
  // the backward pass of the earlier layers is still running (module::AdamWImpl::step_partial).
  using ReducedCallback = std::function<void(const Scheduler &, const std::vector<Tensor> &, Task::Impl::Priority)>;
  void on_reduced(ReducedCallback callback) const;
  // With `skip` the bucket only groups the tensors and hands them to the hook: for a consumer that reduces the
  // gradients itself (the sharded optimizer's reduce-scatter + AdamW + all-gather kernel).
  void skip_reduction(bool skip) const;

 private:
  struct Impl;
  std::shared_ptr<Impl> impl_;
};

struct CS_API AllGather {
  // recv[i] has one tensor per rank; send[i] is this rank's contribution.
  static void run(const Scheduler &scheduler, const Comm &comm, const std::vector<std::vector<Tensor>> &recv,
                  const std::vector<ReadOnlyTensor> &send);
};

struct CS_API ReduceScatter {
  // send[i] has one tensor per rank; recv[i] receives the reduction of everyone's send[i][rank].
  static void run(const Scheduler &scheduler, const Comm &comm, const std::vector<Tensor> &recv,
                  const std::vector<std::vector<ReadOnlyTensor>> &send, Operation operation);
};

struct CS_API AllToAll {
  // send[j] goes to rank j; recv[j] comes from rank j.
  static void run(const Scheduler &scheduler, const Comm &comm, const std::vector<Tensor> &recv,
                  const std::vector<ReadOnlyTensor> &send);
};

// Host-side liveness: every rank bumps a store counter per step; a rank that stops is
// reported by the others after `timeout_ms` without progress. No GPU involvement.
struct CS_API Heartbeat {
  Heartbeat(const Comm &comm, int64_t timeout_ms);
  void beat(int64_t step) const;
  // Ranks whose last beat is older than the timeout (empty = all alive).
  [[nodiscard]] std::vector<int64_t> stale_ranks() const;

 private:
  Comm comm_;
  int64_t timeout_ms_;
};
}  // namespace cs::communication
