// SPDX-License-Identifier: Apache-2.0
// In-process communicator group: `size` ranks that live on threads of one process and exchange tensors through
// shared memory. It exists for host-side tests of everything that sits above a collective (buckets, gradient
// sync, sharded training loops, failure handling) without GPUs, sockets or a launcher: a rank can be delayed, or
// never join, and the others get an error after the group's timeout instead of waiting forever.
// The reference has no such backend (its distributed tests need one GPU per rank, test/test_all_reduce.cpp:55-57).
#include <torch/csrc/distributed/c10d/Work.hpp>

#include <chrono>
#include <condition_variable>
#include <mutex>
#include <thread>

#include "cs/communication.h"

namespace cs::communication {
namespace {
struct DoneWork : c10d::Work {
  bool isCompleted() override { return true; }
  bool isSuccess() const override { return true; }
  bool wait(std::chrono::milliseconds) override { return true; }
};

// Rendezvous of the rank threads. Every collective is: publish a pointer to my arguments, meet, read the others'
// inputs into temporaries, meet again, write my outputs. Nobody writes while anybody may still read.
struct ThreadGroup {
  explicit ThreadGroup(int64_t n) : size{n}, slots(static_cast<size_t>(n), nullptr), delay_ms(static_cast<size_t>(n), 0) {}
  const int64_t size;
  std::mutex mutex;
  std::condition_variable cv;
  int64_t waiting{0};
  uint64_t generation{0};
  bool broken{false};
  int64_t timeout_ms{30000};
  int64_t collectives{0};
  std::vector<const void *> slots;
  std::vector<int64_t> delay_ms;  // injected: the rank sleeps this long before it joins a collective

  void meet(int64_t rank, const char *what) {
    std::unique_lock<std::mutex> lock{mutex};
    CS_ASSERT_TRUE(!broken, "thread communicator: the group is broken (an earlier collective timed out); rank ", rank, " in ", what);
    const uint64_t mine = generation;
    if (++waiting == size) {
      waiting = 0;
      ++generation;
      cv.notify_all();
      return;
    }
    const bool met = cv.wait_for(lock, std::chrono::milliseconds(timeout_ms), [&] { return generation != mine || broken; });
    if (met && generation != mine) return;
    const int64_t missing = size - waiting;
    broken = true;
    cv.notify_all();
    fail(__FILE__, __LINE__, str_cat("thread communicator: ", what, " on rank ", rank, " timed out after ", timeout_ms, " ms; ", missing,
                                     " rank(s) did not join"));
  }
  void enter(int64_t rank, const void *mine, const char *what) {
    int64_t delay = 0;
    {
      std::lock_guard<std::mutex> lock{mutex};
      delay = delay_ms[static_cast<size_t>(rank)];
      slots[static_cast<size_t>(rank)] = mine;
      if (rank == 0) ++collectives;
    }
    if (delay > 0) std::this_thread::sleep_for(std::chrono::milliseconds(delay));
    meet(rank, what);
  }
  template <typename T>
  const T &of(int64_t rank) const {
    return *static_cast<const T *>(slots[static_cast<size_t>(rank)]);
  }
};

at::Tensor reduced(const std::vector<at::Tensor> &parts, const c10d::ReduceOp &op, int64_t size) {
  at::Tensor sum = parts[0].clone();
  for (size_t r = 1; r < parts.size(); ++r) sum.add_(parts[r].to(sum.device()));
  if (op == c10d::ReduceOp::AVG) sum.div_(static_cast<double>(size));
  else CS_ASSERT_TRUE(op == c10d::ReduceOp::SUM, "thread communicator: only SUM and AVG are implemented");
  return sum;
}

struct ThreadBackend : c10d::Backend {
  ThreadBackend(std::shared_ptr<ThreadGroup> group, int rank) : c10d::Backend(rank, static_cast<int>(group->size)), group_{std::move(group)} {}
  const std::string getBackendName() const override { return "cs_threads"; }

  c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor> &tensors, const c10d::AllreduceOptions &opts) override {
    group_->enter(rank_, &tensors, "all_reduce");
    std::vector<at::Tensor> results;
    for (size_t i = 0; i < tensors.size(); ++i) {
      std::vector<at::Tensor> parts;
      for (int64_t r = 0; r < size_; ++r) parts.push_back(group_->of<std::vector<at::Tensor>>(r).at(i));
      results.push_back(reduced(parts, opts.reduceOp, size_));
    }
    group_->meet(rank_, "all_reduce");
    for (size_t i = 0; i < tensors.size(); ++i) tensors[i].copy_(results[i]);
    return c10::make_intrusive<DoneWork>();
  }

  c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor> &tensors, const c10d::BroadcastOptions &opts) override {
    group_->enter(rank_, &tensors, "broadcast");
    std::vector<at::Tensor> results;
    for (size_t i = 0; i < tensors.size(); ++i) results.push_back(group_->of<std::vector<at::Tensor>>(opts.rootRank).at(i).clone());
    group_->meet(rank_, "broadcast");
    for (size_t i = 0; i < tensors.size(); ++i) tensors[i].copy_(results[i]);
    return c10::make_intrusive<DoneWork>();
  }

  c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>> &outputs, std::vector<at::Tensor> &inputs,
                                           const c10d::AllgatherOptions &) override {
    group_->enter(rank_, &inputs, "all_gather");
    for (size_t i = 0; i < inputs.size(); ++i)
      for (int64_t r = 0; r < size_; ++r) outputs[i][static_cast<size_t>(r)].copy_(group_->of<std::vector<at::Tensor>>(r).at(i));
    group_->meet(rank_, "all_gather");  // outputs are private to this rank; inputs stay untouched until everyone has read them
    return c10::make_intrusive<DoneWork>();
  }

  c10::intrusive_ptr<c10d::Work> reduce_scatter(std::vector<at::Tensor> &outputs, std::vector<std::vector<at::Tensor>> &inputs,
                                                const c10d::ReduceScatterOptions &opts) override {
    group_->enter(rank_, &inputs, "reduce_scatter");
    std::vector<at::Tensor> results;
    for (size_t i = 0; i < outputs.size(); ++i) {
      std::vector<at::Tensor> parts;
      for (int64_t r = 0; r < size_; ++r) parts.push_back(group_->of<std::vector<std::vector<at::Tensor>>>(r).at(i).at(static_cast<size_t>(rank_)));
      results.push_back(reduced(parts, opts.reduceOp, size_));
    }
    group_->meet(rank_, "reduce_scatter");
    for (size_t i = 0; i < outputs.size(); ++i) outputs[i].copy_(results[i]);
    return c10::make_intrusive<DoneWork>();
  }

  c10::intrusive_ptr<c10d::Work> alltoall(std::vector<at::Tensor> &outputs, std::vector<at::Tensor> &inputs,
                                          const c10d::AllToAllOptions &) override {
    group_->enter(rank_, &inputs, "all_to_all");
    std::vector<at::Tensor> results;
    for (int64_t r = 0; r < size_; ++r) results.push_back(group_->of<std::vector<at::Tensor>>(r).at(static_cast<size_t>(rank_)).clone());
    group_->meet(rank_, "all_to_all");
    for (int64_t r = 0; r < size_; ++r) outputs[static_cast<size_t>(r)].copy_(results[static_cast<size_t>(r)]);
    return c10::make_intrusive<DoneWork>();
  }

  c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions &) override {
    group_->enter(rank_, nullptr, "barrier");
    return c10::make_intrusive<DoneWork>();
  }

  std::shared_ptr<ThreadGroup> group_;
};
}  // namespace

std::vector<Comm> create_thread_comms(int64_t size, int64_t timeout_ms) {
  CS_ASSERT_TRUE(size >= 1, "a communicator group needs at least one rank");
  auto group = std::make_shared<ThreadGroup>(size);
  group->timeout_ms = timeout_ms;
  std::vector<Comm> comms;
  for (int64_t rank = 0; rank < size; ++rank) {
    auto impl = std::make_shared<Comm::Impl>();
    impl->type = kTHREADS;
    impl->rank = rank;
    impl->size = size;
    if (size > 1) impl->backend = c10::make_intrusive<ThreadBackend>(group, static_cast<int>(rank));
    comms.emplace_back(impl);
  }
  return comms;
}

void set_thread_comm_delay(const Comm &comm, int64_t delay_ms) {
  auto *backend = dynamic_cast<ThreadBackend *>(comm.impl()->backend.get());
  CS_ASSERT_TRUE(backend != nullptr, "not a thread communicator");
  std::lock_guard<std::mutex> lock{backend->group_->mutex};
  backend->group_->delay_ms[static_cast<size_t>(comm.impl()->rank)] = delay_ms;
}

int64_t thread_comm_collectives(const Comm &comm) {
  auto *backend = dynamic_cast<ThreadBackend *>(comm.impl()->backend.get());
  CS_ASSERT_TRUE(backend != nullptr, "not a thread communicator");
  std::lock_guard<std::mutex> lock{backend->group_->mutex};
  return backend->group_->collectives;
}
}  // namespace cs::communication
