// SPDX-License-Identifier: Apache-2.0
// Communicators and library-backed collectives. See cs/communication.h for the parity map.
#include "cs/communication.h"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime.h>
#include <torch/csrc/distributed/c10d/TCPStore.hpp>
#include <torch/csrc/distributed/c10d/Types.hpp>

#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <map>
#include <mutex>

#include "cs/module.h"
#include "cs/symmetric.h"

namespace cs::communication {
int64_t Comm::get_rank() const { return impl_->rank; }
int64_t Comm::get_size() const { return impl_->size; }

void Bucket::apply(const Scheduler &, const Comm &) const {
  CS_ASSERT_TRUE(false, "Bucket::apply is not implemented by this bucket type");
}

// Defined in comm_nccl.cpp (compiled only when the NCCL process group headers are usable).
c10::intrusive_ptr<c10d::Backend> create_nccl_backend(const c10::intrusive_ptr<c10d::Store> &store, int rank, int size);

namespace {
// The library may finish connecting its transports lazily inside the first collective; running
// one tiny all-reduce followed by a device synchronisation here keeps that set-up out of the
// first training step (where it was observed to let a consumer run ahead of the reduction).
void warm_up(Comm::Impl &impl) {
  if (impl.size <= 1 || !impl.backend || (impl.type != kNCCL && impl.type != kNVP2P)) return;
  at::Tensor probe = at::ones({8}, at::TensorOptions().dtype(at::kFloat).device(at::kCUDA));
  std::vector<at::Tensor> one{probe};
  c10d::AllreduceOptions opts;
  auto work = impl.backend->allreduce(one, opts);
  if (work) work->wait();
  cudaDeviceSynchronize();
}
}  // namespace

namespace {
int64_t env_int(const char *name, int64_t fallback) {
  const char *v = std::getenv(name);
  return v ? std::atoll(v) : fallback;
}

std::mutex g_comm_mutex;
// (backend, scope) -> communicator. Heap-allocated and never destroyed: a ProcessGroupNCCL destructor that runs
// during static destruction finds the CUDA driver already shut down and throws; finalize() releases them earlier.
std::map<std::pair<int, int>, Comm> &g_comms = *new std::map<std::pair<int, int>, Comm>();

Comm create_from_env(BackendType type) {
  auto impl = std::make_shared<Comm::Impl>();
  impl->type = type;
  impl->rank = env_int("RANK", 0);
  impl->size = env_int("WORLD_SIZE", 1);
  if (impl->size <= 1) return Comm{impl};
  CS_ASSERT_TRUE(type == kNCCL || type == kNVP2P,
                 "only NCCL-backed communicators can be created from the environment; wrap a torch.distributed "
                 "backend for Gloo");
  const char *addr = std::getenv("MASTER_ADDR");
  const std::string host = addr ? addr : "127.0.0.1";
  // The launcher's MASTER_PORT may already serve torch.distributed; CS_STORE_PORT overrides.
  const int64_t port = env_int("CS_STORE_PORT", env_int("MASTER_PORT", 29500) + 17);
  c10d::TCPStoreOptions opts;
  opts.port = static_cast<uint16_t>(port);
  opts.isServer = impl->rank == 0;
  opts.numWorkers = impl->size;
  opts.waitWorkers = true;
  impl->store = c10::make_intrusive<c10d::TCPStore>(host, opts);
  impl->backend = create_nccl_backend(impl->store, static_cast<int>(impl->rank), static_cast<int>(impl->size));
  warm_up(*impl);
  return Comm{impl};
}

Comm lookup_or_create(BackendType type, int scope) {
  std::lock_guard<std::mutex> lock{g_comm_mutex};
  auto key = std::make_pair(static_cast<int>(type), scope);
  auto it = g_comms.find(key);
  if (it != g_comms.end()) return it->second;
  CS_ASSERT_TRUE(type != kMPI, "the MPI backend is not available; use kNCCL, kNVP2P or a wrapped Gloo backend");
  Comm comm = create_from_env(type);
  g_comms.emplace(key, comm);
  return comm;
}

c10d::ReduceOp reduce_op(Operation op, bool avg_supported) {
  if (op == kAVG && avg_supported) return c10d::ReduceOp::AVG;
  return c10d::ReduceOp::SUM;
}

bool backend_has_avg(const Comm::Impl &impl) { return impl.type == kNCCL || impl.type == kNVP2P; }

void inject_failure(Comm::Impl &impl, const char *what) {
  if (impl.fail_after < 0) return;
  if (impl.fail_after == 0) {
    impl.fail_after = -1;
    fail(__FILE__, __LINE__, str_cat("injected communication failure in ", what, " on rank ", impl.rank));
  }
  --impl.fail_after;
}

void wait_work(const c10::intrusive_ptr<c10d::Work> &work) {
  // NCCL: orders the current (comm) stream after the collective without blocking the host.
  // Gloo: blocks the host until the data arrived.
  if (work) work->wait();

}

// Groups tensors that live in one storage (views of a flat arena) into as few contiguous ranges
// as possible so that a bucket needs one collective and no staging copies. The tensors are
// sorted by address and their byte intervals are united (an interval that lies inside or
// overlaps a previous one is absorbed, so nothing is ever reduced twice). Two intervals are joined across a gap only when
// the second starts exactly where the first one's slot ends, i.e. at the first interval's end
// rounded up to the arena's slot alignment (module::FlatParameters::alignment elements from the
// start of the storage): such a gap is the first slot's own padding, zeros on every rank, and
// cannot hold another tensor. Any wider gap may hold a gradient that belongs to another bucket,
// so it is never bridged. Non-contiguous tensors are returned as they are.
std::vector<at::Tensor> merge_adjacent(const std::vector<at::Tensor> &tensors) {
  struct Piece {
    const char *lo, *hi;
  };
  std::vector<at::Tensor> out;
  std::vector<bool> used(tensors.size(), false);
  constexpr int64_t slot_elems = module::FlatParameters::alignment;
  // Ranges are emitted in the order in which their arena first appears in the bucket and, inside
  // an arena, by address: both are the same on every rank, so all ranks issue the same sequence
  // of collectives (sorting unrelated allocations by address would not be).
  for (size_t i = 0; i < tensors.size(); ++i) {
    if (used[i]) continue;
    const at::Tensor &first = tensors[i];
    used[i] = true;
    if (!first.is_contiguous() || first.numel() == 0) {
      out.push_back(first);
      continue;
    }
    std::vector<Piece> pieces;
    const char *p0 = static_cast<const char *>(first.data_ptr());
    pieces.push_back({p0, p0 + first.nbytes()});
    for (size_t j = i + 1; j < tensors.size(); ++j) {
      const at::Tensor &t = tensors[j];
      if (used[j] || !t.is_contiguous() || t.numel() == 0 || t.scalar_type() != first.scalar_type() ||
          !t.storage().is_alias_of(first.storage()))
        continue;
      used[j] = true;
      const char *p = static_cast<const char *>(t.data_ptr());
      pieces.push_back({p, p + t.nbytes()});
    }
    std::sort(pieces.begin(), pieces.end(), [](const Piece &a, const Piece &b) { return a.lo < b.lo; });
    const int64_t elem = static_cast<int64_t>(first.element_size());
    const char *storage_base = static_cast<const char *>(first.storage().data());
    size_t k = 0;
    while (k < pieces.size()) {
      const char *lo = pieces[k].lo, *hi = pieces[k].hi;
      size_t j = k + 1;
      while (j < pieces.size()) {
        const int64_t slot_bytes = slot_elems * elem;
        const char *slot_end = storage_base + ((hi - storage_base) + slot_bytes - 1) / slot_bytes * slot_bytes;
        if (pieces[j].lo > hi && pieces[j].lo != slot_end) break;
        if (pieces[j].hi > hi) hi = pieces[j].hi;
        ++j;
      }
      out.push_back(at::as_strided(first, {(hi - lo) / elem}, {1}, (lo - storage_base) / elem));
      k = j;
    }
  }
  return out;
}
}  // namespace

#ifdef CS_WITH_MPI
Comm get_comm(MPI_Comm group, BackendType backend_type) {
  CS_ASSERT_TRUE(backend_type == kNCCL || backend_type == kNVP2P, "collectives over an MPI group run on kNCCL or kNVP2P");
  int rank = 0, size = 1;
  CS_CHECK_MPI(MPI_Comm_rank(group, &rank));
  CS_CHECK_MPI(MPI_Comm_size(group, &size));
  auto impl = std::make_shared<Comm::Impl>();
  impl->type = backend_type;
  impl->rank = rank;
  impl->size = size;
  if (size <= 1) return Comm{impl};
  // rank 0 of the group opens the store on a port of its own and tells the others where it is
  char host[256] = "127.0.0.1";
  int port = 0;
  if (rank == 0) {
    if (const char *addr = std::getenv("MASTER_ADDR")) std::snprintf(host, sizeof(host), "%s", addr);
    port = static_cast<int>(env_int("CS_STORE_PORT", 29517));
  }
  CS_CHECK_MPI(MPI_Bcast(host, sizeof(host), MPI_CHAR, 0, group));
  CS_CHECK_MPI(MPI_Bcast(&port, sizeof(port), MPI_CHAR, 0, group));
  c10d::TCPStoreOptions opts;
  opts.port = static_cast<uint16_t>(port);
  opts.isServer = rank == 0;
  opts.numWorkers = size;
  opts.waitWorkers = true;
  impl->store = c10::make_intrusive<c10d::TCPStore>(std::string(host), opts);
  impl->backend = create_nccl_backend(impl->store, rank, size);
  warm_up(*impl);
  return Comm{impl};
}
#endif

Comm get_comm_world(BackendType backend_type) { return lookup_or_create(backend_type, 0); }
Comm get_comm_node(BackendType backend_type) { return lookup_or_create(backend_type, 1); }
Comm get_comm_self() {
  auto impl = std::make_shared<Comm::Impl>();
  return Comm{impl};
}
Comm wrap_backend(c10::intrusive_ptr<c10d::Backend> backend, int64_t rank, int64_t size, BackendType type,
                  c10::intrusive_ptr<c10d::Store> store) {
  auto impl = std::make_shared<Comm::Impl>();
  impl->backend = std::move(backend);
  impl->store = std::move(store);
  impl->rank = rank;
  impl->size = size;
  impl->type = type;
  warm_up(*impl);
  return Comm{impl};
}

// ------------------------------------------------------------------------- all-reduce ----
void AllReduce::run_inplace(const Scheduler &scheduler, const Comm &comm, const std::vector<Tensor> &tensors,
                            Operation operation) {
  if (tensors.empty()) return;
  std::vector<ReadOnlyTensor> ins(tensors.begin(), tensors.end());
  submit(scheduler, "cs::communication::AllReduce::run_inplace", Task::Impl::kComm, Task::Impl::kNccl, tensors, ins,
         [tensors, comm, operation](const FnTask &task) {
           auto &impl = *comm.impl();
           inject_failure(impl, "all_reduce");
           std::vector<at::Tensor> raw;
           for (auto &t : tensors) {
             CS_ASSERT_TRUE(t.impl()->tensor.defined(), "all-reduce of an undefined tensor");
             raw.push_back(t.impl()->tensor);
           }
           if (impl.size <= 1 || !impl.backend) return;
           std::vector<at::Tensor> ranges = merge_adjacent(raw);
           if (impl.type == kNVP2P && impl.symmetric && symmetric_all_reduce(*impl.symmetric, ranges, operation)) return;
           const bool avg = backend_has_avg(impl);
           c10d::AllreduceOptions opts;
           opts.reduceOp = reduce_op(operation, avg);
           opts.asyncOp = false;  // run on the current (comm) stream, not on a stream of the library
           for (auto &r : ranges) {
             at::Tensor buf = r.is_contiguous() ? r : r.contiguous();
             std::vector<at::Tensor> one{buf};
             wait_work(impl.backend->allreduce(one, opts));
             if (operation == kAVG && !avg) buf.div_(static_cast<double>(impl.size));
             if (!buf.is_alias_of(r)) {
               r.copy_(buf);
               task.intermediate().push_back(buf);
             }
           }
         });
}

struct AllReduceBucket::Impl {
  int64_t threshold;
  Operation op;
  std::vector<Tensor> pending;
  int64_t pending_bytes{0};
  int64_t launches{0};
  ReducedCallback callback{};
  bool skip_reduction{false};
};

AllReduceBucket::AllReduceBucket(int64_t byteThreshold, Operation operation)
    : impl_{std::make_shared<Impl>(Impl{byteThreshold, operation, {}, 0, 0, {}, false})} {}

void AllReduceBucket::skip_reduction(bool skip) const { impl_->skip_reduction = skip; }

void AllReduceBucket::on_reduced(ReducedCallback callback) const { impl_->callback = std::move(callback); }

int64_t AllReduceBucket::launches() const { return impl_->launches; }

void AllReduceBucket::push_back(const Scheduler &scheduler, const Comm &comm, Tensor tensor) const {
  CS_ASSERT_TRUE(tensor.defined(), "only materialised tensors can be queued for all-reduce");
  impl_->pending_bytes += static_cast<int64_t>(tensor.impl()->tensor.nbytes());
  impl_->pending.push_back(std::move(tensor));
  if (impl_->pending_bytes >= impl_->threshold) sync(scheduler, comm);
}

void AllReduceBucket::sync(const Scheduler &scheduler, const Comm &comm) const {
  if (impl_->pending.empty()) return;
  const bool alone = comm.get_size() <= 1 || impl_->skip_reduction;
  if (!alone) AllReduce::run_inplace(scheduler, comm, impl_->pending, impl_->op);
  ++impl_->launches;
  // The communication stream has the highest priority and the longest re-join gap, so work hooked in here runs
  // beside the backward pass instead of holding up the weight-gradient GEMMs of the assist stream.
  if (impl_->callback) impl_->callback(scheduler, impl_->pending, Task::Impl::kComm);
  impl_->pending.clear();
  impl_->pending_bytes = 0;
}

// ------------------------------------------------------------------------- all-gather ----
void AllGather::run(const Scheduler &scheduler, const Comm &comm, const std::vector<std::vector<Tensor>> &recv,
                    const std::vector<ReadOnlyTensor> &send) {
  CS_ASSERT_TRUE(recv.size() == send.size(), "all-gather needs one receive list per send tensor");
  std::vector<Tensor> outs;
  for (auto &list : recv) outs.insert(outs.end(), list.begin(), list.end());
  submit(scheduler, "cs::communication::AllGather::run", Task::Impl::kComm, Task::Impl::kNccl, outs, send,
         [recv, send, comm](const FnTask &) {
           auto &impl = *comm.impl();
           inject_failure(impl, "all_gather");
           std::vector<std::vector<at::Tensor>> r;
           std::vector<at::Tensor> s;
           for (size_t i = 0; i < send.size(); ++i) {
             CS_ASSERT_TRUE(static_cast<int64_t>(recv[i].size()) == impl.size, "receive list must have one tensor per rank");
             s.push_back(send[i].impl()->tensor);
             r.emplace_back();
             for (auto &t : recv[i]) r.back().push_back(t.impl()->tensor);
           }
           if (impl.size <= 1 || !impl.backend) {
             for (size_t i = 0; i < s.size(); ++i) r[i][0].copy_(s[i]);
             return;
           }
           if (impl.type == kNVP2P && impl.symmetric && symmetric_all_gather(*impl.symmetric, r, s)) return;
           c10d::AllgatherOptions ag_opts;
           ag_opts.asyncOp = false;
           wait_work(impl.backend->allgather(r, s, ag_opts));
         });
}

// --------------------------------------------------------------------- reduce-scatter ----
void ReduceScatter::run(const Scheduler &scheduler, const Comm &comm, const std::vector<Tensor> &recv,
                        const std::vector<std::vector<ReadOnlyTensor>> &send, Operation operation) {
  CS_ASSERT_TRUE(recv.size() == send.size(), "reduce-scatter needs one send list per receive tensor");
  std::vector<ReadOnlyTensor> ins;
  for (auto &list : send) ins.insert(ins.end(), list.begin(), list.end());
  submit(scheduler, "cs::communication::ReduceScatter::run", Task::Impl::kComm, Task::Impl::kNccl, recv, ins,
         [recv, send, comm, operation](const FnTask &) {
           auto &impl = *comm.impl();
           inject_failure(impl, "reduce_scatter");
           std::vector<at::Tensor> r;
           std::vector<std::vector<at::Tensor>> s;
           for (size_t i = 0; i < recv.size(); ++i) {
             CS_ASSERT_TRUE(static_cast<int64_t>(send[i].size()) == impl.size, "send list must have one tensor per rank");
             r.push_back(recv[i].impl()->tensor);
             s.emplace_back();
             for (auto &t : send[i]) s.back().push_back(t.impl()->tensor);
           }
           if (impl.size <= 1 || !impl.backend) {
             for (size_t i = 0; i < r.size(); ++i) r[i].copy_(s[i][0]);
             return;
           }
           if (impl.type == kNVP2P && impl.symmetric && symmetric_reduce_scatter(*impl.symmetric, r, s, operation)) return;
           if (impl.type == kGLOO) {
             // Gloo has no reduce-scatter: all-reduce each rank's slot and keep our own.
             c10d::AllreduceOptions opts;
             for (size_t i = 0; i < r.size(); ++i) {
               for (int64_t peer = 0; peer < impl.size; ++peer) {
                 std::vector<at::Tensor> one{s[i][peer].clone()};
                 wait_work(impl.backend->allreduce(one, opts));
                 if (peer == impl.rank) {
                   r[i].copy_(one[0]);
                   if (operation == kAVG) r[i].div_(static_cast<double>(impl.size));
                 }
               }
             }
             return;
           }
           c10d::ReduceScatterOptions opts;
           opts.reduceOp = reduce_op(operation, true);
           opts.asyncOp = false;
           wait_work(impl.backend->reduce_scatter(r, s, opts));
         });
}

// ------------------------------------------------------------------------- all-to-all ----
void AllToAll::run(const Scheduler &scheduler, const Comm &comm, const std::vector<Tensor> &recv,
                   const std::vector<ReadOnlyTensor> &send) {
  submit(scheduler, "cs::communication::AllToAll::run", Task::Impl::kComm, Task::Impl::kNccl, recv, send,
         [recv, send, comm](const FnTask &) {
           auto &impl = *comm.impl();
           inject_failure(impl, "all_to_all");
           CS_ASSERT_TRUE(static_cast<int64_t>(recv.size()) == impl.size && static_cast<int64_t>(send.size()) == impl.size,
                          "all-to-all needs one send and one receive tensor per rank");
           std::vector<at::Tensor> r, s;
           for (auto &t : recv) r.push_back(t.impl()->tensor);
           for (auto &t : send) s.push_back(t.impl()->tensor);
           if (impl.size <= 1 || !impl.backend) {
             r[0].copy_(s[0]);
             return;
           }
           if (impl.type == kNVP2P && impl.symmetric && symmetric_all_to_all(*impl.symmetric, r, s)) return;
           if (impl.type == kGLOO) {
             // Gloo's list form is missing on some builds: gather everything and pick our column.
             for (int64_t src = 0; src < impl.size; ++src) {
               for (int64_t dst = 0; dst < impl.size; ++dst) {
                 at::Tensor buf = src == impl.rank ? s[dst].clone() : at::empty_like(r[src]);
                 c10d::BroadcastOptions b;
                 b.rootRank = src;
                 std::vector<at::Tensor> one{buf};
                 wait_work(impl.backend->broadcast(one, b));
                 if (dst == impl.rank) r[src].copy_(buf);
               }
             }
             return;
           }
           c10d::AllToAllOptions a2a_opts;
           a2a_opts.asyncOp = false;
           wait_work(impl.backend->alltoall(r, s, a2a_opts));
         });
}

void finalize() {
  std::lock_guard<std::mutex> lock{g_comm_mutex};
  for (auto &kv : g_comms) {
    auto &impl = *kv.second.impl();
    impl.symmetric.reset();
    if (impl.backend) {
      try {
        impl.backend->shutdown();
      } catch (...) {  // a peer may already be gone; nothing left to do
      }
    }
  }
  g_comms.clear();
}

// -------------------------------------------------------------------------- heartbeat ----
namespace {
int64_t now_ms() {
  return std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
std::string beat_key(int64_t rank) { return str_cat("cs/heartbeat/", rank); }
}  // namespace

Heartbeat::Heartbeat(const Comm &comm, int64_t timeout_ms) : comm_{comm}, timeout_ms_{timeout_ms} {}

void Heartbeat::beat(int64_t step) const {
  auto &impl = *comm_.impl();
  if (!impl.store) return;
  const std::string value = str_cat(step, ":", now_ms());
  impl.store->set(beat_key(impl.rank), std::vector<uint8_t>(value.begin(), value.end()));
}

std::vector<int64_t> Heartbeat::stale_ranks() const {
  std::vector<int64_t> stale;
  auto &impl = *comm_.impl();
  if (!impl.store) return stale;
  const int64_t now = now_ms();
  for (int64_t r = 0; r < impl.size; ++r) {
    if (r == impl.rank) continue;
    if (!impl.store->check({beat_key(r)})) {
      stale.push_back(r);
      continue;
    }
    auto raw = impl.store->get(beat_key(r));
    const std::string value(raw.begin(), raw.end());
    const auto colon = value.find(':');
    const int64_t stamp = colon == std::string::npos ? 0 : std::atoll(value.c_str() + colon + 1);
    if (now - stamp > timeout_ms_) stale.push_back(r);
  }
  return stale;
}
}  // namespace cs::communication
