// SPDX-License-Identifier: Apache-2.0
// Runtime core: logger, pooled events, tensor handles, tasks, the three-stream scheduler,
// autocast guard and the blocking to_torch bridge. See cs/core.h for the parity map.
#include "cs/core.h"

#include <ATen/CPUGeneratorImpl.h>
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAGeneratorImpl.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>
#include <unistd.h>

#include <cstdlib>
#include <cstring>
#include <deque>
#include <iostream>
#include <mutex>

namespace cs {
// ---------------------------------------------------------------------------- logging ----
namespace {
LogLevel level_from_env() {
  const char *e = std::getenv("CS_LOG_LEVEL");
  if (!e) return LogLevel::kInfo;
  static const char *names[] = {"trace", "debug", "info", "warn", "error", "critical", "off"};
  for (int i = 0; i < 7; ++i)
    if (strcasecmp(e, names[i]) == 0) return static_cast<LogLevel>(i);
  return LogLevel::kInfo;
}
}  // namespace

void Logger::log(LogLevel level, const std::string &msg) {
  static const char *tags[] = {"trace", "debug", "info", "warning", "error", "critical", "off"};
  static const char *colours[] = {"\033[37m", "\033[36m", "\033[32m", "\033[33m", "\033[31m", "\033[1;41m", ""};
  static const bool tty = isatty(fileno(stdout));
  static std::mutex mu;
  std::lock_guard<std::mutex> lock{mu};
  const int l = static_cast<int>(level);
  if (tty)
    std::cout << "[CS] [" << colours[l] << tags[l] << "\033[0m] " << msg << std::endl;
  else
    std::cout << "[CS] [" << tags[l] << "] " << msg << std::endl;
}

Logger &logger() {
  static Logger instance = [] {
    Logger l;
    l.set_level(level_from_env());
    return l;
  }();
  return instance;
}

void fail(const char *file, int line, const std::string &what) {
  std::string msg = str_cat(file, ":", line, " ", what);
  const char *abort_env = std::getenv("CS_ABORT_ON_ERROR");
  if (abort_env && abort_env[0] == '1') {
    logger().critical(msg);
    std::abort();
  }
  throw Error(msg);
}

std::string cuda_error_string(int code) {
  return str_cat(cudaGetErrorName(static_cast<cudaError_t>(code)), " (", code, "): ",
                 cudaGetErrorString(static_cast<cudaError_t>(code)));
}

NvtxRange::NvtxRange(const char *name) { nvtxRangePushA(name); }
NvtxRange::~NvtxRange() { nvtxRangePop(); }

void manual_seed(int64_t seed) {
  at::manual_seed(seed);  // CPU + all CUDA default generators
  if (at::hasCUDA() && at::cuda::is_available()) {
    const int n = at::cuda::getNumGPUs();
    for (int i = 0; i < n; ++i) {
      auto gen = at::cuda::detail::getDefaultCUDAGenerator(i);
      std::lock_guard<std::mutex> lock(gen.mutex());
      gen.set_current_seed(static_cast<uint64_t>(seed));
      gen.set_offset(0);
    }
  }
}

// ----------------------------------------------------------------------------- events ----
namespace {
// What stream context the calling thread is in. Set by the scheduler around task bodies.
struct ExecContext {
  bool cuda{false};
  int device{-1};
};
thread_local ExecContext tls_exec{};

bool cuda_usable() {
  static const bool ok = at::hasCUDA() && at::cuda::is_available();
  return ok;
}

struct EventPool {
  std::mutex mu;
  std::vector<std::vector<cudaEvent_t>> free_list;  // per device
  std::atomic<int64_t> parked{0};
  cudaEvent_t acquire(int device) {
    {
      std::lock_guard<std::mutex> lock{mu};
      if (static_cast<int>(free_list.size()) > device && !free_list[device].empty()) {
        cudaEvent_t e = free_list[device].back();
        free_list[device].pop_back();
        parked.fetch_sub(1, std::memory_order_relaxed);
        return e;
      }
    }
    c10::cuda::CUDAGuard guard{static_cast<c10::DeviceIndex>(device)};
    cudaEvent_t e = nullptr;
    CS_CHECK_CUDART(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    return e;
  }
  void release(int device, cudaEvent_t e) {
    std::lock_guard<std::mutex> lock{mu};
    if (static_cast<int>(free_list.size()) <= device) free_list.resize(device + 1);
    free_list[device].push_back(e);
    parked.fetch_add(1, std::memory_order_relaxed);
  }
};
EventPool &event_pool() {
  static auto *pool = new EventPool;  // leaked on purpose: events may die after static teardown
  return *pool;
}
}  // namespace

struct Event::Impl {
  cudaEvent_t ev{nullptr};
  int device{-1};
  bool recorded{false};
  ~Impl() {
    if (ev) event_pool().release(device, ev);
  }
};

Event::Event() : impl_{std::make_shared<Impl>()} {}
Event::Event(std::shared_ptr<Impl> impl) : impl_{std::move(impl)} {}
int64_t Event::pooled() { return event_pool().parked.load(); }

void Event::record() const {
  impl_->recorded = true;
  bool use_cuda = tls_exec.cuda;
  int device = tls_exec.device;
  if (!use_cuda && tls_exec.device < 0 && cuda_usable()) {  // outside any scheduler: follow the current device
    use_cuda = true;
    device = c10::cuda::current_device();
  }
  if (!use_cuda) return;
  if (!impl_->ev || impl_->device != device) {
    if (impl_->ev) event_pool().release(impl_->device, impl_->ev);
    impl_->ev = event_pool().acquire(device);
    impl_->device = device;
  }
  CS_CHECK_CUDART(cudaEventRecord(impl_->ev, c10::cuda::getCurrentCUDAStream(static_cast<c10::DeviceIndex>(device)).stream()));
}

void Event::block() const {
  if (!impl_->ev) return;
  int device = tls_exec.cuda ? tls_exec.device : static_cast<int>(c10::cuda::current_device());
  CS_CHECK_CUDART(cudaStreamWaitEvent(c10::cuda::getCurrentCUDAStream(static_cast<c10::DeviceIndex>(device)).stream(), impl_->ev, 0));
}

bool Event::query() const {
  if (!impl_->ev) return true;
  const cudaError_t code = cudaEventQuery(impl_->ev);
  if (code == cudaSuccess) return true;
  if (code == cudaErrorNotReady) {
    (void)cudaGetLastError();
    return false;
  }
  CS_CHECK_CUDART(code);
  return false;
}

void Event::synchronize() const {
  if (!impl_->ev) return;
  CS_CHECK_CUDART(cudaEventSynchronize(impl_->ev));
}

// ---------------------------------------------------------------------------- tensors ----
ReadOnlyTensor::ReadOnlyTensor() : impl_{std::make_shared<Impl>()} {}
TensorOptions ReadOnlyTensor::options() const { return impl_->tensor.options(); }
IntArrayRef ReadOnlyTensor::sizes() const { return impl_->tensor.sizes(); }
int64_t ReadOnlyTensor::size(int64_t dim) const { return impl_->tensor.size(dim); }
int64_t ReadOnlyTensor::numel() const { return impl_->tensor.numel(); }
bool ReadOnlyTensor::defined() const { return impl_ && impl_->tensor.defined(); }
void ReadOnlyTensor::wait() const { impl_->event.synchronize(); }
void ReadOnlyTensor::reset() { impl_ = std::make_shared<Impl>(); }

Tensor Tensor::wrap(at::Tensor t) {
  Tensor out;
  out.impl()->tensor = std::move(t);
  const at::Tensor &held = out.impl()->tensor;
  if (held.defined() && held.is_cuda() && cuda_usable()) {
    // The tensor may still be being produced by work queued on the caller's current stream (for
    // example a copy launched by PyTorch on its default stream). The scheduler's streams do not
    // synchronise with that stream implicitly, so remember its state: the tag below matches no
    // scheduler stream, which makes the first consumer on any of them wait for this event.
    c10::cuda::CUDAGuard guard{held.device()};
    out.impl()->event.record();
    out.impl()->stream_class = StreamClass::kNumStreamClass;
    out.impl()->external = true;
  }
  return out;
}

std::ostream &print(std::ostream &os, const ReadOnlyTensor &t, int64_t linesize) {
  t.wait();
  if (t.impl()->tensor.defined() && t.impl()->tensor.is_cuda()) {
    c10::cuda::CUDAGuard guard{t.impl()->tensor.device()};
    CS_CHECK_CUDART(cudaDeviceSynchronize());
  }
  return at::print(os, t.impl()->tensor, linesize);
}
std::ostream &operator<<(std::ostream &os, const ReadOnlyTensor &t) { return print(os, t, 80); }

void Task::operator()() const { (*impl_)(); }

// -------------------------------------------------------------------------- scheduler ----
int64_t Scheduler::get_device_rank() const { return impl_->device_rank(); }
at::Device Scheduler::device() const { return impl_->device(); }

void Scheduler::Impl::submit(Task &&task) {
  CS_ASSERT_TRUE(false, "task `", task.impl()->name(), "` was submitted to a scheduler that cannot run it");
}

void submit(const Scheduler &scheduler, const char *name, Task::Impl::Priority priority, Task::Impl::Type type,
            std::vector<Tensor> output, std::vector<ReadOnlyTensor> input, FnTask::Body body) {
  scheduler.impl()->submit(
      Task{std::make_shared<FnTask>(name, std::move(output), std::move(input), priority, type, std::move(body))});
}

namespace {
[[noreturn]] void rethrow_with_task(const Task &task, const std::exception &e) {
  fail(__FILE__, __LINE__, str_cat("task `", task.impl()->name(), "` failed: ", e.what()));
}

// Inline execution for CPU tensors. Keeps the bookkeeping (stream class tags, counters) so
// scheduling logic can be tested without a GPU.
struct CpuImpl final : Scheduler::Impl {
  explicit CpuImpl(int64_t rank) : Impl{rank, at::Device{at::kCPU}} {}
  void submit(Task &&task) override {
    const auto &t = *task.impl();
    if (t.type() == Task::Impl::kConfig) {
      ++submitted[3];
      task();
      return;
    }
    ++submitted[t.priority()];
    CS_NVTX_RANGE_FN(t.name());
    try {
      task();
    } catch (const Error &) {
      throw;
    } catch (const std::exception &e) {
      rethrow_with_task(task, e);
    }
    for (auto &o : t.output()) o.impl()->stream_class = static_cast<StreamClass>(t.priority());
  }
};

struct SideEntry {
  int count;
  Event event;
  std::vector<at::Tensor> keep_alive;
};

struct TimedTask {
  std::string name;
  int stream_class;
  cudaEvent_t start, stop;
};

struct CudaImpl final : Scheduler::Impl {
  CudaImpl(int64_t rank, int assist_gap, int comm_gap)
      : Impl{rank, at::Device{at::kCUDA, static_cast<c10::DeviceIndex>(rank)}}, gaps_{0, assist_gap, comm_gap} {
    const auto dev = static_cast<c10::DeviceIndex>(rank);
    CS_ASSERT_TRUE(rank >= 0 && rank < at::cuda::getNumGPUs(), "local rank ", rank, " has no GPU");
    // Lower number = higher priority. The comm stream goes first so that fused
    // compute+collective kernels that only need a few SMs are scheduled promptly.
    streams_.push_back(c10::cuda::getStreamFromPool(0, dev));
    streams_.push_back(c10::cuda::getStreamFromPool(-1, dev));
    streams_.push_back(c10::cuda::getStreamFromPool(-2, dev));
    const char *p = std::getenv("CS_PROFILE");
    profiling_ = p && p[0] == '1';
    // Experiment switch: run assist-class tasks on the main stream (no compute/compute overlap).
    const char *a = std::getenv("CS_ASSIST_ON_MAIN");
    if (a && a[0] == '1') streams_[Task::Impl::kAssist] = streams_[Task::Impl::kMain];
  }

  ~CudaImpl() override {
    for (auto &t : timed_) {
      cudaEventDestroy(t.start);
      cudaEventDestroy(t.stop);
    }
  }

  [[nodiscard]] void *raw_stream(StreamClass c) const override { return streams_[static_cast<int>(c)].stream(); }
  void set_profiling(bool on) override { profiling_ = on; }

  void synchronize() override {
    c10::cuda::CUDAGuard guard{device_};
    for (auto &s : streams_) CS_CHECK_CUDART(cudaStreamSynchronize(s.stream()));
    for (auto &q : queues_) q.clear();
  }

  std::vector<TaskTiming> drain_timings() override {
    synchronize();
    std::vector<TaskTiming> out;
    out.reserve(timed_.size());
    for (auto &t : timed_) {
      float ms = 0.f;
      CS_CHECK_CUDART(cudaEventElapsedTime(&ms, t.start, t.stop));
      float since_first = 0.f;
      if (&t != &timed_.front()) (void)cudaEventElapsedTime(&since_first, timed_.front().start, t.start);
      out.push_back({t.name, t.stream_class, static_cast<double>(ms), static_cast<double>(since_first)});
    }
    for (auto &t : timed_) {  // only now: the first start event anchors every offset above
      cudaEventDestroy(t.start);
      cudaEventDestroy(t.stop);
    }
    timed_.clear();
    return out;
  }

  // The main stream re-joins every side task that has been passed by `gap` main tasks.
  void age(std::deque<SideEntry> &queue) {
    for (auto &e : queue) --e.count;
    while (!queue.empty() && queue.front().count <= 0) {
      queue.front().event.block();
      queue.pop_front();
    }
  }

  void run(const Task &task, Task::Impl::Priority tag) {
    const auto &t = *task.impl();
    const auto cls = static_cast<StreamClass>(tag);
    auto adopt = [&](ReadOnlyTensor::Impl &ti) {  // see Tensor::Impl::external
      const auto bit = static_cast<uint8_t>(1u << tag);
      if (!ti.external || (ti.external_streams & bit) || !ti.tensor.defined() || !ti.tensor.is_cuda()) return;
      ti.external_streams |= bit;
      if (ti.tensor.has_storage()) c10::cuda::CUDACachingAllocator::recordStream(ti.tensor.storage().data_ptr(), streams_[tag]);
    };
    for (auto &in : t.input()) {  // read-after-write across streams
      auto &ti = *in.impl();
      adopt(ti);
      if (ti.stream_class != cls && !ti.event.query()) ti.event.block();
    }
    for (auto &out : t.output()) {  // write-after-write / write-after-read across streams
      auto &ti = *out.impl();
      adopt(ti);
      if (ti.stream_class != cls && !ti.event.query()) ti.event.block();
      // a writer waits for the readers of every side stream other than its own (its own stream
      // orders them already)
      for (int c = 0; c < static_cast<int>(StreamClass::kNumStreamClass); ++c) {
        const auto bit = static_cast<uint8_t>(1u << c);
        if (!(ti.side_readers & bit) || c == static_cast<int>(cls)) continue;
        if (!ti.read_event[c].query()) ti.read_event[c].block();
      }
      ti.side_readers = 0;
    }
    TimedTask timed{};
    if (profiling_) {
      CS_CHECK_CUDART(cudaEventCreate(&timed.start));
      CS_CHECK_CUDART(cudaEventCreate(&timed.stop));
      CS_CHECK_CUDART(cudaEventRecord(timed.start, streams_[tag].stream()));
    }
    {
      CS_NVTX_RANGE_FN(t.name());
      try {
        task();
      } catch (const Error &) {
        throw;
      } catch (const std::exception &e) {
        rethrow_with_task(task, e);
      }
    }
    if (profiling_) {
      CS_CHECK_CUDART(cudaEventRecord(timed.stop, streams_[tag].stream()));
      timed.name = t.name();
      timed.stream_class = tag;
      timed_.push_back(std::move(timed));
    }
    for (auto &out : t.output()) {
      out.impl()->stream_class = cls;
      out.impl()->event.record();
    }
  }

  void submit(Task &&task) override {
    const auto &t = *task.impl();
    if (t.type() == Task::Impl::kConfig) {
      ++submitted[3];
      CS_NVTX_RANGE_FN(t.name());
      task();
      return;
    }
    c10::cuda::CUDAGuard device_guard{device_};
    const auto tag = t.priority();
    ++submitted[tag];
    c10::cuda::CUDAStreamGuard stream_guard{streams_[tag]};
    const ExecContext saved = tls_exec;
    tls_exec = ExecContext{true, static_cast<int>(device_rank_)};
    struct Restore {
      ExecContext saved;
      ~Restore() { tls_exec = saved; }
    } restore{saved};

    if (tag == Task::Impl::kMain) {
      age(queues_[Task::Impl::kAssist]);
      age(queues_[Task::Impl::kComm]);
      run(task, tag);
      main_event_.record();
      return;
    }
    // Side streams never start ahead of the most recent main-stream task.
    main_event_.block();
    run(task, tag);
    SideEntry entry{gaps_[tag], Event{}, {}};
    entry.keep_alive.reserve(t.input().size() + t.output().size() + t.intermediate().size());
    for (auto &in : t.input()) entry.keep_alive.push_back(in.impl()->tensor);
    for (auto &out : t.output()) entry.keep_alive.push_back(out.impl()->tensor);
    for (auto &tmp : t.intermediate()) entry.keep_alive.push_back(tmp);
    entry.event.record();
    for (auto &in : t.input()) {
      auto &ti = *in.impl();
      ti.read_event[tag] = entry.event;
      ti.side_readers |= static_cast<uint8_t>(1u << tag);
    }
    queues_[tag].push_back(std::move(entry));
  }

 private:
  std::vector<c10::cuda::CUDAStream> streams_;
  Event main_event_;
  std::deque<SideEntry> queues_[Task::Impl::kNumPriority];
  int gaps_[Task::Impl::kNumPriority];
  bool profiling_{false};
  std::vector<TimedTask> timed_;
};
}  // namespace

DynamicScheduler::DynamicScheduler(int localRank) : DynamicScheduler(localRank, Options{}) {}

DynamicScheduler::DynamicScheduler(int localRank, const Options &options) {
  at::DeviceType type = options.device_type().has_value() ? *options.device_type()
                                                          : (cuda_usable() ? at::kCUDA : at::kCPU);
  if (type == at::kCUDA) {
    CS_ASSERT_TRUE(cuda_usable(), "a CUDA scheduler was requested but no GPU is visible");
    impl_ = std::make_shared<CudaImpl>(localRank, options.assist_task_gap(), options.comm_task_gap());
  } else {
    impl_ = std::make_shared<CpuImpl>(localRank);
  }
}

// --------------------------------------------------------------------------- autocast ----
namespace autocast {
ContextGuard::ContextGuard(const Scheduler &scheduler, const c10::ScalarType &dtype)
    : scheduler_{scheduler},
      prev_enabled_{scheduler.impl()->autocast_enabled},
      prev_dtype_{scheduler.impl()->autocast_dtype} {
  auto impl = scheduler.impl();
  const at::ScalarType dt = dtype;
  submit(scheduler, "cs::autocast::ContextGuard::enter", Task::Impl::kMain, Task::Impl::kConfig, {}, {},
         [impl, dt](const FnTask &) {
           impl->autocast_enabled = true;
           impl->autocast_dtype = dt;
         });
}

ContextGuard::~ContextGuard() {
  auto impl = scheduler_.impl();
  const bool en = prev_enabled_;
  const at::ScalarType dt = prev_dtype_;
  try {
    submit(scheduler_, "cs::autocast::ContextGuard::exit", Task::Impl::kMain, Task::Impl::kConfig, {}, {},
           [impl, en, dt](const FnTask &) {
             impl->autocast_enabled = en;
             impl->autocast_dtype = dt;
           });
  } catch (...) {
  }
}
}  // namespace autocast

// ----------------------------------------------------------------------------- memory ----
namespace memory {
at::Tensor to_torch(const Scheduler &scheduler, const ReadOnlyTensor &tensor) {
  Tensor out;
  submit(scheduler, "cs::memory::to_torch", Task::Impl::kMain, Task::Impl::kMemcpy, {out}, {tensor},
         [out, tensor](const FnTask &) {
           const auto &src = tensor.impl()->tensor;
           out.impl()->tensor = src.defined() ? src.detach().clone() : at::Tensor{};
         });
  out.wait();
  return out.impl()->tensor;
}
}  // namespace memory
}  // namespace cs

namespace at {
namespace {
at::Tensor settled(const cs::ReadOnlyTensor &t) {
  t.wait();
  return t.impl()->tensor;
}
bool close_enough(const at::Tensor &a, const at::Tensor &b, double rtol, double atol, bool equal_nan) {
  if (a.is_cuda() || b.is_cuda()) cudaDeviceSynchronize();
  if (a.scalar_type() != b.scalar_type() || a.device() != b.device()) {
    return at::allclose(a.to(at::kCPU, at::kDouble), b.to(at::kCPU, at::kDouble), rtol, atol, equal_nan);
  }
  return at::allclose(a, b, rtol, atol, equal_nan);
}
}  // namespace
bool allclose(const cs::ReadOnlyTensor &t1, const at::Tensor &t2, double rtol, double atol, bool equal_nan) {
  return close_enough(settled(t1), t2, rtol, atol, equal_nan);
}
bool allclose(const cs::ReadOnlyTensor &t1, const cs::ReadOnlyTensor &t2, double rtol, double atol, bool equal_nan) {
  return close_enough(settled(t1), settled(t2), rtol, atol, equal_nan);
}
bool allclose(const at::Tensor &t1, const cs::ReadOnlyTensor &t2, double rtol, double atol, bool equal_nan) {
  return close_enough(t1, settled(t2), rtol, atol, equal_nan);
}
}  // namespace at
