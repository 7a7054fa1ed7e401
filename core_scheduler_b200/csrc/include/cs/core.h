// SPDX-License-Identifier: Apache-2.0
// Core runtime types of the B200 scheduler framework: logging/check macros, NVTX
// ranges, pooled events, future-tensor handles, tasks and the multi-stream scheduler.
//
// Capability parity (reference paths are relative to the reference project root):
//   include/tensor.h:36-83, include/internal/tensor_impl.h:30-59   -> cs::ReadOnlyTensor / cs::Tensor
//   include/threading/event.h:21-42, src/threading/event.cpp:24-77 -> cs::Event (pooled)
//   include/threading/task.h:24-37, include/internal/threading/task_impl.h:23-61 -> cs::Task
//   include/threading/scheduler.h:23-32, src/threading/dynamic_scheduler.cpp:101-221 -> cs::Scheduler / cs::DynamicScheduler
//   include/logger.h:26-91, include/nvtx_helper.h:21-41, include/random.h:23, include/autocast.h:23-30
//
// Design differences (deliberate): events are raw cudaEvent_t objects kept in a per-device
// pool and degrade to host no-ops when the scheduler runs on the CPU; tensors additionally
// carry a "last side-stream reader" event so write-after-read hazards across streams are
// ordered explicitly; streams are created with priorities (comm > assist > main); the
// re-join distances of side tasks are runtime options; failures raise cs::Error with the
// task name instead of aborting the process (set CS_ABORT_ON_ERROR=1 for abort semantics).
#pragma once
#include <ATen/ATen.h>
#include <c10/util/Optional.h>

#include <atomic>
#include <cstdint>
#include <functional>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#if defined(_WIN32)
#define CS_API
#else
#define CS_API __attribute__((visibility("default")))
#endif

// Chainable option setter: `CS_ARG(int64_t, in_futures);` declares `in_futures_`,
// a getter `in_futures()` and a setter `in_futures(v)` returning *this.
#define CS_ARG(T, name)                                        \
 public:                                                       \
  inline auto name(const T &new_##name) -> decltype(*this) {   \
    this->name##_ = new_##name;                                \
    return *this;                                              \
  }                                                            \
  inline const T &name() const noexcept { return this->name##_; } \
  inline T &name() noexcept { return this->name##_; }          \
                                                               \
 private:                                                      \
  T name##_

namespace cs {
using Scalar = at::Scalar;
using IntArrayRef = at::IntArrayRef;
using IntArray = c10::SmallVector<int64_t>;
using TensorOptions = at::TensorOptions;
template <typename T>
using optional = std::optional<T>;

// ----------------------------------------------------------------------------------------
// errors & logging
// ----------------------------------------------------------------------------------------
struct CS_API Error : std::runtime_error {
  using std::runtime_error::runtime_error;
};

enum class LogLevel : int { kTrace = 0, kDebug, kInfo, kWarn, kError, kCritical, kOff };

// Minimal levelled logger named "CS" (stdout, colourised when attached to a tty).
// Level comes from CS_LOG_LEVEL={trace,debug,info,warn,error,critical,off}.
struct CS_API Logger {
  void log(LogLevel level, const std::string &msg);
  void set_level(LogLevel level) { level_ = level; }
  [[nodiscard]] LogLevel level() const { return level_; }
  template <typename... Args>
  void info(const Args &...a) { emit(LogLevel::kInfo, a...); }
  template <typename... Args>
  void warn(const Args &...a) { emit(LogLevel::kWarn, a...); }
  template <typename... Args>
  void error(const Args &...a) { emit(LogLevel::kError, a...); }
  template <typename... Args>
  void critical(const Args &...a) { emit(LogLevel::kCritical, a...); }
  template <typename... Args>
  void debug(const Args &...a) { emit(LogLevel::kDebug, a...); }

 private:
  template <typename... Args>
  void emit(LogLevel l, const Args &...a) {
    if (l < level_) return;
    std::ostringstream os;
    (os << ... << a);
    log(l, os.str());
  }
  LogLevel level_{LogLevel::kInfo};
};
CS_API Logger &logger();

// Raises cs::Error (or aborts when CS_ABORT_ON_ERROR=1) after logging at critical level.
[[noreturn]] CS_API void fail(const char *file, int line, const std::string &what);
CS_API std::string cuda_error_string(int code);

template <typename... Args>
inline std::string str_cat(const Args &...a) {
  std::ostringstream os;
  (os << ... << a);
  return os.str();
}
}  // namespace cs

#define CS_ASSERT_TRUE(cond, ...)                                       \
  do {                                                                  \
    if (!(cond)) [[unlikely]] {                                         \
      ::cs::fail(__FILE__, __LINE__, ::cs::str_cat("assertion `" #cond "` failed: ", __VA_ARGS__)); \
    }                                                                   \
  } while (0)

#define CS_WARN_TRUE(cond, ...)                                         \
  do {                                                                  \
    if (!(cond)) [[unlikely]] {                                         \
      ::cs::logger().warn(__FILE__, ":", __LINE__, " ", ::cs::str_cat(__VA_ARGS__)); \
    }                                                                   \
  } while (0)

#define CS_CHECK_CUDART(expr)                                           \
  do {                                                                  \
    const int cs_code_ = static_cast<int>(expr);                        \
    if (cs_code_ != 0) [[unlikely]] {                                   \
      ::cs::fail(__FILE__, __LINE__, ::cs::str_cat("CUDA runtime call `" #expr "` failed: ", ::cs::cuda_error_string(cs_code_))); \
    }                                                                   \
  } while (0)

// Status checks for the other libraries a program built on this one may call (same names as in the reference's
// logger.h:51-89). They are plain macros over the status value and need the respective library header only where
// they are used; this library itself calls none of cuBLAS, cuDNN or NCCL directly.
#define CS_CHECK_STATUS_(expr, ok_value, what)                                                          \
  do {                                                                                                   \
    const auto cs_status_ = (expr);                                                                      \
    if (!(cs_status_ == (ok_value))) [[unlikely]] {                                                      \
      ::cs::fail(__FILE__, __LINE__, ::cs::str_cat(what " call `" #expr "` returned code ", static_cast<long long>(cs_status_))); \
    }                                                                                                    \
  } while (0)
#define CS_CHECK_CUBLAS(expr) CS_CHECK_STATUS_(expr, CUBLAS_STATUS_SUCCESS, "cuBLAS")
#define CS_CHECK_MPI(expr) CS_CHECK_STATUS_(expr, MPI_SUCCESS, "MPI")
#define CS_CHECK_NCCL(expr) CS_CHECK_STATUS_(expr, ncclSuccess, "NCCL")
#define CS_CHECK_CUDNN(expr) CS_CHECK_STATUS_(expr, CUDNN_STATUS_SUCCESS, "cuDNN")
#define CS_CHECK_CUDNN_FE(expr)                                                                          \
  do {                                                                                                   \
    const auto cs_status_ = (expr);                                                                      \
    if (!cs_status_.is_good()) [[unlikely]] {                                                            \
      ::cs::fail(__FILE__, __LINE__, ::cs::str_cat("cuDNN frontend call `" #expr "` failed: ", cs_status_.get_message())); \
    }                                                                                                    \
  } while (0)

namespace cs {
// ----------------------------------------------------------------------------------------
// NVTX
// ----------------------------------------------------------------------------------------
struct CS_API NvtxRange {
  explicit NvtxRange(const char *name);
  ~NvtxRange();
  NvtxRange(const NvtxRange &) = delete;
  NvtxRange &operator=(const NvtxRange &) = delete;
};
#define CS_NVTX_CAT_(a, b) a##b
#define CS_NVTX_CAT(a, b) CS_NVTX_CAT_(a, b)
#define CS_NVTX_RANGE_FN(name) ::cs::NvtxRange CS_NVTX_CAT(cs_nvtx_range_, __LINE__)(name)

// Seeds the CPU generator and every visible CUDA generator (offset 0).
CS_API void manual_seed(int64_t seed);

// ----------------------------------------------------------------------------------------
// Event
// ----------------------------------------------------------------------------------------
// Completion marker of a piece of stream work. A default-constructed Event has never been
// recorded: query() is true and block()/synchronize() return immediately. On a CPU
// scheduler every method is a no-op. CUDA events come from a per-device free list and go
// back to it when the last handle is dropped.
struct CS_API Event {
  struct Impl;
  Event();
  explicit Event(std::shared_ptr<Impl> impl);
  void block() const;        // make the calling thread's current stream wait for this event
  void record() const;       // record on the calling thread's current stream
  [[nodiscard]] bool query() const;
  void synchronize() const;  // host wait
  [[nodiscard]] const std::shared_ptr<Impl> &impl() const { return impl_; }
  // Number of CUDA events currently parked in the pool (for tests).
  static int64_t pooled();

 private:
  std::shared_ptr<Impl> impl_;
};

// ----------------------------------------------------------------------------------------
// Tensor handles
// ----------------------------------------------------------------------------------------
enum class StreamClass : int8_t { kMain = 0, kAssist = 1, kComm = 2, kNumStreamClass = 3 };

struct CS_API ReadOnlyTensor {
  struct Impl;
  ReadOnlyTensor();
  [[nodiscard]] TensorOptions options() const;
  [[nodiscard]] IntArrayRef sizes() const;
  [[nodiscard]] int64_t size(int64_t dim) const;
  [[nodiscard]] int64_t numel() const;
  [[nodiscard]] bool defined() const;
  void wait() const;   // host-blocks until the last writer finished
  void reset();        // drop this handle's reference; the handle becomes a fresh empty slot
  [[nodiscard]] const std::shared_ptr<Impl> &impl() const { return impl_; }

 protected:
  std::shared_ptr<Impl> impl_;
};

struct CS_API Tensor : ReadOnlyTensor {
  Tensor() = default;
  // Wraps an existing ATen tensor (no copy); the result is immediately ready.
  static Tensor wrap(at::Tensor t);
};

struct ReadOnlyTensor::Impl {
  at::Tensor tensor;                       // undefined until the producing task ran
  Event event;                             // completion of the last writer
  // Completion of the last reader on each side stream (index = stream class; bit set in
  // side_readers while that reader has not been waited for by a later writer).
  Event read_event[static_cast<int>(StreamClass::kNumStreamClass)];
  StreamClass stream_class{StreamClass::kMain};
  uint8_t side_readers{0};
  // Memory that came from the caller's allocator stream (Tensor::wrap): every scheduler stream
  // that touches it is reported to the caching allocator once (bit per stream class), so a
  // block freed on the host is not handed out again while a queued kernel still reads it.
  bool external{false};
  uint8_t external_streams{0};
  // Mixed-precision stamp set by forward ops running under autocast; backward ops use it to
  // pick the compute dtype.
  bool autocast_enabled{false};
  at::ScalarType autocast_dtype{at::kFloat};
  // Bumped whenever the values of a parameter change (optimizer step, load, init); lets
  // low-precision working copies detect staleness.
  uint64_t version{0};
  // Low-precision working copy of a parameter (`lp`, same shape) and its 2-D transpose
  // (`lp_t`), valid while their version equals `version`. Written by the mixed-precision
  // optimizer in the same kernel that updates the master value, or lazily by forward ops.
  at::Tensor lp, lp_t;
  uint64_t lp_version{~0ull}, lp_t_version{~0ull};
  // Gradient slots that live in a flat arena are persistent: zero_grad() marks them
  // `fresh` (the next backward overwrites instead of accumulating) and keeps the storage.
  bool persistent{false};
  bool fresh{false};
  // Optional tensor travelling with this one (e.g. GELU(x) emitted by the epilogue of the
  // GEMM that produced x, consumed by GeluLinear without a separate activation kernel).
  at::Tensor companion;
};

CS_API std::ostream &print(std::ostream &os, const ReadOnlyTensor &t, int64_t linesize = 80);
CS_API std::ostream &operator<<(std::ostream &os, const ReadOnlyTensor &t);

// ----------------------------------------------------------------------------------------
// Task
// ----------------------------------------------------------------------------------------
struct CS_API Task {
  struct Impl;
  explicit Task(std::shared_ptr<Impl> impl) : impl_{std::move(impl)} {}
  void operator()() const;
  [[nodiscard]] const std::shared_ptr<Impl> &impl() const { return impl_; }
  void reset() { impl_.reset(); }

 private:
  std::shared_ptr<Impl> impl_;
};

struct CS_API Task::Impl {
  enum Type { kConfig = 0, kCompute, kLoader, kMemcpy, kNccl, kNumType };
  enum Priority { kMain = 0, kAssist, kComm, kNumPriority };
  Impl(std::vector<Tensor> output, std::vector<ReadOnlyTensor> input, Priority priority, Type type)
      : output_{std::move(output)}, input_{std::move(input)}, priority_{priority}, type_{type} {}
  virtual ~Impl() = default;
  [[nodiscard]] const std::vector<ReadOnlyTensor> &input() const { return input_; }
  [[nodiscard]] const std::vector<Tensor> &output() const { return output_; }
  // Temporaries that must outlive the asynchronous work of this task.
  [[nodiscard]] std::vector<at::Tensor> &intermediate() const { return intermediate_; }
  [[nodiscard]] Type type() const { return type_; }
  [[nodiscard]] Priority priority() const { return priority_; }
  virtual void operator()() const = 0;
  [[nodiscard]] virtual const char *name() const = 0;

 private:
  std::vector<Tensor> output_;
  std::vector<ReadOnlyTensor> input_;
  mutable std::vector<at::Tensor> intermediate_;
  Priority priority_;
  Type type_;
};

// A task whose body is a closure; what every built-in op uses.
struct CS_API FnTask final : Task::Impl {
  using Body = std::function<void(const FnTask &)>;
  FnTask(const char *name, std::vector<Tensor> output, std::vector<ReadOnlyTensor> input,
         Priority priority, Type type, Body body)
      : Task::Impl{std::move(output), std::move(input), priority, type}, name_{name}, body_{std::move(body)} {}
  void operator()() const override { body_(*this); }
  [[nodiscard]] const char *name() const override { return name_; }

 private:
  const char *name_;
  Body body_;
};

// ----------------------------------------------------------------------------------------
// Scheduler
// ----------------------------------------------------------------------------------------
struct TaskTiming {
  std::string name;
  int stream_class;
  double device_ms;
  double start_ms{0};  // start on the device, relative to the first task of the drained batch
};

struct CS_API Scheduler {
  struct Impl;
  [[nodiscard]] const std::shared_ptr<Impl> &impl() const { return impl_; }
  [[nodiscard]] int64_t get_device_rank() const;
  [[nodiscard]] at::Device device() const;

 protected:
  std::shared_ptr<Impl> impl_;
};

struct CS_API Scheduler::Impl {
  explicit Impl(int64_t device_rank, at::Device device) : device_rank_{device_rank}, device_{device} {}
  virtual ~Impl() = default;
  virtual void submit(Task &&task);
  // Host-blocks until everything submitted so far has finished on every stream.
  virtual void synchronize() {}
  // Raw stream handle (cudaStream_t) of a stream class, nullptr on CPU.
  [[nodiscard]] virtual void *raw_stream(StreamClass) const { return nullptr; }
  // Per-task device timings gathered while profiling is on (CS_PROFILE=1 or set_profiling).
  virtual std::vector<TaskTiming> drain_timings() { return {}; }
  virtual void set_profiling(bool) {}
  [[nodiscard]] int64_t device_rank() const { return device_rank_; }
  [[nodiscard]] at::Device device() const { return device_; }
  // number of tasks submitted so far, per stream class (+ config tasks in slot 3)
  int64_t submitted[4] = {0, 0, 0, 0};

  // autocast state (set by autocast::ContextGuard through a kConfig task)
  bool autocast_enabled{false};
  at::ScalarType autocast_dtype{at::kBFloat16};

 protected:
  int64_t device_rank_;
  at::Device device_;
};

struct CS_API DynamicScheduler : Scheduler {
  struct Options {
    Options() {}
    // After how many further main-stream tasks the main stream re-joins a side task.
    CS_ARG(int, assist_task_gap) = 2;
    CS_ARG(int, comm_task_gap) = 5;
    // kCUDA, kCPU, or nullopt = CUDA when a GPU is visible, else CPU.
    CS_ARG(optional<at::DeviceType>, device_type) = {};
  };
  explicit DynamicScheduler(int localRank);
  DynamicScheduler(int localRank, const Options &options);
};

// Convenience used by every op: build an FnTask and hand it to the scheduler.
CS_API void submit(const Scheduler &scheduler, const char *name, Task::Impl::Priority priority,
                   Task::Impl::Type type, std::vector<Tensor> output, std::vector<ReadOnlyTensor> input,
                   FnTask::Body body);

namespace autocast {
// RAII: enables mixed precision for ops submitted to `scheduler` while alive.
struct CS_API ContextGuard {
  ContextGuard(const Scheduler &scheduler, const c10::ScalarType &dtype);
  ~ContextGuard();
  ContextGuard(const ContextGuard &) = delete;
  ContextGuard &operator=(const ContextGuard &) = delete;

 private:
  Scheduler scheduler_;
  bool prev_enabled_;
  at::ScalarType prev_dtype_;
};
}  // namespace autocast

namespace memory {
// Blocking bridge for tests/debugging: returns a detached clone of the current value.
CS_API at::Tensor to_torch(const Scheduler &scheduler, const ReadOnlyTensor &tensor);
}  // namespace memory
}  // namespace cs

namespace at {
CS_API bool allclose(const cs::ReadOnlyTensor &t1, const at::Tensor &t2, double rtol = 1e-5, double atol = 1e-8, bool equal_nan = false);
CS_API bool allclose(const cs::ReadOnlyTensor &t1, const cs::ReadOnlyTensor &t2, double rtol = 1e-5, double atol = 1e-8, bool equal_nan = false);
CS_API bool allclose(const at::Tensor &t1, const cs::ReadOnlyTensor &t2, double rtol = 1e-5, double atol = 1e-8, bool equal_nan = false);
}  // namespace at
