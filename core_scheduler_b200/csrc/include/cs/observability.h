// SPDX-License-Identifier: Apache-2.0
// Metrics, progress watchdog and resumable training state.
//
// The reference prints one console line per step from its examples
// (example/gpt2/gpt2_ddp.cpp:725-729) and appends "Step,Loss" rows to a CSV
// (example/gpt2/gpt2_single_device.cpp:606-607); it has no watchdog and stores parameters only
// (src/module/module.cpp save/load). Everything beyond the console line and the CSV is an addition.
#pragma once

#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <fstream>
#include <functional>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "cs/communication.h"
#include "cs/core.h"
#include "cs/module.h"

namespace cs::metrics {
// One training step as it is reported. Fields that were not measured stay negative and are
// left out of the JSON line.
struct CS_API StepRecord {
  int64_t step{0};
  double loss{-1};
  double lr{-1};
  double grad_norm{-1};
  double dt_host_ms{-1};
  double dt_device_ms{-1};  // max over ranks when the caller reduced it
  double tokens_per_sec{-1};
  double mfu{-1};
  double comm_bytes{-1};
  std::map<std::string, double> extra;  // e.g. per-stream busy fractions, roofline fractions
};

// Writes the reference's console line, its CSV, and a JSON-lines file. Only the rank given as
// `writer_rank` writes; the others are no-ops so that call sites need no rank test.
struct CS_API MetricsLogger {
  struct Options {
    CS_ARG(std::string, jsonl_path) = {};
    CS_ARG(std::string, csv_path) = {};
    CS_ARG(bool, console) = true;
    CS_ARG(int64_t, rank) = 0;
    CS_ARG(int64_t, writer_rank) = 0;
  };
  explicit MetricsLogger(const Options &options);
  void log(const StepRecord &record);
  [[nodiscard]] int64_t records_written() const { return written_; }
  static std::string to_json(const StepRecord &record);
  static std::string console_line(const StepRecord &record);

 private:
  Options options_;
  std::ofstream jsonl_, csv_;
  int64_t written_{0};
};

// Model FLOPs utilisation of a step: flops_per_token * tokens / seconds / peak.
CS_API double mfu(double flops_per_token, double tokens, double seconds, double peak_flops);
}  // namespace cs::metrics

namespace cs::fault {
// Host thread that notices a stalled training loop. The loop calls `progress(step)`; when no
// progress arrives within the timeout the watchdog marks itself tripped, publishes
// "cs/failed/<rank>" in the communicator's store (when there is one) and calls `on_timeout`
// once. It also polls the store for other ranks' failure keys so that a healthy rank learns of
// a peer's stall before its next launch. It never touches a GPU.
struct CS_API Watchdog {
  struct Options {
    CS_ARG(int64_t, timeout_ms) = 60000;
    CS_ARG(int64_t, poll_ms) = 50;
  };
  Watchdog(const communication::Comm &comm, const Options &options, std::function<void(int64_t)> on_timeout = {});
  explicit Watchdog(const Options &options, std::function<void(int64_t)> on_timeout = {});
  ~Watchdog();
  Watchdog(const Watchdog &) = delete;
  Watchdog &operator=(const Watchdog &) = delete;

  void progress(int64_t step);
  void stop();
  [[nodiscard]] bool tripped() const { return tripped_.load(); }
  [[nodiscard]] int64_t last_step() const { return last_step_.load(); }
  // Ranks (other than this one) that published a failure.
  [[nodiscard]] std::vector<int64_t> failed_peers() const;
  // Throws cs::Error when this rank stalled or a peer reported a failure; call it before a launch.
  void check() const;

 private:
  void loop();
  std::shared_ptr<communication::Comm::Impl> comm_;
  Options options_;
  std::function<void(int64_t)> on_timeout_;
  std::atomic<bool> tripped_{false}, stop_{false};
  std::atomic<int64_t> last_step_{-1}, last_ms_{0};
  mutable std::mutex mutex_;
  std::condition_variable cv_;
  std::vector<int64_t> failed_peers_;
  std::thread thread_;
};
}  // namespace cs::fault

namespace cs::checkpoint {
// Everything besides tensors that a run needs to continue where it stopped.
struct CS_API Meta {
  int64_t step{0};
  double lr{0};
  uint64_t seed{0};
  int64_t data_cursor{0};  // batches already consumed by this rank's loader
  int64_t world_size{1};
  int64_t tp_size{1};
  bool zero{false};
  std::string model{};
};
CS_API void save_meta(const Meta &meta, const std::string &path);
CS_API Meta load_meta(const std::string &path);

// Directory layout: model.parquet (the reference's parameter file, loadable by its cs::load),
// optimizer.parquet (moments, step, lr) and meta.json. Written by `writer_rank` only.
CS_API void save_training_state(const Scheduler &scheduler, const std::string &dir, const module::Module &model,
                                const module::OptimizerModule *optimizer, const Meta &meta, int64_t rank = 0,
                                int64_t writer_rank = 0);
CS_API Meta load_training_state(const Scheduler &scheduler, const std::string &dir, const module::Module &model,
                                module::OptimizerModule *optimizer);
}  // namespace cs::checkpoint
