// SPDX-License-Identifier: Apache-2.0
// Metrics logger, host watchdog and resumable training state (see cs/observability.h).
#include "cs/observability.h"

#include <sys/stat.h>

#include <chrono>
#include <cmath>
#include <cstdio>
#include <iomanip>
#include <sstream>

namespace cs::metrics {
namespace {
void put(std::ostringstream &os, bool &first, const std::string &key, double value) {
  if (!std::isfinite(value)) return;
  os << (first ? "" : ", ") << '"' << key << "\": " << std::setprecision(10) << value;
  first = false;
}
std::string escaped(const std::string &s) {
  std::string out;
  for (char c : s) {
    if (c == '"' || c == '\\') out.push_back('\\');
    if (c == '\n') {
      out += "\\n";
      continue;
    }
    out.push_back(c);
  }
  return out;
}
}  // namespace

std::string MetricsLogger::to_json(const StepRecord &r) {
  std::ostringstream os;
  bool first = false;
  os << "{\"step\": " << r.step;
  if (r.loss >= 0) put(os, first, "loss", r.loss);
  if (r.lr >= 0) put(os, first, "lr", r.lr);
  if (r.grad_norm >= 0) put(os, first, "grad_norm", r.grad_norm);
  if (r.dt_host_ms >= 0) put(os, first, "dt_host_ms", r.dt_host_ms);
  if (r.dt_device_ms >= 0) put(os, first, "dt_device_ms_max_over_ranks", r.dt_device_ms);
  if (r.tokens_per_sec >= 0) put(os, first, "tokens_per_sec", r.tokens_per_sec);
  if (r.mfu >= 0) put(os, first, "mfu", r.mfu);
  if (r.comm_bytes >= 0) put(os, first, "comm_bytes", r.comm_bytes);
  for (auto &kv : r.extra) put(os, first, escaped(kv.first), kv.second);
  os << "}";
  return os.str();
}

std::string MetricsLogger::console_line(const StepRecord &r) {
  char buf[256];
  std::snprintf(buf, sizeof(buf), "step %4lld | loss %.6f | lr %.4e | grad norm %.4f | dt %.2f ms | tok/sec %.0f",
                static_cast<long long>(r.step), r.loss, r.lr, r.grad_norm, r.dt_host_ms >= 0 ? r.dt_host_ms : r.dt_device_ms,
                r.tokens_per_sec);
  return buf;
}

MetricsLogger::MetricsLogger(const Options &options) : options_{options} {
  if (options_.rank() != options_.writer_rank()) return;
  if (!options_.jsonl_path().empty()) {
    jsonl_.open(options_.jsonl_path(), std::ios::app);
    CS_ASSERT_TRUE(jsonl_.good(), "cannot open metrics file ", options_.jsonl_path());
  }
  if (!options_.csv_path().empty()) {
    struct stat st {};
    const bool fresh = ::stat(options_.csv_path().c_str(), &st) != 0 || st.st_size == 0;
    csv_.open(options_.csv_path(), std::ios::app);
    CS_ASSERT_TRUE(csv_.good(), "cannot open csv file ", options_.csv_path());
    if (fresh) csv_ << "Step,Loss\n";
  }
}

void MetricsLogger::log(const StepRecord &record) {
  if (options_.rank() != options_.writer_rank()) return;
  if (options_.console()) std::printf("%s\n", console_line(record).c_str());
  if (jsonl_.is_open()) jsonl_ << to_json(record) << std::endl;
  if (csv_.is_open()) csv_ << record.step << "," << std::setprecision(9) << record.loss << std::endl;
  ++written_;
}

double mfu(double flops_per_token, double tokens, double seconds, double peak_flops) {
  if (seconds <= 0 || peak_flops <= 0) return 0.0;
  return flops_per_token * tokens / seconds / peak_flops;
}
}  // namespace cs::metrics

namespace cs::fault {
namespace {
int64_t now_ms() {
  return std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
std::string failed_key(int64_t rank) { return "cs/failed/" + std::to_string(rank); }
}  // namespace

Watchdog::Watchdog(const communication::Comm &comm, const Options &options, std::function<void(int64_t)> on_timeout)
    : comm_{comm.impl()}, options_{options}, on_timeout_{std::move(on_timeout)} {
  last_ms_ = now_ms();
  thread_ = std::thread([this] { loop(); });
}

Watchdog::Watchdog(const Options &options, std::function<void(int64_t)> on_timeout)
    : options_{options}, on_timeout_{std::move(on_timeout)} {
  last_ms_ = now_ms();
  thread_ = std::thread([this] { loop(); });
}

Watchdog::~Watchdog() { stop(); }

void Watchdog::stop() {
  if (!stop_.exchange(true)) cv_.notify_all();
  if (thread_.joinable() && std::this_thread::get_id() != thread_.get_id()) thread_.join();
}

void Watchdog::progress(int64_t step) {
  last_step_ = step;
  last_ms_ = now_ms();
}

std::vector<int64_t> Watchdog::failed_peers() const {
  std::lock_guard<std::mutex> lock{mutex_};
  return failed_peers_;
}

void Watchdog::check() const {
  CS_ASSERT_TRUE(!tripped(), "watchdog: no progress for more than ", options_.timeout_ms(), " ms after step ", last_step());
  const auto peers = failed_peers();
  CS_ASSERT_TRUE(peers.empty(), "watchdog: rank ", peers.empty() ? -1 : peers.front(), " reported a failure");
}

void Watchdog::loop() {
  std::unique_lock<std::mutex> lock{mutex_};
  while (!stop_) {
    cv_.wait_for(lock, std::chrono::milliseconds(options_.poll_ms()), [this] { return stop_.load(); });
    if (stop_) break;
    if (!tripped_ && now_ms() - last_ms_ > options_.timeout_ms()) {
      tripped_ = true;
      const int64_t step = last_step_;
      lock.unlock();
      try {
        if (comm_ && comm_->store) {
          const std::string v = std::to_string(step);
          comm_->store->set(failed_key(comm_->rank), std::vector<uint8_t>(v.begin(), v.end()));
        }
      } catch (...) {  // the store may be gone with its host rank; the local flag still stands
      }
      if (on_timeout_) on_timeout_(step);
      lock.lock();
    }
    if (comm_ && comm_->store) {
      std::vector<int64_t> failed;
      lock.unlock();
      try {
        for (int64_t r = 0; r < comm_->size; ++r)
          if (r != comm_->rank && comm_->store->check({failed_key(r)})) failed.push_back(r);
      } catch (...) {
      }
      lock.lock();
      failed_peers_ = std::move(failed);
    }
  }
}
}  // namespace cs::fault

namespace cs::checkpoint {
namespace {
std::string read_file(const std::string &path) {
  std::ifstream in(path);
  CS_ASSERT_TRUE(in.good(), "cannot open ", path);
  std::stringstream ss;
  ss << in.rdbuf();
  return ss.str();
}
// The file is written by save_meta below: a flat object of numbers, booleans and one string.
std::string raw_value(const std::string &text, const std::string &key) {
  const auto k = text.find("\"" + key + "\"");
  CS_ASSERT_TRUE(k != std::string::npos, "meta file lacks `", key, "`");
  auto p = text.find(':', k);
  CS_ASSERT_TRUE(p != std::string::npos, "meta file: malformed entry `", key, "`");
  ++p;
  while (p < text.size() && std::isspace(static_cast<unsigned char>(text[p]))) ++p;
  CS_ASSERT_TRUE(p < text.size(), "meta file: entry `", key, "` has no value");
  if (text[p] == '"') {
    std::string out;
    for (++p; p < text.size() && text[p] != '"'; ++p) {
      if (text[p] == '\\' && p + 1 < text.size()) ++p;
      out.push_back(text[p]);
    }
    return out;
  }
  auto e = p;
  while (e < text.size() && text[e] != ',' && text[e] != '}' && text[e] != '\n') ++e;
  return text.substr(p, e - p);
}
void make_dir(const std::string &dir) {  // like mkdir -p
  for (size_t pos = 1; pos <= dir.size(); ++pos) {
    if (pos != dir.size() && dir[pos] != '/') continue;
    const std::string part = dir.substr(0, pos);
    if (::mkdir(part.c_str(), 0755) != 0) {
      struct stat st {};
      CS_ASSERT_TRUE(::stat(part.c_str(), &st) == 0 && S_ISDIR(st.st_mode), "cannot create directory ", part);
    }
  }
}
}  // namespace

void save_meta(const Meta &m, const std::string &path) {
  const std::string tmp = path + ".tmp";
  {
    std::ofstream out(tmp, std::ios::trunc);
    CS_ASSERT_TRUE(out.good(), "cannot write ", tmp);
    std::string model;
    for (char c : m.model) {
      if (c == '"' || c == '\\') model.push_back('\\');
      model.push_back(c);
    }
    out << "{\n  \"step\": " << m.step << ",\n  \"lr\": " << std::setprecision(17) << m.lr << ",\n  \"seed\": " << m.seed
        << ",\n  \"data_cursor\": " << m.data_cursor << ",\n  \"world_size\": " << m.world_size << ",\n  \"tp_size\": " << m.tp_size
        << ",\n  \"zero\": " << (m.zero ? "true" : "false") << ",\n  \"model\": \"" << model << "\"\n}\n";
  }
  CS_ASSERT_TRUE(std::rename(tmp.c_str(), path.c_str()) == 0, "cannot move ", tmp, " to ", path);
}

Meta load_meta(const std::string &path) {
  const std::string text = read_file(path);
  Meta m;
  m.step = std::stoll(raw_value(text, "step"));
  m.lr = std::stod(raw_value(text, "lr"));
  m.seed = std::stoull(raw_value(text, "seed"));
  m.data_cursor = std::stoll(raw_value(text, "data_cursor"));
  m.world_size = std::stoll(raw_value(text, "world_size"));
  m.tp_size = std::stoll(raw_value(text, "tp_size"));
  m.zero = raw_value(text, "zero").rfind("true", 0) == 0;
  m.model = raw_value(text, "model");
  return m;
}

void save_training_state(const Scheduler &scheduler, const std::string &dir, const module::Module &model,
                         const module::OptimizerModule *optimizer, const Meta &meta, int64_t rank, int64_t writer_rank) {
  // Every rank drains its queues (parameters and moments settle); one rank writes. The meta file
  // goes last and atomically, so a directory with a meta file is complete.
  scheduler.impl()->synchronize();
  if (rank != writer_rank) return;
  make_dir(dir);
  cs::save(model, dir + "/model.parquet");
  if (optimizer) cs::save(*optimizer, dir + "/optimizer.parquet");
  save_meta(meta, dir + "/meta.json");
}

Meta load_training_state(const Scheduler &scheduler, const std::string &dir, const module::Module &model,
                         module::OptimizerModule *optimizer) {
  scheduler.impl()->synchronize();
  const Meta meta = load_meta(dir + "/meta.json");
  cs::load(model, dir + "/model.parquet");
  if (optimizer) cs::load(*optimizer, dir + "/optimizer.parquet");
  return meta;
}
}  // namespace cs::checkpoint
