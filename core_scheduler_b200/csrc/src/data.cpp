// SPDX-License-Identifier: Apache-2.0
// Dataset listing and threaded loaders. See cs/data.h for the parity map.
#include "cs/data.h"

#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <condition_variable>
#include <filesystem>
#include <mutex>
#include <random>
#include <thread>

#include "parquet_io.h"

namespace cs::data {
// ----------------------------------------------------------------------------- dataset ----
struct LlmDataset::Impl {
  std::vector<std::string> files;
  std::vector<int64_t> offsets;  // offsets[i] = rows before file i; back() = total
};

LlmDataset::LlmDataset(const std::string &directory) : impl_{std::make_shared<Impl>()} {
  namespace fs = std::filesystem;
  CS_ASSERT_TRUE(fs::is_directory(directory), "dataset directory `", directory, "` does not exist");
  for (auto &entry : fs::directory_iterator(directory)) {
    if (entry.is_regular_file() && entry.path().extension() == ".parquet") impl_->files.push_back(entry.path().string());
  }
  CS_ASSERT_TRUE(!impl_->files.empty(), "no .parquet files in `", directory, "`");
  std::sort(impl_->files.begin(), impl_->files.end());
  impl_->offsets.push_back(0);
  for (auto &f : impl_->files) impl_->offsets.push_back(impl_->offsets.back() + io::parquet_row_count(f));
}
int64_t LlmDataset::size() const { return impl_->offsets.back(); }
const std::vector<std::string> &LlmDataset::files() const { return impl_->files; }
const std::vector<int64_t> &LlmDataset::file_offsets() const { return impl_->offsets; }

// ------------------------------------------------------------------- pinned staging ----
namespace {
struct HostBuffer {
  int64_t *ptr{nullptr};
  int64_t capacity{0};  // elements
  bool pinned{false};
  void ensure(int64_t elements, bool want_pinned) {
    if (elements <= capacity) return;
    free_now();
    if (want_pinned && cudaMallocHost(reinterpret_cast<void **>(&ptr), elements * sizeof(int64_t)) == cudaSuccess) {
      pinned = true;
    } else {
      (void)cudaGetLastError();
      ptr = static_cast<int64_t *>(std::malloc(elements * sizeof(int64_t)));
      pinned = false;
    }
    CS_ASSERT_TRUE(ptr != nullptr, "host staging allocation failed");
    capacity = elements;
  }
  void free_now() {
    if (!ptr) return;
    if (pinned) {
      cudaFreeHost(ptr);
    } else {
      std::free(ptr);
    }
    ptr = nullptr;
    capacity = 0;
  }
  ~HostBuffer() { free_now(); }
};

bool cuda_present() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  return n > 0;
}

// One producer thread, two slots. The producer fills a slot when it is free and the
// host-to-device copy that last used it has finished; the consumer takes slots in order.
struct Slot {
  HostBuffer ids, labels;
  int64_t rows{0}, cols{0};
  bool ready{false};
  Event copied;  // completion of the H2D copy that read this slot
};

struct Producer {
  std::mutex mu;
  std::condition_variable cv;
  Slot slots[2];
  int fill{0}, take{0};
  bool stop{false};
  std::string error;
  std::thread thread;
  int device{-1};  // CUDA device of the thread that created the loader (-1: none); the worker selects it

  // `make(slot)` fills ids/labels/rows/cols; returns false when it failed (error set).
  template <typename Make>
  void start(Make make) {
    if (cuda_present() && cudaGetDevice(&device) != cudaSuccess) {
      (void)cudaGetLastError();
      device = -1;
    }
    thread = std::thread([this, make] {
      // Pinned allocations and event waits of this thread belong to the creating rank's device;
      // without this every rank's worker would open a context on device 0.
      if (device >= 0 && cudaSetDevice(device) != cudaSuccess) (void)cudaGetLastError();
      for (;;) {
        Slot *slot;
        {
          std::unique_lock<std::mutex> lock{mu};
          cv.wait(lock, [&] { return stop || !slots[fill].ready; });
          if (stop) return;
          slot = &slots[fill];
        }
        slot->copied.synchronize();  // the device must be done reading this pinned buffer
        try {
          make(*slot);
        } catch (const std::exception &e) {
          std::lock_guard<std::mutex> lock{mu};
          error = e.what();
          slot->ready = true;
          cv.notify_all();
          return;
        }
        {
          std::lock_guard<std::mutex> lock{mu};
          slot->ready = true;
          fill ^= 1;
        }
        cv.notify_all();
      }
    });
  }

  Slot &acquire() {
    std::unique_lock<std::mutex> lock{mu};
    cv.wait(lock, [&] { return slots[take].ready || !error.empty(); });
    CS_ASSERT_TRUE(error.empty(), "data worker failed: ", error);
    return slots[take];
  }
  void release() {
    {
      std::lock_guard<std::mutex> lock{mu};
      slots[take].ready = false;
      take ^= 1;
    }
    cv.notify_all();
  }
  ~Producer() {
    {
      std::lock_guard<std::mutex> lock{mu};
      stop = true;
    }
    cv.notify_all();
    if (thread.joinable()) thread.join();
  }
};

// Copies a ready slot to the device inside a main-stream loader task.
std::unordered_map<std::string, Tensor> upload(const Scheduler &scheduler, Producer &producer, const char *name) {
  Slot &slot = producer.acquire();
  Tensor ids, labels;
  submit(scheduler, name, Task::Impl::kMain, Task::Impl::kLoader, {ids, labels}, {},
         [&slot, ids, labels, device = scheduler.device()](const FnTask &) {
           auto opts = at::TensorOptions().dtype(at::kLong).device(device);
           at::Tensor a = at::empty({slot.rows, slot.cols}, opts);
           at::Tensor b = at::empty({slot.rows, slot.cols}, opts);
           const size_t bytes = static_cast<size_t>(slot.rows * slot.cols) * sizeof(int64_t);
           if (device.is_cuda()) {
             auto stream = c10::cuda::getCurrentCUDAStream().stream();
             CS_CHECK_CUDART(cudaMemcpyAsync(a.data_ptr(), slot.ids.ptr, bytes, cudaMemcpyHostToDevice, stream));
             CS_CHECK_CUDART(cudaMemcpyAsync(b.data_ptr(), slot.labels.ptr, bytes, cudaMemcpyHostToDevice, stream));
             slot.copied.record();
           } else {
             std::memcpy(a.data_ptr(), slot.ids.ptr, bytes);
             std::memcpy(b.data_ptr(), slot.labels.ptr, bytes);
           }
           ids.impl()->tensor = a;
           labels.impl()->tensor = b;
         });
  producer.release();
  return {{"input_ids", ids}, {"labels", labels}};
}
}  // namespace

// ------------------------------------------------------------------------- data loader ----
struct LlmDataLoader::Impl {
  LlmDataset dataset;
  int64_t batch{0};
  int64_t rank{0}, world{1};
  int64_t iterations{0};
  std::vector<std::unique_ptr<Producer>> workers;
  mutable size_t next_worker{0};
  Impl(const LlmDataset &d) : dataset{d} {}
};

namespace {
// Streams rows [begin, begin + rows) of the dataset forever (wrapping), in batches.
struct RowStream {
  const LlmDataset::Impl *ds;
  int64_t begin, rows, batch;
  int64_t produced{0};
  size_t file{0};
  std::unique_ptr<io::TokenFileReader> reader;
  int64_t cols{-1};

  void open_at(int64_t row) {
    file = static_cast<size_t>(std::upper_bound(ds->offsets.begin(), ds->offsets.end(), row) - ds->offsets.begin()) - 1;
    reader = std::make_unique<io::TokenFileReader>(ds->files[file], batch);
    reader->skip_rows(row - ds->offsets[file]);
  }
  void fill(Slot &slot, bool pinned) {
    const int64_t usable = rows / batch * batch;  // whole batches only
    if (produced >= usable) {                     // wrap around: next epoch
      produced = 0;
      reader.reset();
    }
    if (!reader) open_at(begin + produced);
    int64_t done = 0;
    int64_t width = cols;
    while (done < batch) {
      // The staging buffers are sized from the row length, which the first row of the stream fixes.
      if (width <= 0) width = reader->row_width();
      int64_t got = 0;
      if (width > 0) {
        slot.ids.ensure(batch * width, pinned);
        slot.labels.ensure(batch * width, pinned);
        int64_t w = width;
        got = reader->next(slot.ids.ptr + done * width, slot.labels.ptr + done * width, batch - done, &w);
      }
      if (got == 0) {  // end of file: continue in the next one
        ++file;
        CS_ASSERT_TRUE(file < ds->files.size(), "ran past the last dataset file");
        reader = std::make_unique<io::TokenFileReader>(ds->files[file], batch);
        continue;
      }
      done += got;
    }
    cols = width;
    slot.rows = batch;
    slot.cols = width;
    produced += batch;
  }
};
}  // namespace

namespace {
std::shared_ptr<LlmDataLoader::Impl> make_loader(const LlmDataset &dataset, int64_t rank, int64_t world, int64_t batch,
                                                 int64_t workers, bool shuffle) {
  CS_ASSERT_TRUE(!shuffle, "shuffling is not supported");
  CS_ASSERT_TRUE(batch > 0 && workers > 0, "batch size and worker count must be positive");
  auto impl = std::make_shared<LlmDataLoader::Impl>(dataset);
  impl->batch = batch;
  impl->rank = rank;
  impl->world = world;
  const int64_t rows = dataset.size();
  const int64_t per_rank = rows / world;
  const int64_t per_worker = per_rank / workers;
  CS_ASSERT_TRUE(per_worker >= batch, "each worker needs at least one batch of rows (", per_worker, " < ", batch, ")");
  impl->iterations = rows / (batch * world);
  const bool pinned = cuda_present();
  for (int64_t w = 0; w < workers; ++w) {
    auto producer = std::make_unique<Producer>();
    auto stream = std::make_shared<RowStream>();
    stream->ds = dataset.impl().get();
    stream->begin = per_rank * rank + w * per_worker;
    stream->rows = per_worker;
    stream->batch = batch;
    producer->start([stream, pinned, keep = dataset.impl()](Slot &slot) { stream->fill(slot, pinned); });
    impl->workers.push_back(std::move(producer));
  }
  return impl;
}
}  // namespace

LlmDataLoader::LlmDataLoader(const LlmDataset &dataset, int64_t batchSize, int64_t numWorkers, bool shuffle)
    : impl_{make_loader(dataset, 0, 1, batchSize, numWorkers, shuffle)} {}
LlmDataLoader::LlmDataLoader(const LlmDataset &dataset, const communication::Comm &comm, int64_t batchSize,
                             int64_t numWorkers, bool shuffle)
    : impl_{make_loader(dataset, comm.get_rank(), comm.get_size(), batchSize, numWorkers, shuffle)} {}

int64_t LlmDataLoader::iterations_per_epoch() const { return impl_->iterations; }

std::unordered_map<std::string, Tensor> LlmDataLoader::load(const Scheduler &scheduler) const {
  Producer &p = *impl_->workers[impl_->next_worker];
  impl_->next_worker = (impl_->next_worker + 1) % impl_->workers.size();
  return upload(scheduler, p, "cs::data::LlmDataLoader::load");
}

// ---------------------------------------------------------------------- synthetic loader ----
struct SyntheticDataLoader::Impl {
  int64_t batch, seq, vocab;
  Producer producer;
};

SyntheticDataLoader::SyntheticDataLoader(int64_t batchSize, int64_t seqLen, int64_t vocab, uint64_t seed)
    : impl_{std::make_shared<Impl>()} {
  impl_->batch = batchSize;
  impl_->seq = seqLen;
  impl_->vocab = vocab;
  const bool pinned = cuda_present();
  auto rng = std::make_shared<std::mt19937_64>(seed);
  impl_->producer.start([rng, batchSize, seqLen, vocab, pinned](Slot &slot) {
    slot.ids.ensure(batchSize * seqLen, pinned);
    slot.labels.ensure(batchSize * seqLen, pinned);
    std::uniform_int_distribution<int64_t> dist(0, vocab - 1);
    for (int64_t b = 0; b < batchSize; ++b) {
      int64_t *ids = slot.ids.ptr + b * seqLen;
      int64_t *lab = slot.labels.ptr + b * seqLen;
      int64_t prev = dist(*rng);
      for (int64_t t = 0; t < seqLen; ++t) {
        ids[t] = prev;
        prev = dist(*rng);
        lab[t] = prev;  // next token
      }
    }
    slot.rows = batchSize;
    slot.cols = seqLen;
  });
}
int64_t SyntheticDataLoader::bytes_per_batch() const { return 2 * impl_->batch * impl_->seq * 8; }
std::unordered_map<std::string, Tensor> SyntheticDataLoader::load(const Scheduler &scheduler) const {
  return upload(scheduler, impl_->producer, "cs::data::SyntheticDataLoader::load");
}
}  // namespace cs::data
