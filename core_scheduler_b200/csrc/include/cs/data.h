// SPDX-License-Identifier: Apache-2.0
// Token datasets and loaders.
//
// Capability parity (reference project paths): include/data/dataset.h:35-41 +
// src/data/dataset.cpp:50-106 (sorted *.parquet listing, per-file row counts, prefix sums);
// include/data/dataloader.h:26-47 + src/data/dataloader.cpp:109-426 (rows split per rank then
// per worker thread, each worker streams its files into pinned host buffers, load() copies a
// batch to the device inside a main-stream task and returns {"input_ids","labels"}).
//
// Differences: each worker owns two pinned buffer pairs, so it decodes the next batch while
// the previous host-to-device copy is still in flight; a synthetic loader (uniform random
// token ids, labels shifted by one) goes through the same pinned staging path.
#pragma once
#include <string>
#include <unordered_map>

#include "cs/communication.h"
#include "cs/core.h"

namespace cs::data {
struct CS_API LlmDataset {
  struct Impl;
  explicit LlmDataset(const std::string &directory);
  [[nodiscard]] int64_t size() const;
  [[nodiscard]] const std::vector<std::string> &files() const;
  [[nodiscard]] const std::vector<int64_t> &file_offsets() const;  // prefix sums, size = files + 1
  [[nodiscard]] const std::shared_ptr<Impl> &impl() const { return impl_; }

 private:
  std::shared_ptr<Impl> impl_;
};

struct CS_API LlmDataLoader {
  struct Impl;
  LlmDataLoader(const LlmDataset &dataset, int64_t batchSize, int64_t numWorkers, bool shuffle);
  LlmDataLoader(const LlmDataset &dataset, const communication::Comm &comm, int64_t batchSize, int64_t numWorkers,
                bool shuffle);
  // Returns device tensors [batch, seq] (int64) for "input_ids" and "labels".
  [[nodiscard]] std::unordered_map<std::string, Tensor> load(const Scheduler &scheduler) const;
  [[nodiscard]] int64_t iterations_per_epoch() const;

 private:
  std::shared_ptr<Impl> impl_;
};

// extension: uniform random token ids in [0, vocab) produced on the host into pinned double
// buffers by a worker thread; labels are the inputs shifted by one position.
struct CS_API SyntheticDataLoader {
  struct Impl;
  SyntheticDataLoader(int64_t batchSize, int64_t seqLen, int64_t vocab, uint64_t seed);
  [[nodiscard]] std::unordered_map<std::string, Tensor> load(const Scheduler &scheduler) const;
  [[nodiscard]] int64_t bytes_per_batch() const;

 private:
  std::shared_ptr<Impl> impl_;
};
}  // namespace cs::data
