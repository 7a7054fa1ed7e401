// SPDX-License-Identifier: Apache-2.0
// Force-included (-include) when compiling the reference project's src/module/module.cpp and
// src/data/dataloader.cpp against Arrow 24: the sources are not touched. Arrow dropped the
// three-argument parquet::arrow::OpenFile(file, pool, &reader) that module.cpp calls, and
// dataloader.cpp relies on arrow::RecordBatch being complete through a transitive include that
// is gone.
#pragma once
#include <arrow/api.h>
#include <arrow/io/api.h>
#include <arrow/record_batch.h>
#include <parquet/arrow/reader.h>

namespace parquet::arrow {
inline ::arrow::Status OpenFile(std::shared_ptr<::arrow::io::RandomAccessFile> file, ::arrow::MemoryPool *pool,
                                std::unique_ptr<FileReader> *reader) {
  auto result = OpenFile(std::move(file), pool);
  if (!result.ok()) return result.status();
  *reader = std::move(result).ValueUnsafe();
  return ::arrow::Status::OK();
}
}  // namespace parquet::arrow
