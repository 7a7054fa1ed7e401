// SPDX-License-Identifier: Apache-2.0
// Narrow Parquet interface (the only translation unit that includes Arrow headers is
// parquet_io.cpp). Used by checkpoints and by the token dataset.
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

namespace cs::io {
struct FloatListTable {
  std::vector<std::string> keys;
  std::vector<std::vector<float>> values;
};
// Columns: key (utf8), value (list<item: float32>), one row per entry, a single row group.
void write_float_list_table(const std::string &path, const std::vector<std::string> &keys,
                            const std::vector<const float *> &data, const std::vector<int64_t> &lengths);
FloatListTable read_float_list_table(const std::string &path);

int64_t parquet_row_count(const std::string &path);

// Sequential reader of the `input_ids` / `labels` list columns (int32 or int64 items) of one
// Parquet file. next() widens one batch of rows into the two int64 buffers.
class TokenFileReader {
 public:
  TokenFileReader(const std::string &path, int64_t batch_rows);
  ~TokenFileReader();
  // Skips `rows` rows from the current position.
  void skip_rows(int64_t rows);
  // Reads up to batch_rows rows; returns the number of rows read (0 at end of file). `cols`
  // receives the row length; every row must have that many items.
  int64_t next(int64_t *input_ids, int64_t *labels, int64_t capacity_rows, int64_t *cols);
  [[nodiscard]] int64_t rows() const;
  // Length of the row at the current position (-1 at end of file); reads ahead, consumes nothing.
  int64_t row_width();

 private:
  struct Impl;
  std::unique_ptr<Impl> impl_;
};
}  // namespace cs::io
