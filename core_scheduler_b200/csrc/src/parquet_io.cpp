// SPDX-License-Identifier: Apache-2.0
// Arrow/Parquet glue. Checkpoint layout parity: src/module/module.cpp:129-220 of the reference
// project (key: utf8, value: list<float32>, one row per parameter); token files parity:
// src/data/dataloader.cpp:118-205 (list columns input_ids / labels, int32 or int64 items).
#include "parquet_io.h"

#include <arrow/api.h>
#include <arrow/io/api.h>
#include <parquet/arrow/reader.h>
#include <parquet/arrow/writer.h>
#include <parquet/file_reader.h>

#include <stdexcept>

namespace cs::io {
namespace {
void check(const arrow::Status &st, const char *what) {
  if (!st.ok()) throw std::runtime_error(std::string(what) + ": " + st.ToString());
}
template <typename T>
T take(arrow::Result<T> r, const char *what) {
  if (!r.ok()) throw std::runtime_error(std::string(what) + ": " + r.status().ToString());
  return std::move(r).ValueUnsafe();
}
}  // namespace

void write_float_list_table(const std::string &path, const std::vector<std::string> &keys,
                            const std::vector<const float *> &data, const std::vector<int64_t> &lengths) {
  auto *pool = arrow::default_memory_pool();
  arrow::StringBuilder key_builder(pool);
  auto value_builder = std::make_shared<arrow::FloatBuilder>(pool);
  arrow::ListBuilder list_builder(pool, value_builder);
  for (size_t i = 0; i < keys.size(); ++i) {
    check(key_builder.Append(keys[i]), "append key");
    check(list_builder.Append(), "open list");
    check(value_builder->AppendValues(data[i], lengths[i]), "append values");  // bulk copy, no per-element loop
  }
  std::shared_ptr<arrow::Array> key_array, value_array;
  check(key_builder.Finish(&key_array), "finish keys");
  check(list_builder.Finish(&value_array), "finish values");
  auto schema = arrow::schema({arrow::field("key", arrow::utf8()), arrow::field("value", arrow::list(arrow::float32()))});
  auto table = arrow::Table::Make(schema, {key_array, value_array});
  auto sink = take(arrow::io::FileOutputStream::Open(path), "open output file");
  const int64_t rows = std::max<int64_t>(1, static_cast<int64_t>(keys.size()));
  check(parquet::arrow::WriteTable(*table, pool, sink, rows), "write parquet table");
  check(sink->Close(), "close output file");
}

FloatListTable read_float_list_table(const std::string &path) {
  auto input = take(arrow::io::ReadableFile::Open(path), "open checkpoint");
  auto reader = take(parquet::arrow::OpenFile(input, arrow::default_memory_pool()), "open parquet reader");
  std::shared_ptr<arrow::Table> table = take(reader->ReadTable(), "read table");
  if (table->num_columns() < 2) throw std::runtime_error("checkpoint needs the columns key and value");
  FloatListTable out;
  auto key_col = table->column(0);
  auto val_col = table->column(1);
  for (int c = 0; c < key_col->num_chunks(); ++c) {
    auto chunk = key_col->chunk(c);
    if (chunk->type_id() == arrow::Type::STRING) {
      auto keys = std::static_pointer_cast<arrow::StringArray>(chunk);
      for (int64_t i = 0; i < keys->length(); ++i) out.keys.push_back(keys->GetString(i));
    } else if (chunk->type_id() == arrow::Type::LARGE_STRING) {
      auto keys = std::static_pointer_cast<arrow::LargeStringArray>(chunk);
      for (int64_t i = 0; i < keys->length(); ++i) out.keys.push_back(keys->GetString(i));
    } else {
      throw std::runtime_error("checkpoint column `key` must hold strings");
    }
  }
  for (int c = 0; c < val_col->num_chunks(); ++c) {
    auto lists = std::dynamic_pointer_cast<arrow::ListArray>(val_col->chunk(c));
    if (!lists) throw std::runtime_error("checkpoint column `value` must be a list column");
    auto values = lists->values();
    for (int64_t i = 0; i < lists->length(); ++i) {
      const int64_t begin = lists->value_offset(i), len = lists->value_length(i);
      if (values->type_id() == arrow::Type::FLOAT) {
        const float *p = std::static_pointer_cast<arrow::FloatArray>(values)->raw_values() + begin;
        out.values.emplace_back(p, p + len);
      } else if (values->type_id() == arrow::Type::DOUBLE) {
        const double *p = std::static_pointer_cast<arrow::DoubleArray>(values)->raw_values() + begin;
        out.values.emplace_back(p, p + len);
      } else {
        throw std::runtime_error("checkpoint values must be float32 (or float64) lists");
      }
    }
  }
  if (out.keys.size() != out.values.size()) throw std::runtime_error("checkpoint columns have different lengths");
  return out;
}

int64_t parquet_row_count(const std::string &path) {
  auto reader = parquet::ParquetFileReader::OpenFile(path, false);
  return reader->metadata()->num_rows();
}

struct TokenFileReader::Impl {
  std::unique_ptr<parquet::arrow::FileReader> reader;
  std::shared_ptr<arrow::RecordBatchReader> batches;
  std::shared_ptr<arrow::RecordBatch> current;
  int64_t cursor{0};  // row inside `current`
  int64_t total_rows{0};
  int64_t batch_rows{0};
  bool pull() {
    current.reset();
    cursor = 0;
    check(batches->ReadNext(&current), "read record batch");
    return current != nullptr && current->num_rows() > 0;
  }
};

namespace {
void widen_rows(const std::shared_ptr<arrow::Array> &column, int64_t first, int64_t count, int64_t *dst, int64_t *cols) {
  auto lists = std::dynamic_pointer_cast<arrow::ListArray>(column);
  if (!lists) throw std::runtime_error("token columns must be list arrays");
  auto values = lists->values();
  for (int64_t r = 0; r < count; ++r) {
    const int64_t begin = lists->value_offset(first + r), len = lists->value_length(first + r);
    if (*cols < 0) *cols = len;
    if (len != *cols) throw std::runtime_error("token rows must all have the same length");
    int64_t *out = dst + r * len;
    if (values->type_id() == arrow::Type::INT32) {
      const int32_t *p = std::static_pointer_cast<arrow::Int32Array>(values)->raw_values() + begin;
      for (int64_t k = 0; k < len; ++k) out[k] = p[k];
    } else if (values->type_id() == arrow::Type::INT64) {
      const int64_t *p = std::static_pointer_cast<arrow::Int64Array>(values)->raw_values() + begin;
      std::copy(p, p + len, out);
    } else {
      throw std::runtime_error("token items must be int32 or int64");
    }
  }
}
}  // namespace

TokenFileReader::TokenFileReader(const std::string &path, int64_t batch_rows) : impl_{std::make_unique<Impl>()} {
  auto input = take(arrow::io::ReadableFile::Open(path), "open token file");
  parquet::ArrowReaderProperties props;
  props.set_batch_size(batch_rows);
  parquet::arrow::FileReaderBuilder builder;
  check(builder.Open(input), "open parquet file");
  builder.properties(props);
  impl_->reader = take(builder.Build(), "build parquet reader");
  impl_->total_rows = impl_->reader->parquet_reader()->metadata()->num_rows();
  impl_->batch_rows = batch_rows;
  std::shared_ptr<arrow::Schema> schema;
  check(impl_->reader->GetSchema(&schema), "read schema");
  const int ids = schema->GetFieldIndex("input_ids"), labels = schema->GetFieldIndex("labels");
  if (ids < 0 || labels < 0) throw std::runtime_error("token file needs the columns input_ids and labels");
  std::vector<int> row_groups(impl_->reader->num_row_groups());
  for (size_t i = 0; i < row_groups.size(); ++i) row_groups[i] = static_cast<int>(i);
  impl_->batches = take(impl_->reader->GetRecordBatchReader(row_groups, {ids, labels}), "open batch reader");
}
TokenFileReader::~TokenFileReader() = default;
int64_t TokenFileReader::rows() const { return impl_->total_rows; }

void TokenFileReader::skip_rows(int64_t rows) {
  while (rows > 0) {
    if (!impl_->current || impl_->cursor >= impl_->current->num_rows()) {
      if (!impl_->pull()) return;
    }
    const int64_t step = std::min<int64_t>(rows, impl_->current->num_rows() - impl_->cursor);
    impl_->cursor += step;
    rows -= step;
  }
}

int64_t TokenFileReader::row_width() {
  if (!impl_->current || impl_->cursor >= impl_->current->num_rows()) {
    if (!impl_->pull()) return -1;
  }
  auto lists = std::dynamic_pointer_cast<arrow::ListArray>(impl_->current->GetColumnByName("input_ids"));
  if (!lists) throw std::runtime_error("token columns must be list arrays");
  return lists->value_length(impl_->cursor);
}

int64_t TokenFileReader::next(int64_t *input_ids, int64_t *labels, int64_t capacity_rows, int64_t *cols) {
  int64_t done = 0;
  int64_t width = *cols > 0 ? *cols : -1;
  while (done < capacity_rows) {
    if (!impl_->current || impl_->cursor >= impl_->current->num_rows()) {
      if (!impl_->pull()) break;
    }
    const int64_t take_rows = std::min<int64_t>(capacity_rows - done, impl_->current->num_rows() - impl_->cursor);
    auto ids = impl_->current->GetColumnByName("input_ids");
    auto lab = impl_->current->GetColumnByName("labels");
    int64_t w = width;
    widen_rows(ids, impl_->cursor, take_rows, input_ids + done * (width > 0 ? width : 0), &w);
    if (width < 0) {
      // first rows fixed the width; redo with the right stride if this was not the first row block
      width = w;
      widen_rows(ids, impl_->cursor, take_rows, input_ids + done * width, &w);
    }
    widen_rows(lab, impl_->cursor, take_rows, labels + done * width, &w);
    impl_->cursor += take_rows;
    done += take_rows;
  }
  *cols = width;
  return done;
}
}  // namespace cs::io
