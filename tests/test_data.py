# SPDX-License-Identifier: Apache-2.0
"""Parquet dataset listing, loader sharding arithmetic, pinned staging and the synthetic loader."""
import os

import numpy as np
import pyarrow as pa
import pyarrow.parquet as pq
import pytest
import torch

import core_scheduler_b200 as cs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

C = cs._C


def write_files(tmp_path, rows_per_file, cols=16, dtype=pa.int32()):
    """Row r of the whole dataset holds input_ids = r*1000 + arange(cols), labels = input_ids + 1."""
    start = 0
    for i, rows in enumerate(rows_per_file):
        ids = [list(range((start + r) * 1000, (start + r) * 1000 + cols)) for r in range(rows)]
        lab = [[v + 1 for v in row] for row in ids]
        table = pa.table({"input_ids": pa.array(ids, type=pa.list_(dtype)), "labels": pa.array(lab, type=pa.list_(dtype))})
        pq.write_table(table, tmp_path / f"data-{i:05d}-of-{len(rows_per_file):05d}.parquet")
        start += rows
    return start


def first_ids(batch):
    return (batch["input_ids"].raw()[:, 0] // 1000).tolist()


def test_dataset_lists_sorted_files_with_prefix_sums(tmp_path):
    total = write_files(tmp_path, [10, 7, 13])
    (tmp_path / "notes.txt").write_text("ignored")
    ds = C.LlmDataset(str(tmp_path))
    assert ds.size() == total == 30
    assert [f.split("/")[-1] for f in ds.files()] == sorted(f.name for f in tmp_path.glob("*.parquet"))
    assert ds.file_offsets() == [0, 10, 17, 30]


def test_loader_single_worker_streams_in_order_across_files_and_wraps(tmp_path, cpu_scheduler):
    write_files(tmp_path, [5, 6, 5])  # 16 rows
    ds = C.LlmDataset(str(tmp_path))
    loader = C.LlmDataLoader(ds, 4, 1, False)
    assert loader.iterations_per_epoch() == 4
    seen = [first_ids(loader.load(cpu_scheduler)) for _ in range(5)]
    assert seen[:4] == [[0, 1, 2, 3], [4, 5, 6, 7], [8, 9, 10, 11], [12, 13, 14, 15]]
    assert seen[4] == [0, 1, 2, 3]  # next epoch
    batch = loader.load(cpu_scheduler)
    ids, lab = batch["input_ids"].raw(), batch["labels"].raw()
    assert ids.dtype == torch.int64 and ids.shape == (4, 16)
    assert torch.equal(lab, ids + 1)


def test_loader_two_workers_round_robin(tmp_path, cpu_scheduler):
    write_files(tmp_path, [8, 8], dtype=pa.int64())  # 16 rows: worker 0 gets rows 0-7, worker 1 rows 8-15
    loader = C.LlmDataLoader(C.LlmDataset(str(tmp_path)), 2, 2, False)
    seen = [first_ids(loader.load(cpu_scheduler)) for _ in range(4)]
    assert seen == [[0, 1], [8, 9], [2, 3], [10, 11]]


def test_loader_rejects_shuffle(tmp_path):
    write_files(tmp_path, [8])
    with pytest.raises(RuntimeError):
        C.LlmDataLoader(C.LlmDataset(str(tmp_path)), 2, 1, True)


def test_synthetic_loader_shapes_and_shift(cpu_scheduler):
    loader = C.SyntheticDataLoader(4, 32, 1000, seed=3)
    assert loader.bytes_per_batch() == 2 * 4 * 32 * 8
    b = loader.load(cpu_scheduler)
    ids, lab = b["input_ids"].raw(), b["labels"].raw()
    assert ids.shape == (4, 32) and ids.min() >= 0 and ids.max() < 1000
    assert torch.equal(lab[:, :-1], ids[:, 1:])  # next-token labels
    b2 = loader.load(cpu_scheduler)
    assert not torch.equal(b2["input_ids"].raw(), ids)


@pytest.mark.gpu
def test_loader_uploads_through_pinned_buffers(tmp_path, gpu_scheduler):
    write_files(tmp_path, [64], cols=128)
    loader = C.LlmDataLoader(C.LlmDataset(str(tmp_path)), 8, 2, False)
    for i in range(6):
        b = loader.load(gpu_scheduler)
        ids = cs.to_torch(gpu_scheduler, b["input_ids"])
        assert ids.is_cuda and ids.shape == (8, 128)
        assert torch.equal(cs.to_torch(gpu_scheduler, b["labels"]), ids + 1)


def test_prepare_text_gen_splits_windows_and_shards(tmp_path):
    """examples/prepare_text_gen.py: two sources (text file with a carved-out validation set, jsonl), windows of
    block_size tokens with labels shifted by one, the test split falling back to validation, shard count from the
    byte budget, and files that LlmDataset / LlmDataLoader read back."""
    import importlib.util
    import json
    import sys

    import pyarrow.parquet as pq

    spec = importlib.util.spec_from_file_location("prepare_text_gen", os.path.join(ROOT, "examples", "prepare_text_gen.py"))
    prep = importlib.util.module_from_spec(spec)
    sys.modules["prepare_text_gen"] = prep  # the shard writers of its process pool are looked up by module name
    spec.loader.exec_module(prep)
    docs = ["".join(chr(97 + (i + j) % 26) for j in range(40 + i % 7)) for i in range(200)]
    (tmp_path / "a.txt").write_text("\n\n".join(docs[:120]))
    with open(tmp_path / "b.jsonl", "w") as f:
        for d in docs[120:]:
            f.write(json.dumps({"body": d}) + "\n")
    config = {"out": str(tmp_path / "out"), "block_size": 16, "tokenizer": None, "seed": 1, "num_proc": 2,
              "max_shard_size": 2 * 16 * 4 * 60,  # 60 rows per shard
              "sources": [{"path": str(tmp_path / "a.txt"), "split_ratio": 0.25},
                          {"path": str(tmp_path / "b.jsonl"), "text_column": "body", "split_ratio": 0.25, "sampling_rate": 0.5}]}
    report = prep.prepare(config)
    assert set(report) == {"train", "validation", "test"}
    rows, shards = report["train"]
    assert shards == (rows * 2 * 16 * 4 + config["max_shard_size"] - 1) // config["max_shard_size"] and shards >= 2
    files = sorted(os.listdir(tmp_path / "out" / "train"))
    assert files[0] == f"data-00000-of-{shards:05d}.parquet" and len(files) == shards
    table = pq.read_table(tmp_path / "out" / "train" / files[0])
    ids, labels = table.column("input_ids").to_pylist(), table.column("labels").to_pylist()
    assert all(len(r) == 16 for r in ids) and all(len(r) == 16 for r in labels)
    assert all(a[1:] == b[:-1] for a, b in zip(ids, labels))  # labels are the window shifted by one token
    assert report["test"] == report["validation"]  # no test split given: the validation set serves
    ds = cs._C.LlmDataset(str(tmp_path / "out" / "train"))
    assert ds.size() == rows
    loader = cs._C.LlmDataLoader(ds, 4, 1, False)
    s = cs.DynamicScheduler(0, device="cpu")
    batch = loader.load(s)
    assert cs.to_torch(s, batch["input_ids"]).shape == (4, 16)
