# SPDX-License-Identifier: Apache-2.0
"""Tokenise text corpora into the Parquet layout the data loader reads.

Counterpart of the reference project's example/dataset/prepare_text_gen.py (lines 24-66 configuration, 95-110 windowing,
115-180 sharding, 182-322 split handling). Same behaviour, driven by a JSON description or command-line flags instead of
an edited dictionary:

* several sources are tokenised, grouped, concatenated and shuffled together;
* a source is a local file (.txt with blank-line separated documents, .jsonl or .parquet with a text column) or, when
  the `datasets` package and the data are available locally, a Hugging Face dataset name;
* per source: split names for train / validation / test, a text column, a sampling rate, and a split ratio that carves
  the validation set out of the training set when the source has none; the test set falls back to the validation set;
* every document is tokenised and truncated to `block_size` tokens, the token streams of a split are concatenated, and
  every window of `block_size` tokens becomes one row `input_ids`, with `labels` the same window shifted by one token
  (the tail that does not fill a window is dropped);
* each split is written to `<out>/<split>/data-XXXXX-of-YYYYY.parquet`, the number of shards chosen from a byte budget
  per shard (default 1 GiB) or given directly, the shards written by a pool of processes.

The tokenizer is a local Hugging Face tokenizer (`--tokenizer`, no network access is attempted) or, when that is not
available, a byte-level stand-in (ids 0..255, end of text = 0) so that the pipeline can be exercised anywhere.

  python examples/prepare_text_gen.py --out data/ --source corpus.txt --block-size 1024
  python examples/prepare_text_gen.py --out data/ --config sources.json

sources.json:
  {"block_size": 1024, "tokenizer": "openai-community/gpt2", "seed": 42, "max_shard_size": 1073741824,
   "sources": [{"path": "a.jsonl", "text_column": "text", "split_ratio": 0.01, "sampling_rate": 1.0},
               {"path": "HuggingFaceFW/fineweb-edu", "name": "sample-10BT", "train": "train", "validation": null,
                "test": null, "text_column": "text", "split_ratio": 0.001}]}
"""
from __future__ import annotations

import argparse
import json
import os
import random
from multiprocessing import Pool, cpu_count

import numpy as np
import pyarrow as pa
import pyarrow.parquet as pq

SPLITS = ("train", "validation", "test")


def load_tokenizer(name):
    """(encode(text) -> list of ids, end-of-text id)."""
    if name:
        try:
            from transformers import AutoTokenizer

            tok = AutoTokenizer.from_pretrained(name, local_files_only=True, use_fast=True)
            eos = tok.eos_token_id if tok.eos_token_id is not None else 0
            return (lambda text: tok(text)["input_ids"]), eos
        except Exception as exc:  # noqa: BLE001
            print(f"tokenizer {name!r} unavailable ({type(exc).__name__}); using the byte-level stand-in")
    return (lambda text: list(text.encode("utf-8"))), 0


def read_local(path, text_column):
    """Documents of one local file."""
    if path.endswith(".jsonl") or path.endswith(".json"):
        with open(path, encoding="utf-8") as f:
            return [json.loads(line)[text_column] for line in f if line.strip()]
    if path.endswith(".parquet"):
        return pq.read_table(path, columns=[text_column]).column(text_column).to_pylist()
    with open(path, encoding="utf-8") as f:
        return [doc for doc in f.read().split("\n\n") if doc.strip()]


def load_source(spec):
    """{'train': [docs], 'validation': [docs] or None, 'test': [docs] or None} of one source, before sampling."""
    column = spec.get("text_column", "text")
    path = spec["path"]
    if os.path.exists(path):
        if os.path.isdir(path):  # <dir>/<split>.{txt,jsonl,parquet}
            out = {}
            for split in SPLITS:
                name = spec.get(split, split)
                found = [os.path.join(path, f) for f in sorted(os.listdir(path)) if name and os.path.splitext(f)[0] == name]
                out[split] = read_local(found[0], column) if found else None
            if out["train"] is None:
                raise ValueError(f"{path} has no file for the training split")
            return out
        return {"train": read_local(path, column), "validation": None, "test": None}
    try:
        from datasets import load_dataset
    except ImportError as exc:
        raise FileNotFoundError(f"{path} is not a local file and the `datasets` package is not installed") from exc
    data = load_dataset(path=path, name=spec.get("name"))
    train_name = spec.get("train", "train")
    if train_name is None:
        raise ValueError("a source needs a training split")
    out = {"train": list(data[train_name][column])}
    for split in ("validation", "test"):
        name = spec.get(split)
        out[split] = list(data[name][column]) if name else None
    return out


def split_source(docs, spec, rng):
    """Sampling and the train / validation / test rules of the reference script."""
    train = list(docs["train"])
    rng.shuffle(train)
    train = train[: int(len(train) * float(spec.get("sampling_rate", 1.0)))]
    validation = docs["validation"]
    if validation is None:
        ratio = spec.get("split_ratio")
        if ratio is not None:
            cut = int(len(train) * float(ratio))
            validation, train = train[:cut], train[cut:]
    test = docs["test"] if docs["test"] is not None else validation
    return {"train": train, "validation": validation, "test": test}


def windows(documents, encode, block):
    """Token windows of `block` ids and the same windows shifted by one token."""
    stream = []
    for doc in documents:
        stream.extend(encode(doc)[:block])  # truncation per document, as the reference tokenises
    total = len(stream)
    if total <= block:
        return np.zeros((0, block), np.int32), np.zeros((0, block), np.int32)
    total = (total - 1) // block * block
    tokens = np.asarray(stream[: total + 1], dtype=np.int32)
    return tokens[:total].reshape(-1, block), tokens[1:total + 1].reshape(-1, block)


def _write_shard(job):
    path, ids, labels = job
    block = ids.shape[1]
    offsets = pa.array(np.arange(len(ids) + 1, dtype=np.int32) * block)
    table = pa.table({"input_ids": pa.ListArray.from_arrays(offsets, pa.array(ids.reshape(-1))),
                      "labels": pa.ListArray.from_arrays(offsets, pa.array(labels.reshape(-1)))})
    pq.write_table(table, path)
    return path


def write_split(ids, labels, out_dir, max_shard_size, num_shards, num_proc):
    """Shard count from the byte budget (rows are 2 * block int32 values), or as given; at least one."""
    os.makedirs(out_dir, exist_ok=True)
    rows = len(ids)
    row_bytes = 2 * ids.shape[1] * 4
    if max_shard_size:
        shards = max(1, (rows * row_bytes + max_shard_size - 1) // max_shard_size)
    else:
        shards = max(1, num_shards or 1)
    per = (rows + shards - 1) // shards
    jobs = [(os.path.join(out_dir, f"data-{s:05d}-of-{shards:05d}.parquet"), ids[s * per:(s + 1) * per], labels[s * per:(s + 1) * per])
            for s in range(shards)]
    workers = max(1, min(num_proc, shards, cpu_count()))
    if workers == 1:
        for job in jobs:
            _write_shard(job)
    else:
        with Pool(workers) as pool:
            pool.map(_write_shard, jobs)
    return shards


def prepare(config):
    rng = random.Random(config.get("seed", 42))
    encode, _ = load_tokenizer(config.get("tokenizer"))
    block = int(config.get("block_size", 1024))
    gathered = {split: [] for split in SPLITS}
    for spec in config["sources"]:
        if isinstance(spec, str):
            spec = {"path": spec}
        spec.setdefault("split_ratio", config.get("split_ratio", 0.01))
        print(f"processing {spec['path']} ...")
        parts = split_source(load_source(spec), spec, rng)
        for split in SPLITS:
            if parts[split]:
                gathered[split].append(windows(parts[split], encode, block))
    report = {}
    for split in SPLITS:
        if not gathered[split]:
            continue
        ids = np.concatenate([g[0] for g in gathered[split]])
        labels = np.concatenate([g[1] for g in gathered[split]])
        if len(ids) == 0:
            continue
        order = np.random.default_rng(config.get("seed", 42)).permutation(len(ids))  # shuffle rows across the sources
        shards = write_split(ids[order], labels[order], os.path.join(config["out"], split), config.get("max_shard_size", 1 << 30),
                             config.get("num_shards"), int(config.get("num_proc", 8)))
        report[split] = (len(ids), shards)
        print(f"{split}: {len(ids)} rows of {block} tokens in {shards} shard(s)")
    return report


def main(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--out", required=True)
    p.add_argument("--config", help="JSON description of the sources (see the module text); flags below override it")
    p.add_argument("--source", action="append", default=[], help="local text / jsonl / parquet file, directory of split files, or dataset name")
    p.add_argument("--text-column", default="text")
    p.add_argument("--block-size", type=int)
    p.add_argument("--tokenizer")
    p.add_argument("--split-ratio", type=float, help="share of the training documents that becomes the validation set")
    p.add_argument("--max-shard-size", type=int, help="bytes per shard (default 1 GiB); 0 = use --num-shards")
    p.add_argument("--num-shards", type=int)
    p.add_argument("--num-proc", type=int)
    p.add_argument("--seed", type=int)
    args = p.parse_args(argv)
    config = {"tokenizer": "openai-community/gpt2", "sources": []}
    if args.config:
        with open(args.config, encoding="utf-8") as f:
            config.update(json.load(f))
    config["out"] = args.out
    config["sources"] = list(config["sources"]) + [{"path": s, "text_column": args.text_column} for s in args.source]
    for key in ("block_size", "tokenizer", "split_ratio", "max_shard_size", "num_shards", "num_proc", "seed"):
        value = getattr(args, key)
        if value is not None:
            config[key] = value
    if not config["sources"]:
        p.error("give at least one --source or a --config with sources")
    prepare(config)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
