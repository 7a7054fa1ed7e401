"""Tokenise a text corpus into the Parquet layout the data loader reads.

Counterpart of the reference project's example/dataset/prepare_text_gen.py: every output row holds
`input_ids` (block_size token ids) and `labels` (the same window shifted by one token); rows are
written to `data-XXXXX-of-YYYYY.parquet` shards under <out>/{train,validation}.

Offline-friendly: the tokenizer is a local Hugging Face tokenizer directory/name when available
(`--tokenizer`), else a byte-level fallback (ids 0..255) so the pipeline can be exercised
without network access.

  python examples/prepare_text_gen.py --input corpus.txt --out data/ --block-size 1024
"""
from __future__ import annotations

import argparse
import os

import numpy as np
import pyarrow as pa
import pyarrow.parquet as pq


def load_tokenizer(name):
    if name:
        try:
            from transformers import AutoTokenizer

            tok = AutoTokenizer.from_pretrained(name, local_files_only=True)
            return lambda text: tok(text)["input_ids"], (tok.eos_token_id if tok.eos_token_id is not None else 0)
        except Exception as exc:  # noqa: BLE001
            print(f"tokenizer {name!r} unavailable ({exc}); using the byte-level fallback")
    return lambda text: list(text.encode("utf-8")), 0


def chunk(tokens: np.ndarray, block: int):
    """Windows of block+1 tokens -> (input_ids, labels) with labels = next token."""
    n = (len(tokens) - 1) // block
    ids = np.stack([tokens[i * block:(i + 1) * block] for i in range(n)]) if n else np.zeros((0, block), np.int32)
    lab = np.stack([tokens[i * block + 1:(i + 1) * block + 1] for i in range(n)]) if n else np.zeros((0, block), np.int32)
    return ids, lab


def write_shards(ids, lab, out_dir, rows_per_shard):
    os.makedirs(out_dir, exist_ok=True)
    shards = max(1, (len(ids) + rows_per_shard - 1) // rows_per_shard)
    for s in range(shards):
        a, b = s * rows_per_shard, min(len(ids), (s + 1) * rows_per_shard)
        table = pa.table({
            "input_ids": pa.array(ids[a:b].tolist(), type=pa.list_(pa.int32())),
            "labels": pa.array(lab[a:b].tolist(), type=pa.list_(pa.int32())),
        })
        pq.write_table(table, os.path.join(out_dir, f"data-{s:05d}-of-{shards:05d}.parquet"))
    return shards


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--input", required=True, help="UTF-8 text file; documents separated by blank lines")
    p.add_argument("--out", required=True)
    p.add_argument("--block-size", type=int, default=1024)
    p.add_argument("--tokenizer", default="openai-community/gpt2")
    p.add_argument("--validation-fraction", type=float, default=0.01)
    p.add_argument("--rows-per-shard", type=int, default=100_000)
    args = p.parse_args()
    encode, eos = load_tokenizer(args.tokenizer)
    tokens = []
    with open(args.input, encoding="utf-8") as f:
        for doc in f.read().split("\n\n"):
            if doc.strip():
                tokens.extend(encode(doc)[: 1 << 30])
                tokens.append(eos)
    tokens = np.asarray(tokens, dtype=np.int32)
    ids, lab = chunk(tokens, args.block_size)
    n_val = max(1, int(len(ids) * args.validation_fraction)) if len(ids) > 1 else 0
    for split, sl in (("train", slice(0, len(ids) - n_val)), ("validation", slice(len(ids) - n_val, len(ids)))):
        if sl.stop - sl.start > 0:
            shards = write_shards(ids[sl], lab[sl], os.path.join(args.out, split), args.rows_per_shard)
            print(f"{split}: {sl.stop - sl.start} rows in {shards} shard(s)")


if __name__ == "__main__":
    main()
