# SPDX-License-Identifier: Apache-2.0
"""Checkpoint files outside a training process: reading and writing the parameter table, and uniting the
per-rank files of a tensor-parallel run into the canonical single-model file.

The layout is the reference's (src/module/module.cpp:129-220 in the reference project): one Parquet file, column
`key` (utf8, the dotted parameter path) and column `value` (list<float32>, the parameter flattened), one row per
parameter, no shapes. `cs::load` of either project reads what `write_parameters` writes.

    python -m core_scheduler_b200.utils.checkpoint merge --n-head 20 --n-embd 1280 --out model.parquet \
        ckpt/tp_rank0/model.parquet ckpt/tp_rank1/model.parquet ...
    python -m core_scheduler_b200.utils.checkpoint merge-zero --model ckpt/model.parquet --out ckpt/optimizer.parquet \
        ckpt/zero_rank0/optimizer.parquet ckpt/zero_rank1/optimizer.parquet ...
"""
from __future__ import annotations

import argparse
import sys
from collections import OrderedDict

import numpy as np
import pyarrow as pa
import pyarrow.parquet as pq


def read_parameters(path: str) -> "OrderedDict[str, np.ndarray]":
    """key -> flat float32 array, in file order."""
    table = pq.read_table(path)
    keys = table.column(0).to_pylist()
    values = table.column(1).combine_chunks()
    flat = values.values.to_numpy(zero_copy_only=False).astype(np.float32, copy=False)
    offsets = values.offsets.to_numpy()
    return OrderedDict((k, flat[offsets[i]:offsets[i + 1]]) for i, k in enumerate(keys))


def write_parameters(parameters: "OrderedDict[str, np.ndarray]", path: str) -> None:
    keys = list(parameters)
    arrays = [np.ascontiguousarray(parameters[k], dtype=np.float32).reshape(-1) for k in keys]
    offsets = np.zeros(len(arrays) + 1, dtype=np.int32)
    np.cumsum([a.size for a in arrays], out=offsets[1:])
    values = pa.ListArray.from_arrays(pa.array(offsets), pa.array(np.concatenate(arrays) if arrays else np.zeros(0, np.float32)))
    table = pa.table([pa.array(keys, type=pa.utf8()), values], names=["key", "value"])
    pq.write_table(table, path, row_group_size=max(1, len(keys)))


def head_range(n_head: int, rank: int, world: int):
    """Heads that tensor-parallel rank `rank` owns: the first n_head % world ranks own one more."""
    base, extra = divmod(n_head, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def canonical_key(key: str) -> str:
    """Parameter path of the unsharded model for a path of the tensor-parallel one (its blocks hold the sharded
    Linears directly, the unsharded model nests them in `attn` and `mlp`)."""
    for short, full in ((".c_attn", ".attn.c_attn"), (".c_proj", ".attn.c_proj"), (".fc1", ".mlp.fc1"), (".fc2", ".mlp.fc2")):
        if short in key and full not in key:
            key = key.replace(short, full)
    return key


def merge_tensor_parallel(shards: "list[OrderedDict[str, np.ndarray]]", n_head: int, n_embd: int) -> "OrderedDict[str, np.ndarray]":
    """Unites the parameter tables of all tensor-parallel ranks (in rank order) into the unsharded model's table.

    Column-parallel Linears (c_attn: the q, k and v rows of the rank's heads; fc1: a contiguous block of rows) are
    concatenated along the output dimension, row-parallel ones (c_proj, fc2) along the input dimension; the classifier
    is concatenated along the vocabulary when the ranks hold slices of it; everything else is replicated and taken
    from rank 0."""
    world = len(shards)
    d, head_dim = n_embd, n_embd // n_head
    merged: "OrderedDict[str, np.ndarray]" = OrderedDict()
    for key, first in shards[0].items():
        parts = [s[key] for s in shards]
        heads = [head_range(n_head, r, world) for r in range(world)]
        if key.endswith("c_attn.weight"):
            blocks = [p.reshape(3, h1 - h0, head_dim, d) for p, (h0, h1) in zip(parts, heads)]
            value = np.concatenate(blocks, axis=1)
        elif key.endswith("c_attn.bias"):
            value = np.concatenate([p.reshape(3, h1 - h0, head_dim) for p, (h0, h1) in zip(parts, heads)], axis=1)
        elif key.endswith("c_proj.weight"):
            value = np.concatenate([p.reshape(d, (h1 - h0) * head_dim) for p, (h0, h1) in zip(parts, heads)], axis=1)
        elif key.endswith("fc1.weight"):
            value = np.concatenate([p.reshape(-1, d) for p in parts], axis=0)
        elif key.endswith("fc1.bias"):
            value = np.concatenate(parts)
        elif key.endswith("fc2.weight"):
            value = np.concatenate([p.reshape(d, -1) for p in parts], axis=1)
        elif key == "lm_head.weight" and "wte.weight" in shards[0] and first.size * world == shards[0]["wte.weight"].size:
            # vocabulary-parallel classifier: rank r holds rows [r * V/world, (r + 1) * V/world)
            value = np.concatenate([p.reshape(-1, d) for p in parts], axis=0)
        else:
            value = first
        merged[canonical_key(key)] = np.ascontiguousarray(value, dtype=np.float32).reshape(-1)
    return merged


ZERO_BLOCK = 16384   # parallel::ZeroAdamWImpl::kBlock: block j of the arenas belongs to rank j % world
SLOT_ALIGNMENT = 128  # module::FlatParameters::alignment: every parameter starts at a multiple of this many elements


def merge_zero(shards: "list[OrderedDict[str, np.ndarray]]", model: "OrderedDict[str, np.ndarray]") -> "OrderedDict[str, np.ndarray]":
    """Unites the optimizer shard files of a sharded-optimizer (ZeRO) run into the per-parameter table that the
    replicated AdamW writes and reads (`<parameter>.m`, `<parameter>.v`, `__step__`, `__lr__`), plus `<parameter>.master`
    (the fp32 master weights, identical to the model file's values after `gather_master`).

    `shards` are the ranks' `zero_rank<r>/optimizer.parquet` tables in rank order; `model` is the model file of the same
    step. Its key order and sizes give the arena layout: parameters in order, each starting at the next multiple of
    128 elements. Rank r holds the arena's blocks r, r + world, ... (16384 elements each) back to back."""
    world = len(shards)
    offsets, cursor = OrderedDict(), 0
    for key, value in model.items():
        offsets[key] = (cursor, value.size)
        cursor += (value.size + SLOT_ALIGNMENT - 1) // SLOT_ALIGNMENT * SLOT_ALIGNMENT
    merged: "OrderedDict[str, np.ndarray]" = OrderedDict()
    arenas = {}
    for what in ("m", "v", "master"):
        parts = [s[f"shard{r}.{what}"] for r, s in enumerate(shards)]
        per = parts[0].size // ZERO_BLOCK
        # [world, per, block] -> arena order [per, world, block]
        arenas[what] = np.stack([p.reshape(per, ZERO_BLOCK) for p in parts]).transpose(1, 0, 2).reshape(-1)
        if arenas[what].size < cursor:
            raise ValueError(f"the shards hold {arenas[what].size} values, the model needs {cursor}")
    for key, (begin, size) in offsets.items():
        for what in ("m", "v", "master"):
            merged[f"{key}.{what}"] = arenas[what][begin:begin + size]
    for extra in ("__step__", "__lr__"):
        if extra in shards[0]:
            merged[extra] = shards[0][extra]
    return merged


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = parser.add_subparsers(dest="command", required=True)
    merge = sub.add_parser("merge", help="unite tensor-parallel per-rank parameter files (given in rank order)")
    merge.add_argument("--n-head", type=int, required=True)
    merge.add_argument("--n-embd", type=int, required=True)
    merge.add_argument("--out", required=True)
    merge.add_argument("shards", nargs="+")
    zero = sub.add_parser("merge-zero", help="unite the optimizer shard files of a sharded-optimizer run (given in rank order)")
    zero.add_argument("--model", required=True, help="model file of the same step (gives the parameter order and sizes)")
    zero.add_argument("--out", required=True)
    zero.add_argument("--with-master", action="store_true", help="also keep the `<parameter>.master` rows")
    zero.add_argument("shards", nargs="+")
    show = sub.add_parser("list", help="print the keys and sizes of a parameter file")
    show.add_argument("file")
    args = parser.parse_args(argv)
    if args.command == "merge":
        import re

        ranks = [re.search(r"tp_rank(\d+)", p) for p in args.shards]
        if all(ranks):  # a shell glob lists tp_rank10 before tp_rank2
            args.shards = [p for _, p in sorted(zip((int(m.group(1)) for m in ranks), args.shards))]
        merged = merge_tensor_parallel([read_parameters(p) for p in args.shards], args.n_head, args.n_embd)
        write_parameters(merged, args.out)
        print(f"wrote {len(merged)} parameters, {sum(v.size for v in merged.values())} values to {args.out}")
    elif args.command == "merge-zero":
        import re

        ranks = [re.search(r"zero_rank(\d+)", p) for p in args.shards]
        if all(ranks):
            args.shards = [p for _, p in sorted(zip((int(m.group(1)) for m in ranks), args.shards))]
        merged = merge_zero([read_parameters(p) for p in args.shards], read_parameters(args.model))
        if not args.with_master:
            merged = OrderedDict((k, v) for k, v in merged.items() if not k.endswith(".master"))
        write_parameters(merged, args.out)
        print(f"wrote {len(merged)} rows, {sum(v.size for v in merged.values())} values to {args.out}")
    else:
        for key, value in read_parameters(args.file).items():
            print(f"{value.size:12d}  {key}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
