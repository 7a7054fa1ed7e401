# SPDX-License-Identifier: Apache-2.0
"""core_scheduler_b200.utils.checkpoint: the parameter table outside a training process."""
import subprocess
import sys

from collections import OrderedDict

import numpy as np
import torch

import core_scheduler_b200 as cs
from core_scheduler_b200.utils.checkpoint import canonical_key, head_range, merge_tensor_parallel, read_parameters, write_parameters


def test_parameter_files_interchange_with_the_native_loader(tmp_path, cpu_scheduler):
    s = cpu_scheduler
    cfg = cs.GPT2Config(n_layer=1, n_head=2, n_embd=32, block_size=16, vocab_size=64, padded_vocab_size=64)
    cs.manual_seed(1)
    model = cs.GPT2(s, cfg)
    model.save(str(tmp_path / "native.parquet"))
    table = read_parameters(str(tmp_path / "native.parquet"))
    named = model.named_parameters()
    assert list(table) == list(named)
    for k, v in table.items():
        assert v.dtype == np.float32 and np.array_equal(v, named[k].raw().reshape(-1).numpy())
    # written here, loaded natively into a model with another initialisation
    doubled = type(table)((k, 2 * v) for k, v in table.items())
    write_parameters(doubled, str(tmp_path / "python.parquet"))
    cs.manual_seed(2)
    other = cs.GPT2(s, cfg)
    other.load(str(tmp_path / "python.parquet"))
    for k, p in other.named_parameters().items():
        assert torch.equal(p.raw(), 2 * named[k].raw())
    out = subprocess.run([sys.executable, "-m", "core_scheduler_b200.utils.checkpoint", "list", str(tmp_path / "python.parquet")],
                         capture_output=True, text=True, timeout=120)
    assert out.returncode == 0 and "wte.weight" in out.stdout and str(64 * 32) in out.stdout


def test_merge_inverts_the_tensor_parallel_slicing():
    n_head, d, world = 5, 40, 3  # 5 heads over 3 ranks: 2, 2, 1
    D = d // n_head
    rng = np.random.default_rng(0)
    full = {"0.attn.c_attn.weight": rng.standard_normal((3 * d, d)), "0.attn.c_proj.weight": rng.standard_normal((d, d)),
            "0.mlp.fc1.weight": rng.standard_normal((6 * world, d)), "0.mlp.fc2.weight": rng.standard_normal((d, 6 * world)),
            "0.ln1.weight": rng.standard_normal(d), "wte.weight": rng.standard_normal((16, d))}
    shards = []
    for r in range(world):
        h0, h1 = head_range(n_head, r, world)
        shards.append({
            "0.c_attn.weight": full["0.attn.c_attn.weight"].reshape(3, n_head, D, d)[:, h0:h1].reshape(-1),
            "0.c_proj.weight": full["0.attn.c_proj.weight"][:, h0 * D:h1 * D].reshape(-1),
            "0.fc1.weight": full["0.mlp.fc1.weight"][r * 6:(r + 1) * 6].reshape(-1),
            "0.fc2.weight": full["0.mlp.fc2.weight"][:, r * 6:(r + 1) * 6].reshape(-1),
            "0.ln1.weight": full["0.ln1.weight"], "wte.weight": full["wte.weight"].reshape(-1)})
    assert [head_range(n_head, r, world) for r in range(world)] == [(0, 2), (2, 4), (4, 5)]
    assert canonical_key("3.c_attn.weight") == "3.attn.c_attn.weight" and canonical_key("3.attn.c_attn.weight") == "3.attn.c_attn.weight"
    merged = merge_tensor_parallel(shards, n_head, d)
    assert sorted(merged) == sorted(full)
    for k, v in full.items():
        assert np.allclose(merged[k], v.reshape(-1).astype(np.float32)), k


def test_merge_zero_rebuilds_per_parameter_moments_from_block_interleaved_shards():
    """Rank r of a sharded-optimizer run holds arena blocks r, r + world, ...; the merge puts every parameter's
    moments and master weights back together from the ranks' files and the model file's parameter order."""
    from core_scheduler_b200.utils.checkpoint import SLOT_ALIGNMENT, ZERO_BLOCK, merge_zero

    rng = np.random.default_rng(3)
    sizes = OrderedDict([("a.weight", 40000), ("a.bias", 100), ("b.weight", 3 * ZERO_BLOCK + 17), ("c", 128)])
    model = OrderedDict((k, rng.standard_normal(n).astype(np.float32)) for k, n in sizes.items())
    total = sum((n + SLOT_ALIGNMENT - 1) // SLOT_ALIGNMENT * SLOT_ALIGNMENT for n in sizes.values())
    world = 4
    blocks = (total + ZERO_BLOCK - 1) // ZERO_BLOCK
    per = (blocks + world - 1) // world
    arena = {w: np.zeros(per * world * ZERO_BLOCK, np.float32) for w in ("m", "v", "master")}
    cursor, expect = 0, {}
    for k, n in sizes.items():
        for w in arena:
            values = model[k] if w == "master" else rng.standard_normal(n).astype(np.float32)
            arena[w][cursor:cursor + n] = values
            expect[f"{k}.{w}"] = values
        cursor += (n + SLOT_ALIGNMENT - 1) // SLOT_ALIGNMENT * SLOT_ALIGNMENT
    shards = []
    for r in range(world):
        shard = OrderedDict()
        for w in ("m", "v", "master"):
            shard[f"shard{r}.{w}"] = arena[w].reshape(per, world, ZERO_BLOCK)[:, r].reshape(-1).copy()
        shard["__step__"] = np.asarray([7], np.float32)
        shards.append(shard)
    merged = merge_zero(shards, model)
    for k, v in expect.items():
        assert np.array_equal(merged[k], v), k
    assert merged["__step__"][0] == 7
