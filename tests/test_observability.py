# SPDX-License-Identifier: Apache-2.0
"""Metrics logger, host watchdog and resumable training state (CPU)."""
import json
import os
import time

import pytest
import torch

import core_scheduler_b200 as cs

C = cs._C


def test_metrics_logger_writes_console_csv_jsonl(tmp_path, capfd):
    log = C.MetricsLogger(jsonl_path=str(tmp_path / "m.jsonl"), csv_path=str(tmp_path / "log.csv"))
    for step in range(3):
        r = C.StepRecord()
        r.step, r.loss, r.lr, r.grad_norm, r.dt_host_ms, r.tokens_per_sec = step, 4.0 - step, 3e-4, 1.5, 20.0, 8e5
        r.mfu = C.mfu(6 * 124e6, 16384, 0.02, 1.3e15)
        r.extra = {"main_busy": 0.9}
        log.log(r)
    assert log.records_written() == 3
    out = capfd.readouterr().out
    assert out.count("tok/sec") == 3 and "grad norm 1.5000" in out
    rows = [json.loads(l) for l in open(tmp_path / "m.jsonl")]
    assert [r["step"] for r in rows] == [0, 1, 2]
    assert rows[1]["loss"] == 3.0 and rows[0]["main_busy"] == 0.9 and 0 < rows[0]["mfu"] < 1
    assert "comm_bytes" not in rows[0]  # unmeasured fields are left out
    csv = open(tmp_path / "log.csv").read().splitlines()
    assert csv[0] == "Step,Loss" and csv[1:] == ["0,4", "1,3", "2,2"]


def test_metrics_logger_other_ranks_are_silent(tmp_path, capfd):
    log = C.MetricsLogger(jsonl_path=str(tmp_path / "m.jsonl"), rank=1, writer_rank=0)
    log.log(C.StepRecord())
    assert log.records_written() == 0 and capfd.readouterr().out == "" and not (tmp_path / "m.jsonl").exists()


def test_watchdog_trips_only_without_progress():
    dog = C.Watchdog(timeout_ms=150, poll_ms=10)
    for step in range(10):
        dog.progress(step)
        time.sleep(0.03)
    assert not dog.tripped()
    dog.check()
    time.sleep(0.4)
    assert dog.tripped() and dog.last_step() == 9
    with pytest.raises(RuntimeError, match="no progress"):
        dog.check()
    dog.stop()


def test_meta_round_trip(tmp_path):
    m = C.CheckpointMeta()
    m.step, m.lr, m.seed, m.data_cursor, m.world_size, m.tp_size, m.zero, m.model = 17, 2.5e-4, 2**40 + 3, 99, 8, 2, True, 'gpt2 "124M"'
    C.save_meta(m, str(tmp_path / "meta.json"))
    json.load(open(tmp_path / "meta.json"))  # valid JSON
    r = C.load_meta(str(tmp_path / "meta.json"))
    assert (r.step, r.lr, r.seed, r.data_cursor, r.world_size, r.tp_size, r.zero, r.model) == (
        17, 2.5e-4, 2**40 + 3, 99, 8, 2, True, 'gpt2 "124M"')


def test_training_state_resume_continues_bit_identically(tmp_path):
    """Stop after two steps, save, load into fresh objects, continue: same as an uninterrupted run."""
    s = cs.DynamicScheduler(0, device="cpu")
    cfg = cs.GPT2Config(n_layer=2, n_head=2, n_embd=32, block_size=16, vocab_size=64, padded_vocab_size=64)
    g = torch.Generator().manual_seed(3)
    batches = [torch.randint(0, 64, (2, 17), generator=g) for _ in range(4)]

    def make():
        cs.manual_seed(5)
        model = cs.GPT2(s, cfg)
        flat = C.flatten_parameters(s, model)
        return model, cs.AdamW(s, model, lr=1e-2, weight_decay=0.1, flat=flat)

    def step(model, opt, b):
        loss = model.forward_loss(s, cs.from_torch(b[:, :-1].contiguous()), cs.from_torch(b[:, 1:].contiguous()))
        model.backward_loss(s)
        opt.step(s)
        opt.zero_grad(s)
        return loss.raw().item()

    model, opt = make()
    full = [step(model, opt, b) for b in batches]

    model, opt = make()
    for b in batches[:2]:
        step(model, opt, b)
    meta = C.CheckpointMeta()
    meta.step, meta.data_cursor, meta.model = 2, 2, "tiny"
    C.save_training_state(s, str(tmp_path / "nested" / "ckpt"), model, opt, meta)  # parents are created
    os.rename(tmp_path / "nested" / "ckpt", tmp_path / "ckpt")
    assert sorted(os.listdir(tmp_path / "ckpt")) == ["meta.json", "model.parquet", "optimizer.parquet"]

    cs.manual_seed(1234)  # a different init: everything must come from the files
    model2 = cs.GPT2(s, cfg)
    opt2 = cs.AdamW(s, model2, lr=1e-2, weight_decay=0.1, flat=C.flatten_parameters(s, model2))
    got = C.load_training_state(s, str(tmp_path / "ckpt"), model2, opt2)
    assert got.step == 2 and got.data_cursor == 2 and got.model == "tiny"
    resumed = [step(model2, opt2, b) for b in batches[got.data_cursor:]]
    assert resumed == full[2:]


def test_descriptor_of_another_process_can_be_duplicated(tmp_path):
    """Arena handles travel between ranks as (pid, fd) pairs through the store; the importer duplicates the
    descriptor with pidfd_getfd. Here the 'handle' is a memfd of this process read by a child process."""
    import subprocess
    import sys

    fd = os.memfd_create("cs_handle")
    os.write(fd, b"symmetric")
    code = ("import os, sys; sys.path.insert(0, %r); import core_scheduler_b200 as cs; "
            "n = cs._C.duplicate_descriptor(%d, %d); assert n >= 0, n; print(os.pread(n, 9, 0).decode())"
            % (os.path.dirname(os.path.dirname(os.path.abspath(__file__))), os.getpid(), fd))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120, env=dict(os.environ, CS_NO_AUTOBUILD="1"))
    assert out.returncode == 0 and out.stdout.strip() == "symmetric", out.stdout + out.stderr
    assert cs._C.duplicate_descriptor(os.getpid(), fd) >= 0  # own descriptors are dup()ed
    assert cs._C.duplicate_descriptor(os.getpid(), 10 ** 6) == -1
