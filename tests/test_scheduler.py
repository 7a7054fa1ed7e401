# SPDX-License-Identifier: Apache-2.0
"""Scheduler semantics: stream classes, ordering across streams, re-join of side tasks, errors."""
import pytest
import torch

import core_scheduler_b200 as cs

C = cs._C


def test_cpu_scheduler_runs_tasks_inline_and_tags_outputs(cpu_scheduler):
    s = cpu_scheduler
    out = cs.Tensor()
    seen = []
    s.submit_python("t0", 1, [out], [], lambda: (seen.append(1), out.set_raw(torch.ones(3)))[0])
    assert seen == [1]
    assert out.stream_class() == 1
    assert s.submitted()[1] == 1


def test_task_failure_carries_task_name(cpu_scheduler):
    def boom():
        raise ValueError("bad thing")

    with pytest.raises(RuntimeError) as e:
        cpu_scheduler.submit_python("my_failing_task", 0, [], [], boom)
    assert "my_failing_task" in str(e.value)


def test_autocast_guard_sets_and_restores(cpu_scheduler):
    s = cpu_scheduler
    assert not s.autocast_enabled()
    with cs.autocast(s, torch.bfloat16):
        assert s.autocast_enabled()
    assert not s.autocast_enabled()
    assert s.submitted()[3] == 2  # two config tasks


def test_to_torch_returns_detached_clone(cpu_scheduler):
    x = torch.arange(6.0)
    t = cs.from_torch(x)
    y = cs.to_torch(cpu_scheduler, t)
    y += 1
    assert torch.equal(x, torch.arange(6.0))


@pytest.mark.gpu
def test_cross_stream_read_after_write_is_ordered(gpu_scheduler):
    """A slow writer on the assist stream must be visible to a main-stream reader."""
    s = gpu_scheduler
    n = 1 << 24
    src = torch.zeros(n, device="cuda")
    out = cs.Tensor()
    res = cs.Tensor()

    def writer():
        t = src
        for _ in range(50):  # long chain of kernels on the assist stream
            t = t + 1
        out.set_raw(t)

    def reader():
        res.set_raw(out.raw().sum())

    s.submit_python("writer", 1, [out], [], writer)
    s.submit_python("reader", 0, [res], [out], reader)
    val = cs.to_torch(s, res).item()
    assert val == 50 * n


@pytest.mark.gpu
def test_write_after_read_across_streams_is_ordered(gpu_scheduler):
    """A main-stream writer must wait for a side-stream reader of the same tensor."""
    s = gpu_scheduler
    n = 1 << 24
    buf = cs.from_torch(torch.ones(n, device="cuda"))
    res = cs.Tensor()

    def slow_reader():
        t = buf.raw()
        acc = torch.zeros((), device="cuda")
        for _ in range(40):
            acc = acc + t.sum()
        res.set_raw(acc)

    def overwriter():
        buf.raw().zero_()

    s.submit_python("slow_reader", 2, [res], [buf], slow_reader)
    s.submit_python("overwriter", 0, [buf], [], overwriter)
    assert cs.to_torch(s, res).item() == 40 * n


@pytest.mark.gpu
def test_writer_waits_for_readers_on_both_side_streams(gpu_scheduler):
    """An assist-stream reader followed by a comm-stream reader of the same tensor: a later main-stream writer
    must wait for both, not only for the most recent one."""
    s = gpu_scheduler
    n = 1 << 24
    buf = cs.from_torch(torch.ones(n, device="cuda"))
    slow, fast = cs.Tensor(), cs.Tensor()

    def slow_reader():
        t = buf.raw()
        acc = torch.zeros((), device="cuda")
        for _ in range(60):
            acc = acc + t.sum()
        slow.set_raw(acc)

    s.submit_python("slow_assist_reader", 1, [slow], [buf], slow_reader)
    s.submit_python("fast_comm_reader", 2, [fast], [buf], lambda: fast.set_raw(buf.raw()[:16].sum()))
    s.submit_python("overwriter", 0, [buf], [], lambda: buf.raw().zero_())
    assert cs.to_torch(s, slow).item() == 60 * n
    assert cs.to_torch(s, fast).item() == 16


@pytest.mark.gpu
def test_side_tasks_rejoin_and_events_are_pooled(gpu_scheduler):
    s = gpu_scheduler
    x = cs.from_torch(torch.ones(1024, device="cuda"))
    for i in range(20):
        o = cs.Tensor()
        s.submit_python("side", 1 + (i % 2), [o], [x], lambda o=o: o.set_raw(x.raw() * 2))
        m = cs.Tensor()
        s.submit_python("main", 0, [m], [o], lambda m=m, o=o: m.set_raw(o.raw() + 1))
    s.synchronize()
    assert cs.to_torch(s, m).eq(3).all()
    del o, m
    assert C.event_pool_size() > 0


@pytest.mark.gpu
def test_profiling_reports_task_times(gpu_scheduler):
    s = gpu_scheduler
    s.set_profiling(True)
    x = cs.from_torch(torch.ones(1 << 20, device="cuda"))
    o = cs.Tensor()
    s.submit_python("timed_task", 0, [o], [x], lambda: o.set_raw(x.raw() * 3))
    t = s.drain_timings()
    s.set_profiling(False)
    assert any(r.name == "timed_task" and r.device_ms >= 0 for r in t)


@pytest.mark.gpu
def test_chrome_trace_export_orders_tasks_by_device_start(gpu_scheduler, tmp_path):
    import json

    from core_scheduler_b200.utils.trace import write_chrome_trace

    s = gpu_scheduler
    s.set_profiling(True)
    x = cs.from_torch(torch.ones(1 << 22, device="cuda"))
    outs = [cs.Tensor() for _ in range(3)]
    prev = x
    for i, o in enumerate(outs):
        s.submit_python(f"stage{i}", i % 2, [o], [prev], lambda o=o, prev=prev: o.set_raw(prev.raw() * 2))
        prev = o
    rows = s.drain_timings()
    s.set_profiling(False)
    n = write_chrome_trace(rows, str(tmp_path / "t.json"))
    assert n == len(rows) >= 3
    trace = json.load(open(tmp_path / "t.json"))["traceEvents"]
    tasks = {e["name"]: e for e in trace if e["ph"] == "X"}
    assert tasks["stage0"]["ts"] == 0 and tasks["stage0"]["ts"] <= tasks["stage1"]["ts"] <= tasks["stage2"]["ts"]
    assert tasks["stage1"]["tid"] == 1 and tasks["stage0"]["tid"] == 0  # lanes are the stream classes


@pytest.mark.gpu
def test_wrapped_tensors_wait_for_their_producer_stream(gpu_scheduler):
    """A tensor still being written on PyTorch's current stream is not read early by a task."""
    s = gpu_scheduler
    n = 1 << 24
    x = torch.zeros(n, device="cuda")
    torch.cuda.synchronize()
    for _ in range(60):  # long chain on the default stream
        x = x + 1
    h = cs.from_torch(x)  # wrapped while the chain is still running
    res = cs.Tensor()
    s.submit_python("reader", 0, [res], [h], lambda: res.set_raw(h.raw().sum()))
    assert cs.to_torch(s, res).item() == 60 * n
