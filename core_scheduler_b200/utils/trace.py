# SPDX-License-Identifier: Apache-2.0
"""Chrome-trace export of the scheduler's per-task device timings.

  s.set_profiling(True); ... one step ...; rows = s.drain_timings()
  write_chrome_trace(rows, "step.json")     # open in chrome://tracing or Perfetto

One lane per stream class (main / assist / comm); times are CUDA-event times on the device, relative to the
first task of the drained batch. The reference only emits NVTX ranges for an external profiler
(include/nvtx_helper.h:21-41); the ranges are kept, this file is an addition for machines without one.
"""
from __future__ import annotations

import json

_LANES = {0: "main stream", 1: "assist stream", 2: "comm stream"}


def chrome_trace_events(timings) -> list[dict]:
    events = [{"name": "thread_name", "ph": "M", "pid": 0, "tid": tid, "args": {"name": lane}} for tid, lane in _LANES.items()]
    for t in timings:
        events.append({"name": t.name, "ph": "X", "pid": 0, "tid": int(t.stream_class), "ts": t.start_ms * 1e3,
                       "dur": t.device_ms * 1e3, "cat": "task"})
    return events


def write_chrome_trace(timings, path: str) -> int:
    events = chrome_trace_events(timings)
    with open(path, "w") as f:
        json.dump({"traceEvents": events, "displayTimeUnit": "ms"}, f)
    return len(events) - len(_LANES)
