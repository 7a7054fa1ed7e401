# SPDX-License-Identifier: Apache-2.0
"""bench.py prints one JSON line with the keys its callers read."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.gpu
def test_bench_prints_one_json_line_with_the_contract_keys():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "3", "--warmup", "3"], capture_output=True,
                         text=True, timeout=900)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, out.stdout[-2000:]
    line = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
                "dtype", "data", "config", "clocks", "e2e", "gpu_launches"):
        assert key in line, key
    assert line["n_gpus"] == 1 and line["steps"] == 3 and line["warmup"] == 3 and line["higher_is_better"] is True
    assert line["dtype"] == "bf16" and line["unit"] == "tokens/s"
    assert line["value"] > 0 and abs(line["value"] - 16 * 1024 / (line["ms_per_step"] / 1e3)) < 1e-6 * line["value"]
    assert line["gpu_launches"] > 0  # this library's kernels ran, not a library fallback
    e2e = line["e2e"]
    assert e2e["value"] > 0 and e2e["h2d_bytes_per_step"] == 2 * 16 * 1024 * 8 and e2e["d2h_bytes_per_step"] == 4
    for key in ("model", "global_batch", "seq_len", "parallelism"):
        assert key in line["config"], key
