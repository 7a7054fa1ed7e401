# SPDX-License-Identifier: Apache-2.0
"""Read-only sampling of GPU clocks and throttle reasons while a benchmark runs."""
from __future__ import annotations

import shutil
import statistics
import subprocess
import threading

_QUERY = (
    "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
    "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
    "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
)
_REASONS = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]


class ClockSampler:
    """Polls `nvidia-smi --query-gpu` (never sets anything) every `period_ms` for one GPU index."""

    def __init__(self, gpu_index: int = 0, period_ms: int = 50):
        self.gpu_index = gpu_index
        self.period_ms = period_ms
        self.samples: list[dict] = []
        self._proc = None
        self._thread = None

    def start(self) -> "ClockSampler":
        exe = shutil.which("nvidia-smi")
        if exe is None:
            return self
        self._proc = subprocess.Popen(
            [exe, f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits", "-i", str(self.gpu_index), "-lms",
             str(self.period_ms)],
            stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        self._thread = threading.Thread(target=self._read, daemon=True)
        self._thread.start()
        return self

    def _read(self) -> None:
        for line in self._proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                self.samples.append({
                    "sm_mhz": float(parts[1]), "sm_max_mhz": float(parts[2]), "power_w": float(parts[3]),
                    "flags": {name: parts[5 + i].lower().startswith("active") for i, name in enumerate(_REASONS)},
                })
            except ValueError:
                continue

    def stop(self) -> dict:
        if self._proc is not None:
            self._proc.terminate()  # the exact child started above
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
            if self._thread is not None:
                self._thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        busy = [s for s in self.samples if s["power_w"] > 300] or self.samples
        reasons = sorted({name for s in busy for name, on in s["flags"].items() if on})
        return {
            "sm_mhz": statistics.median(s["sm_mhz"] for s in busy),
            "sm_max_mhz": max(s["sm_max_mhz"] for s in self.samples),
            "power_w_max": max(s["power_w"] for s in self.samples),
            "reasons": reasons,
            "samples": len(self.samples),
        }
