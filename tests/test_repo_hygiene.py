# SPDX-License-Identifier: Apache-2.0
"""The licence-line check that CI runs: clean on this checkout, finds and repairs a file without the line."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPT = os.path.join(ROOT, "ci", "license_headers.py")


def test_every_source_of_this_checkout_carries_the_licence_line():
    run = subprocess.run([sys.executable, SCRIPT], capture_output=True, text=True)
    assert run.returncode == 0, run.stdout


def test_missing_line_is_reported_and_fixed(tmp_path):
    (tmp_path / "a.py").write_text("#!/usr/bin/env python\nprint(1)\n")
    (tmp_path / "b.cu").write_text("__global__ void k() {}\n")
    (tmp_path / "c.txt").write_text("not a source\n")
    run = subprocess.run([sys.executable, SCRIPT, "--root", str(tmp_path)], capture_output=True, text=True)
    assert run.returncode == 1 and "a.py" in run.stdout and "b.cu" in run.stdout and "c.txt" not in run.stdout
    subprocess.run([sys.executable, SCRIPT, "--root", str(tmp_path), "--fix"], check=True, capture_output=True)
    assert (tmp_path / "a.py").read_text().splitlines()[:2] == ["#!/usr/bin/env python", "# SPDX-License-Identifier: Apache-2.0"]
    assert (tmp_path / "b.cu").read_text().startswith("// SPDX-License-Identifier: Apache-2.0\n")
    assert subprocess.run([sys.executable, SCRIPT, "--root", str(tmp_path)]).returncode == 0
