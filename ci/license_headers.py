# SPDX-License-Identifier: Apache-2.0
"""Checks (or adds) the licence line at the top of every source file.

Counterpart of the reference project's script/add-copyright.py and .github/workflows/copyright.yml: every C++ / CUDA /
Python / CMake source must carry the line `SPDX-License-Identifier: Apache-2.0` within its first five lines.

  python ci/license_headers.py            # list files without the line; exit status 1 if there are any
  python ci/license_headers.py --fix      # insert the line (after a shebang, before everything else)
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys

TAG = "SPDX-License-Identifier: Apache-2.0"
STYLES = {".cpp": "//", ".h": "//", ".cu": "//", ".cuh": "//", ".c": "//", ".py": "#", ".cmake": "#", ".sh": "#"}
SKIP_DIRS = {".git", "build", "__pycache__", "_ref", ".pytest_cache", "lib", "lib_checked", "lib_asan", "bin"}


def candidates(root):
    """Files of the checkout that git tracks or would track (ignored files are nobody's sources); outside a git
    checkout, every file below `root` except build products."""
    try:
        out = subprocess.run(["git", "-C", root, "ls-files", "--cached", "--others", "--exclude-standard"], capture_output=True,
                             text=True, check=True).stdout
        return [os.path.join(root, line) for line in out.splitlines() if line and os.path.isfile(os.path.join(root, line))]
    except (OSError, subprocess.CalledProcessError):
        found = []
        for base, dirs, files in os.walk(root):
            dirs[:] = [d for d in dirs if d not in SKIP_DIRS]
            found.extend(os.path.join(base, name) for name in files)
        return found


def sources(root):
    for path in sorted(candidates(root)):
        name = os.path.basename(path)
        ext = os.path.splitext(name)[1]
        if ext in STYLES or name == "CMakeLists.txt":
            yield path, STYLES.get(ext, "#")


def has_tag(path):
    with open(path, encoding="utf-8", errors="replace") as f:
        return any(TAG in f.readline() for _ in range(5))


def add_tag(path, comment):
    with open(path, encoding="utf-8") as f:
        text = f.read()
    line = f"{comment} {TAG}\n"
    if text.startswith("#!"):
        first, rest = text.split("\n", 1)
        text = first + "\n" + line + rest
    else:
        text = line + text
    with open(path, "w", encoding="utf-8") as f:
        f.write(text)


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--fix", action="store_true")
    parser.add_argument("--root", default=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    args = parser.parse_args(argv)
    missing = [(p, c) for p, c in sources(args.root) if not has_tag(p)]
    for path, comment in missing:
        if args.fix:
            add_tag(path, comment)
        print(("added: " if args.fix else "missing: ") + os.path.relpath(path, args.root))
    return 0 if args.fix or not missing else 1


if __name__ == "__main__":
    sys.exit(main())
