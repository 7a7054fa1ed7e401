# SPDX-License-Identifier: Apache-2.0
"""Starts one process per GPU with the rendezvous environment the C++ examples read.

  python examples/launch.py --nproc 8 [--master-port 29500] -- examples/bin/gpt2_ddp --model 124M --steps 20

Every child gets RANK, LOCAL_RANK, WORLD_SIZE, MASTER_ADDR=127.0.0.1 and MASTER_PORT (the role mpirun plays for
the reference project's examples). The launcher waits for all children, stops the others when one fails, and
returns the first non-zero exit code.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import time


def main() -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--nproc", type=int, required=True)
    p.add_argument("--master-port", type=int, default=29500)
    p.add_argument("cmd", nargs=argparse.REMAINDER)
    args = p.parse_args()
    cmd = args.cmd[1:] if args.cmd and args.cmd[0] == "--" else args.cmd
    if not cmd:
        p.error("no command given")
    children = []
    for rank in range(args.nproc):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(args.nproc), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(args.master_port))
        children.append(subprocess.Popen(cmd, env=env))
    code = 0
    alive = set(range(args.nproc))
    while alive:
        for r in list(alive):
            rc = children[r].poll()
            if rc is None:
                continue
            alive.discard(r)
            if rc != 0 and code == 0:
                code = rc
                for other in alive:  # exactly the processes started above
                    children[other].terminate()
        time.sleep(0.05)
    return code


if __name__ == "__main__":
    sys.exit(main())
