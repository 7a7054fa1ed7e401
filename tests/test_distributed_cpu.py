# SPDX-License-Identifier: Apache-2.0
"""Host-side logic of the communication layer with two Gloo ranks on the CPU (no GPU involved)."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def run_case(case, nproc=2, device="cpu", extra=(), timeout=240, env_extra=None):
    env = dict(os.environ)
    env.update({"CS_NO_AUTOBUILD": "1", "OMP_NUM_THREADS": "1", "NCCL_NVLS_ENABLE": "0"})
    if env_extra:
        env.update(env_extra)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1", "--nnodes=1",
           f"--nproc-per-node={nproc}", os.path.join(HERE, "dist_worker.py"), device, case, *extra]
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    if proc.returncode != 0 or f"OK {case}" not in proc.stdout:
        lines = [l for l in (proc.stdout + proc.stderr).splitlines()
                 if any(k in l for k in ("Error", "error", "assert", "Assert", "Traceback", "File \"/"))]
        raise AssertionError("\n".join(lines[-40:]))


@pytest.mark.parametrize("case", ["all_reduce", "bucket", "bucket_arena_order", "bucket_gradients_bias", "all_gather", "reduce_scatter", "all_to_all", "dp_training",
                                  "failure_injection", "watchdog", "tp_training", "tp_uneven_heads", "resume_smaller_world", "loader_shards_by_rank", "trainer", "tp_trainer_uneven", "tp_checkpoint_merge"])
def test_two_gloo_ranks(case):
    run_case(case)
