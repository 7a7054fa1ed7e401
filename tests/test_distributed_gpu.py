# SPDX-License-Identifier: Apache-2.0
"""Collectives and parallel training on 2 GPUs: NCCL path and this library's peer-memory kernels.

Runs as child processes (one per GPU) with NVLS switched off, as multi-rank GPU tests should on
shared machines. Skipped when fewer than two GPUs are visible.
"""
import os
import subprocess
import sys

import pytest
import torch

from test_distributed_cpu import run_case

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytestmark = pytest.mark.gpu
needs2 = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")


@needs2
@pytest.mark.parametrize("case", ["all_reduce", "bucket", "bucket_arena_order", "bucket_gradients_bias", "all_gather", "reduce_scatter", "all_to_all", "dp_training"])
@pytest.mark.parametrize("backend", ["nccl", "nvp2p"])
def test_two_gpu_ranks(case, backend):
    run_case(case, device="cuda", extra=(backend,), timeout=600)


@needs2
@pytest.mark.parametrize("backend", ["nccl", "nvp2p"])
def test_tensor_parallel_matches_single_device(backend):
    run_case("tp_training", device="cuda", extra=(backend,), timeout=600)


@needs2
def test_tensor_parallel_fused_gemm_collectives():
    run_case("tp_training_fused", device="cuda", extra=("nvp2p",), timeout=600)


@needs2
def test_tensor_parallel_uneven_heads_fused():
    run_case("tp_uneven_heads_fused", device="cuda", extra=("nvp2p",), timeout=600)


@needs2
def test_tensor_parallel_trainer_with_unequal_shards_in_symmetric_memory():
    run_case("tp_trainer_uneven", device="cuda", extra=("nvp2p",), timeout=600)


@needs2
def test_in_place_arena_all_reduce():
    run_case("all_reduce_arena", device="cuda", extra=("nvp2p",), timeout=600)


@needs2
@pytest.mark.parametrize("memory", ["multicast", "peer", "ipc"])
def test_collectives_on_arena_buffers_every_memory_path(memory):
    """The same collectives over the three ways the arena can exist: virtual-memory allocation with an NVLink
    multicast object (multimem kernels), the same without multicast (peer loads/stores), and cudaMalloc + CUDA
    IPC. Every rank runs to completion and all ranks leave together."""
    env = {"multicast": {"NCCL_NVLS_ENABLE": "1", "CS_EXPECT_MULTICAST": "1"},
           "peer": {"NCCL_NVLS_ENABLE": "0", "CS_EXPECT_MULTICAST": "0"},
           "ipc": {"CS_SYMMETRIC_IPC": "1", "CS_EXPECT_MULTICAST": "0"}}[memory]
    run_case("collectives_arena", device="cuda", extra=("nvp2p",), timeout=600, env_extra=env)


@needs2
@pytest.mark.parametrize("case", ["all_reduce_arena", "dp_training", "zero_training"])
def test_multicast_paths_of_training(case):
    """Data-parallel and sharded-optimizer steps with the multicast mapping on (all ranks run to completion)."""
    run_case(case, device="cuda", extra=("nvp2p",), timeout=600, env_extra={"NCCL_NVLS_ENABLE": "1"})


@needs2
def test_zero_fused_step_matches_replicated_adamw():
    run_case("zero_training", device="cuda", extra=("nvp2p",), timeout=600)


@needs2
def test_zero_per_bucket_steps_and_shard_files():
    run_case("zero_bucketed", device="cuda", extra=("nvp2p",), timeout=600)


@needs2
def test_peer_wait_times_out_with_status_instead_of_hanging():
    run_case("timeout_status", device="cuda", extra=("nvp2p",), timeout=600)


@needs2
@pytest.mark.parametrize("exe,args", [("gpt2_ddp", ["--backend", "nvp2p"]), ("gpt2_ddp", ["--backend", "nccl"]),
                                      ("gpt2_zero_tp", ["--mode", "zero"]), ("gpt2_zero_tp", ["--mode", "tp"])])
def test_cpp_multi_gpu_examples(exe, args, tmp_path):
    """The C++ entry points bootstrap from the launcher's environment and train the tiny model on two GPUs."""
    path = os.path.join(ROOT, "examples", "bin", exe)
    if not os.path.exists(path):
        pytest.skip("examples not built (python -m core_scheduler_b200.build examples)")
    extra = ["--batch", "16"] if exe == "gpt2_zero_tp" else ["--micro-batch", "4"]
    if exe == "gpt2_zero_tp":
        extra += ["--metrics", str(tmp_path / "m.jsonl"), "--save-dir", str(tmp_path / "ckpt")]
    cmd = [sys.executable, os.path.join(ROOT, "examples", "launch.py"), "--nproc", "2", "--master-port", "29631", "--",
           path, "--model", "tiny", "--steps", "4", *args, *extra]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, (out.stdout + out.stderr)[-3000:]
    assert sum("tok/s" in line for line in out.stdout.splitlines()) == 4, out.stdout
    if exe == "gpt2_zero_tp":
        import json
        rows = [json.loads(l) for l in open(tmp_path / "m.jsonl")]
        assert [r["step"] for r in rows] == [1, 2, 3, 4] and rows[-1]["loss"] < rows[0]["loss"] + 0.5
        assert os.path.exists(tmp_path / "ckpt" / ("tp_rank0" if "tp" in args else "") / "meta.json")
