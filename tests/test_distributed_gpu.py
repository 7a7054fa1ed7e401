"""Collectives and parallel training on 2 GPUs: NCCL path and this library's peer-memory kernels.

Runs as child processes (one per GPU) with NVLS switched off, as multi-rank GPU tests should on
shared machines. Skipped when fewer than two GPUs are visible.
"""
import pytest
import torch

from test_distributed_cpu import run_case

pytestmark = pytest.mark.gpu
needs2 = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")


@needs2
@pytest.mark.parametrize("case", ["all_reduce", "bucket", "bucket_arena_order", "all_gather", "reduce_scatter", "all_to_all", "dp_training"])
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
def test_in_place_arena_all_reduce():
    run_case("all_reduce_arena", device="cuda", extra=("nvp2p",), timeout=600)


@needs2
def test_zero_fused_step_matches_replicated_adamw():
    run_case("zero_training", device="cuda", extra=("nvp2p",), timeout=600)


@needs2
def test_peer_wait_times_out_with_status_instead_of_hanging():
    run_case("timeout_status", device="cuda", extra=("nvp2p",), timeout=600)
