# SPDX-License-Identifier: Apache-2.0
"""The C++ test programs (tests/cpp/): cs_b200_tests for one device, cs_b200_communication_tests for the collectives.
They mirror the reference project's two GoogleTest executables (test/CMakeLists.txt:15-48) with a small harness of
their own, since the image has no GoogleTest."""
import os
import subprocess
import sys

import pytest
import torch

from core_scheduler_b200 import build as native_build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def program(name):
    return [e for e in native_build.build_cpp_tests() if e.endswith(name)][0]


def check(out, tests):
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert f"{tests} tests ran, 0 failed" in out.stdout, out.stdout[-3000:]


def test_cpp_single_device_tests_on_the_cpu():
    out = subprocess.run([program("cs_b200_tests")], env=dict(os.environ, CUDA_VISIBLE_DEVICES=""), capture_output=True, text=True,
                         timeout=600)
    assert "device: cpu" in out.stdout
    check(out, 20)


def test_cpp_communication_tests_as_a_single_rank_on_the_cpu():
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    out = subprocess.run([program("cs_b200_communication_tests")], env=dict(env, CUDA_VISIBLE_DEVICES=""), capture_output=True,
                         text=True, timeout=600)
    assert "rank 0 of 1 on cpu" in out.stdout
    check(out, 9)


@pytest.mark.parametrize("ranks", [2, 4])
def test_cpp_communication_tests_with_rank_threads(ranks):
    """Real multi-rank semantics without GPUs or a launcher: the ranks are threads of one process (kTHREADS group),
    including a rank that never joins (error after the rendezvous timeout) and a slow rank."""
    out = subprocess.run([program("cs_b200_communication_tests"), "--threads", str(ranks)],
                         env=dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1"), capture_output=True, text=True, timeout=600)
    assert f"{ranks} rank threads on cpu" in out.stdout
    check(out, 9)


def test_cpp_harness_reports_a_filter_and_counts(tmp_path):
    out = subprocess.run([program("cs_b200_tests"), "--filter", "GeLU"], env=dict(os.environ, CUDA_VISIBLE_DEVICES=""),
                         capture_output=True, text=True, timeout=600)
    check(out, 1)


@pytest.mark.gpu
def test_cpp_single_device_tests_on_the_gpu():
    out = subprocess.run([program("cs_b200_tests")], capture_output=True, text=True, timeout=600)
    assert "device: cuda" in out.stdout
    check(out, 20)


@pytest.mark.gpu
def test_cpp_communication_tests_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "launch.py"), "--nproc", "2", "--master-port", "29613", "--",
                          program("cs_b200_communication_tests")], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert out.stdout.count("9 tests ran, 0 failed") == 2, out.stdout[-3000:]


@pytest.mark.skipif(os.environ.get("CS_RUN_SANITIZERS") != "1", reason="set CS_RUN_SANITIZERS=1 (builds the host code with the sanitizers, several minutes)")
@pytest.mark.parametrize("kind", ["address", "thread"])
def test_host_code_is_clean_under_the_sanitizers(kind):
    """The scheduler, the rank-thread communicator, bucketing, the loader's producer thread, the module tree and the
    optimizer run the two C++ test programs on the CPU under AddressSanitizer + UndefinedBehaviorSanitizer and under
    ThreadSanitizer without a report. ThreadSanitizer runs with tests/cpp/tsan.supp (NVTX's and oneDNN's own lazy
    initialisation) and without mutex-misuse reports, which uninstrumented libtorch triggers by itself."""
    from core_scheduler_b200.build import build_sanitized

    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1",
               ASAN_OPTIONS="detect_leaks=0:protect_shadow_gap=0:detect_odr_violation=0",
               UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=1",
               TSAN_OPTIONS=f"suppressions={os.path.join(ROOT, 'tests', 'cpp', 'tsan.supp')} report_signal_unsafe=0 report_mutex_bugs=0")
    for exe in build_sanitized(kind):
        args = [exe, "--threads", "2"] if "communication" in exe else [exe]
        run = subprocess.run(args, env=env, capture_output=True, text=True, timeout=1800)
        text = run.stdout + run.stderr
        assert run.returncode == 0 and "0 failed" in text, text[-3000:]
        assert "ERROR: AddressSanitizer" not in text and "runtime error:" not in text and "WARNING: ThreadSanitizer" not in text, text[-3000:]
