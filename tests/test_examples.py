# SPDX-License-Identifier: Apache-2.0
"""C++ entry points and the data preparation script."""
import os

import pytest
import subprocess
import sys

import core_scheduler_b200 as cs
from core_scheduler_b200 import build as native_build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
C = cs._C


def test_cpp_single_device_example_trains_and_saves(tmp_path):
    exes = native_build.build_examples()
    exe = [e for e in exes if e.endswith("gpt2_single_device")][0]
    ckpt = tmp_path / "tiny.parquet"
    log = tmp_path / "log.csv"
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    out = subprocess.run([exe, "--model", "tiny", "--steps", "3", "--save", str(ckpt), "--log", str(log)], env=env,
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert out.stdout.count("tok/s") == 3
    assert ckpt.exists() and log.read_text().startswith("Step,Loss")
    # the checkpoint written by the C++ program loads into a Python-built model of the same config
    s = cs.DynamicScheduler(0, device="cpu")
    m = cs.GPT2(s, cs.GPT2Config(n_layer=2, n_head=4, n_embd=128, block_size=64, vocab_size=512, padded_vocab_size=512))
    m.load(str(ckpt))


def test_prepare_text_gen_feeds_the_loader(tmp_path, cpu_scheduler):
    corpus = tmp_path / "corpus.txt"
    corpus.write_text("\n\n".join("document %d " % i + "lorem ipsum dolor sit amet " * 40 for i in range(30)))
    out = tmp_path / "data"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "prepare_text_gen.py"), "--source", str(corpus), "--out",
                        str(out), "--block-size", "64", "--tokenizer", "", "--split-ratio", "0.1"],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    ds = C.LlmDataset(str(out / "train"))
    assert ds.size() > 8
    batch = C.LlmDataLoader(ds, 4, 1, False).load(cpu_scheduler)
    ids, lab = batch["input_ids"].raw(), batch["labels"].raw()
    assert ids.shape == (4, 64)
    assert (ids[:, 1:] == lab[:, :-1]).all()


def test_launcher_sets_rendezvous_environment_and_propagates_failure():
    launch = os.path.join(ROOT, "examples", "launch.py")
    ok = subprocess.run([sys.executable, launch, "--nproc", "3", "--master-port", "29777", "--", sys.executable, "-c",
                         "import os; print('R', os.environ['RANK'], os.environ['LOCAL_RANK'], os.environ['WORLD_SIZE'], "
                         "os.environ['MASTER_ADDR'], os.environ['MASTER_PORT'])"], capture_output=True, text=True, timeout=180)
    assert ok.returncode == 0, ok.stdout + ok.stderr
    assert sorted(l for l in ok.stdout.splitlines() if l.startswith("R ")) == [f"R {r} {r} 3 127.0.0.1 29777" for r in range(3)]
    bad = subprocess.run([sys.executable, launch, "--nproc", "2", "--", sys.executable, "-c",
                          "import os, sys, time; sys.exit(7) if os.environ['RANK'] == '1' else time.sleep(30)"],
                         capture_output=True, text=True, timeout=180)
    assert bad.returncode == 7, (bad.returncode, bad.stdout + bad.stderr)  # rank 1 failed; the sleeping rank 0 was stopped, not waited for


@pytest.mark.gpu
def test_program_written_for_the_reference_api_runs_on_this_library(tmp_path):
    """baseline/ref_gpt2_driver.cpp uses only the reference's public headers (include/compute/*.h, module/*.h, ...).
    Compiled unchanged against this repository's compatibility headers and library it must train the tiny model."""
    import torch

    from core_scheduler_b200.build import _paths

    p = _paths()
    csrc = os.path.join(ROOT, "core_scheduler_b200", "csrc")
    lib = os.path.join(ROOT, "core_scheduler_b200", "lib")
    shim = os.path.join(ROOT, "baseline", "shims")
    exe = tmp_path / "ref_api_gpt2"
    # the driver initialises Arrow's compute kernels for its data path: Arrow headers and both Arrow libraries
    import glob
    arrow_libs = ["-l:" + os.path.basename(sorted(glob.glob(os.path.join(str(p["arrow_lib"]), pat)))[0])
                  for pat in ("libarrow_compute.so.*", "libarrow.so.*")]
    subprocess.run(["gcc", "-O1", "-c", os.path.join(shim, "mpi_shim.c"), f"-I{shim}", "-o", str(tmp_path / "mpi_shim.o")], check=True)
    cmd = ["g++", "-std=c++20", "-O1", "-w", f"-D_GLIBCXX_USE_CXX11_ABI={p['cxx11_abi']}", "-DUSE_C10D_NCCL", "-DUSE_DISTRIBUTED",
           f"-I{shim}", f"-I{csrc}/include", f"-I{csrc}", f"-I{p['arrow_inc']}"] + [f"-I{i}" for i in p["torch_inc"]] + [f"-I{p['cuda_home'] / 'include'}",
           os.path.join(ROOT, "baseline", "ref_gpt2_driver.cpp"), str(tmp_path / "mpi_shim.o"), "-o", str(exe), f"-L{lib}", "-lcs_b200",
           f"-L{p['torch_lib']}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", f"-L{p['cuda_home'] / 'lib64'}", "-lcudart",
           f"-L{p['arrow_lib']}", *arrow_libs, f"-Wl,-rpath,{lib}", f"-Wl,-rpath,{p['torch_lib']}", f"-Wl,-rpath,{p['arrow_lib']}", "-Wl,--no-as-needed"]
    build = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert build.returncode == 0, build.stderr[-3000:]
    env = dict(os.environ, CS_MPISHIM_KEY=f"api{os.getpid()}")
    run = subprocess.run([str(exe), "--model", "tiny", "--micro-batch", "2", "--seq", "64", "--steps", "3", "--warmup", "1"], env=env,
                         capture_output=True, text=True, timeout=300)
    line = next((l for l in run.stdout.splitlines() if l.startswith("REF_RESULT")), None)
    assert line is not None, (run.stdout + run.stderr)[-2000:]
    fields = dict(kv.split("=") for kv in line.split()[1:])
    assert 0.0 < float(fields["final_loss"]) < 7.0 and float(fields["ms_per_step"]) > 0.0


def test_cmake_project_configures_and_builds_the_library(tmp_path):
    """The CMake entry (for C++ projects that linked the reference's `core_scheduler` target) builds the same sources."""
    import shutil

    if shutil.which("cmake") is None:
        pytest.skip("cmake not installed")
    cfg = subprocess.run(["cmake", "-S", ROOT, "-B", str(tmp_path / "b"), f"-DPython3_EXECUTABLE={sys.executable}",
                          "-DCORE_SCHEDULER_ENABLE_EXAMPLES=ON"], capture_output=True, text=True, timeout=600)
    assert cfg.returncode == 0, cfg.stdout[-2000:] + cfg.stderr[-2000:]
    build = subprocess.run(["cmake", "--build", str(tmp_path / "b"), "-j", "16", "--target", "gpt2_single_device"],
                           capture_output=True, text=True, timeout=3000)
    assert build.returncode == 0, build.stdout[-3000:] + build.stderr[-3000:]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    run = subprocess.run([str(tmp_path / "b" / "gpt2_single_device"), "--model", "tiny", "--steps", "2"], env=env,
                         capture_output=True, text=True, timeout=300)
    assert run.returncode == 0 and run.stdout.count("tok/s") == 2, run.stdout + run.stderr
