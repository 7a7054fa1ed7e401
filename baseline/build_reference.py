# SPDX-License-Identifier: Apache-2.0
"""Builds the unmodified reference sources into baseline/_ref/ (git-ignored) and the GPT-2 driver.

  python baseline/build_reference.py [--reference <checkout>]      (default: $CS_REFERENCE_DIR or ../reference beside the repo)

The reference is a CMake project that wants MPI, hwloc, gtest and cxxopts, none of which is in the
image. Its library sources compile unchanged against the libtorch, Arrow, cuDNN-frontend, fmt and
spdlog copies that the Python packages of the image ship, with two stand-in headers on the include
path (baseline/shims/mpi.h: single-node rank/size/broadcast; baseline/shims/hwloc.h: no-ops for
code that is never called). Nothing of this repository's library is linked into the result.
"""
from __future__ import annotations

import argparse
import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"


def paths():
    import torch
    import pyarrow

    site = Path(torch.__file__).resolve().parent.parent
    return {
        "torch": Path(torch.__file__).resolve().parent,
        "site": site,
        "arrow_inc": Path(pyarrow.get_include()),
        "arrow_lib": Path(pyarrow.get_library_dirs()[0]),
        "cuda": Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")),
        "abi": int(torch._C._GLIBCXX_USE_CXX11_ABI),
    }


def run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    return r.returncode, (r.stdout + r.stderr)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("CS_REFERENCE_DIR", str(HERE.parent.parent / "reference")))
    ap.add_argument("--jobs", type=int, default=8)
    args = ap.parse_args()
    ref = Path(args.reference)
    if not (ref / "src" / "tensor.cpp").exists():
        print(f"reference checkout not found at {ref}")
        return 2
    p = paths()
    OUT.mkdir(exist_ok=True)
    obj_dir = OUT / "obj"
    obj_dir.mkdir(exist_ok=True)
    inc = [HERE / "shims", ref / "include", ref / "include" / "internal", p["torch"] / "include",
           p["torch"] / "include" / "torch" / "csrc" / "api" / "include", p["cuda"] / "include", p["arrow_inc"],
           p["site"] / "include", p["site"] / "nvidia" / "cudnn" / "include", p["site"] / "nvidia" / "nccl" / "include",
           p["site"] / "flashinfer" / "data" / "spdlog" / "include"]
    defs = [f"-D_GLIBCXX_USE_CXX11_ABI={p['abi']}", "-DCORE_SCHEDULER_ENABLE_INTERNAL_BUILD", "-DUSE_C10D_NCCL", "-DUSE_DISTRIBUTED",
            "-DUSE_CUDA", "-DFMT_HEADER_ONLY", "-DSPDLOG_USE_STD_FORMAT", "-DSPDLOG_HEADER_ONLY"]
    cxx = [os.environ.get("CS_CXX", "g++"), "-std=c++20", "-O2", "-fPIC", "-fopenmp", "-w", "-fvisibility=hidden"] + defs + [f"-I{i}" for i in inc]
    nvcc = [str(p["cuda"] / "bin" / "nvcc"), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++20", "--expt-relaxed-constexpr",
            "--extended-lambda", "-Xcompiler", "-fPIC,-w", "-w"] + defs + [f"-I{i}" for i in inc]
    sources = sorted(glob.glob(str(ref / "src" / "**" / "*.cpp"), recursive=True)) + sorted(glob.glob(str(ref / "src" / "**" / "*.cu"), recursive=True))
    jobs = []
    for src in sources:
        obj = obj_dir / (Path(src).relative_to(ref / "src").as_posix().replace("/", "_") + ".o")
        cmd = (nvcc if src.endswith(".cu") else cxx) + ["-c", src, "-o", str(obj)]
        if src.endswith(("module/module.cpp", "data/dataloader.cpp")):  # Arrow 24 API drift, see shims/arrow_compat.h
            cmd += ["-include", str(HERE / "shims" / "arrow_compat.h")]
        jobs.append((src, obj, cmd))
    shim_obj = obj_dir / "mpi_shim.o"
    jobs.append((str(HERE / "shims" / "mpi_shim.c"), shim_obj, ["gcc", "-O2", "-fPIC", "-c", str(HERE / "shims" / "mpi_shim.c"), "-o", str(shim_obj)]))
    jobs_to_run = [j for j in jobs if not j[1].exists() or os.path.getmtime(j[1]) < os.path.getmtime(j[0])]
    failed = []
    with ThreadPoolExecutor(args.jobs) as pool:
        for (src, obj, cmd), (rc, out) in zip(jobs_to_run, pool.map(lambda j: run(j[2]), jobs_to_run)):
            if rc != 0:
                failed.append(src)
                print(f"FAILED {src}\n{out[-3000:]}")
    if failed:
        print(f"{len(failed)} of {len(jobs)} sources failed")
        return 1
    lib = OUT / "libcore_scheduler_core.so"
    cuda_lib = p["cuda"] / "lib64"
    link = [cxx[0], "-shared", "-fopenmp"] + [str(j[1]) for j in jobs] + ["-o", str(lib), f"-L{p['torch'] / 'lib'}", "-ltorch", "-ltorch_cpu",
            "-ltorch_cuda", "-lc10", "-lc10_cuda", f"-L{p['arrow_lib']}", "-l:libarrow.so.2400", "-l:libparquet.so.2400",
            "-l:libarrow_dataset.so.2400", "-l:libarrow_acero.so.2400", f"-L{cuda_lib}", "-lcudart", f"-L{cuda_lib / 'stubs'}", "-lnvidia-ml",
            f"-L{p['site'] / 'nvidia' / 'cudnn' / 'lib'}", "-l:libcudnn.so.9", "-ldl", "-lpthread",
            f"-Wl,-rpath,{p['torch'] / 'lib'}", f"-Wl,-rpath,{p['arrow_lib']}", f"-Wl,-rpath,{cuda_lib}",
            f"-Wl,-rpath,{p['site'] / 'nvidia' / 'cudnn' / 'lib'}", "-Wl,--no-as-needed"]
    rc, out = run(link)
    if rc != 0:
        print("link failed\n" + out[-3000:])
        return 1
    driver_src = HERE / "ref_gpt2_driver.cpp"
    exe = OUT / "ref_gpt2"
    if driver_src.exists():
        cmd = [c for c in cxx if c != "-fvisibility=hidden"] + [str(driver_src), "-o", str(exe), f"-L{OUT}", "-lcore_scheduler_core",
              f"-L{p['torch'] / 'lib'}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", f"-L{cuda_lib}", "-lcudart",
              f"-L{p['arrow_lib']}", "-l:libarrow.so.2400", "-l:libarrow_compute.so.2400", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{p['torch'] / 'lib'}", f"-Wl,-rpath,{p['arrow_lib']}", f"-Wl,-rpath,{cuda_lib}",
              f"-Wl,-rpath,{p['site'] / 'nvidia' / 'cudnn' / 'lib'}", "-Wl,--no-as-needed"]
        rc, out = run(cmd)
        if rc != 0:
            print("driver failed\n" + out[-4000:])
            return 1
    print(f"built {lib}" + (f" and {exe}" if driver_src.exists() else ""))
    return 0


if __name__ == "__main__":
    sys.exit(main())
