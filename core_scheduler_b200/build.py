# SPDX-License-Identifier: Apache-2.0
"""In-tree build of the native runtime.

Produces, next to this file:
  lib/libcs_b200.so   C++ framework + sm_100a kernels (what C++ programs link against)
  _C.<abi>.so         pybind11 bindings over the same library

CUDA sources are compiled by nvcc for sm_100a only (-gencode arch=compute_100a,code=sm_100a);
they include no torch headers, so they build in seconds. C++ sources are compiled by g++
against the libtorch headers of the running interpreter. A ninja file is generated and run,
so rebuilds are incremental.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
BUILD = HERE / "build"
LIBDIR = HERE / "lib"
CHECKED_LIBDIR = HERE / "lib_checked"

CPP_SOURCES = [
    "src/core.cpp",
    "src/compute_ops.cpp",
    "src/attention_utils.cpp",
    "src/optimizer.cpp",
    "src/module.cpp",
    "src/modules.cpp",
    "src/parquet_io.cpp",
    "src/communication.cpp",
    "src/comm_nccl.cpp",
    "src/comm_threads.cpp",
    "src/symmetric.cpp",
    "src/vmm.cpp",
    "src/data.cpp",
    "src/observability.cpp",
    "src/models_gpt2.cpp",
]
CUDA_SOURCES = [
    "kernels/elementwise.cu",
    "kernels/gemm_tcgen05.cu",
    "kernels/collectives.cu",
    "kernels/attention_tcgen05.cu",
]
BINDING_SOURCES = ["python/bindings.cpp"]


def _optional_sources():
    extra_cpp, extra_cu = [], []
    for name in ("src/parallel.cpp",):
        if (CSRC / name).exists():
            extra_cpp.append(name)
    for name in ():
        if (CSRC / name).exists():
            extra_cu.append(name)
    return extra_cpp, extra_cu


def _paths():
    import torch
    import pyarrow

    torch_dir = Path(torch.__file__).resolve().parent
    site = torch_dir.parent
    nccl_inc = site / "nvidia" / "nccl" / "include"
    cuda_home = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
    return {
        "torch_inc": [torch_dir / "include", torch_dir / "include" / "torch" / "csrc" / "api" / "include"],
        "torch_lib": torch_dir / "lib",
        "arrow_inc": Path(pyarrow.get_include()),
        "arrow_lib": Path(pyarrow.get_library_dirs()[0]),
        "nccl_inc": nccl_inc if nccl_inc.exists() else Path("/usr/include"),
        "cuda_home": cuda_home,
        "py_inc": Path(sysconfig.get_paths()["include"]),
        "pybind_flags": [
            f'-DPYBIND11_COMPILER_TYPE=\\"{getattr(torch._C, "_PYBIND11_COMPILER_TYPE", "_gcc")}\\"',
            f'-DPYBIND11_STDLIB=\\"{getattr(torch._C, "_PYBIND11_STDLIB", "_libstdcpp")}\\"',
            f'-DPYBIND11_BUILD_ABI=\\"{getattr(torch._C, "_PYBIND11_BUILD_ABI", "_cxxabi1018")}\\"',
        ],
        "cxx11_abi": int(torch._C._GLIBCXX_USE_CXX11_ABI),
    }


def ext_suffix() -> str:
    return sysconfig.get_config_var("EXT_SUFFIX")


def generate_ninja() -> Path:
    p = _paths()
    BUILD.mkdir(exist_ok=True)
    LIBDIR.mkdir(exist_ok=True)
    extra_cpp, extra_cu = _optional_sources()
    inc = [CSRC / "include", CSRC, CSRC / "src"] + p["torch_inc"] + [p["cuda_home"] / "include"]
    cxxflags = [
        "-std=c++20", "-O2", "-fPIC", "-Wall", "-Wno-unused-function", "-Wno-interference-size",
        "-Wno-sign-compare", "-Wno-unused-local-typedefs", "-Wno-deprecated-declarations",
        f"-D_GLIBCXX_USE_CXX11_ABI={p['cxx11_abi']}", "-DUSE_C10D_NCCL", "-DUSE_DISTRIBUTED", "-DUSE_RPC", "-DUSE_CUDA",
    ] + [f"-I{i}" for i in inc]
    nvccflags = [
        "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
        "-Xcompiler", "-fPIC", f"-I{CSRC}", f"-I{CSRC / 'kernels'}",
    ]
    lines = [
        "ninja_required_version = 1.5",
        f"cxx = {os.environ.get('CS_CXX', 'g++')}",
        f"nvcc = {p['cuda_home'] / 'bin' / 'nvcc'}",
        f"cxxflags = {' '.join(cxxflags)}",
        f"nvccflags = {' '.join(nvccflags)}",
        "rule cxx",
        "  command = $cxx -MMD -MF $out.d $cxxflags $extra -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "rule nvcc",
        "  command = $nvcc $nvccflags -MD -MF $out.d -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "rule nvcc_checked",
        "  command = $nvcc $nvccflags -DCS_BOUNDS_CHECK -MD -MF $out.d -c $in -o $out",
        "  depfile = $out.d",
        "  deps = gcc",
        "rule link",
        "  command = $cxx -shared $in -o $out $ldflags",
    ]
    objs, checked_objs = [], []
    for src in CPP_SOURCES + extra_cpp:
        obj = BUILD / (src.replace("/", "_") + ".o")
        extra = ""
        if src.endswith("parquet_io.cpp"):
            extra = f"-I{p['arrow_inc']}"
        if src.endswith("comm_nccl.cpp"):
            extra = f"-I{p['nccl_inc']}"
        lines += [f"build {obj}: cxx {CSRC / src}", f"  extra = {extra}"]
        objs.append(obj)
        checked_objs.append(obj)
    for src in CUDA_SOURCES + extra_cu:
        obj = BUILD / (src.replace("/", "_") + ".o")
        lines += [f"build {obj}: nvcc {CSRC / src}"]
        objs.append(obj)
        # diagnostic variant of the same kernels: checked index accessors (kernels/bounds_check.h)
        cobj = BUILD / (src.replace("/", "_") + ".checked.o")
        lines += [f"build {cobj}: nvcc_checked {CSRC / src}"]
        checked_objs.append(cobj)
    cuda_lib = p["cuda_home"] / "lib64"
    lib_ld = [
        f"-L{p['torch_lib']}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
        f"-L{p['arrow_lib']}", "-l:libarrow.so.2400", "-l:libparquet.so.2400",
        f"-L{cuda_lib}", "-lcudart", "-ldl", "-lpthread",
        f"-Wl,-rpath,{p['torch_lib']}", f"-Wl,-rpath,{p['arrow_lib']}", f"-Wl,-rpath,{cuda_lib}",
        "-Wl,--no-as-needed", "-Wl,-soname,libcs_b200.so",
    ]
    libcs = LIBDIR / "libcs_b200.so"
    lines += [f"build {libcs}: link {' '.join(map(str, objs))}", f"  ldflags = {' '.join(lib_ld)}"]
    CHECKED_LIBDIR.mkdir(exist_ok=True)
    libcs_checked = CHECKED_LIBDIR / "libcs_b200.so"
    lines += [f"build {libcs_checked}: link {' '.join(map(str, checked_objs))}", f"  ldflags = {' '.join(lib_ld)}",
              f"build checked: phony {libcs_checked}"]
    bobjs = []
    for src in BINDING_SOURCES:
        obj = BUILD / (src.replace("/", "_") + ".o")
        lines += [f"build {obj}: cxx {CSRC / src}", f"  extra = -I{p['py_inc']} {' '.join(p['pybind_flags'])} -DTORCH_EXTENSION_NAME=_C -DTORCH_API_INCLUDE_EXTENSION_H"]
        bobjs.append(obj)
    ext = HERE / f"_C{ext_suffix()}"
    ext_ld = [
        f"-L{LIBDIR}", "-lcs_b200", f"-L{p['torch_lib']}", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10",
        "-Wl,-rpath,'$$ORIGIN/lib'", f"-Wl,-rpath,{p['torch_lib']}",
    ]
    lines += [f"build {ext}: link {' '.join(map(str, bobjs))} | {libcs}", f"  ldflags = {' '.join(ext_ld)}"]
    lines += [f"default {ext}"]
    ninja_file = BUILD / "build.ninja"
    ninja_file.write_text("\n".join(lines) + "\n")
    return ninja_file


def build(verbose: bool = False, checked: bool = False) -> None:
    """Builds the library and the extension; with `checked` also lib_checked/libcs_b200.so, the same
    library with -DCS_BOUNDS_CHECK kernels (loaded instead of the normal one when CS_BOUNDS_CHECK=1)."""
    ninja_file = generate_ninja()
    cmd = [sys.executable, "-m", "ninja", "-f", str(ninja_file)]
    if checked:
        cmd += [str(HERE / f"_C{ext_suffix()}"), "checked"]
    if verbose:
        cmd.append("-v")
    jobs = os.environ.get("CS_BUILD_JOBS")
    if jobs:
        cmd += ["-j", jobs]
    subprocess.run(cmd, check=True, cwd=str(BUILD))


def build_examples() -> list[str]:
    """Compiles the C++ programs under examples/ against libcs_b200.so into examples/bin/."""
    return _build_programs(HERE.parent / "examples", [])


def build_cpp_tests() -> list[str]:
    """Compiles the C++ test programs under tests/cpp/ (cs_b200_tests, cs_b200_communication_tests) into tests/cpp/bin/."""
    root = HERE.parent / "tests" / "cpp"
    return _build_programs(root, [root], {"test_ops": "cs_b200_tests", "test_communication": "cs_b200_communication_tests"})


def _sources_digest(files) -> str:
    import hashlib

    h = hashlib.sha256()
    for f in sorted(files):
        h.update(str(f.name).encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def _build_programs(root: Path, extra_inc: list, names: dict | None = None) -> list[str]:
    # A shipped snapshot carries the built library but not the object files: there is nothing to bring up to date
    # there, and running the build would compile every kernel again.
    if not (is_built() and not any(BUILD.glob("*.o"))):
        build()
    p = _paths()
    out_dir = root / "bin"
    out_dir.mkdir(exist_ok=True)
    inc = [CSRC / "include", CSRC] + p["torch_inc"] + [p["cuda_home"] / "include"] + extra_inc
    built = []
    for src in sorted(root.glob("*.cpp")):
        exe = out_dir / (names or {}).get(src.stem, src.stem)
        # up to date = same program source and same headers as when it was compiled (content, not time stamps, which
        # a copy of the tree does not keep); the library itself is linked dynamically
        stamp = out_dir / (exe.name + ".stamp")
        digest = _sources_digest([src, *root.glob("*.h"), *(f for f in (CSRC / "include").rglob("*.h"))])
        if exe.exists() and stamp.exists() and stamp.read_text() == digest:
            built.append(str(exe))
            continue
        cmd = [os.environ.get("CS_CXX", "g++"), "-std=c++20", "-O2", "-Wno-interference-size",
               f"-D_GLIBCXX_USE_CXX11_ABI={p['cxx11_abi']}", "-DUSE_C10D_NCCL", "-DUSE_DISTRIBUTED"]
        cmd += [f"-I{i}" for i in inc] + [str(src), "-o", str(exe), f"-L{LIBDIR}", "-lcs_b200", f"-L{p['torch_lib']}",
                "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", f"-L{p['cuda_home'] / 'lib64'}", "-lcudart",
                f"-Wl,-rpath,{LIBDIR}", f"-Wl,-rpath,{p['torch_lib']}", f"-Wl,-rpath,{p['arrow_lib']}", "-Wl,--no-as-needed"]
        subprocess.run(cmd, check=True)
        stamp.write_text(digest)
        built.append(str(exe))
    return built


def build_sanitized(kind: str = "address") -> list[str]:
    """Host-side race and memory checks: compiles the C++ sources (not the kernels) with AddressSanitizer and
    UndefinedBehaviorSanitizer (kind "address") or with ThreadSanitizer (kind "thread") into lib_asan/ or lib_tsan/
    and links the two C++ test programs against it (tests/cpp/bin/*_asan, *_tsan). Run them on the CPU, e.g.
        ASAN_OPTIONS=detect_leaks=0:protect_shadow_gap=0 tests/cpp/bin/cs_b200_communication_tests_asan --threads 4
        TSAN_OPTIONS=suppressions=tests/cpp/tsan.supp tests/cpp/bin/cs_b200_communication_tests_tsan --threads 4
    (scheduler queues, rank-thread communicator, bucket logic, data-loader threads, module tree)."""
    assert kind in ("address", "thread")
    tag = "asan" if kind == "address" else "tsan"
    p = _paths()
    generate_ninja()
    subprocess.run([sys.executable, "-m", "ninja", "-f", str(BUILD / "build.ninja"), str(LIBDIR / "libcs_b200.so")], check=True, cwd=str(BUILD))
    out = HERE / f"lib_{tag}"
    out.mkdir(exist_ok=True)
    extra_cpp, extra_cu = _optional_sources()
    inc = [CSRC / "include", CSRC, CSRC / "src"] + p["torch_inc"] + [p["cuda_home"] / "include"]
    san = [("-fsanitize=address,undefined" if kind == "address" else "-fsanitize=thread"), "-fno-omit-frame-pointer", "-g", "-O1"]
    base = [os.environ.get("CS_CXX", "g++"), "-std=c++20", "-fPIC", "-Wno-interference-size", "-Wno-deprecated-declarations",
            f"-D_GLIBCXX_USE_CXX11_ABI={p['cxx11_abi']}", "-DUSE_C10D_NCCL", "-DUSE_DISTRIBUTED", "-DUSE_RPC", "-DUSE_CUDA"] + [f"-I{i}" for i in inc]
    objs = []
    jobs = []
    for src in CPP_SOURCES + extra_cpp:
        obj = BUILD / (src.replace("/", "_") + f".{tag}.o")
        extra = [f"-I{p['arrow_inc']}"] if src.endswith("parquet_io.cpp") else ([f"-I{p['nccl_inc']}"] if src.endswith("comm_nccl.cpp") else [])
        if not obj.exists() or obj.stat().st_mtime < (CSRC / src).stat().st_mtime:
            jobs.append(subprocess.Popen(base + san + extra + ["-c", str(CSRC / src), "-o", str(obj)]))
        objs.append(str(obj))
    for j in jobs:
        if j.wait() != 0:
            raise RuntimeError("sanitized compile failed")
    objs += [str(BUILD / (src.replace("/", "_") + ".o")) for src in CUDA_SOURCES + extra_cu]  # kernels as they are
    cuda_lib = p["cuda_home"] / "lib64"
    lib = out / "libcs_b200.so"
    subprocess.run([base[0], "-shared", *san, *objs, "-o", str(lib), f"-L{p['torch_lib']}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10",
                    "-lc10_cuda", f"-L{p['arrow_lib']}", "-l:libarrow.so.2400", "-l:libparquet.so.2400", f"-L{cuda_lib}", "-lcudart", "-ldl",
                    "-lpthread", f"-Wl,-rpath,{p['torch_lib']}", f"-Wl,-rpath,{p['arrow_lib']}", f"-Wl,-rpath,{cuda_lib}", "-Wl,--no-as-needed",
                    "-Wl,-soname,libcs_b200.so"], check=True)
    root = HERE.parent / "tests" / "cpp"
    (root / "bin").mkdir(exist_ok=True)
    built = []
    for stem, name in (("test_ops", f"cs_b200_tests_{tag}"), ("test_communication", f"cs_b200_communication_tests_{tag}")):
        exe = root / "bin" / name
        subprocess.run(base + san + [f"-I{root}", str(root / f"{stem}.cpp"), "-o", str(exe), f"-L{out}", "-lcs_b200", f"-L{p['torch_lib']}",
                                     "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", f"-L{cuda_lib}", "-lcudart",
                                     f"-Wl,-rpath,{out}", f"-Wl,-rpath,{p['torch_lib']}", f"-Wl,-rpath,{p['arrow_lib']}", "-Wl,--no-as-needed"],
                       check=True)
        built.append(str(exe))
    return built


def is_checked_built() -> bool:
    return (CHECKED_LIBDIR / "libcs_b200.so").exists()


def is_built() -> bool:
    return (HERE / f"_C{ext_suffix()}").exists() and (LIBDIR / "libcs_b200.so").exists()


if __name__ == "__main__":
    if "examples" in sys.argv:
        print("\n".join(build_examples()))
    elif "tests" in sys.argv:
        print("\n".join(build_cpp_tests()))
    elif "sanitize" in sys.argv:
        print("\n".join(build_sanitized("thread" if "thread" in sys.argv else "address")))
    else:
        build(verbose="-v" in sys.argv, checked="checked" in sys.argv)
