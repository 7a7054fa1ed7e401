# SPDX-License-Identifier: Apache-2.0
"""Plumbing of the reference arm that can be checked without a GPU: the MPI stand-in and bench.py's fallback line."""
import json
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_mpi_stand_in_broadcast_and_max_over_ranks(tmp_path):
    src = tmp_path / "t.c"
    src.write_text(textwrap.dedent("""
        #include <mpi.h>
        #include <stdio.h>
        int main(int argc, char **argv) {
          MPI_Init(&argc, &argv);
          int rank, size;
          MPI_Comm_rank(MPI_COMM_WORLD, &rank);
          MPI_Comm_size(MPI_COMM_WORLD, &size);
          char text[16] = "none";
          uint16_t port = 0;
          if (rank == 0) { snprintf(text, sizeof(text), "10.1.2.3"); port = 29541; }
          MPI_Bcast(text, 16, MPI_CHAR, 0, MPI_COMM_WORLD);
          MPI_Bcast(&port, 1, MPI_UINT16_T, 0, MPI_COMM_WORLD);
          double v = 1.5 * (rank + 1);
          MPI_Shim_max_double(&v);
          MPI_Barrier(MPI_COMM_WORLD);
          printf("R %d/%d %s %d %.1f\\n", rank, size, text, (int)port, v);
          MPI_Finalize();
          return 0;
        }
    """))
    exe = tmp_path / "t"
    shim = os.path.join(ROOT, "baseline", "shims")
    subprocess.run(["gcc", "-O1", f"-I{shim}", str(src), os.path.join(shim, "mpi_shim.c"), "-o", str(exe)], check=True)
    env = dict(os.environ, CS_MPISHIM_KEY=f"test{os.getpid()}")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "launch.py"), "--nproc", "3", "--master-port", "29876", "--",
                          str(exe)], env=env, capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    lines = sorted(l for l in out.stdout.splitlines() if l.startswith("R "))
    assert lines == [f"R {r}/3 10.1.2.3 29541 4.5" for r in range(3)]
    leftovers = [f for f in os.listdir("/tmp") if f.startswith(f"cs_mpishim_test{os.getpid()}_")]
    assert leftovers == []  # every rank removed the files it published


def test_reference_arm_prints_one_json_line_and_exits_zero_without_a_gpu():
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "2", "--warmup", "3"],
                         env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    assert "unavailable" in line or line["metric"].startswith("GPT-2 train tokens/sec")
    zero = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--mode", "zero"], env=env,
                          capture_output=True, text=True, timeout=300)
    assert zero.returncode == 0 and "unavailable" in json.loads(zero.stdout.strip().splitlines()[-1])


def test_reference_dataset_has_the_layout_the_reference_loader_scans():
    """The reference's loader projects `input_ids` and `labels`, asks for batches of the micro-batch size, casts each
    column to a list array of int32/int64 and takes the sequence length from the first row (src/data/dataloader.cpp)."""
    import importlib.util
    import shutil

    import pyarrow as pa
    import pyarrow.dataset as ds

    spec = importlib.util.spec_from_file_location("cs_bench", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    directory = bench.write_reference_dataset(4, 32, 512, 3, f"test{os.getpid()}", batches_per_rank=5)
    try:
        files = sorted(os.listdir(directory))
        assert files == ["train.parquet"]
        scanner = ds.dataset([os.path.join(directory, files[0])], format="parquet").scanner(
            columns=["input_ids", "labels"], batch_size=4, batch_readahead=0)
        batches = list(scanner.to_batches())
        assert len(batches) == 5 * 3  # every rank's shard holds `batches_per_rank` whole batches
        for batch in batches:
            for column in (batch.column(0), batch.column(1)):
                assert isinstance(column, pa.ListArray) and column.type.value_type == pa.int64()
                assert len(column) == 4 and set(column.value_lengths().to_pylist()) == {32}
            tokens = batch.column(0).values.to_numpy().reshape(4, 32)
            labels = batch.column(1).values.to_numpy().reshape(4, 32)
            assert (tokens[:, 1:] == labels[:, :-1]).all() and 0 <= tokens.min() and max(tokens.max(), labels.max()) < 512
    finally:
        shutil.rmtree(directory, ignore_errors=True)
