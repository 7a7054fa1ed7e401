# SPDX-License-Identifier: Apache-2.0
"""Headline benchmark: GPT-2 training tokens/sec (device-timed, max over ranks) on N GPUs of one node.

  python bench.py --gpus 1 --steps 10 --warmup 3
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
      bench.py --gpus N --steps K --warmup W

Prints ONE JSON line from rank 0. `value` is the whole-job tokens/sec with inputs already on the
device; `e2e` repeats the measurement through the public data-loading path (pinned host buffers ->
H2D copy every step, loss read back to the host every step).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "GPT-2 train tokens/sec, device-timed max over ranks"


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--model", default="124M")
    p.add_argument("--micro-batch", type=int, default=16)
    p.add_argument("--seq-len", type=int, default=1024)
    p.add_argument("--mode", default="dp", choices=["dp", "zero", "tp"])
    p.add_argument("--backend", default="fused", choices=["fused", "library"])
    p.add_argument("--bucket-mb", type=float, default=25.0)
    p.add_argument("--comm", default="nvp2p", choices=["nvp2p", "nccl"],
                   help="gradient collectives: this library's peer-memory kernels, or NCCL")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-overlap-optimizer", action="store_true",
                   help="one whole-model AdamW launch after the backward pass instead of per-bucket updates during it")
    p.add_argument("--assist-gap", type=int, default=2, help="main-stream tasks after which an assist-stream task is re-joined")
    p.add_argument("--comm-gap", type=int, default=5, help="main-stream tasks after which a communication task is re-joined")
    p.add_argument("--profile", action="store_true", help="print per-task device time of one step (not a bench value)")
    p.add_argument("--trace", default="", help="with --profile: also write that step as a chrome trace (JSON) to this file")
    return p.parse_args()


def write_reference_dataset(batch, seq_len, vocab, world, tag, batches_per_rank=8):
    """Writes one Parquet file in the layout the reference's LlmDataLoader scans (list<int64> columns `input_ids`
    and `labels`, one row per sequence, one row group per batch) with uniform random token ids, and returns its
    directory. `batches_per_rank` batches per rank are enough: the loader wraps around at the end of its shard."""
    import tempfile

    import numpy as np
    import pyarrow as pa
    import pyarrow.parquet as pq

    rows = batch * batches_per_rank * world
    rng = np.random.default_rng(20240611)
    ids = rng.integers(0, vocab, size=(rows, seq_len + 1), dtype=np.int64)
    offsets = np.arange(rows + 1, dtype=np.int32) * seq_len
    columns = [pa.ListArray.from_arrays(pa.array(offsets), pa.array(np.ascontiguousarray(part).reshape(-1)))
               for part in (ids[:, :-1], ids[:, 1:])]
    directory = os.path.join(tempfile.gettempdir(), f"cs_ref_dataset_{tag}")
    os.makedirs(directory, exist_ok=True)
    pq.write_table(pa.table(columns, names=["input_ids", "labels"]), os.path.join(directory, "train.parquet"), row_group_size=batch)
    return directory


def reference_arm(args):
    """Runs the unmodified reference library (built by baseline/build_reference.py into baseline/_ref/) through
    its own public API: baseline/_ref/ref_gpt2 is a GPT-2 driver that links only that library. One driver process
    per rank; it times K steps on the device between two full synchronisations and takes the max over ranks."""
    import subprocess

    here = os.path.dirname(os.path.abspath(__file__))
    exe = os.path.join(here, "baseline", "_ref", "ref_gpt2")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not os.path.exists(exe):
        if rank == 0:
            print(json.dumps({"impl": "reference",
                              "unavailable": "baseline/_ref/ref_gpt2 is not built: run python baseline/build_reference.py "
                                             "(the reference is a CMake C++ project; pip install of it is not possible)"}))
        return 0
    if args.mode != "dp":
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"the reference has no {args.mode} mode (data parallel only)"}))
        return 0
    # the clock sampler is loaded by file so that nothing of this repository's package (and none of its
    # native libraries) is imported into the reference arm's processes
    import importlib.util

    spec = importlib.util.spec_from_file_location("cs_clocks", os.path.join(here, "core_scheduler_b200", "utils", "clocks.py"))
    clocks_mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(clocks_mod)
    ClockSampler = clocks_mod.ClockSampler

    env = dict(os.environ, CS_MPISHIM_KEY=f"{os.getppid()}")
    cmd = [exe, "--model", args.model, "--micro-batch", str(args.micro_batch), "--seq", str(args.seq_len), "--steps", str(args.steps),
           "--warmup", str(args.warmup), "--bucket-mb", str(args.bucket_mb)]
    dataset_dir = None
    if not args.no_e2e:
        # end-to-end arm: the reference's own data path reads Parquet files, so every rank writes the same
        # synthetic file (same seed) into a directory of its own and the loader shards it by rank
        try:
            dataset_dir = write_reference_dataset(args.micro_batch, args.seq_len, 512 if args.model == "tiny" else 50257, world,
                                                  f"{os.getppid()}_{rank}")
            cmd += ["--dataset", dataset_dir]
        except Exception as e:  # no pyarrow, no space: the device-timed number does not depend on it
            print(f"reference arm: no end-to-end dataset ({e})", file=sys.stderr)
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0"))) if rank == 0 else None
    if sampler:
        sampler.start()
    proc = subprocess.run(cmd, env=env, capture_output=True, text=True)
    clocks = sampler.stop() if sampler else None
    if dataset_dir:
        import shutil

        shutil.rmtree(dataset_dir, ignore_errors=True)
    if os.environ.get("CS_REF_LOG"):  # keep the driver's full output for diagnosis
        with open(f"{os.environ['CS_REF_LOG']}.rank{rank}", "w") as f:
            f.write(proc.stdout + proc.stderr)
    line = next((l for l in proc.stdout.splitlines() if l.startswith("REF_RESULT")), None)
    if rank != 0:
        return 0  # a failed rank shows on rank 0 as a missing result line
    if line is None:
        text = [l for l in (proc.stdout + proc.stderr).strip().splitlines() if "Warning" not in l and not l.startswith("frame #")]
        tail = text[-3:]
        print(json.dumps({"impl": "reference", "unavailable": "reference driver failed: " + " | ".join(tail)[:400]}))
        return 0
    fields = dict(kv.split("=") for kv in line.split()[1:])
    ms = float(fields["ms_per_step"])
    e2e = None
    e2e_line = next((l for l in proc.stdout.splitlines() if l.startswith("REF_E2E")), None)
    if e2e_line:
        f2 = dict(kv.split("=") for kv in e2e_line.split()[1:])
        e2e = {"value": float(f2["tokens_per_s"]), "unit": "tokens/s", "ms_per_step": float(f2["ms_per_step"]),
               "h2d_bytes_per_step": int(f2["h2d_bytes"]), "d2h_bytes_per_step": int(f2["d2h_bytes"]),
               "path": "reference LlmDataset + LlmDataLoader (Parquet -> pinned host -> device), loss read back every step"}
    print(json.dumps({
        "metric": "GPT-2 train tokens/sec, device-timed max over ranks", "value": float(fields["tokens_per_s"]), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform token ids, random-init weights N(0,0.02)", "impl": "reference",
        "config": config_labels(args, world, False),
        "implementation": {"precision": "fp32 parameters under a bf16 autocast guard",
                           "backend": "reference library (cuBLAS / ATen / flash attention / NCCL), unmodified sources"},
        "final_loss": float(fields["final_loss"]), "clocks": clocks, "e2e": e2e, "gpu_launches": None}))
    return 0


def make_trainer(args, cs, comm, world, local_rank):
    """The training step a user of the package gets: core_scheduler_b200.parallel.GPT2Trainer."""
    from core_scheduler_b200.models import gpt2_config
    from core_scheduler_b200.parallel import GPT2Trainer

    scheduler = cs.DynamicScheduler(local_rank, device="cuda", assist_task_gap=args.assist_gap, comm_task_gap=args.comm_gap)
    cs._C.set_backend(args.backend)
    trainer = GPT2Trainer(gpt2_config(args.model, dtype=torch.float32), comm, world, local_rank, mode=args.mode, collectives=args.comm,
                          device="cuda", lr=3e-4, beta1=0.9, beta2=0.95, weight_decay=0.1, bucket_mb=args.bucket_mb, seed=1234,
                          scheduler=scheduler, overlap_optimizer=not args.no_overlap_optimizer,
                          max_tokens=args.micro_batch * args.seq_len)
    trainer.s, trainer.cfg = scheduler, trainer.config
    trainer.tp = args.mode == "tp" and world > 1
    return trainer


def config_labels(args, world, tensor_parallel):
    """The workload description, identical for both arms when the workload is identical."""
    return {"model": f"GPT-2 {args.model}", "global_batch": args.micro_batch * (1 if tensor_parallel else world),
            "micro_batch_per_gpu": args.micro_batch, "seq_len": args.seq_len, "parallelism": f"{args.mode}{world}",
            "bucket_mb": args.bucket_mb, "l2": "per-step working set exceeds the 126 MB L2; no flush needed"}


def max_over_ranks(value: float, world: int) -> float:
    if world <= 1:
        return value
    import torch.distributed as dist

    t = torch.tensor([value], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world: int):
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
    torch.cuda.synchronize()


def main():
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if not torch.cuda.is_available():
        print(json.dumps({"metric": METRIC, "error": "no CUDA device visible"}))
        return 1
    import core_scheduler_b200 as cs
    from core_scheduler_b200.parallel import init_distributed
    from core_scheduler_b200.utils.clocks import ClockSampler

    comm, rank, world, local_rank = init_distributed("cuda")
    torch.cuda.set_device(local_rank)
    C = cs._C
    trainer = make_trainer(args, cs, comm, world, local_rank)
    B, T = args.micro_batch, args.seq_len
    vocab = trainer.cfg.vocab_size

    # ---- device-resident inputs for the kernel-level number (a few distinct batches) -------------
    gen = torch.Generator(device="cuda").manual_seed(1000 + (0 if trainer.tp else rank))
    batches = []
    for _ in range(4):
        ids = torch.randint(0, vocab, (B, T + 1), generator=gen, device="cuda")
        batches.append((cs.from_torch(ids[:, :-1].contiguous()), cs.from_torch(ids[:, 1:].contiguous())))

    for i in range(args.warmup):
        loss = trainer.step(*batches[i % len(batches)])
        if i == 0:
            trainer.s.synchronize()
            trainer.check_device_status()  # a broken configuration shows in the first step: stop before timing anything
    trainer.s.synchronize()
    barrier(world)
    if args.profile:
        trainer.s.set_profiling(True)
        trainer.step(*batches[0])
        rows = trainer.s.drain_timings()
        trainer.s.set_profiling(False)
        if rank == 0:
            agg = {}
            for r in rows:
                a = agg.setdefault((r.name, r.stream_class), [0, 0.0])
                a[0] += 1
                a[1] += r.device_ms
            total = sum(v[1] for v in agg.values())
            print(f"per-task device time of one step (sum over streams {total:.3f} ms; tasks overlap across streams)", file=sys.stderr)
            for (name, cls), (n, ms) in sorted(agg.items(), key=lambda kv: -kv[1][1]):
                print(f"  {ms:8.3f} ms  x{n:4d}  stream{cls}  {name}", file=sys.stderr)
            if args.trace:
                from core_scheduler_b200.utils.trace import write_chrome_trace

                print(f"wrote {write_chrome_trace(rows, args.trace)} task events to {args.trace}", file=sys.stderr)

    sampler = ClockSampler(local_rank).start() if rank == 0 else None
    launches_before = C.kernel_launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    main_stream = torch.cuda.ExternalStream(trainer.s.raw_stream(0))
    start.record(main_stream)
    for i in range(args.steps):
        loss = trainer.step(*batches[i % len(batches)])
    trainer.s.synchronize()  # every stream drained (optimizer runs on the assist stream)
    stop.record(main_stream)
    torch.cuda.synchronize()
    launches = C.kernel_launch_count() - launches_before
    device_ms = start.elapsed_time(stop)
    trainer.check_device_status()  # a kernel that gave up on a bounded wait makes the measurement void: fail loudly
    barrier(world)
    clocks = sampler.stop() if sampler else None
    device_ms = max_over_ranks(device_ms, world)
    final_loss = float(cs.to_torch(trainer.s, loss).item())
    # Random tokens keep the loss near ln(vocabulary) (10.8 for GPT-2); a step whose numbers went wrong (a buffer read
    # before it was complete, ranks disagreeing on an offset) shows up here long before it shows in the timing.
    if not math.isfinite(final_loss) or final_loss > 1.5 * math.log(vocab):
        raise RuntimeError(f"loss {final_loss} after {args.warmup + args.steps} steps is not that of a working training step "
                           f"(expected about ln({vocab}) = {math.log(vocab):.2f}); the measurement is void")

    tokens_per_step = B * T * (1 if trainer.tp else world)  # tensor parallel ranks share one global batch
    ms_per_step = device_ms / args.steps
    value = tokens_per_step / (ms_per_step / 1e3)

    # ---- end to end: pinned host staging + H2D every step, loss read back every step ----------------
    e2e = None
    if not args.no_e2e:
        loader = C.SyntheticDataLoader(B, T, vocab, seed=77 + (0 if trainer.tp else rank))
        for _ in range(2):
            d = loader.load(trainer.s)
            float(cs.to_torch(trainer.s, trainer.step(d["input_ids"], d["labels"])).item())
        trainer.s.synchronize()
        barrier(world)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            d = loader.load(trainer.s)
            loss = trainer.step(d["input_ids"], d["labels"])
            float(cs.to_torch(trainer.s, loss).item())
        trainer.s.synchronize()
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3
        e2e_ms = max_over_ranks(e2e_ms, world)
        e2e = {
            "value": tokens_per_step / (e2e_ms / args.steps / 1e3),
            "unit": "tokens/s",
            "ms_per_step": e2e_ms / args.steps,
            "h2d_bytes_per_step": loader.bytes_per_batch(),
            "d2h_bytes_per_step": 4,
        }

    if rank == 0:
        weights_gb = trainer.cfg.parameter_count() * (4 + 2 + 2) / 1e9
        out = {
            "metric": METRIC,
            "value": value,
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": ms_per_step,
            "higher_is_better": True,
            "scaling": "strong" if trainer.tp else "weak",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic uniform token ids, random-init weights N(0,0.02)",
            "impl": "ours",
            "config": config_labels(args, world, trainer.tp),
            "implementation": {
                "parameters": f"{trainer.cfg.parameter_count() / 1e6:.1f}M, untied lm_head",
                "precision": "bf16 compute, fp32 master weights + AdamW moments",
                "backend": args.backend,
                "scheduler_gaps": {"assist": args.assist_gap, "comm": args.comm_gap},
                "collectives": (args.comm if world > 1 else "none"),
                "optimizer": "per-bucket AdamW overlapped with backward" if not args.no_overlap_optimizer and args.mode != "zero" else "after backward",
                "working_set": f"~{weights_gb:.1f} GB weights/optimizer + activations per step",
                "library_fallbacks": int(C.library_fallbacks()),
            },
            "final_loss": final_loss,
            "mfu_vs_measured_sustained": None,
            "clocks": clocks,
            "e2e": e2e,
            "gpu_launches": int(launches),
        }
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
            flops = trainer.cfg.train_flops_per_token(T) * value / world
            out["mfu_vs_measured_sustained"] = flops / (peaks["bf16_tflops_sustained"] * 1e12)
        except Exception:
            pass
        print(json.dumps(out))
    if world > 1:
        import torch.distributed as dist

        del batches, loss
        trainer.close()
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
