# SPDX-License-Identifier: Apache-2.0
"""Collective microbenchmark: all-reduce, all-gather, reduce-scatter, all-to-all on bf16 tensors.

  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
      -m core_scheduler_b200.utils.collective_bench [--max-mb 1024] [--backends nccl,nvp2p]

For every message size (powers of two from 1 KiB) and both back-ends (NCCL through torch.distributed's
process group, and this library's peer-memory kernels) it reports the device time (CUDA events on
the comm stream, max over ranks, median of the iterations after warm-up) and the bus bandwidth
  all-reduce      2 (N-1)/N * S / t
  all-gather      (N-1)/N * S / t        (S = gathered bytes)
  reduce-scatter  (N-1)/N * S / t        (S = bytes before the reduction)
  all-to-all      (N-1)/N * S / t
next to the NVLink reference figures (900 GB/s nominal, 770 GB/s measured peer copy per direction). The SM clock
and the throttle reasons of GPU 0 are sampled during the whole run and printed with the results.
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys

import torch
import torch.distributed as dist

import core_scheduler_b200 as cs
from core_scheduler_b200.parallel import init_distributed
from core_scheduler_b200.utils.clocks import ClockSampler

C = cs._C
BF = torch.bfloat16


def timed(s, comm_stream, fn, iters, warmup):
    for _ in range(warmup):
        fn()
    s.synchronize()
    times = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(comm_stream)
        fn()
        b.record(comm_stream)
        s.synchronize()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    t = torch.tensor([statistics.median(times)], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--max-mb", type=int, default=1024)
    p.add_argument("--backends", default="nccl,nvp2p")
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--min-mb", type=float, default=0.0, help="first message size (default 1 KiB)")
    p.add_argument("--grid-cap", type=int, default=0, help="most blocks per collective launch (library default when 0)")
    p.add_argument("--multicast-min-ranks", type=int, default=0,
                   help="smallest group that uses the multicast mapping (library default when 0)")
    args = p.parse_args()
    if args.grid_cap:
        C.set_collective_grid_cap(args.grid_cap)
    if args.multicast_min_ranks:
        C.set_multicast_min_ranks(args.multicast_min_ranks)
    comm_nccl, rank, world, local_rank = init_distributed("cuda")
    assert world > 1, "launch with torch.distributed.run on at least 2 GPUs"
    s = cs.DynamicScheduler(local_rank, device="cuda")
    comm_stream = torch.cuda.ExternalStream(s.raw_stream(2))
    pg = dist.distributed_c10d._get_default_group()
    comm_p2p = C.comm_from_process_group(pg.group_name, "cuda", True)
    max_bytes = args.max_mb << 20
    ctx = C.create_symmetric_context(comm_p2p, 3 * max_bytes + (64 << 20))
    comms = {"nccl": comm_nccl, "nvp2p": comm_p2p}
    multicast_used = ctx.has_multicast and world >= C.multicast_min_ranks()
    memory = "multicast" if multicast_used else ("peer mappings (cuMemCreate)" if ctx.virtual_memory else "peer mappings (CUDA IPC)")
    if rank == 0:
        print(f"world {world}; symmetric arena: {memory}; grid cap {C.collective_grid_cap()}", flush=True)
    sampler = ClockSampler(local_rank).start() if rank == 0 else None
    results = []
    size = max(1024, int(args.min_mb * (1 << 20)))
    while size <= max_bytes:
        n = size // 2  # bf16 elements
        chunk = max(8, (n // world) // 8 * 8)
        for backend in args.backends.split(","):
            comm = comms[backend]
            if backend == "nvp2p":
                buf, off, nb = ctx.empty([chunk * world], BF)
                out_buf, off2, nb2 = ctx.empty([chunk * world], BF)
            else:
                buf = torch.empty(chunk * world, device="cuda", dtype=BF)
                out_buf = torch.empty(chunk * world, device="cuda", dtype=BF)
            buf.normal_()
            x = cs.from_torch(buf)
            parts_in = [cs.from_torch(buf[i * chunk:(i + 1) * chunk]) for i in range(world)]
            parts_out = [cs.from_torch(out_buf[i * chunk:(i + 1) * chunk]) for i in range(world)]
            shard = cs.from_torch(out_buf[:chunk])
            cases = {
                "all_reduce": (lambda: C.all_reduce(s, comm, [x], "sum"), 2.0),
                "all_gather": (lambda: C.all_gather(s, comm, [parts_out], [parts_in[rank]]), 1.0),
                "reduce_scatter": (lambda: C.reduce_scatter(s, comm, [shard], [parts_in], "sum"), 1.0),
                "all_to_all": (lambda: C.all_to_all(s, comm, parts_out, parts_in), 1.0),
            }
            for name, (fn, factor) in cases.items():
                ms = timed(s, comm_stream, fn, args.iters, 3)
                total = chunk * world * 2
                bus = factor * (world - 1) / world * total / (ms * 1e-3) / 1e9
                results.append({"op": name, "backend": backend, "bytes": total, "ms": ms, "bus_gbs": bus})
                if rank == 0:
                    print(f"{name:15s} {backend:6s} {total:>12d} B  {ms * 1e3:10.1f} us  bus {bus:8.1f} GB/s "
                          f"({bus / 900:.2f} of 900 nominal, {bus / 770:.2f} of 770 measured copy)", flush=True)
            if backend == "nvp2p":
                ctx.release(off, nb)
                ctx.release(off2, nb2)
            ctx.check_status()
        size *= 4 if size < (1 << 20) else 2
    if rank == 0:
        clocks = sampler.stop()
        print("clocks during the run:", json.dumps(clocks))
        print(json.dumps({"world": world, "memory": memory, "grid_cap": C.collective_grid_cap(), "clocks": clocks, "results": results}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
